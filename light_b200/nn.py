"""The two layer types whose forward pass chooses among the quantized matmuls: the host-side mirror of the
reference's nn.Linear (nn/linear.go:193-354, 476-516) and nn.SparseMoE (nn/moe.go:121-245).

They carry no kernels of their own.  Each forward checks what the reference checks, in the reference's words, and
dispatches to one `ops` call per weight kind:

    weight                       call                       reference branch
    GGUF block-quantized         ops.MatMulQ                nn/linear.go:273-280
    4-bit GPTQ / AWQ (W4)        ops.MatMulInt4             nn/linear.go:476-516
    FP8 with block scales        ops.MatMulF8Block          nn/linear.go:255-258
    F32 / BF16 / F16             the library GEMM           nn/linear.go:300-330

The dense branch is a plain library GEMM on the device, as it is in the reference (cuBLAS); everything else is this
package's own kernels.  LoRA adapters, autograd and per-tensor FP8 (the cuBLASLt FP8 GEMM) are outside this path.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence, Tuple, Union

import torch

from . import ops


@dataclass
class Linear:
    """y = x @ W^T + b.  Exactly one of `W` (dense tensor or ops.QTensor) and `W4` (ops.Int4) is set."""
    in_features: int
    out_features: int
    W: Union[torch.Tensor, ops.QTensor, None] = None
    B: Optional[torch.Tensor] = None
    W4: Optional[ops.Int4] = None
    WBlockScale: Optional[torch.Tensor] = None
    WBlock: Tuple[int, int] = (0, 0)

    def set_weight(self, w) -> None:
        """Linear.SetWeight: shape-checked install of a dense or block-quantized weight."""
        shape = tuple(w.shape)
        if shape != (self.out_features, self.in_features):
            raise ValueError(f"nn.Linear.SetWeight: weight {shape}, want ({self.out_features}, {self.in_features})")
        self.W, self.W4 = w, None

    def set_int4(self, w: ops.Int4) -> None:
        """Linear.SetInt4."""
        if (w.N(), w.K()) != (self.out_features, self.in_features):
            raise ValueError(f"nn.Linear.SetInt4: weight ({w.N()}, {w.K()}), want ({self.out_features}, {self.in_features})")
        self.W4, self.W = w, None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.W4 is not None:
            return self._forward_int4(x)
        if self.W is None:
            raise ValueError(f"nn.Linear: weight not loaded (placeholder layer {self.in_features}→{self.out_features})")
        wdev = self.W.device
        if x.device != wdev:
            raise ValueError(f"nn.Linear: x on {x.device} but W on {wdev}")
        if x.dim() < 1 or x.shape[-1] != self.in_features:
            raise ValueError(f"nn.Linear: last dim of x ({x.shape[-1] if x.dim() else 0}) != in_features ({self.in_features})")
        quantized = isinstance(self.W, ops.QTensor)
        if quantized and x.dtype != torch.float32:
            raise ValueError(f"nn.Linear: quantized weight ({ops.GGUF_NAMES[self.W.ggml_type]}) needs F32 activations, got {x.dtype}")
        fp8 = (not quantized) and self.W.dtype == torch.float8_e4m3fn
        if fp8 and self.WBlockScale is None:
            raise ValueError("nn.Linear: per-tensor FP8 weights run the library's FP8 GEMM in the reference; only block-scaled FP8 is built here")
        if fp8 and x.dtype == torch.float16:
            raise ValueError("nn.Linear: block-scaled FP8 needs F32 or BF16 activations, got F16")
        if fp8 and x.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"nn.Linear: F8E4M3 weight needs F32/BF16/F16 activations, got {x.dtype}")
        w16 = (not quantized) and x.dtype == torch.float32 and self.W.dtype in (torch.bfloat16, torch.float16)
        if not quantized and not fp8 and not w16 and x.dtype != self.W.dtype:
            raise ValueError(f"nn.Linear: x dtype {x.dtype} != W dtype {self.W.dtype} — cast at the boundary, not inside the layer")
        flat = x.reshape(-1, self.in_features).contiguous()
        bias_done = False
        if fp8:
            y = ops.MatMulF8Block(flat, self.W, self.WBlockScale, self.WBlock[0], self.WBlock[1])
        elif quantized:
            y = ops.MatMulQ(flat, self.W)
        elif w16:
            y = flat @ self.W.float().t()          # the 16-bit weight widened exactly, F32 arithmetic (ops.MatMulW16)
        elif self.B is not None and self.W.dtype == torch.bfloat16:
            # one rounding for x W^T + b (nn/linear.go:312-322): F32 product, F32 bias add, then BF16
            y = (torch.mm(flat, self.W.t(), out_dtype=torch.float32) + self.B.float()).to(torch.bfloat16)
            bias_done = True
        else:
            y = flat @ self.W.t()
        if self.B is not None and not bias_done:
            y = y + self.B
        return y.reshape(*x.shape[:-1], self.out_features)

    def _forward_int4(self, x: torch.Tensor) -> torch.Tensor:
        w = self.W4
        if x.device != w.codes.device:
            raise ValueError(f"nn.Linear: x on {x.device} but the 4-bit weight on {w.codes.device}")
        if x.dim() < 1 or x.shape[-1] != self.in_features:
            raise ValueError(f"nn.Linear: last dim of x ({x.shape[-1] if x.dim() else 0}) != in_features ({self.in_features})")
        flat = x.reshape(-1, self.in_features)
        inp = flat.float() if (self.B is not None and x.dtype == torch.bfloat16) else flat   # bias added before the one rounding
        y = ops.MatMulInt4(inp, w)
        if self.B is not None:
            y = (y + self.B.to(y.dtype)).to(x.dtype)
        return y.reshape(*x.shape[:-1], self.out_features)


@dataclass
class SparseMoE:
    """Routed gated-MLP block (nn/moe.go:27-60).  `GateUp` (E, 2 I, H) holds every expert's gate rows then up rows,
    `Down` (E, H, I); both dense tensors at the activation dtype or ops.QTensor (then activations are F32).
    Block-scaled FP8 experts carry `GateUpScale` / `DownScale` with `Block`.  `GateUpQ4` / `DownQ4` are per-expert 4-bit
    weights instead.  `Router`, when set, maps the (T, E) F32 router logits to an ops.MoERouting (the group-limited and
    sigmoid-with-bias routers); otherwise softmax + top-k."""
    Gate: Linear
    GateUp: Union[torch.Tensor, ops.QTensor, None] = None
    Down: Union[torch.Tensor, ops.QTensor, None] = None
    TopK: int = 1
    NormTopK: bool = False
    Gelu: bool = False
    RouterF32: bool = False
    Router: Optional[Callable[[torch.Tensor], ops.MoERouting]] = None
    GateUpQ4: Optional[Sequence[ops.Int4]] = None
    DownQ4: Optional[Sequence[ops.Int4]] = None
    GateUpScale: Optional[torch.Tensor] = None
    DownScale: Optional[torch.Tensor] = None
    Block: Tuple[int, int] = (0, 0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        H = self.Gate.in_features
        if x.shape[-1] != H:
            raise ValueError(f"nn.SparseMoE: last dim {x.shape[-1]} != hidden {H}")
        flat = x.contiguous().reshape(-1, H)
        gate_in = flat.float() if (self.RouterF32 and flat.dtype != torch.float32) else flat
        route = self.route(gate_in)
        if self.GateUpQ4 is not None:
            return ops.MoEInt4(flat, self.GateUpQ4, self.DownQ4, route, self.TopK, self.Gelu).reshape(x.shape)
        return self.run_experts(flat, route).reshape(x.shape)

    def route(self, gate_in: torch.Tensor) -> ops.MoERouting:
        logits = self.Gate.forward(gate_in).float()
        if self.Router is not None:
            return self.Router(logits)
        return ops.MoERoute(torch.softmax(logits, -1), self.TopK, self.NormTopK)

    def run_experts(self, flat: torch.Tensor, route: ops.MoERouting) -> torch.Tensor:
        gu, dn = self.GateUp, self.Down
        quantized = isinstance(gu, ops.QTensor)
        if quantized and flat.dtype != torch.float32:
            raise ValueError(f"nn.SparseMoE: quantized experts ({ops.GGUF_NAMES[gu.ggml_type]}) need F32 activations, got {flat.dtype}")
        if quantized:
            gemm = lambda a, w, tw: ops.MoEGemmQ(a, w, route, tw, self.TopK)
        elif gu.dtype == torch.float8_e4m3fn:
            scale = {id(gu): self.GateUpScale, id(dn): self.DownScale}
            gemm = lambda a, w, tw: ops.MoEGemmF8Block(a, w, scale[id(w)], self.Block[0], self.Block[1], route, tw, self.TopK)
        else:
            gemm = lambda a, w, tw: ops.MoEGemm(a, w, route, tw, self.TopK)
        h = gemm(flat, gu, None)                          # (M, 2 I)
        pair = gemm(ops.MoEGateMul(h, self.Gelu), dn, route.weights)   # (M, H), routing-weighted
        return ops.MoECombine(pair, self.TopK)            # (T, H)
