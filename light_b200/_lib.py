"""ctypes binding of liblight_b200.so -- the C ABI declared in include/light_b200.h.

There is no fallback: if the shared library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liblight_b200.so")

F32, BF16, F16 = 0, 1, 2
Q4_0, Q5_0, Q8_0, Q4_K, Q5_K, Q6_K = 2, 6, 8, 12, 13, 14


class Light200Error(RuntimeError):
    """A call into liblight_b200.so returned non-zero; .code is the return value."""

    def __init__(self, code: int, msg: str):
        super().__init__(msg)
        self.code = code


class Peers(C.Structure):
    _fields_ = [("slots", C.c_void_p * 8), ("world", C.c_int32), ("rank", C.c_int32)]


class TpArgs(C.Structure):
    """lb200_tp: activations as a receive buffer (or NULL), per-output receive buffers of every rank, step word."""
    _fields_ = [("x_slots", C.c_void_p), ("out_slots", (C.c_void_p * 8) * 4), ("step", C.c_void_p),
                ("world", C.c_int32), ("rank", C.c_int32)]


class MoeArgs(C.Structure):
    _fields_ = [
        ("input", C.c_void_p), ("weights", C.c_void_p), ("sorted_pairs", C.c_void_p), ("expert_ids", C.c_void_p),
        ("counts", C.c_void_p), ("offsets", C.c_void_p), ("topk_weights", C.c_void_p), ("out", C.c_void_p),
        ("M", C.c_int64), ("size_m", C.c_int64), ("E", C.c_int32), ("N", C.c_int32), ("K", C.c_int32),
        ("topk", C.c_int32), ("row_per_pair", C.c_int32), ("dtype", C.c_int32),
    ]


class NormArgs(C.Structure):
    """lb200_norm"""
    _fields_ = [("weight", C.c_void_p), ("residual", C.c_void_p), ("sum_out", C.c_void_p), ("eps", C.c_float)]


class ChainOp(C.Structure):
    """lb200_chain_op"""
    _fields_ = [("wtype", C.c_int32), ("K", C.c_int32), ("count", C.c_int32), ("act", C.c_int32), ("w", C.c_void_p * 4),
                ("n", C.c_int32 * 4), ("out", C.c_void_p * 4), ("out_vec", C.c_int32 * 4), ("x", C.c_void_p), ("x_vec", C.c_int32),
                ("res_vec", C.c_int32), ("sum_vec", C.c_int32), ("norm_weight", C.c_void_p), ("norm_eps", C.c_float)]


class DecodeAttnArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("kbuf", C.c_void_p), ("vbuf", C.c_void_p), ("k_new", C.c_void_p), ("v_new", C.c_void_p),
        ("pos", C.c_void_p), ("out", C.c_void_p), ("dtype", C.c_int32), ("B", C.c_int32), ("NH", C.c_int32),
        ("KH", C.c_int32), ("Cap", C.c_int32), ("D", C.c_int32), ("window", C.c_int32), ("scale", C.c_float),
        ("rope_base", C.c_float),
    ]


# name -> (restype, argtypes): every symbol include/light_b200.h declares
SYMBOLS = {
    "light_b200_init": (C.c_int, [C.c_int]),
    "light_b200_last_error": (C.c_int, [C.c_char_p, C.c_size_t]),
    "light_b200_abi_version": (C.c_int, []),
    "light_b200_launch_count": (C.c_ulonglong, []),
    "light_b200_comm_step_begin": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "light_b200_matmul_q_tp": (C.c_int, [C.c_int, C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_int32),
                                         C.c_int, C.c_int, C.POINTER(TpArgs), C.c_int, C.c_void_p]),
    "light_b200_allgather_ll": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(Peers), C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "light_b200_comm_status": (C.c_int, [C.c_int]),
    "light_b200_set_workspace": (C.c_int, [C.c_int, C.c_void_p, C.c_size_t]),
    "light_b200_prefill_status": (C.c_int, [C.c_int]),
    "light_b200_block_elems": (C.c_int, [C.c_int]),
    "light_b200_block_bytes": (C.c_int, [C.c_int]),
    "light_b200_matmul_q": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                      C.c_void_p]),
    "light_b200_matmul_q_multi": (C.c_int, [C.c_int, C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                            C.POINTER(C.c_int32), C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_matmul_q_multi_rows": (C.c_int, [C.c_int, C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                                 C.POINTER(C.c_int32), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_matmul_q_gated": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                            C.c_int, C.c_int, C.c_void_p]),
    "light_b200_matmul_q_fused": (C.c_int, [C.c_int, C.c_void_p, C.POINTER(NormArgs), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                            C.POINTER(C.c_int32), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_dequant": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p]),
    "light_b200_quantize_rows_int8": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_matmul_w8a8": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                         C.c_int, C.c_void_p]),
    "light_b200_moe_route_sigmoid": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_moe_sort_pairs": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int,
                                            C.c_void_p]),
    "light_b200_moe_route_status": (C.c_int, [C.c_int]),
    "light_b200_moe_route_deepseek": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                                C.c_int, C.c_void_p]),
    "light_b200_moe_route_topk": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_moe_gate_mul": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_moe_combine_weighted": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int64, C.c_int, C.c_void_p]),
    "light_b200_moe_combine": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_argmax": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_embedding_q": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_int4_repack": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                         C.c_int, C.c_int, C.c_void_p]),
    "light_b200_int4_dequant": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                          C.c_int, C.c_int64, C.c_int, C.c_void_p]),
    "light_b200_int4_gemv": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                       C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_fp8_block_dequant": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                               C.c_int, C.c_int, C.c_void_p]),
    "light_b200_fp8_block_gemv": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                            C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_moe_gemm": (C.c_int, [C.POINTER(MoeArgs), C.c_int, C.c_void_p]),
    "light_b200_moe_gemm_q": (C.c_int, [C.POINTER(MoeArgs), C.c_int, C.c_void_p]),
    "light_b200_moe_gemm_f8block": (C.c_int, [C.POINTER(MoeArgs), C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_moe_gemm_static_scratch": (C.c_int, [C.POINTER(MoeArgs), C.c_int, C.c_void_p]),
    "light_b200_kv_append": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                       C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_decode_attn": (C.c_int, [C.POINTER(DecodeAttnArgs), C.c_int, C.c_void_p]),
    "light_b200_inc_i64": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_rmsnorm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_float,
                                     C.c_int, C.c_void_p]),
    "light_b200_rope": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_double, C.c_int, C.c_void_p]),
    "light_b200_decode_attn_status": (C.c_int, [C.c_int]),
    "light_b200_matmul_q_workspace_bytes": (C.c_ulonglong, [C.c_int, C.c_int]),
    "light_b200_gather_columns": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_gemv_multi": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_int32), C.c_int, C.c_int, C.c_int,
                                        C.c_int, C.c_void_p]),
    "light_b200_gemv_gated": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_chain_program_bytes": (C.c_size_t, [C.c_int]),
    "light_b200_chain_arena_bytes": (C.c_int64, [C.POINTER(ChainOp), C.c_int, C.c_int, C.c_int]),
    "light_b200_chain_build": (C.c_int, [C.POINTER(ChainOp), C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p), C.c_size_t,
                                         C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "light_b200_chain_run": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "light_b200_chain_status": (C.c_int, [C.c_int]),
}

_lib = None


def lib() -> C.CDLL:
    """Loads liblight_b200.so (built by light_b200/build.py); raises if it is absent."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise Light200Error(-100, f"{LIB_PATH} is missing: run `python -m light_b200.build` (needs nvcc); "
                                      "there is no CPU or PyTorch fallback")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib


def last_error() -> str:
    buf = C.create_string_buffer(512)
    lib().light_b200_last_error(buf, 512)
    return buf.value.decode("utf-8", "replace")


def check(rc: int) -> None:
    if rc != 0:
        raise Light200Error(rc, last_error() or f"light_b200 call failed with code {rc}")


def launch_count() -> int:
    return int(lib().light_b200_launch_count())
