"""Shared test helpers: block builders that restate the reference tests' own builders,
error metrics, and a loader for the reference's CUDA kernels (oracle/_ref/*.cubin)."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")


def f16_bytes(v: float) -> bytes:
    return np.float16(v).tobytes()


def build_q4_k_block(d, dmin, sub_scales, sub_mins, quants) -> np.ndarray:
    """quant/q4_k_test.go:13-47 (buildQ4_KBlock)."""
    buf = np.zeros(144, np.uint8)
    buf[0:2] = np.frombuffer(f16_bytes(d), np.uint8)
    buf[2:4] = np.frombuffer(f16_bytes(dmin), np.uint8)
    for j in range(4):
        buf[4 + j] = (sub_scales[j] & 0x3F) | ((sub_scales[j + 4] & 0x30) << 2)
        buf[4 + j + 4] = (sub_mins[j] & 0x3F) | ((sub_mins[j + 4] & 0x30) << 2)
        buf[4 + j + 8] = (sub_scales[j + 4] & 0x0F) | ((sub_mins[j + 4] & 0x0F) << 4)
    for p in range(4):
        for l in range(32):
            buf[16 + p * 32 + l] = (quants[p * 64 + l] & 0xF) | ((quants[p * 64 + 32 + l] & 0xF) << 4)
    return buf


def build_q6_k_block(d, scales, raw) -> np.ndarray:
    """quant/q6_k_test.go:14-59 (buildQ6_KBlock)."""
    buf = np.zeros(210, np.uint8)
    for half in range(2):
        for l in range(32):
            r1, r2, r3, r4 = (raw[half * 128 + l + 32 * k] & 0x3F for k in range(4))
            buf[half * 64 + l] = (r1 & 0xF) | ((r3 & 0xF) << 4)
            buf[half * 64 + l + 32] = (r2 & 0xF) | ((r4 & 0xF) << 4)
            buf[128 + half * 32 + l] = ((r1 >> 4) & 3) | (((r2 >> 4) & 3) << 2) | (((r3 >> 4) & 3) << 4) | (
                ((r4 >> 4) & 3) << 6)
    buf[192:208] = np.array(scales, np.int8).view(np.uint8)
    buf[208:210] = np.frombuffer(f16_bytes(d), np.uint8)
    return buf


def build_q8_0_block(scale, values) -> np.ndarray:
    """quant/others_test.go:21-28 (buildQ8_0Block)."""
    buf = np.zeros(34, np.uint8)
    buf[0:2] = np.frombuffer(f16_bytes(scale), np.uint8)
    buf[2:] = np.array(values, np.int8).view(np.uint8)
    return buf


def rel_l2(got, want) -> float:
    got = np.asarray(got, np.float64).ravel()
    want = np.asarray(want, np.float64).ravel()
    den = np.linalg.norm(want)
    return float(np.linalg.norm(got - want) / (den if den > 0 else 1.0))


def max_rel(got, want) -> float:
    """max |got - want| / (1 + |want|), the metric of ops/int4_test.go and ops/fp8_block_test.go."""
    got = np.asarray(got, np.float64).ravel()
    want = np.asarray(want, np.float64).ravel()
    return float(np.max(np.abs(got - want) / (1.0 + np.abs(want)))) if got.size else 0.0


# ---------------------------------------------------------------- reference CUDA kernels

class RefCuda:
    """Loads oracle/_ref/<name>.cubin (the reference's own kernels compiled for sm_100a by
    oracle/Makefile) with the driver API and launches kernels from it on torch's current context."""

    def __init__(self):
        self.cu = C.CDLL("libcuda.so.1")
        self.mods = {}
        self.fns = {}

    @staticmethod
    def available(name: str) -> bool:
        return os.path.exists(os.path.join(REF_DIR, name + ".cubin"))

    def _check(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"cuda driver: {what} failed with {rc}")

    def fn(self, module: str, kernel: str):
        key = (module, kernel)
        if key not in self.fns:
            if module not in self.mods:
                import torch

                torch.zeros(1, device="cuda")  # make sure the primary context is current
                mod = C.c_void_p()
                path = os.path.join(REF_DIR, module + ".cubin").encode()
                self._check(self.cu.cuModuleLoad(C.byref(mod), path), f"cuModuleLoad {module}")
                self.mods[module] = mod
            f = C.c_void_p()
            self._check(self.cu.cuModuleGetFunction(C.byref(f), self.mods[module], kernel.encode()),
                        f"cuModuleGetFunction {kernel}")
            self.fns[key] = f
        return self.fns[key]

    def launch(self, module, kernel, grid, block, args, shmem=0):
        """args: list of ctypes scalars (c_void_p for device pointers, c_int, c_ulong ...)."""
        import torch

        f = self.fn(module, kernel)
        arr = (C.c_void_p * len(args))(*[C.cast(C.byref(a), C.c_void_p) for a in args])
        gx, gy, gz = (list(grid) + [1, 1])[:3]
        bx, by, bz = (list(block) + [1, 1])[:3]
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        self._check(self.cu.cuLaunchKernel(f, gx, gy, gz, bx, by, bz, shmem, stream, arr, None), f"launch {kernel}")
