"""light_b200: B200 (sm_100a) kernels for the reference's quantized-weight matmul path.

`light_b200.ops` mirrors the reference operator API; `light_b200._lib` binds the C ABI of
include/light_b200.h; `light_b200.build` compiles the shared library; `light_b200.synth` makes
seeded synthetic weights in the on-disk layouts.
"""
__all__ = ["ops", "synth", "build"]
