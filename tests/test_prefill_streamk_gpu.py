"""The persistent tensor-core kernel (an even split of all K blocks over one CTA per SM, partial tiles summed in a fixed
order) takes a call only where the split pays; here every shape of the prefill, int4 / block-FP8 and grouped (MoE) parity
tests runs through it (LIGHT_B200_PREFILL_SK=2): one K block per CTA with a tile shared by eight of them, runs that start
and end inside tiles, more CTAs than blocks (empty runs), ragged and empty expert groups; the status word stays zero."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FILES = ["test_prefill_gpu.py", "test_moe_gpu.py", "test_int4_fp8_gpu.py", "test_nn_gpu.py"]


def test_parity_suites_through_the_persistent_kernel():
    env = {**os.environ, "LIGHT_B200_PREFILL_SK": "2"}
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-x", "-m", "gpu", "-p", "no:cacheprovider"] + [os.path.join(ROOT, "tests", f) for f in FILES],
                       capture_output=True, text=True, timeout=1500, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-2000:]


CHILD = """
import sys, torch
sys.path.insert(0, %r)
from light_b200 import ops, synth
dev = torch.device("cuda:0")
for dt, M, N, K in ((ops.Q4_K, 2048, 1024, 4096), (ops.Q6_K, 700, 520, 2048), (ops.Q8_0, 300, 300, 1024)):
    w = ops.QTensor(synth.gaussian_weight(7, dt, N, K, device=dev).reshape(-1), dt, (N, K))
    x = torch.randn(M, K, generator=torch.Generator().manual_seed(8)).to(dev)
    a, b = ops.MatMulQ(x, w), ops.MatMulQ(x, w)
    assert torch.equal(a, b), "the partial tiles must be added in a fixed order"
    assert bool(torch.isfinite(a).all())
assert ops.prefill_status(0) == 0
print("CASE OK")
""" % ROOT


def test_same_bits_twice():
    r = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, timeout=600, env={**os.environ, "LIGHT_B200_PREFILL_SK": "2"})
    assert r.returncode == 0 and "CASE OK" in r.stdout, r.stdout + r.stderr[-3000:]
