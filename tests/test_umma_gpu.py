"""The opt-in tensor-memory decode kernel for Q4_K (tcgen05.mma kind::i8, TTQ_Q4K_UMMA=1) against the CPU checker.

The switch is read once per process, so the comparison runs in a child process with the variable set.  Shapes: one
super-block, fewer rows than one 128-row group, a row count that is not a multiple of 16, the Llama-3-8B O and down
projections (many CTAs per group: partial sums through the workspace); batches 1 to 8, with a bias.  Every forward is
run twice: the arrival counters and the workspace must be back in their start state.  Tolerance: relative L2 <= 1e-3.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

CHILD = r"""
import sys
import numpy as np, torch
import oracle, tattletale_b200 as ttq
from tattletale_b200 import quantize as Q
sys.path.insert(0, sys.argv[1])
from gpu_util import make_x, x_bits
ctx = ttq.Context(0)
bad = []
for k, n in [(256, 128), (512, 16), (1024, 200), (4096, 4096), (14336, 4096)]:
    g = torch.Generator(device="cuda").manual_seed(k + n)
    blocks = Q.quantize(ttq.FMT_Q4_K, torch.randn(n, k, generator=g, device="cuda") * 0.02)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(7)) * 0.1
    lin = ttq.QuantLinear(ctx, ttq.FMT_Q4_K, blocks, k, bias=bias.cuda())
    host = blocks.cpu().numpy()
    for m in (1, 2, 3, 4, 5, 8):
        x = make_x(m, k, 100 + m)
        c0 = ctx.launch_count
        y = lin.forward(x.cuda(), out_dtype=torch.float32)
        launches = ctx.launch_count - c0
        y2 = lin.forward(x.cuda(), out_dtype=torch.float32)
        ctx.check_device_status()
        want = oracle.linear(oracle.Q4_K, host, x_bits(x), oracle.BF16, bias=bias.numpy())
        rel = float(np.linalg.norm(y.cpu().numpy().astype(np.float64) - want) / np.linalg.norm(want))
        if not (rel < 1e-3 and bool(torch.isfinite(y).all()) and torch.equal(y, y2) and launches == 2):
            bad.append((k, n, m, rel, launches))
    lin.close()
print("BAD", bad)
sys.exit(1 if bad else 0)
"""


def test_q4k_tensor_memory_decode_matches_checker():
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, TTQ_Q4K_UMMA="1", PYTHONPATH=os.pathsep.join([os.path.dirname(here), os.environ.get("PYTHONPATH", "")]))
    r = subprocess.run([sys.executable, "-c", CHILD, here], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
