"""The two-CTA dense Q4_K GEMM (tcgen05 cta_group::2, tiles of 256 weight rows x 512 activation rows) against the CPU checker.

By default a cost model picks between this kernel and the one-CTA kernel per call; TTQ_GEMM_PAIR=2 takes the two-CTA
kernel wherever it applies (more than 128 rows, no K split), so that small shapes exercise it too.  The switch is read
once per process: the comparison runs in a child process.  Cases: one full tile with masked rows (300 rows), a full and
a half tile (700 rows), several full tiles (1300, 2048 rows), only a half tile (256 rows), a weight row count that is
not a multiple of 256 (1000) or of 16-row tiles per CTA, a bias, the three output types, a strided output, and a shape
whose last weight-tile columns go to the second (K-split) launch.  Tolerance: relative L2 <= 1e-3 on sampled rows;
a second forward must reproduce the first bit for bit.
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
cases = [(512, 512, 256, torch.float32), (1024, 768, 300, torch.bfloat16), (512, 1000, 700, torch.float32),
         (512, 1000, 1300, torch.float16), (4096, 6144, 2048, torch.bfloat16), (1024, 40 * 256, 2048, torch.float32),
         (256, 16, 513, torch.float32)]
for k, n, m, dt in cases:
    g = torch.Generator(device="cuda").manual_seed(k + n)
    blocks = Q.quantize(ttq.FMT_Q4_K, torch.randn(n, k, generator=g, device="cuda") * 0.02)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(7)) * 0.1
    lin = ttq.QuantLinear(ctx, ttq.FMT_Q4_K, blocks, k, bias=bias.cuda())
    host = blocks.cpu().numpy()
    x = make_x(m, k, 100 + m)
    wide = torch.full((m, n + 24), 7.0, dtype=dt, device="cuda")
    y = lin.forward(x.cuda(), out=wide[:, :n])
    y1 = y.clone()
    lin.forward(x.cuda(), out=wide[:, :n])
    torch.cuda.synchronize()
    ctx.check_device_status()
    rows = np.sort(np.random.default_rng(m).choice(m, min(m, 40), replace=False))
    rows[-1] = m - 1
    want = oracle.linear(oracle.Q4_K, host, x_bits(x[rows]), oracle.BF16, bias=bias.numpy())
    got = y[rows].float().cpu().numpy().astype(np.float64)
    rel = float(np.linalg.norm(got - want) / np.linalg.norm(want))
    tol = 1e-3 if dt == torch.float32 else 6e-3
    ok = rel < tol and bool(torch.isfinite(y.float()).all()) and torch.equal(y, y1) and bool((wide[:, n:] == 7.0).all())
    if not ok:
        bad.append((k, n, m, str(dt), rel))
    lin.close()
print("BAD", bad)
sys.exit(1 if bad else 0)
"""


def test_two_cta_gemm_matches_checker():
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, TTQ_GEMM_PAIR="2", PYTHONPATH=os.pathsep.join([os.path.dirname(here), os.environ.get("PYTHONPATH", "")]))
    r = subprocess.run([sys.executable, "-c", CHILD, here], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
