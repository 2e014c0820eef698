"""Size-independent properties of the linear at the headline shapes, through the C ABI, with no checker in the loop:
they hold (or fail) whatever the matrix size, so they cover the full-size configurations every kernel path is
dispatched on -- the integer decode kernel (1-2 rows), the one-launch fp16 decode kernel (3-16 rows) and the
tensor-core GEMM (17 rows and more, including the shape whose ragged last round runs as a second launch).

* Scaling the activations up by a power of two scales the fp32 result by that factor: exactly on the integer path
  (16-bit fixed point per chunk: the planes of 2x are the planes of x), to 1e-6 on the paths that convert the
  activations to fp16 (only draws below fp16's normal range round differently after scaling).
* The result of a row does not depend on where the row sits in the batch: a permuted batch gives the permuted result,
  bit for bit.
* A zero row gives exactly the bias.
* The same row through two different kernels (alone, and inside a batch) agrees within the parity tolerance (1e-3).
"""
import numpy as np
import pytest
import torch

import tattletale_b200 as ttq
from conftest import rel_l2
from gpu_util import make_x
from tattletale_b200 import quantize as Q

pytestmark = pytest.mark.gpu
BATCHES = [1, 2, 4, 8, 16, 40, 300, 2048]


@pytest.fixture(scope="module")
def gate_up(ctx):
    """Llama-3-8B gate|up projection (4096 -> 28672, Q4_K) with a bias."""
    g = torch.Generator(device="cuda").manual_seed(777)
    blocks = Q.quantize(ttq.FMT_Q4_K, torch.randn(28672, 4096, generator=g, device="cuda") * 0.02)
    bias = (torch.randn(28672, generator=torch.Generator().manual_seed(778)) * 0.25).cuda()
    lin = ttq.QuantLinear(ctx, ttq.FMT_Q4_K, blocks, 4096, bias=bias)
    yield lin
    lin.close()


@pytest.mark.parametrize("m", BATCHES)
def test_power_of_two_scaling_is_exact(ctx, gate_up, m):
    x = make_x(m, 4096, 900 + m).cuda()
    y1 = gate_up.forward(x, out_dtype=torch.float32, use_bias=False)
    y2 = gate_up.forward(x * 2, out_dtype=torch.float32, use_bias=False)
    y4 = gate_up.forward(x * 4, out_dtype=torch.float32, use_bias=False)
    ctx.check_device_status()
    if m <= 2:  # 16-bit fixed point per chunk: the planes of 2x are the planes of x
        assert torch.equal(y2, y1 * 2) and torch.equal(y4, y1 * 4)
    else:  # fp16 activations: only draws below the normal range (6e-5) round differently after scaling
        assert rel_l2(y2.cpu().numpy(), (y1 * 2).cpu().numpy()) < 1e-6
        assert rel_l2(y4.cpu().numpy(), (y1 * 4).cpu().numpy()) < 1e-6


@pytest.mark.parametrize("m", [m for m in BATCHES if m > 1])
def test_rows_do_not_depend_on_their_position(ctx, gate_up, m):
    x = make_x(m, 4096, 950 + m).cuda()
    perm = torch.randperm(m, generator=torch.Generator().manual_seed(m)).cuda()
    y = gate_up.forward(x, out_dtype=torch.float32)
    yp = gate_up.forward(x[perm].contiguous(), out_dtype=torch.float32)
    ctx.check_device_status()
    assert torch.equal(yp, y[perm])


@pytest.mark.parametrize("m", BATCHES)
def test_zero_row_gives_the_bias(ctx, gate_up, m):
    x = make_x(m, 4096, 980 + m).cuda()
    x[m // 2] = 0
    y = gate_up.forward(x, out_dtype=torch.float32)
    ctx.check_device_status()
    assert torch.equal(y[m // 2], gate_up.bias.float())


def test_a_row_agrees_across_kernels(ctx, gate_up):
    """Row 0 alone (integer kernel), in batches served by the fp16 decode kernel and by the GEMM."""
    x = make_x(2048, 4096, 999).cuda()
    alone = gate_up.forward(x[:1], out_dtype=torch.float32).cpu().numpy()
    for m in (2, 3, 8, 16, 17, 64, 256, 2048):
        y = gate_up.forward(x[:m], out_dtype=torch.float32)[:1].cpu().numpy()
        assert rel_l2(y, alone) < 1e-3, m
    ctx.check_device_status()
