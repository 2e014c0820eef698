"""Tensor-core (tcgen05) dequant-GEMM (Q4_K beyond 16 rows, Q8_0 / Q6_K from 9) against the CPU checker, through the C ABI.

Weights are expanded to fp16 before the MMA and activations are converted to fp16, so the expected
relative L2 error is a few 1e-4 (bar: 1e-3, fp32 accumulation in tensor memory)."""
import numpy as np
import pytest
import torch

import oracle
import tattletale_b200 as ttq
from conftest import rel_l2
from gpu_util import make_weight, make_x, x_bits

pytestmark = pytest.mark.gpu
TOL = 1e-3


def run(ctx, n, k, m, seed, y_dtype=torch.float32, bias=False, x_dtype=torch.bfloat16):
    blocks = make_weight(ttq.FMT_Q4_K, n, k, seed)
    x = make_x(m, k, seed + 1, x_dtype)
    b = None
    if bias:
        b = torch.from_numpy(np.random.default_rng(seed + 2).normal(0, 0.1, n).astype(np.float32))
    lin = ttq.QuantLinear(ctx, ttq.FMT_Q4_K, torch.from_numpy(blocks), k, bias=None if b is None else b.cuda())
    y = lin.forward(x.cuda(), out_dtype=y_dtype)
    ctx.check_device_status()
    want = oracle.linear(oracle.Q4_K, blocks, x_bits(x), oracle.BF16 if x_dtype == torch.bfloat16 else oracle.F16,
                         None if b is None else b.numpy())
    lin.close()
    return y.float().cpu().numpy(), want


@pytest.mark.parametrize("m", [17, 64, 65, 128, 129, 256, 300])
def test_row_counts(ctx, m):
    got, want = run(ctx, 256, 1024, m, seed=700 + m)
    assert got.shape == want.shape
    assert rel_l2(got, want) < TOL


@pytest.mark.parametrize("n,k", [(128, 256), (100, 512), (130, 768), (16, 256), (384, 2304)])
def test_ragged_weight_shapes(ctx, n, k):
    for m in (40, 150):
        got, want = run(ctx, n, k, m, seed=n + k + m)
        assert rel_l2(got, want) < TOL


def test_bias_and_output_types(ctx):
    for ydt in (torch.float32, torch.bfloat16, torch.float16):
        got, want = run(ctx, 192, 512, 70, seed=720, y_dtype=ydt, bias=True, x_dtype=torch.float16)
        assert rel_l2(got, want) < (TOL if ydt == torch.float32 else 6e-3)


def test_llama_projection_prefill(ctx):
    """4096 -> 4096 at M = 256 (one of the prefill points of the headline configuration)."""
    got, want = run(ctx, 4096, 4096, 256, seed=2001)
    assert rel_l2(got, want) < TOL


def test_same_rows_give_same_result_as_decode_path(ctx):
    """The first rows of a prefill batch agree with the decode kernel on the same rows (both within tolerance)."""
    blocks = make_weight(ttq.FMT_Q4_K, 256, 1024, 730)
    lin = ttq.QuantLinear(ctx, ttq.FMT_Q4_K, torch.from_numpy(blocks), 1024)
    x = make_x(48, 1024, 731).cuda()
    big = lin.forward(x, out_dtype=torch.float32)
    small = lin.forward(x[:4], out_dtype=torch.float32)
    assert rel_l2(big[:4].cpu().numpy(), small.cpu().numpy()) < TOL
    lin.close()


@pytest.mark.parametrize("fmt", [ttq.FMT_Q8_0, ttq.FMT_Q6_K], ids=["q8_0", "q6_k"])
@pytest.mark.parametrize("n,k,m", [(256, 512, 33), (130, 768, 200), (512, 1024, 300), (100, 256, 64), (272, 2304, 9), (4096, 1024, 40)])
def test_q8_0_and_q6_k_fused_dequant_gemm(ctx, fmt, n, k, m):
    """Q8_0 and Q6_K batches from 9 rows: the same tcgen05 kernel as Q4_K, its dequant warps expanding int8 values
    (Q8_0) or nibble + 2-bit planes (Q6_K) to fp16 in shared memory; no whole-weight expansion."""
    from gpu_util import OFMT

    blocks = make_weight(fmt, n, k, seed=n + k + m + fmt)
    x = make_x(m, k, seed=m + 5)
    bias = torch.from_numpy(np.random.default_rng(m).normal(0, 0.1, n).astype(np.float32))
    lin = ttq.QuantLinear(ctx, fmt, torch.from_numpy(blocks), k, bias=bias.cuda())
    c0 = ctx.launch_count
    y = lin.forward(x.cuda(), out_dtype=torch.float32)
    ctx.check_device_status()
    assert ctx.launch_count - c0 <= 3  # activation images, GEMM (+ split-K sum)
    want = oracle.linear(OFMT[fmt], blocks, x_bits(x), oracle.BF16, bias.numpy())
    assert rel_l2(y.cpu().numpy(), want) < TOL
    lin.close()
