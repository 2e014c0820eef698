"""Parity of the CUDA quantized linear against the CPU checker (fp64 accumulation), through the C ABI.

Tolerance: relative L2 error <= 1e-3 (the bar set for this path).  Observed: ~3e-7 for Q4_K batches of
3..16 rows (exact integer products on fp16 tensor-core instructions, fp32 accumulation), ~3e-5 wherever the
activations go through 16-bit fixed point.
"""
import numpy as np
import pytest
import torch

import oracle
import tattletale_b200 as ttq
from conftest import rel_l2
from gpu_util import ALL_FMTS, FMT_IDS, OFMT, make_weight, make_x, odt, random_blocks, x_bits

pytestmark = pytest.mark.gpu
TOL = 1e-3


def run_case(ctx, fmt, n, k, m, seed, x_dtype=torch.bfloat16, y_dtype=torch.float32, bias=False, blocks=None):
    if blocks is None:
        blocks = make_weight(fmt, n, k, seed)
    x = make_x(m, k, seed + 1, x_dtype)
    b = None
    if bias:
        b = torch.from_numpy(np.random.default_rng(seed + 2).normal(0, 0.1, n).astype(np.float32)).to(x_dtype)
    lin = ttq.QuantLinear(ctx, fmt, torch.from_numpy(blocks), k, bias=None if b is None else b.cuda())
    y = lin.forward(x.cuda(), out_dtype=y_dtype)
    ctx.check_device_status()
    want = oracle.linear(OFMT[fmt], blocks, x_bits(x), odt(x_dtype), None if b is None else b.float().numpy())
    lin.close()
    return y.float().cpu().numpy(), want


@pytest.mark.parametrize("fmt", ALL_FMTS, ids=FMT_IDS)
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 8, 9, 16])
def test_decode_sizes(ctx, fmt, m):
    got, want = run_case(ctx, fmt, 128, 1024, m, seed=40 + m)
    assert got.shape == want.shape
    assert rel_l2(got, want) < TOL


@pytest.mark.parametrize("fmt", ALL_FMTS, ids=FMT_IDS)
@pytest.mark.parametrize("n,k", [(16, 256), (1, 256), (17, 512), (100, 768), (48, 2304), (4096, 256)])
def test_ragged_shapes(ctx, fmt, n, k):
    for m in (1, 3, 7):
        got, want = run_case(ctx, fmt, n, k, m, seed=n + k + m)
        assert rel_l2(got, want) < TOL


@pytest.mark.parametrize("fmt", ALL_FMTS, ids=FMT_IDS)
@pytest.mark.parametrize("m", [17, 33, 64])
def test_more_rows_than_one_pass(ctx, fmt, m):
    got, want = run_case(ctx, fmt, 96, 512, m, seed=70 + m)
    assert rel_l2(got, want) < TOL


@pytest.mark.parametrize("fmt", ALL_FMTS, ids=FMT_IDS)
def test_bias_and_dtypes(ctx, fmt):
    for xdt in (torch.bfloat16, torch.float16):
        for ydt in (torch.float32, torch.bfloat16, torch.float16):
            got, want = run_case(ctx, fmt, 64, 512, 3, seed=90, x_dtype=xdt, y_dtype=ydt, bias=True)
            tol = TOL if ydt == torch.float32 else 6e-3  # 16-bit outputs add their own rounding
            assert rel_l2(got, want) < tol


@pytest.mark.parametrize("fmt", ALL_FMTS, ids=FMT_IDS)
def test_random_bytes_weights(ctx, fmt):
    """Extreme quants and scales (every byte pattern) still agree with the checker."""
    per = 8 if fmt == ttq.FMT_Q8_0 else 1
    blocks = random_blocks(fmt, 32, 2 * per, seed=17)
    # keep magnitudes finite in fp32: clear the top exponent bits of the fp16 scale fields
    nb = oracle.BLOCK_BYTES[OFMT[fmt]]
    b3 = blocks.reshape(32, -1, nb)
    for off in {ttq.FMT_Q8_0: (0,), ttq.FMT_Q4_K: (0, 2), ttq.FMT_Q6_K: (208,)}[fmt]:
        b3[:, :, off + 1] &= 0xBF
    for m in (1, 4, 6):
        got, want = run_case(ctx, fmt, 32, 512, m, seed=18 + m, blocks=blocks)
        assert rel_l2(got, want) < TOL


def test_zero_input_gives_bias(ctx):
    fmt = ttq.FMT_Q4_K
    blocks = make_weight(fmt, 32, 512, seed=3)
    b = torch.arange(32, dtype=torch.float32).cuda()
    lin = ttq.QuantLinear(ctx, fmt, torch.from_numpy(blocks), 512, bias=b)
    y = lin.forward(torch.zeros(2, 512, dtype=torch.bfloat16, device="cuda"), out_dtype=torch.float32)
    assert torch.equal(y, b.expand(2, 32))
    lin.close()


def test_linearity(ctx):
    """W(a*x) == a*W(x) for a power-of-two factor, exactly: every product and partial sum scales with it."""
    fmt = ttq.FMT_Q4_K
    lin = ttq.QuantLinear(ctx, fmt, torch.from_numpy(make_weight(fmt, 64, 1024, seed=4)), 1024)
    x = make_x(2, 1024, 5).cuda()
    y1 = lin.forward(x, out_dtype=torch.float32)
    y2 = lin.forward(x * 4, out_dtype=torch.float32)
    assert torch.equal(y2, y1 * 4)
    lin.close()


def test_leading_dimensions_and_strides(ctx):
    fmt = ttq.FMT_Q8_0
    blocks = make_weight(fmt, 48, 512, seed=6)
    lin = ttq.QuantLinear(ctx, fmt, torch.from_numpy(blocks), 512)
    xfull = make_x(3, 640, 7)
    x = xfull[:, 64:576]  # row stride 640, 128-byte aligned start
    y = lin.forward(x.cuda()[...], out_dtype=torch.float32)
    want = oracle.linear(oracle.Q8_0, blocks, x_bits(x.contiguous()), oracle.BF16)
    assert rel_l2(y.cpu().numpy(), want) < TOL
    x3 = make_x(6, 512, 8).reshape(2, 3, 512)
    y3 = lin.forward(x3.cuda())
    assert y3.shape == (2, 3, 48) and y3.dtype == torch.bfloat16
    # misaligned start (odd element offset): falls back to scalar loads inside the kernel
    xo = make_x(2, 513, 9)
    ym = lin.forward(xo.cuda()[:, 1:], out_dtype=torch.float32)
    want = oracle.linear(oracle.Q8_0, blocks, x_bits(xo[:, 1:].contiguous()), oracle.BF16)
    assert rel_l2(ym.cpu().numpy(), want) < TOL
    lin.close()


def test_forward_rejects_bad_arguments(ctx):
    fmt = ttq.FMT_Q4_K
    lin = ttq.QuantLinear(ctx, fmt, torch.from_numpy(make_weight(fmt, 16, 256, seed=1)), 256)
    with pytest.raises(ttq.TtqError):
        lin.forward(torch.zeros(1, 512, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ttq.TtqError):
        lin.forward(torch.zeros(1, 256, dtype=torch.float32, device="cuda"))
    with pytest.raises(ttq.TtqError):
        lin.forward(torch.zeros(1, 256, dtype=torch.bfloat16))
    y = lin.forward(torch.zeros(0, 256, dtype=torch.bfloat16, device="cuda"))
    assert y.shape == (0, 16)
    lin.close()


def test_host_entry_point(ctx):
    fmt = ttq.FMT_Q4_K
    blocks = make_weight(fmt, 64, 512, seed=12)
    lin = ttq.QuantLinear(ctx, fmt, torch.from_numpy(blocks), 512)
    x = make_x(2, 512, 13).pin_memory()
    y = torch.empty(2, 64, dtype=torch.float32).pin_memory()
    lin.forward_host(x, y)
    want = oracle.linear(oracle.Q4_K, blocks, x_bits(x), oracle.BF16)
    assert rel_l2(y.numpy(), want) < TOL
    lin.close()


def test_host_entry_point_enqueue_then_wait(ctx):
    """Several host-buffer calls enqueued without a wait, one ttq_host_sync: results as from the synchronous call; pageable
    buffers are refused (they would need the one staging area per call)."""
    fmt = ttq.FMT_Q4_K
    lins, xs, ys, wants = [], [], [], []
    for i, (n, k) in enumerate([(64, 512), (48, 256), (4096, 4096)]):
        blocks = make_weight(fmt, n, k, seed=40 + i)
        lin = ttq.QuantLinear(ctx, fmt, torch.from_numpy(blocks), k)
        x = make_x(1 + i, k, 50 + i).pin_memory()
        lins.append(lin)
        xs.append(x)
        ys.append(torch.zeros(1 + i, n, dtype=torch.float32).pin_memory())
        wants.append(oracle.linear(oracle.Q4_K, blocks, x_bits(x), oracle.BF16))
    for _ in range(2):
        for lin, x, y in zip(lins, xs, ys):
            lin.forward_host(x, y, wait=False)
        ctx.host_sync()
        for y, want in zip(ys, wants):
            assert rel_l2(y.numpy(), want) < TOL
            y.zero_()
    calls = [lin.host_call(x, y, wait=False) for lin, x, y in zip(lins, xs, ys)]  # the pre-bound form
    for call in calls:
        call()
    ctx.host_sync()
    for y, want in zip(ys, wants):
        assert rel_l2(y.numpy(), want) < TOL
    with pytest.raises(ttq.TtqError):
        lins[0].forward_host(make_x(1, 512, 3), torch.zeros(1, 64), wait=False)
    ctx.host_sync()
    for lin in lins:
        lin.close()


def test_recorded_host_batch(ctx):
    """ttq_host_batch_*: three linears recorded once, run three times on refreshed inputs; every y as from the checker.
    A pageable buffer is refused at creation."""
    fmt = ttq.FMT_Q4_K
    items, blocks_of = [], []
    for i, (n, k) in enumerate([(64, 512), (4096, 4096), (48, 256)]):
        blocks = make_weight(fmt, n, k, seed=60 + i)
        lin = ttq.QuantLinear(ctx, fmt, torch.from_numpy(blocks), k)
        rows = (1, 2, 5)[i]  # batched activation pass twice, gathered activations + one-launch kernel once
        items.append((lin, make_x(rows, k, 70 + i).pin_memory(), torch.zeros(rows, n, dtype=torch.float32).pin_memory()))
        blocks_of.append(blocks)
    batch = ttq.HostBatch(ctx, items)
    for rep in range(3):
        for i, (lin, x, y) in enumerate(items):
            x.copy_(make_x(x.shape[0], x.shape[1], 80 + 7 * rep + i))  # same buffers, new activations
            y.zero_()
        batch.run()
        for (lin, x, y), blocks in zip(items, blocks_of):
            assert rel_l2(y.numpy(), oracle.linear(oracle.Q4_K, blocks, x_bits(x), oracle.BF16)) < TOL
    batch.close()
    with pytest.raises(ttq.TtqError):
        ttq.HostBatch(ctx, [(items[0][0], make_x(1, 512, 3), torch.zeros(1, 64))])
    ctx.host_sync()
    lin = items[0][0]
    y = lin.forward(items[0][1].cuda(), out_dtype=torch.float32)  # the context is still usable
    assert torch.isfinite(y).all()
    for lin, _, _ in items:
        lin.close()


@pytest.mark.parametrize("m", [2, 4, 5, 16, 17])
def test_recorded_batch_on_device_buffers(ctx, m):
    """A recorded batch of Q4_K linears of several rows on device buffers: the linears of up to 16 rows run on the forked
    streams (two rows of a long K and 3-16 rows: the one-launch decode kernel with a workspace per stream), 17 rows stay in
    line; every y is bit-identical to the stand-alone forward on the same input, run after run (within bf16 rounding at 3-4
    rows, where a batch serves small weights with another kernel than the stand-alone call)."""
    fmt = ttq.FMT_Q4_K
    lins = [ttq.QuantLinear(ctx, fmt, torch.from_numpy(make_weight(fmt, n, k, seed=90 + i)), k,
                            bias=(torch.randn(n, generator=torch.Generator().manual_seed(i)) * 0.1).cuda() if i == 0 else None)
            for i, (n, k) in enumerate([(512, 1024), (256, 8192), (1000, 512)])]
    items = []
    for i, lin in enumerate(lins * 2):
        x = make_x(m, lin.in_features, 200 + i).cuda()
        items.append((lin, x, torch.zeros(m, lin.out_features, dtype=torch.bfloat16, device="cuda")))
    torch.cuda.synchronize()
    batch = ttq.HostBatch(ctx, items)
    for rep in range(2):
        for _, _, y in items:
            y.zero_()
        torch.cuda.synchronize()
        batch.run()
        for lin, x, y in items:
            want = lin.forward(x)
            torch.cuda.synchronize()
            if m in (3, 4):
                # small weights at 3-4 rows take the integer GEMV inside a batch, the one-launch fp16 kernel stand-alone
                assert rel_l2(y.float().cpu().numpy(), want.float().cpu().numpy()) < 6e-3
            else:
                assert torch.equal(want, y)
    batch.close()
    ctx.check_device_status()
    for lin in lins:
        lin.close()


def test_config1_q8_0_decode(ctx):
    """Single Q8_0 linear, M=1, K=N=4096, fp16 activations, fp32 output."""
    rng = np.random.default_rng(1001)
    w = rng.normal(0, 0.02, (4096, 4096)).astype(np.float32)
    blocks = oracle.quantize(oracle.Q8_0, w)
    x = torch.from_numpy(rng.normal(0, 1, (1, 4096)).astype(np.float32)).to(torch.float16)
    lin = ttq.QuantLinear(ctx, ttq.FMT_Q8_0, torch.from_numpy(blocks), 4096)
    assert np.array_equal(lin.dequantize().cpu().numpy().view(np.uint32),
                          oracle.dequantize(oracle.Q8_0, blocks).view(np.uint32))
    y = lin.forward(x.cuda(), out_dtype=torch.float32).cpu().numpy()
    want = oracle.linear(oracle.Q8_0, blocks, x_bits(x), oracle.F16)
    assert rel_l2(y, want) < TOL
    lin.close()


LLAMA_SHAPES = [(4096, 6144), (4096, 4096), (4096, 28672), (14336, 4096)]


@pytest.mark.parametrize("idx", range(4))
def test_config2_q4_k_llama_shapes(ctx, idx):
    k, n = LLAMA_SHAPES[idx]
    blocks = make_weight(ttq.FMT_Q4_K, n, k, seed=2000 + idx)
    lin = ttq.QuantLinear(ctx, ttq.FMT_Q4_K, torch.from_numpy(blocks), k)
    for m in (1, 4, 16):
        x = make_x(m, k, 2100 + m)
        y = lin.forward(x.cuda(), out_dtype=torch.float32).cpu().numpy()
        want = oracle.linear(oracle.Q4_K, blocks, x_bits(x), oracle.BF16)
        assert rel_l2(y, want) < TOL, (k, n, m)
    lin.close()


def test_gated_mlp_matches_checker(ctx):
    """GatedMLP dataflow (mlp.nim:43-60): gate|up linear, silu_and_mul, down linear."""
    h, inter, m = 512, 1024, 3
    fmt = ttq.FMT_Q4_K
    g, u, d = (make_weight(fmt, inter, h, 50), make_weight(fmt, inter, h, 51), make_weight(fmt, h, inter, 52))
    mlp = ttq.GatedMLP(ctx, fmt, torch.from_numpy(g), torch.from_numpy(u), torch.from_numpy(d), h, inter)
    x = make_x(m, h, 53)
    y = mlp.forward(x.cuda()).float().cpu().numpy()
    gu = oracle.linear(oracle.Q4_K, np.concatenate([g, u]), x_bits(x), oracle.BF16)
    gu16 = torch.from_numpy(gu).to(torch.bfloat16)  # the operator returns the input dtype, like ATen linear
    act = oracle.silu_and_mul(gu16.float().numpy())
    act16 = torch.from_numpy(act).to(torch.bfloat16)
    want = oracle.linear(oracle.Q4_K, d, x_bits(act16), oracle.BF16)
    assert rel_l2(y, want) < 2e-2  # bf16 intermediates; the reference's own layer tolerance (common_utils.nim:55)


def test_silu_and_mul(ctx, aten_witness):
    x = torch.from_numpy(aten_witness["silu_in"]).cuda()
    got = ttq.silu_and_mul(ctx, x).cpu().numpy()
    np.testing.assert_allclose(got, aten_witness["silu_out"], rtol=1e-5, atol=1e-6)
    xb = x.to(torch.bfloat16)
    gb = ttq.silu_and_mul(ctx, xb).float().cpu().numpy()
    np.testing.assert_allclose(gb, oracle.silu_and_mul(xb.float().cpu().numpy()), rtol=1e-2, atol=1e-3)


def test_launch_counter_moves(ctx):
    fmt = ttq.FMT_Q4_K
    lin = ttq.QuantLinear(ctx, fmt, torch.from_numpy(make_weight(fmt, 16, 256, seed=1)), 256)
    before = ctx.launch_count
    lin.forward(torch.zeros(1, 256, dtype=torch.bfloat16, device="cuda"))
    assert ctx.launch_count == before + 2  # activation conversion pass + integer GEMV
    lin.forward(torch.zeros(8, 256, dtype=torch.bfloat16, device="cuda"))
    assert ctx.launch_count == before + 3  # Q4_K batches of 3..16 rows: one kernel, activations converted inside it
    lin.forward(torch.zeros(64, 256, dtype=torch.bfloat16, device="cuda"))
    assert ctx.launch_count == before + 5  # activation pass + tensor-core GEMM
    lin.close()
    q8 = ttq.QuantLinear(ctx, ttq.FMT_Q8_0, torch.from_numpy(make_weight(ttq.FMT_Q8_0, 16, 256, seed=1)), 256)
    before = ctx.launch_count
    q8.forward(torch.zeros(8, 256, dtype=torch.bfloat16, device="cuda"))
    assert ctx.launch_count == before + 2
    q8.close()


@pytest.mark.parametrize("fmt", ALL_FMTS, ids=FMT_IDS)
@pytest.mark.parametrize("m", [1, 3, 8, 40])
def test_gated_input_conversion(ctx, fmt, m):
    """y = W (silu(gate) * up) with the activation folded into the input conversion (decode kernel, fused GEMM
    for Q4_K, expansion + GEMM for the other formats), against the checker's silu_and_mul + linear."""
    n, k = 96, 512
    blocks = make_weight(fmt, n, k, seed=300 + m)
    gu = make_x(m, 2 * k, seed=301 + m)
    lin = ttq.QuantLinear(ctx, fmt, torch.from_numpy(blocks), k)
    y = lin.forward_gated(gu.cuda(), out_dtype=torch.float32)
    ctx.check_device_status()
    act = oracle.silu_and_mul(gu.float().numpy())
    want = oracle.linear(OFMT[fmt], blocks, act, oracle.F32)
    assert rel_l2(y.cpu().numpy(), want) < TOL
    with pytest.raises(ttq.TtqError):
        lin.forward_gated(gu.cuda()[:, : k])
    lin.close()
