"""Trellis-coded 3-bit linear on the GPU against the CPU checker, through the C ABI: bit-exact decode, the
decode-and-multiply kernel (up to 4 rows), and the expansion + tensor-core GEMM path beyond."""
import os

import numpy as np
import pytest
import torch

import oracle
import tattletale_b200 as ttq
from conftest import rel_l2
from gpu_util import make_x, x_bits

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "trellis_vectors.npz"))


def random_packed(n, k, seed):
    """Uniformly random code bits (every bit pattern is a valid code) with moderate fp16 scales."""
    rng = np.random.default_rng(seed)
    p = rng.integers(0, 256, oracle.tq3_packed_bytes(n, k), dtype=np.uint8)
    scale = (rng.normal(0, 0.02, n) + np.sign(rng.normal(0, 1, n)) * 0.01).astype(np.float16)
    p[n * k * 3 // 8: n * k * 3 // 8 + 2 * n] = scale.view(np.uint8)
    return p


def layer(ctx, packed, n, k, bias=None):
    return ttq.QuantLinear(ctx, ttq.FMT_TQ3, torch.from_numpy(packed), k, bias=bias, out_features=n)


def test_decode_known_answers_bit_exact(ctx):
    n, k = int(GOLD["n"]), int(GOLD["k"])
    lin = layer(ctx, GOLD["packed"], n, k)
    got = lin.dequantize().cpu().numpy()
    assert np.array_equal(got.view(np.uint32), GOLD["decoded"].view(np.uint32))
    lin.close()


@pytest.mark.parametrize("n,k", [(128, 128), (256, 384), (384, 2048)])
def test_decode_random_codes_bit_exact(ctx, n, k):
    packed = random_packed(n, k, seed=n + k)
    lin = layer(ctx, packed, n, k)
    got = lin.dequantize().cpu().numpy()
    want = oracle.tq3_decode(packed, n, k)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    lin.close()


@pytest.mark.parametrize("m", [1, 2, 3, 4])
def test_decode_and_multiply_rows(ctx, m):
    n, k = 256, 1024
    packed = random_packed(n, k, seed=40 + m)
    lin = layer(ctx, packed, n, k)
    x = make_x(m, k, seed=m)
    y = lin.forward(x.cuda(), out_dtype=torch.float32)
    want = oracle.tq3_linear(packed, n, k, x_bits(x), oracle.BF16)
    assert rel_l2(y.cpu().numpy(), want) < 1e-5  # fp32 rotations and accumulation against fp64
    lin.close()


@pytest.mark.parametrize("m", [5, 8, 16, 17, 33, 64, 65, 100, 300, 700])
def test_tensor_core_paths(ctx, m):
    """5..64 rows: decoded weights as the B operand of mma.sync (every weight decoded once, activations in fragment
    order); beyond: whole-weight expansion + plain tcgen05 GEMM."""
    n, k = 384, 640
    packed = random_packed(n, k, seed=60 + m)
    bias = torch.from_numpy(np.random.default_rng(m).normal(0, 0.1, n).astype(np.float32))
    lin = layer(ctx, packed, n, k, bias=bias.cuda())
    x = make_x(m, k, seed=m + 1)
    y = lin.forward(x.cuda(), out_dtype=torch.float32)
    ctx.check_device_status()
    want = oracle.tq3_linear(packed, n, k, x_bits(x), oracle.BF16, bias.numpy())
    assert rel_l2(y.cpu().numpy(), want) < 1e-3  # codes and rotated activations rounded to fp16 for the MMA
    lin.close()


def test_encoded_weight_end_to_end(ctx):
    """Encoder -> device linear reproduces the dense product within the code's own error."""
    rng = np.random.default_rng(9)
    n, k, m = 128, 256, 4
    w = rng.normal(0, 0.015, (n, k)).astype(np.float32)
    packed, _ = oracle.tq3_encode(w, seed=4)
    lin = layer(ctx, packed, n, k)
    x = make_x(m, k, seed=3, dtype=torch.float16)
    y = lin.forward(x.cuda(), out_dtype=torch.float16).float().cpu().numpy()
    want = oracle.tq3_linear(packed, n, k, x_bits(x), oracle.F16)
    assert rel_l2(y, want) < 2e-3
    dense = x.float().numpy() @ w.T
    assert rel_l2(y, dense) < 0.25
    lin.close()


def test_known_answer_linear(ctx):
    n, k = int(GOLD["n"]), int(GOLD["k"])
    lin = layer(ctx, GOLD["packed"], n, k)
    x = torch.from_numpy(GOLD["x"]).to(torch.bfloat16)
    y = lin.forward(x.cuda(), out_dtype=torch.float32).cpu().numpy()
    want = oracle.tq3_linear(GOLD["packed"], n, k, x_bits(x), oracle.BF16)
    assert rel_l2(y, want) < 1e-5
    lin.close()


def test_argument_errors(ctx):
    packed = random_packed(128, 128, 1)
    with pytest.raises(ttq.TtqError):
        ttq.QuantLinear(ctx, ttq.FMT_TQ3, torch.from_numpy(packed), 128, out_features=64)   # N not a multiple of 128
    with pytest.raises(ttq.TtqError):
        ttq.QuantLinear(ctx, ttq.FMT_TQ3, torch.from_numpy(packed[:-1].copy()), 128, out_features=128)  # short buffer
    with pytest.raises(ttq.TtqError):
        ttq.QuantLinear(ctx, ttq.FMT_TQ3, torch.from_numpy(packed), 128, out_features=128, shard=(ttq.SHARD_ROW, 0, 2))
