"""Repack + device dequantization must reproduce the CPU checker bit for bit (through the C ABI)."""
import numpy as np
import pytest
import torch

import oracle
import tattletale_b200 as ttq
from gpu_util import ALL_FMTS, FMT_IDS, OFMT, bits, make_weight, random_blocks

pytestmark = pytest.mark.gpu

GOLD = {ttq.FMT_Q8_0: "q8_0", ttq.FMT_Q4_K: "q4_k", ttq.FMT_Q6_K: "q6_k"}


def gpu_dequant(ctx, fmt, blocks, k, device_blocks=False, shard=None):
    t = torch.from_numpy(blocks)
    if device_blocks:
        t = t.cuda()
    lin = ttq.QuantLinear(ctx, fmt, t, k, shard=shard)
    out = lin.dequantize().cpu().numpy()
    lin.close()
    return out


@pytest.mark.parametrize("fmt", ALL_FMTS, ids=FMT_IDS)
@pytest.mark.parametrize("kind", ["rand", "edge"])
def test_golden_blocks_bit_exact(ctx, gguf_witness, fmt, kind):
    blocks = gguf_witness[f"{GOLD[fmt]}_{kind}_blocks"]
    want = gguf_witness[f"{GOLD[fmt]}_{kind}_deq"]
    got = gpu_dequant(ctx, fmt, blocks, want.shape[1])
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("fmt", ALL_FMTS, ids=FMT_IDS)
@pytest.mark.parametrize("n,kblocks", [(1, 1), (16, 2), (17, 3), (100, 5), (256, 16)])
def test_random_bytes_bit_exact(ctx, fmt, n, kblocks):
    per = 8 if fmt == ttq.FMT_Q8_0 else 1  # keep K a multiple of 256 here; ragged K is tested below
    blocks = random_blocks(fmt, n, kblocks * per, seed=100 + n)
    want = oracle.dequantize(OFMT[fmt], blocks)
    for dev in (False, True):
        got = gpu_dequant(ctx, fmt, blocks, want.shape[1], device_blocks=dev)
        assert np.array_equal(bits(got), bits(want))


def test_q8_0_k_not_multiple_of_256(ctx):
    blocks = random_blocks(ttq.FMT_Q8_0, 20, 11, seed=5)  # K = 352
    want = oracle.dequantize(oracle.Q8_0, blocks)
    got = gpu_dequant(ctx, ttq.FMT_Q8_0, blocks, 352)
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("fmt", ALL_FMTS, ids=FMT_IDS)
def test_quantized_normal_weights_bit_exact(ctx, fmt):
    blocks = make_weight(fmt, 512, 2048, seed=21)
    want = oracle.dequantize(OFMT[fmt], blocks)
    got = gpu_dequant(ctx, fmt, blocks, 2048)
    assert np.array_equal(bits(got), bits(want))


def test_config_sizes_checksum(ctx):
    """Llama-3-8B down projection at full size: every dequantized bit agrees (xor / sum checksums)."""
    fmt = ttq.FMT_Q4_K
    blocks = make_weight(fmt, 4096, 14336, seed=2003)
    want = oracle.dequantize(oracle.Q4_K, blocks)
    got = gpu_dequant(ctx, fmt, blocks, 14336)
    assert np.bitwise_xor.reduce(bits(got).ravel()) == np.bitwise_xor.reduce(bits(want).ravel())
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.parametrize("fmt", ALL_FMTS, ids=FMT_IDS)
def test_shards_are_slices_of_the_full_matrix(ctx, fmt):
    n, k, world = 64, 1024, 2
    blocks = make_weight(fmt, n, k, seed=33)
    full = oracle.dequantize(OFMT[fmt], blocks)
    for rank in range(world):
        col = gpu_dequant(ctx, fmt, blocks, k, shard=(ttq.SHARD_COLUMN, rank, world))
        assert np.array_equal(bits(col), bits(full[rank * 32:(rank + 1) * 32]))
        gated = gpu_dequant(ctx, fmt, blocks, k, shard=(ttq.SHARD_COLUMN_GATED, rank, world))
        want = np.concatenate([full[rank * 16:(rank + 1) * 16], full[32 + rank * 16:32 + (rank + 1) * 16]])
        assert np.array_equal(bits(gated), bits(want))
        row = gpu_dequant(ctx, fmt, blocks, k, shard=(ttq.SHARD_ROW, rank, world))
        assert np.array_equal(bits(row), bits(full[:, rank * 512:(rank + 1) * 512]))


def test_create_rejects_bad_arguments(ctx):
    good = torch.from_numpy(make_weight(ttq.FMT_Q4_K, 16, 256, seed=1))
    with pytest.raises(ttq.TtqError, match="SHAPE"):
        ttq.QuantLinear(ctx, ttq.FMT_Q4_K, good, 512)  # nbytes mismatch
    with pytest.raises(ttq.TtqError, match="SHAPE"):
        ttq.QuantLinear(ctx, ttq.FMT_Q4_K, good, 100)  # K not a multiple of 256
    with pytest.raises(ttq.TtqError, match="INVALID_ARG"):
        ttq.QuantLinear(ctx, 9, good, 256)
    with pytest.raises(ttq.TtqError, match="SHAPE"):
        ttq.QuantLinear(ctx, ttq.FMT_Q4_K, good, 256, shard=(ttq.SHARD_ROW, 0, 2))  # K/world not a block multiple
    with pytest.raises(ttq.TtqError):
        ttq.QuantLinear(ctx, ttq.FMT_Q4_K, good, 256, shard=(ttq.SHARD_COLUMN, 2, 2))
