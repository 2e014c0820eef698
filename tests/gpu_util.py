"""Shared helpers of the GPU parity tests."""
import numpy as np
import torch

import oracle
import tattletale_b200 as ttq

OFMT = {ttq.FMT_Q8_0: oracle.Q8_0, ttq.FMT_Q4_K: oracle.Q4_K, ttq.FMT_Q6_K: oracle.Q6_K}
ALL_FMTS = [ttq.FMT_Q8_0, ttq.FMT_Q4_K, ttq.FMT_Q6_K]
FMT_IDS = ["q8_0", "q4_k", "q6_k"]


def make_weight(fmt, n, k, seed, std=0.02):
    rng = np.random.default_rng(seed)
    w = rng.normal(0.0, std, (n, k)).astype(np.float32)
    return oracle.quantize(OFMT[fmt], w)


def make_x(m, k, seed, dtype=torch.bfloat16):
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.normal(0.0, 1.0, (m, k)).astype(np.float32)).to(dtype)
    return x


def x_bits(x):
    return x.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def odt(dtype):
    return oracle.BF16 if dtype == torch.bfloat16 else oracle.F16


def random_blocks(fmt, rows, blocks_per_row, seed):
    """Uniformly random bytes with finite fp16 fields."""
    rng = np.random.default_rng(seed)
    nb = oracle.BLOCK_BYTES[OFMT[fmt]]
    b = rng.integers(0, 256, (rows, blocks_per_row, nb), dtype=np.uint8)
    offs = {ttq.FMT_Q8_0: (0,), ttq.FMT_Q4_K: (0, 2), ttq.FMT_Q6_K: (208,)}[fmt]
    for off in offs:
        hi = b[:, :, off + 1]
        hi[(hi & 0x7C) == 0x7C] &= 0x3F
    return b.reshape(rows, blocks_per_row * nb)


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
