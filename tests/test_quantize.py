"""Package-side encoders emit valid blocks (checked by decoding them with the CPU checker)."""
import numpy as np
import pytest
import torch

import oracle
from tattletale_b200 import quantize as Q

FMTS = [(Q.FMT_Q8_0, oracle.Q8_0, 0.01), (Q.FMT_Q4_K, oracle.Q4_K, 0.12), (Q.FMT_Q6_K, oracle.Q6_K, 0.03)]


@pytest.mark.parametrize("fmt,ofmt,tol", FMTS)
def test_encoder_round_trip(fmt, ofmt, tol):
    rng = np.random.default_rng(11)
    w = rng.normal(0, 0.02, (32, 1024)).astype(np.float32)
    w[2, :256] = 0.0
    blocks = Q.quantize(fmt, torch.from_numpy(w)).numpy()
    assert blocks.shape == (32, 1024 // oracle.BLOCK_ELEMS[ofmt] * oracle.BLOCK_BYTES[ofmt])
    deq = oracle.dequantize(ofmt, blocks)
    assert np.all(np.isfinite(deq))
    assert np.all(deq[2, :256] == 0.0)
    assert np.linalg.norm(deq - w) / np.linalg.norm(w) < tol


def test_q8_0_encoder_equals_checker_encoder():
    rng = np.random.default_rng(12)
    w = rng.normal(0, 0.02, (16, 512)).astype(np.float32)
    assert np.array_equal(Q.quantize(Q.FMT_Q8_0, torch.from_numpy(w)).numpy(), oracle.quantize(oracle.Q8_0, w))
