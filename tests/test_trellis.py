"""Trellis-coded 3-bit format on the CPU: the C checker against the committed known-answer vectors (made by an
independent Python-integer statement of the format), encoder self-consistency, and the package's beam-search
encoder against the checker's exact search."""
import os

import numpy as np
import pytest
import torch

import oracle
from tattletale_b200 import FMT_TQ3, formats
from tattletale_b200 import quantize as Q

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "trellis_vectors.npz"))


def test_decode_matches_known_answers_bit_exact():
    n, k = int(GOLD["n"]), int(GOLD["k"])
    got = oracle.tq3_decode(GOLD["packed"], n, k)
    assert np.array_equal(got.view(np.uint32), GOLD["decoded"].view(np.uint32))
    # about unit variance, centred: the codebook is a sum of four hashed bytes
    assert abs(float(got.std()) - 1.0) < 0.05 and abs(float(got.mean())) < 0.05


def test_linear_matches_known_answers():
    n, k = int(GOLD["n"]), int(GOLD["k"])
    y = oracle.tq3_linear(GOLD["packed"], n, k, np.ascontiguousarray(GOLD["x"]), oracle.F32)
    assert np.linalg.norm(y - GOLD["y"]) / np.linalg.norm(GOLD["y"]) < 1e-6


def test_packed_size():
    assert oracle.tq3_packed_bytes(128, 256) == 128 * 256 * 3 // 8 + 256 + 32 == formats.packed_bytes(FMT_TQ3, 128, 256)
    with pytest.raises(ValueError):
        formats.packed_bytes(FMT_TQ3, 100, 256)


def test_encoder_roundtrip_and_operator():
    rng = np.random.default_rng(5)
    n, k = 128, 256
    w = rng.normal(0, 0.015, (n, k)).astype(np.float32)
    w[5] *= 8.0  # an outlier row: the per-row scale absorbs it
    packed, mse = oracle.tq3_encode(w, seed=3)
    assert 0.005 < mse < 0.035  # 3 bits per weight on a unit-variance target
    w_eff = oracle.tq3_effective_weight(packed, n, k)
    rel = np.linalg.norm(w_eff - w) / np.linalg.norm(w)
    assert rel < 0.2
    # the operator applies exactly that matrix
    x = rng.normal(0, 1, (4, k)).astype(np.float32)
    y = oracle.tq3_linear(packed, n, k, x, oracle.F32)
    want = x.astype(np.float64) @ w_eff.astype(np.float64).T
    assert np.linalg.norm(y - want) / np.linalg.norm(want) < 1e-5
    # encoding is deterministic
    again, _ = oracle.tq3_encode(w, seed=3)
    assert np.array_equal(packed, again)


def test_zero_rows_do_not_break_the_encoder():
    w = np.zeros((128, 128), dtype=np.float32)
    w[0, 0] = 1.0
    packed, _ = oracle.tq3_encode(w, seed=1)
    assert np.isfinite(oracle.tq3_effective_weight(packed, 128, 128)).all()


def test_beam_encoder_is_a_valid_code_close_to_the_exact_search():
    rng = np.random.default_rng(6)
    n, k = 128, 128
    w = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    packed = Q.quantize_tq3(torch.from_numpy(w), seed=2, beam=64).numpy()
    assert packed.size == oracle.tq3_packed_bytes(n, k)
    rel_beam = np.linalg.norm(oracle.tq3_effective_weight(packed, n, k) - w) / np.linalg.norm(w)
    exact, _ = oracle.tq3_encode(w, seed=2)
    rel_exact = np.linalg.norm(oracle.tq3_effective_weight(exact, n, k) - w) / np.linalg.norm(w)
    assert rel_exact < 0.2
    assert rel_beam < 1.35 * rel_exact


def test_tensor_parallel_slices_add_up():
    """Column slices concatenate and row slices sum to the full operator (host-side shard helper + checker)."""
    from tattletale_b200 import SHARD_COLUMN, SHARD_ROW, tp

    rng = np.random.default_rng(8)
    n, k, world = 256, 512, 2
    packed = rng.integers(0, 256, oracle.tq3_packed_bytes(n, k), dtype=np.uint8)
    packed[n * k * 3 // 8: n * k * 3 // 8 + 2 * n] = rng.normal(0, 0.02, n).astype(np.float16).view(np.uint8)
    x = rng.normal(0, 1, (3, k)).astype(np.float32)
    full = oracle.tq3_linear(packed, n, k, x, oracle.F32)
    cols, rows = [], np.zeros_like(full, dtype=np.float64)
    for r in range(world):
        p, nl, kl = tp.shard_trellis(torch.from_numpy(packed), n, k, SHARD_COLUMN, r, world)
        assert (nl, kl) == (n // world, k) and p.numel() == oracle.tq3_packed_bytes(nl, kl)
        cols.append(oracle.tq3_linear(p.numpy(), nl, kl, x, oracle.F32))
        p, nl, kl = tp.shard_trellis(torch.from_numpy(packed), n, k, SHARD_ROW, r, world)
        assert (nl, kl) == (n, k // world) and p.numel() == oracle.tq3_packed_bytes(nl, kl)
        rows += oracle.tq3_linear(p.numpy(), nl, kl, np.ascontiguousarray(x[:, r * kl:(r + 1) * kl]), oracle.F32)
    assert np.array_equal(np.concatenate(cols, axis=1), full)
    assert np.linalg.norm(rows - full) / np.linalg.norm(full) < 1e-6
    with pytest.raises(ValueError):
        tp.shard_trellis(torch.from_numpy(packed), n, k, SHARD_ROW, 0, 8)
