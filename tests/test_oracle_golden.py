"""Pins the CPU checker (oracle/) against the committed witness fixtures (tests/golden/)."""
import numpy as np
import pytest

import oracle

FMTS = {"q8_0": oracle.Q8_0, "q4_k": oracle.Q4_K, "q6_k": oracle.Q6_K}


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("name", list(FMTS))
@pytest.mark.parametrize("kind", ["rand", "edge"])
def test_dequant_matches_witness_bit_exact(gguf_witness, name, kind):
    blocks = gguf_witness[f"{name}_{kind}_blocks"]
    want = gguf_witness[f"{name}_{kind}_deq"]
    got = oracle.dequantize(FMTS[name], blocks)
    assert got.shape == want.shape
    assert np.array_equal(bits(got), bits(want))


def test_q8_0_quantizer_matches_witness(gguf_witness):
    got = oracle.quantize(oracle.Q8_0, gguf_witness["q8_0_w"])
    assert np.array_equal(got, gguf_witness["q8_0_w_blocks"])


@pytest.mark.parametrize("name", list(FMTS))
def test_quantize_dequantize_is_close(name):
    rng = np.random.default_rng(7)
    w = rng.normal(0, 0.02, (8, 512)).astype(np.float32)
    fmt = FMTS[name]
    deq = oracle.dequantize(fmt, oracle.quantize(fmt, w))
    err = np.linalg.norm(deq - w) / np.linalg.norm(w)
    assert err < {"q8_0": 0.01, "q4_k": 0.12, "q6_k": 0.03}[name]


@pytest.mark.parametrize("name", list(FMTS))
def test_requantize_is_stable(name):
    """Dequantized weights are a fixed point of encode->decode up to the format's own rounding."""
    rng = np.random.default_rng(8)
    fmt = FMTS[name]
    w = rng.normal(0, 0.02, (4, 256)).astype(np.float32)
    d1 = oracle.dequantize(fmt, oracle.quantize(fmt, w))
    d2 = oracle.dequantize(fmt, oracle.quantize(fmt, d1))
    assert np.linalg.norm(d2 - d1) / np.linalg.norm(d1) < 0.05


@pytest.mark.parametrize("tag", ["a", "b"])
def test_dense_operator_matches_aten(aten_witness, tag):
    W, x = aten_witness[f"{tag}_W"], aten_witness[f"{tag}_x_bits"]
    b = aten_witness.get(f"{tag}_b")
    y = oracle.linear_dense(W, x, oracle.BF16, b)
    np.testing.assert_allclose(y, aten_witness[f"{tag}_y"], rtol=1e-5, atol=1e-6)


def test_quantized_operator_equals_dense_on_dequantized_weights():
    rng = np.random.default_rng(9)
    for fmt in FMTS.values():
        w = rng.normal(0, 0.02, (24, 512)).astype(np.float32)
        blocks = oracle.quantize(fmt, w)
        x = oracle.to_bf16_bits(rng.normal(0, 1, (3, 512)).astype(np.float32))
        bias = rng.normal(0, 0.1, 24).astype(np.float32)
        y = oracle.linear(fmt, blocks, x, oracle.BF16, bias)
        y_dense = oracle.linear_dense(oracle.dequantize(fmt, blocks), x, oracle.BF16, bias)
        assert np.array_equal(y, y_dense)
        y_fast = oracle.linear(fmt, blocks, x, oracle.BF16, bias, fast=True)
        np.testing.assert_allclose(y_fast, y, rtol=1e-4, atol=1e-5)


def test_silu_and_mul_matches_aten(aten_witness):
    got = oracle.silu_and_mul(aten_witness["silu_in"])
    np.testing.assert_allclose(got, aten_witness["silu_out"], rtol=1e-6, atol=1e-7)


def test_half_conversions_exhaustive():
    L = oracle.lib()
    allh = np.arange(65536, dtype=np.uint16)
    ref = allh.view(np.float16).astype(np.float32)
    mine = np.array([L.ttq_ref_f16_to_f32(int(h)) for h in allh], dtype=np.float32)
    ok = ~np.isnan(ref)
    assert np.array_equal(bits(ref)[ok], bits(mine)[ok])
    back = np.array([L.ttq_ref_f32_to_f16(float(v)) for v in ref[ok]], dtype=np.uint16)
    assert np.array_equal(back, allh[ok])


def test_bf16_bits_helper():
    x = np.array([1.0, -2.5, 3.1415927, 1e-8, 65504.0], dtype=np.float32)
    import torch

    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.to_bf16_bits(x), want)
