"""CPU checker for the quantized-linear path (test infrastructure, not a product code path).

Thin ctypes binding over ``oracle/libttq_oracle.so`` (built from ``ttq_oracle.c`` by
``oracle/Makefile``).  Only the test-suite, the smoke check and the CPU-baseline leg of the
benchmark import this module; the product package never does.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libttq_oracle.so")

Q8_0, Q4_K, Q6_K = 0, 1, 2
BF16, F16, F32 = 0, 1, 2
BLOCK_ELEMS = {Q8_0: 32, Q4_K: 256, Q6_K: 256}
BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q6_K: 210}

_lib = None


def build(force: bool = False) -> str:
    """Compile the checker with gcc if the shared object is missing or stale."""
    src = os.path.join(_HERE, "ttq_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libttq_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        i64, vp, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        L.ttq_ref_dequantize.argtypes = [ci, vp, i64, vp]
        L.ttq_ref_quantize.argtypes = [ci, vp, i64, vp]
        for name in ("ttq_ref_linear", "ttq_ref_linear_fast"):
            getattr(L, name).argtypes = [ci, vp, i64, i64, vp, ci, i64, i64, vp, vp, i64]
        L.ttq_ref_linear_dense.argtypes = [vp, i64, i64, vp, ci, i64, i64, vp, vp, i64]
        L.ttq_ref_silu_and_mul.argtypes = [vp, i64, i64, vp]
        L.ttq_ref_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.ttq_ref_f16_to_f32.restype = ctypes.c_float
        L.ttq_ref_f32_to_f16.argtypes = [ctypes.c_float]
        L.ttq_ref_f32_to_f16.restype = ctypes.c_uint16
        L.ttq_ref_num_threads.restype = ci
        L.ttq_tq3_packed_bytes.argtypes = [i64, i64]
        L.ttq_tq3_packed_bytes.restype = i64
        L.ttq_tq3_decode.argtypes = [vp, i64, i64, vp]
        L.ttq_tq3_effective_weight.argtypes = [vp, i64, i64, vp]
        L.ttq_tq3_linear.argtypes = [vp, i64, i64, vp, ci, i64, i64, vp, vp, i64]
        L.ttq_tq3_encode.argtypes = [vp, i64, i64, ctypes.c_uint32, vp, vp]
        _lib = L
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def quantize(fmt: int, w: np.ndarray) -> np.ndarray:
    """fp32 [N, K] -> canonical blocks, uint8 [N, K / block_elems * block_bytes]."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    assert k % BLOCK_ELEMS[fmt] == 0
    out = np.zeros((n, k // BLOCK_ELEMS[fmt] * BLOCK_BYTES[fmt]), dtype=np.uint8)
    rc = lib().ttq_ref_quantize(fmt, _ptr(w), w.size, _ptr(out))
    assert rc == 0, rc
    return out


def dequantize(fmt: int, blocks: np.ndarray) -> np.ndarray:
    """canonical blocks uint8 [N, bytes_per_row] -> fp32 [N, K]."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    n, nbytes = blocks.shape
    assert nbytes % BLOCK_BYTES[fmt] == 0
    nb = nbytes // BLOCK_BYTES[fmt]
    out = np.empty((n, nb * BLOCK_ELEMS[fmt]), dtype=np.float32)
    rc = lib().ttq_ref_dequantize(fmt, _ptr(blocks), n * nb, _ptr(out))
    assert rc == 0, rc
    return out


def _act(x: np.ndarray, x_dtype: int) -> np.ndarray:
    if x_dtype in (BF16, F16):
        assert x.dtype == np.uint16, "16-bit activations are passed as raw uint16 bit patterns"
    else:
        assert x.dtype == np.float32
    return np.ascontiguousarray(x)


def linear(fmt: int, blocks: np.ndarray, x: np.ndarray, x_dtype: int, bias: np.ndarray | None = None,
           fast: bool = False) -> np.ndarray:
    """y = x . W^T + b, fp64 accumulation (fp32 when ``fast``).  x: [M, K]; returns fp32 [M, N]."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    x = _act(x, x_dtype)
    m, k = x.shape
    n = blocks.shape[0]
    assert blocks.shape[1] == k // BLOCK_ELEMS[fmt] * BLOCK_BYTES[fmt]
    y = np.empty((m, n), dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    fn = lib().ttq_ref_linear_fast if fast else lib().ttq_ref_linear
    rc = fn(fmt, _ptr(blocks), n, k, _ptr(x), x_dtype, m, k, None if b is None else _ptr(b), _ptr(y), n)
    assert rc == 0, rc
    return y


def linear_dense(w: np.ndarray, x: np.ndarray, x_dtype: int, bias: np.ndarray | None = None) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.float32)
    x = _act(x, x_dtype)
    m, k = x.shape
    n = w.shape[0]
    y = np.empty((m, n), dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    rc = lib().ttq_ref_linear_dense(_ptr(w), n, k, _ptr(x), x_dtype, m, k, None if b is None else _ptr(b),
                                    _ptr(y), n)
    assert rc == 0, rc
    return y


def silu_and_mul(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    m, h2 = x.shape
    out = np.empty((m, h2 // 2), dtype=np.float32)
    lib().ttq_ref_silu_and_mul(_ptr(x), m, h2 // 2, _ptr(out))
    return out


def moe(fmt: int, gate_up_blocks, down_blocks, x: np.ndarray, x_dtype: int, topk_ids: np.ndarray,
        topk_weights: np.ndarray, f16_intermediates: bool = True) -> np.ndarray:
    """Mixture of gated-MLP experts: y[t] = sum_j w[t, j] * down_e(silu(gate_e x[t]) * up_e x[t]), e = ids[t, j].

    The per-expert MLP is the dataflow of the reference's GatedMLP (workspace/transformers/src/layers/mlp.nim:56-60)
    built from this module's own linear and silu_and_mul.  With ``f16_intermediates`` the two intermediate
    tensors are rounded to fp16 where the device path stores them (after gate|up, after down); without, everything
    between the projections stays fp32.  ids outside 0..E-1 contribute nothing.  Sum over j in fp64, ascending j.
    """
    t, k = topk_ids.shape
    n_exp = len(gate_up_blocks)
    hidden = down_blocks[0].shape[0]
    y = np.zeros((t, hidden), dtype=np.float64)
    for e in range(n_exp):
        tok, j = np.nonzero(topk_ids == e)
        if tok.size == 0:
            continue
        h = linear(fmt, gate_up_blocks[e], np.ascontiguousarray(x[tok]), x_dtype)
        if f16_intermediates:
            h = h.astype(np.float16).astype(np.float32)
        a = silu_and_mul(h)
        o = linear(fmt, down_blocks[e], to_f16_bits(a), F16)
        if f16_intermediates:
            o = o.astype(np.float16).astype(np.float32)
        np.add.at(y, tok, o.astype(np.float64) * topk_weights[tok, j].astype(np.float64)[:, None])
    return y.astype(np.float32)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit patterns (round to nearest even)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def to_f16_bits(x: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def num_threads() -> int:
    return int(lib().ttq_ref_num_threads())


# ---- trellis-coded 3-bit format (oracle/ttq_trellis.c) ---------------------------------------------------
TQ3 = 3


def tq3_packed_bytes(n: int, k: int) -> int:
    return int(lib().ttq_tq3_packed_bytes(n, k))


def tq3_encode(w: np.ndarray, seed: int = 1):
    """fp32 [N, K] -> (packed uint8 buffer, mean squared code error against the rotated unit-variance target)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    out = np.zeros(tq3_packed_bytes(n, k), dtype=np.uint8)
    mse = ctypes.c_double()
    rc = lib().ttq_tq3_encode(_ptr(w), n, k, seed, _ptr(out), ctypes.addressof(mse))
    assert rc == 0, rc
    return out, float(mse.value)


def tq3_decode(packed: np.ndarray, n: int, k: int) -> np.ndarray:
    """The decoded codes q [N, K] (before rotations and scales): bit-exact target of the device decode."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    assert packed.size == tq3_packed_bytes(n, k)
    out = np.empty((n, k), dtype=np.float32)
    assert lib().ttq_tq3_decode(_ptr(packed), n, k, _ptr(out)) == 0
    return out


def tq3_effective_weight(packed: np.ndarray, n: int, k: int) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty((n, k), dtype=np.float32)
    assert lib().ttq_tq3_effective_weight(_ptr(packed), n, k, _ptr(out)) == 0
    return out


def tq3_linear(packed: np.ndarray, n: int, k: int, x: np.ndarray, x_dtype: int, bias: np.ndarray | None = None) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    x = _act(x, x_dtype)
    m = x.shape[0]
    assert x.shape[1] == k
    y = np.empty((m, n), dtype=np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    rc = lib().ttq_tq3_linear(_ptr(packed), n, k, _ptr(x), x_dtype, m, k, None if b is None else _ptr(b), _ptr(y), n)
    assert rc == 0, rc
    return y
