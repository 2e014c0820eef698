"""Regenerates tests/golden/trellis_vectors.npz: known-answer vectors of the trellis-coded 3-bit format.

    python tests/golden/make_trellis_golden.py

The decode below is a second, independent statement of the format text in include/ttq.h (TTQ_FMT_TQ3),
written with Python integers (one arbitrary-precision integer per tile stream) and sharing no code with the
C checker or the device kernels.  No reference implementation or third-party witness of this format
exists, so these vectors pin the three implementations against each other, not against the reference.
"""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def decode(packed: np.ndarray, n: int, k: int) -> np.ndarray:
    out = np.empty((n, k), dtype=np.float32)
    unit = np.float32(1.0) / np.float32(147.8)
    tk = k // 16
    for tile in range((n // 16) * tk):
        stream = int.from_bytes(packed[tile * 96:(tile + 1) * 96].tobytes(), "little")
        n0, k0 = (tile // tk) * 16, (tile % tk) * 16
        for t in range(256):
            state = (stream >> (3 * t)) & 0xFFFF
            h = (state * 2654435761) % (1 << 32)
            s = sum((h >> (8 * i)) & 0xFF for i in range(4)) - 510
            out[n0 + t // 16, k0 + t % 16] = np.float32(s) * unit
    return out


def hadamard128(v: np.ndarray) -> np.ndarray:
    """Rows of v (length a multiple of 128) times the orthonormal Sylvester matrix, built explicitly."""
    h = np.array([[1.0]])
    while h.shape[0] < 128:
        h = np.block([[h, h], [h, -h]])
    h /= np.sqrt(128.0)
    return (v.reshape(v.shape[0], -1, 128) @ h).reshape(v.shape)


def linear(packed: np.ndarray, n: int, k: int, x: np.ndarray) -> np.ndarray:
    q = decode(packed, n, k).astype(np.float64)
    scale = packed[n * k * 3 // 8: n * k * 3 // 8 + 2 * n].view(np.float16).astype(np.float64)
    sign_bytes = packed[n * k * 3 // 8 + 2 * n:]
    neg = (sign_bytes[np.arange(k) >> 3] >> (np.arange(k) & 7)) & 1
    x1 = hadamard128(x.astype(np.float64) * np.where(neg == 1, -1.0, 1.0))
    y1 = x1 @ q.T
    return (hadamard128(y1) * scale).astype(np.float32)


def main():
    rng = np.random.default_rng(20250117)
    n, k, m = 128, 256, 3
    nbytes = n * k * 3 // 8 + 2 * n + k // 8
    packed = rng.integers(0, 256, nbytes, dtype=np.uint8)
    # finite, moderate fp16 scales
    scale = rng.normal(0, 0.02, n).astype(np.float16)
    packed[n * k * 3 // 8: n * k * 3 // 8 + 2 * n] = scale.view(np.uint8)
    x = rng.normal(0, 1, (m, k)).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "trellis_vectors.npz"), n=n, k=k, packed=packed, decoded=decode(packed, n, k),
                        x=x, y=linear(packed, n, k, x))


if __name__ == "__main__":
    main()
