"""Regenerates the golden fixtures in this directory.  Run once, by hand, where the witnesses exist:

    python tests/golden/make_golden.py

Two witnesses, neither of them this repository's code:
  * the PyPI package ``gguf`` (gguf/quants.py): dequantization of Q8_0 / Q4_K / Q6_K blocks and the
    Q8_0 quantizer.  The reference tree has no quantized format, so this third-party package is the
    only independent statement of the block layouts available.
  * ATen ``torch.nn.functional.linear`` / ``silu`` on CPU: the exact library call behind the
    reference's ``Linear.forward`` (workspace/transformers/src/layers/linear.nim:45-57) and
    ``silu_and_mul`` (workspace/transformers/src/kernels/activations.nim:37-38).

Inputs are seeded; the fixtures hold inputs and witness outputs only.
"""
import os

import numpy as np
import torch
import torch.nn.functional as F
from gguf import GGMLQuantizationType as T
from gguf import quants

HERE = os.path.dirname(os.path.abspath(__file__))
SIZES = {"q8_0": (32, 34, T.Q8_0), "q4_k": (256, 144, T.Q4_K), "q6_k": (256, 210, T.Q6_K)}
# byte offsets of the fp16 fields inside a block
F16_FIELDS = {"q8_0": (0,), "q4_k": (0, 2), "q6_k": (208,)}


def random_blocks(rng, name, rows, blocks_per_row):
    """Uniformly random bytes with every fp16 field forced finite (exponent != 31)."""
    _, nbytes, _ = SIZES[name]
    b = rng.integers(0, 256, (rows, blocks_per_row, nbytes), dtype=np.uint8)
    for off in F16_FIELDS[name]:
        hi = b[:, :, off + 1]
        hi[(hi & 0x7C) == 0x7C] &= 0x3F
    return b.reshape(rows, blocks_per_row * nbytes)


def main():
    rng = np.random.default_rng(20240611)
    out = {}
    # (1) witness dequantization of random bytes, every format
    for name, (_, _, t) in SIZES.items():
        blocks = random_blocks(rng, name, 8, 3 if name != "q8_0" else 24)
        out[f"{name}_rand_blocks"] = blocks
        out[f"{name}_rand_deq"] = quants.dequantize(blocks, t).astype(np.float32)
    # edge patterns: all-zero block, all-ones bytes with finite scales, extreme quants
    for name, (_, nbytes, t) in SIZES.items():
        z = np.zeros((1, nbytes), dtype=np.uint8)
        o = np.full((1, nbytes), 0xFF, dtype=np.uint8)
        for off in F16_FIELDS[name]:
            o[0, off] = 0x00
            o[0, off + 1] = 0x3C  # fp16 1.0
        edge = np.concatenate([z, o], axis=0)
        out[f"{name}_edge_blocks"] = edge
        out[f"{name}_edge_deq"] = quants.dequantize(edge, t).astype(np.float32)
    # (2) witness Q8_0 quantizer on N(0, 0.02) weights (the only quantizer the package implements)
    w = rng.normal(0.0, 0.02, (16, 256)).astype(np.float32)
    w[3, :32] = 0.0  # an all-zero block
    out["q8_0_w"] = w
    out["q8_0_w_blocks"] = quants.quantize(w, T.Q8_0)
    np.savez_compressed(os.path.join(HERE, "gguf_witness.npz"), **out)

    # (3) ATen linear / silu on CPU, bf16 like the reference's layer fixtures
    torch.manual_seed(42)
    dense = {}
    for tag, (m, k, n, with_bias) in {"a": (3, 64, 48, True), "b": (1, 256, 32, False)}.items():
        W = (torch.randn(n, k) * 0.02).to(torch.bfloat16)
        x = torch.randn(m, k).to(torch.bfloat16)
        b = (torch.randn(n) * 0.1).to(torch.bfloat16) if with_bias else None
        y = F.linear(x.float(), W.float(), None if b is None else b.float())
        dense[f"{tag}_W"] = W.float().numpy()
        dense[f"{tag}_x_bits"] = x.view(torch.int16).numpy().view(np.uint16)
        if b is not None:
            dense[f"{tag}_b"] = b.float().numpy()
        dense[f"{tag}_y"] = y.numpy()
    g = torch.randn(4, 96)
    gate, up = g.chunk(2, -1)
    dense["silu_in"] = g.numpy()
    dense["silu_out"] = (F.silu(gate) * up).numpy()
    np.savez_compressed(os.path.join(HERE, "aten_witness.npz"), **dense)
    print("wrote gguf_witness.npz, aten_witness.npz")


if __name__ == "__main__":
    main()
