"""tattletale_b200 -- B200 (sm_100a) quantized-linear kernels behind tattletale's ``Linear`` API.

Host-side mirror of the reference operator interface (workspace/transformers/src/layers):

  ``Linear.init(weight, bias)`` / ``Linear.forward(x)``          linear.nim:29-57
  ``GatedMLP.init(gate, up, down, activation)`` / ``.forward``   mlp.nim:31-60
  ``silu_and_mul``                                               kernels/activations.nim:14-38

with the dense weight replaced by GGUF-style block-quantized bytes.  All compute happens in
``libttq.so`` through the C ABI of ``include/ttq.h``; torch is used only for device buffers and
streams.  Importing this package does not need a GPU; creating a :class:`Context` does.
"""
from ._lib import (DT_BF16, DT_F16, DT_F32, FMT_Q4_K, FMT_Q6_K, FMT_Q8_0, FMT_TQ3, SHARD_COLUMN,
                   SHARD_COLUMN_GATED, SHARD_NONE, SHARD_ROW, TtqError)
from .layers import (ActivationKind, Context, GatedMLP, HostBatch, MoELayer, QuantLinear, add_rmsnorm, decode_attention,
                     rope_kv_append, silu_and_mul)
from .formats import BLOCK_BYTES, BLOCK_ELEMS, FORMAT_NAMES, packed_bytes
from . import tp

__all__ = [
    "Context", "QuantLinear", "HostBatch", "GatedMLP", "MoELayer", "add_rmsnorm", "rope_kv_append", "decode_attention", "ActivationKind", "silu_and_mul", "TtqError",
    "FMT_Q8_0", "FMT_Q4_K", "FMT_Q6_K", "FMT_TQ3", "DT_BF16", "DT_F16", "DT_F32",
    "SHARD_NONE", "SHARD_COLUMN", "SHARD_COLUMN_GATED", "SHARD_ROW",
    "BLOCK_BYTES", "BLOCK_ELEMS", "FORMAT_NAMES", "packed_bytes",
]
