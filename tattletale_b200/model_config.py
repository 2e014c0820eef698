"""Model-configuration plumbing: which linear a checkpoint's ``quantization_config`` asks for, and the decoder
geometry of a Hugging Face style ``config.json``.

The reference parses the geometry fields of such a file (``parseQwen3Config``,
workspace/transformers/src/models/qwen3.nim:51-89) and carries quantized-checkpoint configurations only as test
fixtures (tests/fixtures/configs/: GPTQ, AWQ, FP8, EXL3 variants) without acting on ``quantization_config``.
This module adds that decision: a checkpoint is served by ``QuantLinear`` when its weights are in one of the
formats this library multiplies (GGUF-style Q8_0 / Q4_K / Q6_K blocks, the trellis-coded TQ3 format); for every
other method it says so instead of guessing.  Pure Python, no GPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

from ._lib import FMT_Q4_K, FMT_Q6_K, FMT_Q8_0, FMT_TQ3
from .decoder import DecoderConfig

_BLOCK_FORMATS = {"q8_0": FMT_Q8_0, "q4_k": FMT_Q4_K, "q6_k": FMT_Q6_K, "tq3": FMT_TQ3}
# quantization methods of other tools seen in model configurations; none of them stores weights in a format
# this library reads
_FOREIGN = {
    "gptq": "GPTQ group-wise integer weights (qweight / qzeros / scales tensors)",
    "awq": "AWQ group-wise integer weights",
    "fp8": "FP8 (e4m3) weights with scale tensors",
    "compressed-tensors": "compressed-tensors schemes",
    "bitsandbytes": "bitsandbytes NF4 / int8",
    "exl3": "EXL3 trellis-coded weights (a different codec from this library's TQ3: not interchangeable)",
    "exl2": "EXL2 mixed-precision weights",
}


@dataclass(frozen=True)
class QuantSpec:
    """What ``quantization_config`` says.  ``ttq_format`` is the library format when the checkpoint is servable by
    ``QuantLinear`` (then ``servable`` is True), else None and ``reason`` explains why."""
    method: str
    bits: Optional[float]
    group_size: Optional[int]
    ttq_format: Optional[int]
    servable: bool
    reason: str


def parse_quantization_config(config: Mapping[str, Any]) -> Optional[QuantSpec]:
    """``config``: the parsed ``config.json``.  Returns None for an unquantized checkpoint (dense ``Linear``)."""
    qc = config.get("quantization_config")
    if not qc:
        return None
    method = str(qc.get("quant_method", "")).lower()
    bits = qc.get("bits", qc.get("w_bit"))
    group = qc.get("group_size", qc.get("q_group_size"))
    if method in ("ttq", "gguf"):
        name = str(qc.get("format", qc.get("weight_format", ""))).lower()
        if name not in _BLOCK_FORMATS:
            raise ValueError(f"quantization_config.format {name!r}: expected one of {sorted(_BLOCK_FORMATS)}")
        fmt = _BLOCK_FORMATS[name]
        bpw = {FMT_Q8_0: 8.5, FMT_Q4_K: 4.5, FMT_Q6_K: 6.5625, FMT_TQ3: 3.0}[fmt]
        return QuantSpec(method, bpw, {FMT_Q8_0: 32, FMT_TQ3: 256}.get(fmt, 256), fmt, True, "block format of this library")
    if method in _FOREIGN:
        return QuantSpec(method, None if bits is None else float(bits), None if group is None else int(group), None, False,
                         f"{_FOREIGN[method]}: no kernel in this library reads that layout; re-encode the weights "
                         "(tattletale_b200.quantize) or load them dense")
    raise ValueError(f"unknown quantization method {method!r}")


def decoder_config_from_hf(config: Mapping[str, Any], context: int = 2048) -> DecoderConfig:
    """Decoder geometry from the fields the reference reads (qwen3.nim:51-89); ``head_dim`` defaults to
    ``hidden_size / num_attention_heads`` when the file omits it."""
    try:
        hidden, heads = int(config["hidden_size"]), int(config["num_attention_heads"])
        return DecoderConfig(
            n_layers=int(config["num_hidden_layers"]), hidden=hidden, n_q_heads=heads,
            n_kv_heads=int(config.get("num_key_value_heads", heads)), head_dim=int(config.get("head_dim") or hidden // heads),
            ffn=int(config["intermediate_size"]), vocab=int(config["vocab_size"]),
            rope_theta=float(config.get("rope_theta", 10000.0)), rms_eps=float(config.get("rms_norm_eps", 1e-6)), context=context)
    except KeyError as exc:
        raise ValueError(f"config.json lacks {exc.args[0]!r}") from None
