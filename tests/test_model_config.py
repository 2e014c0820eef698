"""quantization_config and geometry parsing (CPU): the decision between QuantLinear and a dense linear."""
import pytest

from tattletale_b200 import FMT_Q4_K, FMT_TQ3
from tattletale_b200.model_config import decoder_config_from_hf, parse_quantization_config

BASE = {"hidden_size": 1024, "num_hidden_layers": 4, "num_attention_heads": 16, "num_key_value_heads": 8, "intermediate_size": 3072,
        "vocab_size": 32000, "rms_norm_eps": 1e-6, "rope_theta": 1e6}


def test_dense_checkpoint():
    assert parse_quantization_config(BASE) is None
    cfg = decoder_config_from_hf(BASE, context=512)
    assert (cfg.n_layers, cfg.hidden, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab, cfg.context) == \
        (4, 1024, 16, 8, 64, 3072, 32000, 512)
    assert decoder_config_from_hf({**BASE, "head_dim": 128}).head_dim == 128


def test_own_formats_are_servable():
    spec = parse_quantization_config({**BASE, "quantization_config": {"quant_method": "gguf", "format": "Q4_K"}})
    assert spec.servable and spec.ttq_format == FMT_Q4_K and spec.bits == 4.5
    spec = parse_quantization_config({**BASE, "quantization_config": {"quant_method": "ttq", "format": "tq3"}})
    assert spec.servable and spec.ttq_format == FMT_TQ3 and spec.bits == 3.0


@pytest.mark.parametrize("qc", [{"quant_method": "gptq", "bits": 4, "group_size": 128}, {"quant_method": "awq", "w_bit": 4, "q_group_size": 128},
                                {"quant_method": "fp8"}, {"quant_method": "exl3", "bits": 3.84}, {"quant_method": "compressed-tensors"}])
def test_foreign_methods_are_named_not_guessed(qc):
    spec = parse_quantization_config({**BASE, "quantization_config": qc})
    assert not spec.servable and spec.ttq_format is None and spec.method == qc["quant_method"]
    assert "re-encode" in spec.reason


def test_errors():
    with pytest.raises(ValueError):
        parse_quantization_config({"quantization_config": {"quant_method": "mystery"}})
    with pytest.raises(ValueError):
        parse_quantization_config({"quantization_config": {"quant_method": "gguf", "format": "q2_k"}})
    with pytest.raises(ValueError):
        decoder_config_from_hf({"hidden_size": 8})
