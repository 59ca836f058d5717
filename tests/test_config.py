"""Configuration parsing and the architecture registry (CPU)."""
import json

import pytest

from conftest import TINY_A, TINY_B
from llmi_b200.config import ConfigError, LlamaConfig, parse_config, registered_architectures

SMOLLM2_135M = {
    "architectures": ["LlamaForCausalLM"], "attention_bias": False, "attention_dropout": 0.0, "bos_token_id": 0,
    "eos_token_id": 0, "hidden_act": "silu", "hidden_size": 576, "initializer_range": 0.041666666666666664,
    "intermediate_size": 1536, "is_llama_config": True, "max_position_embeddings": 8192, "model_type": "llama",
    "num_attention_heads": 9, "num_hidden_layers": 30, "num_key_value_heads": 3, "pretraining_tp": 1,
    "rms_norm_eps": 1e-05, "rope_interleaved": False, "rope_scaling": None, "rope_theta": 100000,
    "tie_word_embeddings": True, "torch_dtype": "bfloat16", "transformers_version": "4.40.1", "use_cache": True,
    "vocab_size": 49152,
}


def test_real_config_shape():
    arch, c = parse_config(json.dumps(SMOLLM2_135M))
    assert arch.name == "LlamaForCausalLM" and isinstance(c, LlamaConfig)
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (49152, 576, 1536, 30)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (9, 3, 64)
    assert c.rms_norm_eps == 1e-5 and c.rope_theta == 100000.0 and c.tie_word_embeddings and not c.attention_bias
    assert c.eos_token_ids == (0,) and c.max_position_embeddings == 8192


def test_defaults_and_options():
    base = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "tie_word_embeddings", "eos_token_id")}
    _, c = parse_config(base)
    assert c.num_key_value_heads == c.num_attention_heads and c.head_dim == 16
    assert not c.tie_word_embeddings and c.eos_token_ids == ()
    _, b = parse_config(TINY_B)
    assert b.attention_bias and b.eos_token_ids == (7, 11) and b.head_dim == 24
    _, n = parse_config(dict(base, eos_token_id=None, rope_scaling=None, use_sliding_window=False))
    assert n.eos_token_ids == ()
    _, wide = parse_config(dict(base, head_dim=32))          # head_dim is a size of its own here
    assert wide.head_dim == 32


def test_spec_is_built_from_config_numbers():
    arch, c = parse_config(TINY_B)
    spec = arch.model_spec(c)
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    m = spec.layers[1].mixer
    assert m.kind == "gqa" and m.params["n_heads"] == 5 and m.params["n_kv_heads"] == 1 and m.params["head_dim"] == 24
    assert m.params["bias"] and m.params["position"].params["theta"] == 100000.0
    assert spec.layers[0].ffn.params == {"width": 120, "inner": 320}
    assert spec.final_norm.params["eps"] == 1e-6 and not spec.head.params["tied"]
    assert spec.stop_ids == (7, 11)


@pytest.mark.parametrize("change,message", [
    ({"architectures": ["GPT2LMHeadModel"]}, "unsupported architecture GPT2LMHeadModel"),
    ({"architectures": []}, "exactly one architecture"),
    ({"architectures": ["LlamaForCausalLM", "X"]}, "exactly one architecture"),
    ({"vocab_size": None}, 'missing "vocab_size"'),
    ({"vocab_size": 0}, '"vocab_size" must be an integer'),
    ({"vocab_size": 1 << 23}, '"vocab_size" must be an integer'),
    ({"hidden_size": 2.5}, '"hidden_size" must be an integer'),
    ({"num_hidden_layers": 2000}, '"num_hidden_layers" must be an integer'),
    ({"rms_norm_eps": 0}, '"rms_norm_eps" must be a positive number'),
    ({"rope_theta": -1}, '"rope_theta" must be a positive number'),
    ({"tie_word_embeddings": "yes"}, '"tie_word_embeddings" must be true or false'),
    ({"num_key_value_heads": 3}, "not a multiple of num_key_value_heads"),
    ({"head_dim": 15}, "head_dim must be even"),
    ({"hidden_act": "gelu"}, 'only hidden_act "silu"'),
    ({"eos_token_id": 256}, "eos_token_id out of range"),
    ({"eos_token_id": [1, -2]}, "eos_token_id out of range"),
    ({"rope_scaling": {"type": "linear", "factor": 2}}, "rope_scaling is not supported"),
    ({"use_sliding_window": True}, "sliding-window attention is not supported"),
])
def test_rejections(change, message):
    with pytest.raises(ConfigError, match=message):
        parse_config(dict(TINY_A, **change))


def test_required_keys_have_no_defaults():
    for key in ("rms_norm_eps", "rope_theta", "max_position_embeddings", "intermediate_size", "num_attention_heads"):
        cfg = {k: v for k, v in TINY_A.items() if k != key}
        with pytest.raises(ConfigError, match=f'missing "{key}"'):
            parse_config(cfg)
    no_hd = {k: v for k, v in TINY_A.items() if k != "head_dim"}
    with pytest.raises(ConfigError, match="not a multiple of num_attention_heads"):
        parse_config(dict(no_hd, hidden_size=66))


def test_text_level_errors(tmp_path):
    from llmi_b200.config import read_model_config
    with pytest.raises(ConfigError, match="config:"):
        parse_config("{not json")
    with pytest.raises(ConfigError, match="not a JSON object"):
        parse_config("[1, 2]")
    with pytest.raises(ConfigError, match="duplicate key"):
        parse_config('{"vocab_size": 1, "vocab_size": 2}')
    with pytest.raises(ConfigError, match="cannot open"):
        read_model_config(str(tmp_path))
    (tmp_path / "config.json").write_text(" " * ((1 << 20) + 1))
    with pytest.raises(ConfigError, match="larger than"):
        read_model_config(str(tmp_path))


def test_registry_maps_name_to_recipe():
    from llmi_b200.config.registry import Architecture, get_architecture, register_architecture
    assert "LlamaForCausalLM" in registered_architectures()
    with pytest.raises(ValueError, match="already registered"):
        register_architecture(get_architecture("LlamaForCausalLM"))
    register_architecture(Architecture("CpuTestLM", lambda root: root, lambda c: c), replace=True)
    arch, c = parse_config({"architectures": ["CpuTestLM"], "x": 1})
    assert arch.name == "CpuTestLM" and c["x"] == 1


def test_roundtrip_to_dict():
    _, c = parse_config(TINY_B)
    _, again = parse_config(c.to_dict())
    assert again == c
