"""Typed configuration and the architecture registry."""
import json

import pytest

from tensorline_b200.config import ConfigError, EngineConfig, Qwen2Config
from tensorline_b200.models import architecture, expected_tensors, load_config, registered_architectures
from tests.tiny import CONFIGS, TINY_A, TINY_B


def test_reads_every_size_from_config_json():
    a, b = Qwen2Config.from_dict(TINY_A), Qwen2Config.from_dict(TINY_B)
    assert (a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 4, 2, 16)
    assert (b.intermediate_size, b.vocab_size, b.rope_theta, b.rms_norm_eps) == (200, 384, 1e6, 1e-5)
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert [a.layer_window(i) for i in range(2)] == [None, None]
    assert [b.layer_window(i) for i in range(3)] == [None, 24, 24]


def test_defaults_and_nested_rope_theta():
    raw = dict(TINY_A)
    del raw["head_dim"], raw["rope_theta"], raw["num_key_value_heads"]
    raw["rope_parameters"] = {"rope_theta": 123456.0, "rope_type": "default"}
    c = Qwen2Config.from_dict(raw)
    assert c.head_dim == 16 and c.num_key_value_heads == 4 and c.rope_theta == 123456.0


@pytest.mark.parametrize("key,value,word", [
    ("hidden_size", None, "hidden_size"), ("vocab_size", "many", "vocab_size"),
    ("num_key_value_heads", 3, "num_key_value_heads"), ("hidden_act", "gelu", "hidden_act"),
    ("rope_scaling", {"rope_type": "yarn", "factor": 4.0}, "rope_scaling"), ("rms_norm_eps", -1.0, "rms_norm_eps"),
    ("head_dim", 15, "head_dim"), ("tie_word_embeddings", "yes", "tie_word_embeddings"),
])
def test_errors_name_the_key(key, value, word):
    raw = dict(TINY_A)
    if value is None:
        del raw[key]
    else:
        raw[key] = value
    with pytest.raises(ConfigError, match=word):
        Qwen2Config.from_dict(raw)


def test_window_without_size_is_refused():
    raw = dict(TINY_B)
    del raw["sliding_window"]
    with pytest.raises(ConfigError, match="sliding_window"):
        Qwen2Config.from_dict(raw)


def test_registry_maps_name_to_model(tmp_path):
    assert "Qwen2ForCausalLM" in registered_architectures()
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    arch, cfg = load_config(tmp_path)
    assert arch.name == "Qwen2ForCausalLM" and isinstance(cfg, Qwen2Config)
    spec = arch.describe(cfg)
    assert len(spec.layers) == 3 and [e.layer for e in spec.run] == [0, 1, 2]
    assert spec.layers[1].block.params["mixer"].params["window"] == 24
    with pytest.raises(ConfigError, match="NoSuchModel"):
        architecture("NoSuchModel")
    (tmp_path / "config.json").write_text(json.dumps(dict(TINY_B, architectures=["LlamaForCausalLM"])))
    with pytest.raises(ConfigError, match="LlamaForCausalLM"):
        load_config(tmp_path)


def test_expected_tensors_follow_the_configuration():
    for name, raw in CONFIGS.items():
        cfg = Qwen2Config.from_dict(raw)
        exp = expected_tensors(cfg)
        n = sum(int(__import__("math").prod(s.shape)) for k, s in exp.items() if not s.optional)
        assert n == cfg.num_parameters(), name
        assert exp["model.layers.0.self_attn.k_proj.bias"].shape == (cfg.num_key_value_heads * cfg.head_dim,)
        assert exp["lm_head.weight"].optional == cfg.tie_word_embeddings


def test_engine_config_defaults_are_the_reference_ones():
    e = EngineConfig()
    assert (e.block_size, e.max_num_seqs, e.max_batched_tokens, e.max_model_len) == (16, 64, 2048, 4096)
    assert e.cuda_graphs and e.prefix_caching and e.kv_mem_fraction == 0.6
    assert e.resolved_dtype() == "bfloat16" and EngineConfig(dtype="fp32").resolved_dtype() == "float32"
    with pytest.raises(ValueError):
        EngineConfig(dtype="int8").resolved_dtype()
    with pytest.raises(ValueError):
        EngineConfig(block_size=24).validate()
