"""Configuration and registry (no GPU)."""
import json

import pytest

from ember_b200.config import (AttentionSpec, ConfigError, Qwen3Config, RMSNormSpec, RotarySpec, config_from_dict,
                               load_config, registered_architectures)
from tests.tiny_configs import TINY, tiny_config


def test_keys_defaults_and_derived():
    c = Qwen3Config.from_json(dict(model_type="qwen3", vocab_size=100, hidden_size=48, intermediate_size=80,
                                   num_hidden_layers=2, num_attention_heads=3))
    assert (c.num_key_value_heads, c.head_dim, c.rms_norm_eps, c.rope_theta) == (3, 16, 1e-6, 10000.0)
    assert c.max_position_embeddings == 4096 and not c.tie_word_embeddings and not c.attention_bias
    assert c.q_dim == 48 and c.kv_dim == 48


def test_head_dim_independent_of_hidden():
    c = Qwen3Config.from_json(TINY["b"]["json"])
    assert c.q_dim == 192 and c.hidden_size == 96
    spec = c.to_model_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    a = spec.layers[1].part("mixer")[0]
    assert isinstance(a, AttentionSpec) and a.qk_norm and a.qk_norm_eps == 1e-5 and a.num_kv_heads == 1
    assert isinstance(a.position, RotarySpec) and a.position.theta == 1e6 and a.position.rotary_dim == 32
    assert isinstance(spec.final_norm, RMSNormSpec) and spec.final_norm.eps == 1e-5
    assert not spec.tie_embeddings and spec.layers[2].part("mixer")[1] == "model.layers.2.self_attn."


@pytest.mark.parametrize("patch,msg", [
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"num_key_value_heads": 4}, "multiple"),
    ({"head_dim": 15}, "head_dim"),
    ({"head_dim": 512}, "head_dim"),
    ({"hidden_size": 0}, "non-positive"),
    ({"use_sliding_window": True}, "sliding"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"vocab_size": None}, "vocab_size"),
])
def test_rejections(patch, msg):
    d = dict(TINY["b"]["json"])
    d.update(patch)
    with pytest.raises(ConfigError, match=msg):
        Qwen3Config.from_json(d)


def test_registry_by_architecture_and_model_type():
    assert "Qwen3ForCausalLM" in registered_architectures()
    d = dict(TINY["a"]["json"])
    assert isinstance(config_from_dict(d), Qwen3Config)
    d2 = dict(d)
    del d2["architectures"]
    assert isinstance(config_from_dict(d2), Qwen3Config)            # falls back to model_type
    d3 = dict(d, architectures=["LlamaForCausalLM"], model_type="llama")
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        config_from_dict(d3)


def test_eos_from_generation_config(tmp_path):
    d = dict(TINY["a"]["json"], eos_token_id=7)
    (tmp_path / "config.json").write_text(json.dumps(d))
    assert load_config(str(tmp_path)).eos_token_ids == (7,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [3, 4]}))
    assert load_config(str(tmp_path)).eos_token_ids == (3, 4)


def test_round_trip_and_parameter_count():
    c = Qwen3Config.from_json(TINY["a"]["json"])
    assert Qwen3Config.from_json(c.to_json()) == c
    # 1.7B shape: the count the reference's formula gives (src/model/config.cpp:10-16)
    big = Qwen3Config.from_json(dict(model_type="qwen3", vocab_size=151936, hidden_size=2048, intermediate_size=6144,
                                     num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                                     head_dim=128, tie_word_embeddings=True))
    assert abs(big.parameters() / 1e9 - 1.72) < 0.01
    assert big.kv_bytes_per_token(2) == 114688


def test_sliding_window_keys_give_layers_of_two_kinds():
    """use_sliding_window / sliding_window / max_window_layers: the first layers see all keys, the rest a window;
    the model then needs two cache groups.  Without use_sliding_window the other two keys mean nothing."""
    from ember_b200.cache import CacheManager
    from ember_b200.model.causal_lm import CausalLM
    cfg = tiny_config("f")
    assert [cfg.layer_window(i) for i in range(3)] == [0, 24, 24]
    spec = cfg.to_model_spec()
    assert [l.part("mixer")[0].window for l in spec.layers] == [0, 24, 24]
    assert Qwen3Config.from_json(cfg.to_json()) == cfg
    groups = CacheManager(CausalLM(spec).cache_needs(), 16, 256, 4).groups
    assert [(g.need.kind, g.layers) for g in groups] == [("full", [0]), ("window", [1, 2])]
    d = dict(TINY["f"]["json"], use_sliding_window=False)
    assert [l.part("mixer")[0].window for l in Qwen3Config.from_json(d).to_model_spec().layers] == [0, 0, 0]
