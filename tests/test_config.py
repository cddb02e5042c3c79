"""Configuration reading and the architecture registry (no GPU)."""
import json

import pytest

import helpers
from hk_b200.config import (ConfigError, Qwen3Config, config_from_dict, load_config, resolve_architecture,
                            supported_architectures)


def test_reads_every_key_of_both_tiny_configs():
    a = config_from_dict(helpers.TINY_A)
    b = config_from_dict(helpers.TINY_B)
    assert isinstance(a, Qwen3Config)
    assert (a.hidden_size, a.num_hidden_layers, a.intermediate_size) == (64, 2, 128)
    assert (a.num_attention_heads, a.num_key_value_heads, a.head_dim, a.vocab_size) == (4, 2, 16, 256)
    assert (a.rope_theta, a.rms_norm_eps, a.tie_word_embeddings, a.max_position_embeddings) == (1e4, 1e-6, True, 128)
    assert (b.q_width, b.kv_width, b.hidden_size) == (192, 64, 96)     # q width differs from hidden
    assert (b.rope_theta, b.rms_norm_eps, b.tie_word_embeddings) == (1e6, 1e-5, False)
    for k in ("hidden_size", "num_hidden_layers", "head_dim", "vocab_size", "rms_norm_eps", "rope_theta"):
        assert getattr(a, k) != getattr(b, k)


def test_defaults_follow_the_reference():
    # src/convert/hf.zig:269-313: kv heads = heads, head_dim = hidden/heads, eps 1e-6, theta 1e4, ctx 4096, untied
    c = config_from_dict(dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, num_hidden_layers=1,
                              intermediate_size=32, num_attention_heads=4, vocab_size=10))
    assert (c.num_key_value_heads, c.head_dim, c.rms_norm_eps, c.rope_theta) == (4, 16, 1e-6, 10000.0)
    assert (c.max_position_embeddings, c.tie_word_embeddings, c.partial_rotary_factor) == (4096, False, 1.0)
    assert c.layer_window(0) is None


def test_round_trip_through_to_dict():
    for raw in (helpers.TINY_A, helpers.TINY_B, helpers.TINY_C):
        c = config_from_dict(raw)
        assert config_from_dict(json.loads(json.dumps(c.to_dict()))) == c


def test_window_layers_from_layer_types_and_max_window_layers():
    c = config_from_dict(helpers.TINY_C)
    assert [c.layer_window(i) for i in range(4)] == [None, 20, 20, None]
    raw = dict(helpers.TINY_C)
    del raw["layer_types"]
    raw["max_window_layers"] = 3
    assert [config_from_dict(raw).layer_window(i) for i in range(4)] == [None, None, None, 20]
    raw["use_sliding_window"] = False
    assert config_from_dict(raw).layer_window(3) is None


@pytest.mark.parametrize("change,needle", [
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"rope_type": "dynamic", "factor": 4.0}}, "rope_scaling"),
    ({"rope_scaling": {"rope_type": "yarn"}}, "factor"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 0.5}}, "rope_scaling"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 4.0, "high_freq_factor": 1.0}}, "low_freq_factor"),
    ({"rope_scaling": "yarn"}, "rope_scaling"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"head_dim": 258}, "head_dim"),
    ({"head_dim": 15}, "head_dim"),
    ({"hidden_size": None}, "hidden_size"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"partial_rotary_factor": 0.2}, "partial_rotary_factor"),
    ({"use_sliding_window": True, "sliding_window": 8, "layer_types": ["full_attention"]}, "layer_types"),
    ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
])
def test_bad_values_name_the_key(change, needle):
    raw = dict(helpers.TINY_A)
    raw.update(change)
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert needle in str(e.value)


def test_rope_scaling_kinds_are_read_with_the_reference_defaults():
    raw = dict(helpers.TINY_B, rope_scaling={"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64})
    c = config_from_dict(raw)
    assert c.rope_scaling == {"kind": "yarn", "factor": 4.0, "orig_ctx": 64}
    assert config_from_dict(c.to_dict()).rope_scaling == c.rope_scaling
    c = config_from_dict(dict(helpers.TINY_B, rope_scaling={"factor": 2.0}))                 # a factor alone means linear
    assert c.rope_scaling["kind"] == "linear"
    c = config_from_dict(dict(helpers.TINY_B, rope_scaling={"rope_type": "llama3", "factor": 8.0}))
    assert c.rope_scaling["orig_ctx"] == helpers.TINY_B["max_position_embeddings"]         # defaults to the training context
    assert config_from_dict(dict(helpers.TINY_B, rope_scaling={"rope_type": "default"})).rope_scaling is None
    from hk_b200.models.qwen3 import build_qwen3
    rope = build_qwen3(config_from_dict(raw), 32).layers[0].mixer.position
    assert rope.scaling.kind == "yarn" and rope.pairing == "half"


def test_registry_names_what_it_supports():
    assert "Qwen3ForCausalLM" in supported_architectures()
    cfg_cls, builder = resolve_architecture("Qwen3ForCausalLM")
    assert cfg_cls is Qwen3Config and callable(builder)
    with pytest.raises(ConfigError) as e:
        config_from_dict(dict(architectures=["GPTNeoXForCausalLM"]))
    assert "GPTNeoXForCausalLM" in str(e.value) and "Qwen3ForCausalLM" in str(e.value)
    assert config_from_dict(dict(helpers.TINY_A, architectures=None, model_type="qwen3")).hidden_size == 64
    with pytest.raises(ConfigError):
        config_from_dict({"hidden_size": 4})


def test_load_config_errors(tmp_path):
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(helpers.TINY_B))
    assert load_config(str(tmp_path)).num_hidden_layers == 3


def test_model_is_built_from_the_configuration_layer_by_layer():
    from hk_b200.parts import GQAAttention, SwiGLUFeedForward
    cfg = config_from_dict(helpers.TINY_C)
    _, build = resolve_architecture(cfg.architecture)
    spec = build(cfg, 64)
    assert len(spec.layers) == 4 and [c.layer for c in spec.schedule] == [0, 1, 2, 3]
    assert [blk.mixer.window for blk in spec.layers] == [None, 20, 20, None]
    m = spec.layers[1].mixer
    assert isinstance(m, GQAAttention) and (m.H, m.G, m.hd, m.hidden) == (5, 1, 48, 72)
    assert m.position.rotary_dim == 24 and m.position.theta == 50000.0 and m.qk_norm_eps == 3e-6
    assert isinstance(spec.layers[0].feed_forward, SwiGLUFeedForward) and spec.layers[0].feed_forward.F == 200
    names = spec.param_specs()
    assert names["model.layers.3.self_attn.q_proj.weight"].shape == (240, 72)
    assert names["model.layers.0.self_attn.k_norm.weight"].shape == (48,)
    assert names["lm_head.weight"].shape == (333, 72) and not names["lm_head.weight"].optional
    tied = build(config_from_dict(helpers.TINY_A), 64).param_specs()
    assert tied["lm_head.weight"].optional
