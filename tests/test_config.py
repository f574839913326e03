"""Configuration and registry (CPU)."""
import json

import pytest

import tiny_configs
from supersonic_b200.config import (ConfigError, LlamaConfig, config_from_dict, known_architectures,
                                    load_config, preset_config, preset_names, register_architecture)
from supersonic_b200.config.base import ModelSpec, ScheduleEntry


def test_every_key_is_read():
    c = config_from_dict(tiny_configs.B)
    assert isinstance(c, LlamaConfig)
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (384, 96, 256, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (3, 1, 32)
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 500000.0 and not c.tie_word_embeddings
    assert c.rope_scaling.factor == 8.0 and c.rope_scaling.original_max_position_embeddings == 16
    assert c.eos_token_ids == [5, 9]
    assert config_from_dict(tiny_configs.A).eos_token_ids == [7]


def test_defaults():
    d = dict(tiny_configs.A)
    for k in ("head_dim", "num_key_value_heads", "rope_theta", "tie_word_embeddings", "eos_token_id"):
        d.pop(k)
    c = config_from_dict(d)
    assert c.head_dim == 16 and c.num_key_value_heads == 4 and c.rope_theta == 10000.0
    assert c.tie_word_embeddings is False and c.eos_token_ids == [] and c.rope_scaling is None


def test_head_dim_need_not_divide_hidden():
    c = config_from_dict(tiny_configs.C)
    assert c.num_attention_heads * c.head_dim != c.hidden_size
    shapes = c.tensor_shapes()
    assert shapes["model.layers.0.self_attn.q_proj.weight"] == [288, 72]
    assert shapes["model.layers.0.self_attn.o_proj.weight"] == [72, 288]
    assert "lm_head.weight" not in shapes


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "max_position_embeddings", "rms_norm_eps"])
def test_missing_required_key(key):
    d = dict(tiny_configs.A)
    d.pop(key)
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


@pytest.mark.parametrize("change,word", [
    (dict(hidden_act="gelu"), "hidden_act"), (dict(attention_bias=True), "bias"),
    (dict(mlp_bias=True), "bias"), (dict(num_key_value_heads=3), "multiple"),
    (dict(head_dim=15), "even"), (dict(rms_norm_eps=0.0), "rms_norm_eps"),
    (dict(rope_scaling=dict(rope_type="yarn", factor=2.0)), "rope_type"),
    (dict(rope_scaling=dict(rope_type="llama3", factor=2.0)), "missing"),
    (dict(eos_token_id=999), "vocabulary"), (dict(eos_token_id="x"), "eos_token_id"),
    (dict(architectures=["NopeForCausalLM"]), "unknown architecture"),
    (dict(architectures=[]), "architectures"),
])
def test_rejects(change, word):
    d = dict(tiny_configs.A)
    d.update(change)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_round_trip_through_json(tmp_path):
    c = config_from_dict(tiny_configs.C)
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert load_config(str(tmp_path)) == c
    with pytest.raises(ConfigError, match="read config.json"):
        load_config(str(tmp_path / "nowhere"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="parse config.json"):
        load_config(str(tmp_path))


def test_rope_default_type_means_unscaled():
    d = dict(tiny_configs.A, rope_scaling=dict(rope_type="default"))
    assert config_from_dict(d).rope_scaling is None


def test_spec_is_data():
    spec = config_from_dict(tiny_configs.B).build_spec()
    assert isinstance(spec, ModelSpec) and len(spec.blocks) == 3
    assert [s.layer for s in spec.schedule] == [0, 1, 2] and [s.cache for s in spec.schedule] == [0, 1, 2]
    b = spec.blocks[1]
    assert b.kind == "pre_norm" and b.mixer.kind == "attention" and b.feed_forward.kind == "swiglu"
    assert b.mixer.params["num_kv_heads"] == 1 and b.mixer.params["scale"] == 32 ** -0.5
    assert b.mixer.weights["q"] == "model.layers.1.self_attn.q_proj.weight"
    assert b.position.params["scaling"]["factor"] == 8.0
    assert spec.head.weights["weight"] == "lm_head.weight"
    assert config_from_dict(tiny_configs.A).build_spec().head.weights["weight"] == "model.embed_tokens.weight"
    assert spec.stop_token_ids == [5, 9]


def test_schedule_validation():
    spec = config_from_dict(tiny_configs.A).build_spec()
    bad = ModelSpec(**{**spec.__dict__, "schedule": [ScheduleEntry(0, 0), ScheduleEntry(5, 1)]})
    with pytest.raises(ConfigError, match="names layer 5"):
        bad.validate()
    bad = ModelSpec(**{**spec.__dict__, "schedule": [ScheduleEntry(0, 3, writes_cache=False)]})
    with pytest.raises(ConfigError, match="before any stop has written"):
        bad.validate()
    ok = ModelSpec(**{**spec.__dict__, "schedule": [ScheduleEntry(0, 0), ScheduleEntry(1, 0, False),
                                                    ScheduleEntry(0, 1)]})
    ok.validate()          # a layer twice, and a layer reading another layer's cache


def test_registry_and_presets():
    assert "LlamaForCausalLM" in known_architectures()
    with pytest.raises(TypeError):
        register_architecture("Broken", object)
    assert {"tiny-a", "tiny-b", "llama3.1-8b", "llama3.2-3b", "llama3.2-1b"} <= set(preset_names())
    c = preset_config("llama3.1-8b")
    assert c.parameter_count() == 8030261248 and c.kv_bytes_per_token(2) == 131072
    assert preset_config("llama3.2-1b").head_dim == 64 and preset_config("llama3.2-3b").tie_word_embeddings
    with pytest.raises(ConfigError, match="unknown preset"):
        preset_config("llama-9000")


def test_memory_estimate_of_the_8b_preset():
    """Weights + cache + workspace from the model's description alone: 16.06 GB of bfloat16 weights,
    64 GiB for 64 slots of 8,192 tokens at 131,072 bytes a token."""
    import torch
    from supersonic_b200.config import preset_config
    from supersonic_b200.engine import preflight
    from supersonic_b200.weights import RandomWeightStore
    cfg = preset_config("llama3.1-8b")
    est = preflight.estimate(cfg.build_spec(), RandomWeightStore(cfg, 2), torch.bfloat16, 64 * 8192, 8192, 64, 32768)
    assert est.weights == 2 * cfg.parameter_count() == 16_060_522_496
    assert abs(est.cache - 64 * 8192 * cfg.kv_bytes_per_token(2)) < (1 << 20)
    assert est.cache >= 64 * (1 << 30)
    # a step of 32,768 tokens: float32 residual, two bfloat16 copies, and the widest part (3 x 14,336)
    assert est.workspace == 32768 * (4 * 4096 + 2 * (2 * 4096 + 3 * 14336)) + 2 * 64 * 128256 * 4
    assert "kv_cache=64.0" in est.line(64 * 8192)
    f32 = preflight.estimate(cfg.build_spec(), RandomWeightStore(cfg, 2), torch.float32, 4096, 4096, 1, 4096)
    assert f32.weights == 4 * cfg.parameter_count() - 2 * (2 * 32 + 1) * 4096      # norm vectors stay as stored
