"""Configuration and registries (CPU)."""
import json

import pytest

import helpers
from mini_llama_cpp_release_b200.config import (ConfigError, ModelConfig, PartSpec, ScheduleEntry, build_model_spec,
                                                known_architectures, part_class, register_architecture)
from mini_llama_cpp_release_b200.config.specs import ModelSpec


def test_reads_the_architectures_own_keys():
    c = ModelConfig.from_dict(helpers.TINY_B)
    assert (c.architecture, c.hidden_size, c.intermediate_size, c.num_hidden_layers) == ("Qwen2ForCausalLM", 128, 344, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.vocab_size) == (8, 1, 16, 1000)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and c.tie_word_embeddings is False
    assert c.q_size == 128 and c.kv_size == 16


def test_defaults_follow_from_other_keys():
    raw = dict(helpers.TINY_A)
    del raw["head_dim"], raw["num_key_value_heads"], raw["rope_theta"]
    c = ModelConfig.from_dict(raw)
    assert c.head_dim == 16 and c.num_key_value_heads == 4 and c.rope_theta == 10000.0
    assert c.eos_token_id == (2,)


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                                 "vocab_size", "max_position_embeddings", "architectures"])
def test_missing_key_is_named(key):
    raw = dict(helpers.TINY_A)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        ModelConfig.from_dict(raw)


@pytest.mark.parametrize("patch,word", [
    (dict(num_key_value_heads=3), "multiple"),
    (dict(head_dim=15), "even"),
    (dict(rope_theta=0.0), "rope_theta"),
    (dict(rms_norm_eps=float("nan")), "rms_norm_eps"),
    (dict(num_hidden_layers=0), "num_hidden_layers"),
    (dict(rope_scaling={"type": "yarn"}), "rope_scaling"),
    (dict(use_sliding_window=True, sliding_window=None), "sliding_window"),
    (dict(hidden_size=2.5), "integer"),
])
def test_bad_values_are_refused(patch, word):
    raw = dict(helpers.TINY_A)
    raw.update(patch)
    with pytest.raises(ConfigError, match=word):
        ModelConfig.from_dict(raw)


def test_round_trip_through_a_folder(tmp_path):
    c = ModelConfig.from_dict(helpers.TINY_W)
    c.save(str(tmp_path))
    assert ModelConfig.from_folder(str(tmp_path)) == c
    with pytest.raises(ConfigError, match="config.json"):
        ModelConfig.from_folder(str(tmp_path / "nowhere"))
    (tmp_path / "bad").mkdir()
    (tmp_path / "bad" / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        ModelConfig.from_folder(str(tmp_path / "bad"))


def test_window_applies_from_max_window_layers_upward():
    c = ModelConfig.from_dict(helpers.TINY_W)
    assert [c.window_of_layer(i) for i in range(3)] == [None, 24, 24]
    assert ModelConfig.from_dict(helpers.TINY_A).window_of_layer(1) is None


def test_registry_maps_the_name_to_a_model_and_lists_known_names():
    assert "Qwen2ForCausalLM" in known_architectures()
    spec = build_model_spec(ModelConfig.from_dict(helpers.TINY_W))
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert spec.layers[0].mixer.params["window"] is None and spec.layers[2].mixer.params["window"] == 24
    assert spec.layers[1].mixer.kind == "gqa_attention" and spec.layers[1].feed_forward.kind == "swiglu"
    raw = dict(helpers.TINY_A, architectures=["NoSuchModel"])
    with pytest.raises(ConfigError, match="Qwen2ForCausalLM"):
        build_model_spec(ModelConfig.from_dict(raw))
    with pytest.raises(ConfigError, match="rmsnorm"):
        part_class("norm", "nope")


def test_unsupported_activation_is_refused():
    with pytest.raises(ConfigError, match="hidden_act"):
        build_model_spec(ModelConfig.from_dict(dict(helpers.TINY_A, hidden_act="gelu")))


def test_schedule_is_checked():
    spec = build_model_spec(ModelConfig.from_dict(helpers.TINY_A))
    def with_schedule(s):
        return ModelSpec(spec.config, spec.embedding, spec.layers, tuple(s), spec.final_norm, spec.head)
    with_schedule([ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, reads_cache_of=1)]).validate()
    with pytest.raises(ValueError, match="layer 5"):
        with_schedule([ScheduleEntry(5)]).validate()
    with pytest.raises(ValueError, match="does not run before"):
        with_schedule([ScheduleEntry(0, reads_cache_of=0)]).validate()
    with pytest.raises(ValueError, match="none of its own"):
        with_schedule([ScheduleEntry(0), ScheduleEntry(1, reads_cache_of=0), ScheduleEntry(0, reads_cache_of=1)]).validate()
