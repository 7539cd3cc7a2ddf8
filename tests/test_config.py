"""Typed configuration, validation and the architecture registry."""
import json

import pytest

from tinyinfer_b200.config import (ConfigError, Qwen3Config, get_architecture, known_architectures,
                                   load_config)
from tinyinfer_b200.config.plan import ModelPlan, PartSpec, ScheduleEntry
from util import TINY, TINY_A, TINY_B, TINY_C


def test_reads_every_key():
    c = Qwen3Config.from_dict(TINY_B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads,
            c.head_dim, c.intermediate_size, c.vocab_size, c.max_position_embeddings) == \
        (3, 96, 8, 2, 32, 224, 512, 256)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and c.tie_word_embeddings is False
    assert c.layer_types == ("full_attention",) * 3 and c.sliding_window is None


def test_head_dim_defaults_to_hidden_over_heads():
    cfg = dict(TINY_A)
    del cfg["head_dim"]
    assert Qwen3Config.from_dict(cfg).head_dim == 16


def test_defaults_of_theta_and_eps_are_the_reference_ones():
    cfg = {k: v for k, v in TINY_A.items() if k not in ("rope_theta", "rms_norm_eps")}
    c = Qwen3Config.from_dict(cfg)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-6


@pytest.mark.parametrize("name", list(TINY))
def test_round_trip(name):
    c = Qwen3Config.from_dict(TINY[name])
    assert Qwen3Config.from_dict(json.loads(json.dumps(c.to_dict()))) == c


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads",
                                 "num_key_value_heads", "intermediate_size", "vocab_size",
                                 "max_position_embeddings"])
def test_missing_or_bad_size_is_an_error(key):
    cfg = dict(TINY_A)
    del cfg[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_dict(cfg)
    for bad in (0, -3, 2.5, "8", True):
        cfg[key] = bad
        with pytest.raises(ConfigError, match=key):
            Qwen3Config.from_dict(cfg)


@pytest.mark.parametrize("change,match", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"rope_scaling": {"type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"rope_theta": -1}, "rope_theta"),
    ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
    ({"use_sliding_window": True}, "layer_types"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"layer_types": ["full_attention", "local"]}, "layer_types"),
    ({"layer_types": ["full_attention", "sliding_attention"]}, "sliding_window"),
    ({"eos_token_id": 99999}, "eos_token_id"),
])
def test_refused_options(change, match):
    with pytest.raises(ConfigError, match=match):
        Qwen3Config.from_dict({**TINY_A, **change})


def test_window_layers_reach_the_plan():
    arch = get_architecture("Qwen3ForCausalLM")
    plan = arch.build_plan(arch.from_dict(TINY_C))
    windows = [lp.mixer.params["window"] for lp in plan.layers]
    assert windows == [None, 24, 24, None]
    assert [e.layer for e in plan.schedule] == [0, 1, 2, 3]
    assert plan.layers[2].names["mixer"] == "model.layers.2.self_attn."
    assert plan.layers[0].mixer.params["position"].params == {"head_dim": 48, "theta": 50000.0}


def test_registry_by_both_names_and_unknown():
    assert get_architecture("qwen3") is get_architecture("Qwen3ForCausalLM")
    assert "Qwen3ForCausalLM" in known_architectures()
    with pytest.raises(ConfigError, match="known: .*Qwen3ForCausalLM"):
        get_architecture("LlamaForCausalLM")


def test_load_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    arch, cfg = load_config(str(tmp_path))
    assert arch.name == "Qwen3ForCausalLM" and cfg.hidden_size == 64
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps({"hidden_size": 4}))
    with pytest.raises(ConfigError, match="architectures"):
        load_config(str(tmp_path))
    with pytest.raises(ConfigError, match="no such file"):
        load_config(str(tmp_path / "nowhere"))


def _plan(schedule):
    lp = get_architecture("qwen3").build_plan(Qwen3Config.from_dict(TINY_A)).layers
    return ModelPlan(architecture="x", hidden_size=64, vocab_size=256, max_position=128, layers=lp,
                     schedule=schedule, embedding=PartSpec("embedding"),
                     final_norm=PartSpec("rmsnorm"), head=PartSpec("lm_head"), names={})


def test_schedule_is_data_and_is_checked():
    # a layer named twice, and an entry that reads the slot another entry writes
    p = _plan([ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2),
               ScheduleEntry(1, 1, writes_cache=False)])
    assert p.num_cache_slots == 3
    with pytest.raises(ValueError, match="names layer 5"):
        _plan([ScheduleEntry(5, 0)])
    with pytest.raises(ValueError, match="written by"):
        _plan([ScheduleEntry(0, 0), ScheduleEntry(1, 0)])
    with pytest.raises(ValueError, match="before any entry"):
        _plan([ScheduleEntry(0, 1, writes_cache=False), ScheduleEntry(1, 1)])
