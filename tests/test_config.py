"""Configuration and registry (CPU)."""
import json

import pytest

from conftest import TINY_A, TINY_B
from pico_engine.config import (ConfigError, GQAAttentionSpec, Qwen2Config, architecture, config_from_dict,
                                known_architectures, read_config, register_architecture)


def test_reads_every_size_from_config_json():
    a, b = config_from_dict(TINY_A), config_from_dict(TINY_B)
    assert isinstance(a, Qwen2Config)
    for cfg, d in ((a, TINY_A), (b, TINY_B)):
        for key in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                    "head_dim", "intermediate_size", "rope_theta", "rms_norm_eps", "max_position_embeddings",
                    "tie_word_embeddings"):
            assert getattr(cfg, key) == d[key], key
    assert b.sliding_window == 32 and b.max_window_layers == 1


def test_head_dim_defaults_to_hidden_over_heads():
    d = dict(TINY_A); del d["head_dim"]
    assert config_from_dict(d).head_dim == 16
    d["hidden_size"] = 66
    with pytest.raises(ConfigError, match="head_dim"):
        config_from_dict(d)


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                                 "num_key_value_heads", "intermediate_size", "rope_theta", "rms_norm_eps",
                                 "max_position_embeddings"])
def test_missing_size_is_an_error_that_names_it(key):
    d = dict(TINY_A); del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


def test_rejects_what_it_cannot_compute():
    for patch, word in (({"hidden_act": "gelu"}, "hidden_act"), ({"rope_scaling": {"type": "yarn", "factor": 4}}, "rope_scaling"),
                        ({"num_key_value_heads": 3}, "multiple"), ({"vocab_size": -1}, "vocab_size"),
                        ({"use_sliding_window": True}, "sliding_window"), ({"hidden_size": 64.5}, "hidden_size")):
        with pytest.raises(ConfigError, match=word):
            config_from_dict({**TINY_A, **patch})


def test_unknown_architecture_lists_known_ones():
    with pytest.raises(ConfigError, match="Qwen2ForCausalLM"):
        config_from_dict({**TINY_A, "architectures": ["NoSuchModel"]})
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "architectures"})
    assert "Qwen2ForCausalLM" in known_architectures()


def test_plan_chooses_parts_layer_by_layer():
    plan = config_from_dict(TINY_B).plan()
    assert [l.mixer.window for l in plan.layers] == [None, 32, 32]
    assert all(isinstance(l.mixer, GQAAttentionSpec) and l.mixer.qkv_bias for l in plan.layers)
    assert plan.layers[0].mixer.position.theta == 1e6 and plan.layers[0].mixer_norm.eps == 1e-5
    assert plan.head == "lm_head.weight" and [e.layer for e in plan.schedule] == [0, 1, 2]
    a = config_from_dict(TINY_A).plan()
    assert a.head is None and a.ignorable_tensors == ("lm_head.weight",) and a.layers[1].mixer.scale == 16 ** -0.5
    off = config_from_dict({**TINY_B, "use_sliding_window": False}).plan()
    assert [l.mixer.window for l in off.layers] == [None, None, None]


def test_round_trip_through_config_json(tmp_path):
    cfg = config_from_dict(TINY_B)
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    assert read_config(str(tmp_path)) == cfg
    with pytest.raises(ConfigError, match="config.json"):
        read_config(str(tmp_path / "nowhere"))


def test_registering_another_architecture():
    class Other(Qwen2Config):
        ARCHITECTURE = "OtherForCausalLM"
    register_architecture("OtherForCausalLM", Other)
    cfg = config_from_dict({**TINY_A, "architectures": ["OtherForCausalLM"]})
    assert type(cfg) is Other and architecture("OtherForCausalLM").config_class is Other


def test_schedule_validation():
    from dataclasses import replace
    from pico_engine.config import ScheduleEntry
    plan = config_from_dict(TINY_A).plan()
    replace(plan, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1))).validate()
    for bad in ((ScheduleEntry(5),), (ScheduleEntry(0, cache_of=0),), (ScheduleEntry(0), ScheduleEntry(1, cache_of=0), ScheduleEntry(0, cache_of=1))):
        with pytest.raises(ConfigError):
            replace(plan, schedule=bad).validate()


def test_layers_share_their_rotary_tables():
    """One pair of cos/sin tables per (head size, base, device), grown when a longer one is asked for."""
    import torch
    from pico_engine.config.specs import RotaryHalfSpec
    from pico_engine.parts.position import RotaryHalf, rotary_tables
    a, b, c = (RotaryHalf(RotaryHalfSpec(hd, th), torch.float32, "cpu") for hd, th in ((16, 1e4), (16, 1e4), (16, 1e6)))
    for part in (a, b, c):
        part.prepare(100)
    assert a.cos.data_ptr() == b.cos.data_ptr() and a.cos.data_ptr() != c.cos.data_ptr() and a.cos.shape == (100, 8)
    longer = rotary_tables(16, 1e4, 300, "cpu")[0]
    assert longer.shape[0] == 300 and torch.equal(longer[:100], a.cos)
    b.prepare(200)
    assert b.cos.data_ptr() == longer.data_ptr()                # what is there already is long enough
    inv = 1.0 / (1e4 ** (torch.arange(0, 16, 2, dtype=torch.float32) / 16))
    assert torch.allclose(a.sin[7], torch.sin(7 * inv))
