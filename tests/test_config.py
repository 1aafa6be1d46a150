"""Configuration: the LFM2 keys, their alternative spellings, derived sizes and errors."""

import copy
import json

import pytest

from lalamo_b200.config import (
    AttentionSpec,
    ConfigError,
    Lfm2Config,
    ModelPlan,
    ScheduleEntry,
    ShortConvSpec,
    UnknownArchitectureError,
    config_from_dict,
    load_config,
)
from tiny import TINY_A, TINY_B


def test_tiny_a_sizes():
    config = Lfm2Config.from_dict(TINY_A)
    assert (config.hidden_size, config.num_attention_heads, config.num_key_value_heads, config.head_dim) == (64, 4, 2, 16)
    assert config.ffn_dim == 192 and config.vocab_size == 512 and config.conv_kernel_size == 3
    assert config.layer_types == ("conv", "full_attention", "conv", "full_attention")
    assert config.rope_theta == 10000.0 and config.tie_embedding and not config.conv_bias


def test_tiny_b_alternative_spellings():
    config = Lfm2Config.from_dict(TINY_B)
    # full_attn_idxs -> layer kinds; auto-adjusted width 384 * 2/3 = 256 -> multiple of 256; nested theta
    assert config.layer_types == ("full_attention", "conv", "conv", "full_attention", "conv", "full_attention")
    assert config.ffn_dim == 256
    assert config.rope_theta == 1e6
    assert config.head_dim == 32 and config.num_key_value_heads == 1
    assert config.block_norm_eps == 1e-6 and config.norm_eps == 3e-6
    assert not config.tie_embedding and config.conv_bias


@pytest.mark.parametrize("block_ff_dim,expected", [(12288, 8192), (6656, 4608), (10240, 6912)])
def test_published_widths(block_ff_dim, expected):
    raw = dict(TINY_B, block_ff_dim=block_ff_dim)
    assert Lfm2Config.from_dict(raw).ffn_dim == expected


def test_intermediate_size_wins_without_auto_adjust():
    raw = dict(TINY_A, intermediate_size=320)
    assert Lfm2Config.from_dict(raw).ffn_dim == 320


def test_block_norm_eps_defaults_to_norm_eps():
    raw = {k: v for k, v in TINY_A.items() if k != "block_norm_eps"}
    raw["norm_eps"] = 2e-5
    assert Lfm2Config.from_dict(raw).block_norm_eps == 2e-5


@pytest.mark.parametrize(
    "change,key",
    [
        ({"hidden_size": None}, "hidden_size"),
        ({"vocab_size": "big"}, "vocab_size"),
        ({"num_attention_heads": 5, "num_heads": 5}, "hidden_size"),
        ({"num_key_value_heads": 3}, "num_key_value_heads"),
        ({"layer_types": None}, "layer_types"),
        ({"layer_types": ["conv", "attention", "conv", "conv"]}, "layer_types"),
        ({"layer_types": ["conv"]}, "layer_types"),
        ({"rope_theta": None}, "rope_theta"),
        ({"rope_theta": 1e4, "rope_parameters": {"rope_theta": 1e6}}, "rope_theta"),
        ({"num_heads": 8}, "num_heads"),
        ({"conv_L_cache": 0}, "conv_L_cache"),
        ({"norm_eps": None}, "norm_eps"),
        ({"model_type": "llama"}, "model_type"),
    ],
)
def test_errors_name_the_key(change, key):
    raw = copy.deepcopy(TINY_A)
    raw.update(change)
    with pytest.raises(ConfigError) as info:
        Lfm2Config.from_dict(raw)
    assert info.value.key == key


def test_registry(tmp_path):
    assert isinstance(config_from_dict(TINY_A), Lfm2Config)
    with pytest.raises(UnknownArchitectureError):
        config_from_dict(dict(TINY_A, architectures=["SomethingElse"]))
    with pytest.raises(ConfigError):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "architectures"})
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert load_config(tmp_path) == Lfm2Config.from_dict(TINY_B)
    with pytest.raises(FileNotFoundError):
        load_config(tmp_path / "nowhere")


def test_json_round_trip():
    for raw in (TINY_A, TINY_B):
        config = Lfm2Config.from_dict(raw)
        assert Lfm2Config.from_dict(json.loads(json.dumps(config.to_json_dict()))) == config


def test_plan_from_config():
    plan = Lfm2Config.from_dict(TINY_B).to_plan()
    assert len(plan.layers) == 6 and [entry.layer for entry in plan.schedule] == list(range(6))
    attention = plan.layers[0].mixer
    assert isinstance(attention, AttentionSpec)
    assert (attention.num_heads, attention.num_groups, attention.head_dim) == (3, 1, 32)
    assert attention.qk_norm.eps == 1e-6 and attention.position.theta == 1e6 and attention.window is None
    conv = plan.layers[1].mixer
    assert isinstance(conv, ShortConvSpec) and conv.kernel_size == 4 and conv.has_bias
    assert plan.final_norm.eps == 3e-6 and plan.layers[0].pre_mixer_norm.eps == 1e-6
    assert plan.layers[0].ffn.hidden_dim == 256 and not plan.tie_embeddings


def test_schedule_is_data():
    plan = Lfm2Config.from_dict(TINY_A).to_plan()
    twice = ModelPlan(plan.vocab_size, plan.model_dim, plan.layers, plan.final_norm, schedule=(
        ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(3, cache_from=1)))
    assert [entry.layer for entry in twice.schedule] == [0, 1, 0, 3]
    with pytest.raises(ValueError):
        ModelPlan(plan.vocab_size, plan.model_dim, plan.layers, plan.final_norm, schedule=(ScheduleEntry(7),))
    with pytest.raises(ValueError):
        ModelPlan(plan.vocab_size, plan.model_dim, plan.layers, plan.final_norm, schedule=(ScheduleEntry(1, cache_from=0),))
