"""What the Python entry point decides on the host: the default generation options of a model
(``generation_config.json``, else the registry's options for the model, merged with the stop token of
``config.json``), as the reference settles them at import (``lalamo/model_import/common.py:251-271``,
``lalamo/model_import/model_specs/lfm2.py:30,58``)."""

from __future__ import annotations

import json

import pytest

from lalamo_b200.language_model import load_generation_config
from lalamo_b200.model_registry import ModelRegistry


def test_generation_config_json_wins_and_merges_the_stop_tokens(tmp_path):
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [7, 9], "temperature": 0.6, "top_k": 20}))
    config = load_generation_config(tmp_path, 2, spec="LiquidAI/LFM2-1.2B")
    assert config.stop_token_ids == (2, 7, 9) and config.temperature == 0.6 and config.top_k == 20 and config.min_p is None


def test_registry_defaults_apply_when_the_folder_brings_none(tmp_path):
    by_spec = load_generation_config(tmp_path, 7, spec="LiquidAI/LFM2-1.2B")
    assert (by_spec.temperature, by_spec.min_p, by_spec.top_k, by_spec.stop_token_ids) == (0.3, 0.15, None, (7,))
    newer = load_generation_config(tmp_path, [7, 2], spec="LiquidAI/LFM2.5-1.2B-Instruct")
    assert (newer.temperature, newer.top_k, newer.top_p, newer.stop_token_ids) == (0.1, 50, 0.1, (2, 7))
    # a folder named after a known model needs no spec
    folder = tmp_path / "lfm2-350m"
    folder.mkdir()
    assert load_generation_config(folder, 7).min_p == 0.15
    # an unknown folder gets neutral options, an unknown spec is an error
    neutral = load_generation_config(tmp_path, 7)
    assert neutral.temperature is None and neutral.min_p is None and neutral.stop_token_ids == (7,)
    with pytest.raises(ValueError, match="not a known model"):
        load_generation_config(tmp_path, 7, spec="LiquidAI/LFM9-1T")


def test_registry_lookup():
    registry = ModelRegistry.build()
    assert registry.find("LiquidAI/LFM2-700M").size == "700M"
    assert registry.find("models/LFM2.5-350M/").family == "LFM2.5"
    assert registry.find("something-else") is None
