"""The known models of the supported architecture, for ``list-models`` and for random-weight presets.

Mirrors ``lalamo/model_registry.py:45-58`` and ``lalamo/model_import/model_specs/lfm2.py:21-67``
(full-precision LiquidAI repositories only; the quantised MLX variants are out of scope), with the
default generation options the reference gives each family.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .sampling.policy import GenerationConfig

__all__ = ["ModelRegistry", "ModelSpec", "PRESETS"]


@dataclass(frozen=True)
class ModelSpec:
    vendor: str
    family: str
    name: str
    size: str
    repo: str
    architecture: str
    generation_config: GenerationConfig

    @property
    def description(self) -> str:
        return self.repo


def _size_to_number(size: str) -> float:
    factors = {"K": 1e3, "M": 1e6, "B": 1e9, "T": 1e12}
    return float(size[:-1]) * factors[size[-1].upper()]


_LFM2 = [
    ModelSpec("LiquidAI", "LFM2", f"LFM2-{size}", size, f"LiquidAI/LFM2-{size}", "Lfm2ForCausalLM",
              GenerationConfig(temperature=0.3, min_p=0.15))
    for size in ("350M", "700M", "1.2B", "2.6B")
]
_LFM25 = [
    ModelSpec("LiquidAI", "LFM2.5", name, size, f"LiquidAI/{name}", "Lfm2ForCausalLM",
              GenerationConfig(temperature=0.1, top_k=50, top_p=0.1))
    for name, size in (("LFM2.5-350M", "350M"), ("LFM2.5-1.2B-Instruct", "1.2B"), ("LFM2.5-1.2B-Thinking", "1.2B"))
]


class ModelRegistry:
    def __init__(self, specs: list[ModelSpec]) -> None:
        self.repo_to_model = {spec.repo: spec for spec in specs}

    @classmethod
    def build(cls) -> "ModelRegistry":
        return cls(_LFM2 + _LFM25)

    def find(self, name: str) -> ModelSpec | None:
        """The spec of a repository (``"LiquidAI/LFM2-1.2B"``) or of a folder named after one
        (``"LFM2-1.2B"``, any case)."""
        if name in self.repo_to_model:
            return self.repo_to_model[name]
        wanted = name.rstrip("/").split("/")[-1].lower()
        for spec in self.repo_to_model.values():
            if spec.name.lower() == wanted:
                return spec
        return None

    def sorted_specs(self) -> list[ModelSpec]:
        """Sorted as the reference's ``list-models`` sorts (``lalamo/main.py:591-599``)."""
        return sorted(
            self.repo_to_model.values(),
            key=lambda spec: (spec.vendor.lower(), spec.family.lower(), _size_to_number(spec.size), spec.name.lower()),
        )


def _lfm2_shape(hidden: int, heads: int, ff_dim: int) -> dict[str, Any]:
    return {
        "architectures": ["Lfm2ForCausalLM"],
        "model_type": "lfm2",
        "vocab_size": 65536,
        "hidden_size": hidden,
        "num_hidden_layers": 16,
        "num_attention_heads": heads,
        "num_heads": heads,
        "num_key_value_heads": 8,
        "full_attn_idxs": [2, 5, 8, 10, 12, 14],
        "block_auto_adjust_ff_dim": True,
        "block_ff_dim": ff_dim,
        "block_ffn_dim_multiplier": 1.0,
        "block_multiple_of": 256,
        "conv_L_cache": 3,
        "conv_bias": False,
        "rope_theta": 1000000.0,
        "block_norm_eps": 1e-5,
        "norm_eps": 1e-5,
        "tie_embedding": True,
        "max_position_embeddings": 128000,
        "bos_token_id": 1,
        "eos_token_id": 7,
        "pad_token_id": 0,
    }


# Shapes of the published checkpoints, for the random-weights mode (no weights are downloaded).
PRESETS: dict[str, dict[str, Any]] = {
    "lfm2-350m": _lfm2_shape(1024, 16, 6656),
    "lfm2-700m": _lfm2_shape(1536, 24, 10240),
    "lfm2-1.2b": _lfm2_shape(2048, 32, 12288),
}
