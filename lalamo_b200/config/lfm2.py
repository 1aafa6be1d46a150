"""Typed configuration of the LFM2 architecture (``"Lfm2ForCausalLM"``).

Every size and constant is read from the architecture's own ``config.json`` keys, with the
meanings the reference gives them (``lalamo/model_import/model_configs/huggingface/lfm2.py:33-212``):

* ``head_dim`` is *computed* as ``hidden_size // num_attention_heads`` (``lfm2.py:103``);
* the layer kinds come from ``layer_types`` or, failing that, ``full_attn_idxs`` (``lfm2.py:164-171``);
* the feed-forward width is ``intermediate_size``/``block_ff_dim`` or, with
  ``block_auto_adjust_ff_dim``, ``block_ff_dim * block_ffn_dim_multiplier * 2/3`` rounded up to a
  multiple of ``block_multiple_of`` (``lfm2.py:193-199``);
* ``rope_theta`` may be flat or nested under ``rope_parameters`` (``lfm2.py:81-94``);
* block norms (operator, ffn, q/k) use ``block_norm_eps``, the final norm ``norm_eps``
  (``lfm2.py:124-129``, ``186-191``);
* the tying key is ``tie_embedding`` (``lfm2.py:73``).
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .errors import ConfigError
from .plan import (
    AttentionSpec,
    BlockSpec,
    GatedMLPSpec,
    ModelPlan,
    RMSNormSpec,
    RopeSpec,
    ShortConvSpec,
)

__all__ = ["Lfm2Config"]

_LAYER_KINDS = ("conv", "full_attention")


def _require(raw: Mapping[str, Any], key: str, kind: type | tuple[type, ...]) -> Any:
    if key not in raw or raw[key] is None:
        raise ConfigError(key, "is required but missing")
    value = raw[key]
    if isinstance(value, bool) and kind in (int, float, (int, float)):
        raise ConfigError(key, f"must be a number, got {value!r}")
    if not isinstance(value, kind):
        raise ConfigError(key, f"has the wrong type: {value!r}")
    return value


def _optional(raw: Mapping[str, Any], key: str, kind: type | tuple[type, ...], default: Any) -> Any:
    if key not in raw or raw[key] is None:
        return default
    return _require(raw, key, kind)


@dataclass(frozen=True)
class Lfm2Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    ffn_dim: int
    layer_types: tuple[str, ...]
    conv_kernel_size: int
    conv_bias: bool
    rope_theta: float
    block_norm_eps: float
    norm_eps: float
    tie_embedding: bool
    max_position_embeddings: int | None
    eos_token_id: int | None
    bos_token_id: int | None
    pad_token_id: int | None

    architecture = "Lfm2ForCausalLM"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Lfm2Config":
        architectures = raw.get("architectures")
        if architectures is not None and "Lfm2ForCausalLM" not in architectures:
            raise ConfigError("architectures", f"expected ['Lfm2ForCausalLM'], got {architectures!r}")
        model_type = raw.get("model_type")
        if model_type is not None and model_type != "lfm2":
            raise ConfigError("model_type", f"expected 'lfm2', got {model_type!r}")

        hidden_size = _require(raw, "hidden_size", int)
        num_layers = _require(raw, "num_hidden_layers", int)
        num_heads = _require(raw, "num_attention_heads", int)
        num_groups = _require(raw, "num_key_value_heads", int)
        vocab_size = _require(raw, "vocab_size", int)
        conv_kernel_size = _require(raw, "conv_L_cache", int)
        norm_eps = float(_require(raw, "norm_eps", (int, float)))
        block_norm_eps = float(_optional(raw, "block_norm_eps", (int, float), norm_eps))
        conv_bias = _optional(raw, "conv_bias", bool, False)
        tie_embedding = _optional(raw, "tie_embedding", bool, True)

        alias = raw.get("num_heads")
        if alias is not None and alias != num_heads:
            raise ConfigError("num_heads", f"{alias} conflicts with num_attention_heads={num_heads}")
        for key, value in (
            ("hidden_size", hidden_size),
            ("num_hidden_layers", num_layers),
            ("num_attention_heads", num_heads),
            ("num_key_value_heads", num_groups),
            ("vocab_size", vocab_size),
            ("conv_L_cache", conv_kernel_size),
        ):
            if value < 1:
                raise ConfigError(key, f"must be positive, got {value}")
        if hidden_size % num_heads != 0:
            raise ConfigError("hidden_size", f"{hidden_size} is not divisible by num_attention_heads={num_heads}")
        if num_heads % num_groups != 0:
            raise ConfigError(
                "num_key_value_heads", f"{num_groups} does not divide num_attention_heads={num_heads}"
            )
        head_dim = hidden_size // num_heads
        if head_dim % 2 != 0:
            raise ConfigError("hidden_size", f"head_dim={head_dim} must be even for rotary embeddings")

        layer_types = cls._resolve_layer_types(raw, num_layers)
        rope_theta = cls._resolve_rope_theta(raw)
        ffn_dim = cls._resolve_ffn_dim(raw)

        return cls(
            vocab_size=vocab_size,
            hidden_size=hidden_size,
            num_hidden_layers=num_layers,
            num_attention_heads=num_heads,
            num_key_value_heads=num_groups,
            head_dim=head_dim,
            ffn_dim=ffn_dim,
            layer_types=layer_types,
            conv_kernel_size=conv_kernel_size,
            conv_bias=conv_bias,
            rope_theta=rope_theta,
            block_norm_eps=block_norm_eps,
            norm_eps=norm_eps,
            tie_embedding=tie_embedding,
            max_position_embeddings=_optional(raw, "max_position_embeddings", int, None),
            eos_token_id=_optional(raw, "eos_token_id", int, None),
            bos_token_id=_optional(raw, "bos_token_id", int, None),
            pad_token_id=_optional(raw, "pad_token_id", int, None),
        )

    @classmethod
    def from_json(cls, path: str | Path) -> "Lfm2Config":
        with open(path) as stream:
            return cls.from_dict(json.load(stream))

    @staticmethod
    def _resolve_layer_types(raw: Mapping[str, Any], num_layers: int) -> tuple[str, ...]:
        layer_types = raw.get("layer_types")
        if layer_types is not None:
            if not isinstance(layer_types, list) or len(layer_types) != num_layers:
                raise ConfigError("layer_types", f"must list {num_layers} layer kinds, got {layer_types!r}")
            for kind in layer_types:
                if kind not in _LAYER_KINDS:
                    raise ConfigError("layer_types", f"unknown layer kind {kind!r}; known: {_LAYER_KINDS}")
            return tuple(layer_types)
        indices = raw.get("full_attn_idxs")
        if indices is not None:
            if not isinstance(indices, list) or any(
                isinstance(i, bool) or not isinstance(i, int) or not 0 <= i < num_layers for i in indices
            ):
                raise ConfigError("full_attn_idxs", f"must list layer indices below {num_layers}, got {indices!r}")
            return tuple("full_attention" if i in indices else "conv" for i in range(num_layers))
        raise ConfigError("layer_types", "either layer_types or full_attn_idxs must be present")

    @staticmethod
    def _resolve_rope_theta(raw: Mapping[str, Any]) -> float:
        flat = raw.get("rope_theta")
        nested_block = raw.get("rope_parameters")
        nested = nested_block.get("rope_theta") if isinstance(nested_block, dict) else None
        if flat is None and nested is None:
            raise ConfigError("rope_theta", "neither rope_theta nor rope_parameters.rope_theta is given")
        if flat is not None and nested is not None and flat != nested:
            raise ConfigError("rope_theta", f"{flat} conflicts with rope_parameters.rope_theta={nested}")
        value = nested if nested is not None else flat
        if isinstance(value, bool) or not isinstance(value, (int, float)) or value <= 0:
            raise ConfigError("rope_theta", f"must be a positive number, got {value!r}")
        return float(value)

    @staticmethod
    def _resolve_ffn_dim(raw: Mapping[str, Any]) -> int:
        auto_adjust = _optional(raw, "block_auto_adjust_ff_dim", bool, False)
        if not auto_adjust:
            if raw.get("intermediate_size") is not None:
                result = _require(raw, "intermediate_size", int)
            else:
                result = _require(raw, "block_ff_dim", int)
        else:
            block_ff_dim = _require(raw, "block_ff_dim", int)
            multiplier = float(_optional(raw, "block_ffn_dim_multiplier", (int, float), 1.0))
            multiple_of = _require(raw, "block_multiple_of", int)
            if multiple_of < 1:
                raise ConfigError("block_multiple_of", f"must be positive, got {multiple_of}")
            adjusted = block_ff_dim * multiplier * (2 / 3)
            result = int((adjusted + multiple_of - 1) // multiple_of * multiple_of)
        if result < 1:
            raise ConfigError("block_ff_dim", f"feed-forward width must be positive, got {result}")
        return result

    # ------------------------------------------------------------------ plan
    def to_plan(self) -> ModelPlan:
        block_norm = RMSNormSpec(dim=self.hidden_size, eps=self.block_norm_eps)
        head_norm = RMSNormSpec(dim=self.head_dim, eps=self.block_norm_eps)
        attention = AttentionSpec(
            model_dim=self.hidden_size,
            num_heads=self.num_attention_heads,
            num_groups=self.num_key_value_heads,
            head_dim=self.head_dim,
            qk_norm=head_norm,
            position=RopeSpec(rotary_dim=self.head_dim, theta=self.rope_theta),
            window=None,
            scale=None,
        )
        short_conv = ShortConvSpec(
            model_dim=self.hidden_size,
            kernel_size=self.conv_kernel_size,
            has_bias=self.conv_bias,
        )
        ffn = GatedMLPSpec(model_dim=self.hidden_size, hidden_dim=self.ffn_dim, activation="silu")
        layers = tuple(
            BlockSpec(
                pre_mixer_norm=block_norm,
                mixer=attention if kind == "full_attention" else short_conv,
                pre_ffn_norm=block_norm,
                ffn=ffn,
            )
            for kind in self.layer_types
        )
        return ModelPlan(
            vocab_size=self.vocab_size,
            model_dim=self.hidden_size,
            layers=layers,
            final_norm=RMSNormSpec(dim=self.hidden_size, eps=self.norm_eps),
            tie_embeddings=self.tie_embedding,
        )

    # ------------------------------------------------------ checkpoint names
    def checkpoint_names(self, path: tuple, local: str) -> list[str]:
        """Candidate tensor names in a checkpoint for the tensor ``local`` of the part at
        ``path`` (first = canonical, rest = accepted aliases;
        ``lalamo/model_import/loaders/huggingface.py:1298-1310``, ``766-863``, ``426-461``)."""
        if path == ("embedding",):
            return ["model.embed_tokens.weight"]
        if path == ("lm_head",):
            return ["lm_head.weight"]
        if path == ("final_norm",):
            return ["model.embedding_norm.weight"]
        if path[0] == "layers":
            index, role = path[1], path[2]
            root = f"model.layers.{index}"
            if role == "pre_mixer_norm":
                return [f"{root}.operator_norm.weight"]
            if role == "pre_ffn_norm":
                return [f"{root}.ffn_norm.weight"]
            if role == "ffn":
                name = {"gate_proj": "w1", "up_proj": "w3", "down_proj": "w2"}[local]
                return [f"{root}.feed_forward.{name}.weight"]
            if role == "mixer" and self.layer_types[index] == "conv":
                table = {
                    "in_proj": ["conv.in_proj.weight"],
                    "out_proj": ["conv.out_proj.weight"],
                    "conv_weight": ["conv.conv.weight", "conv.conv1d.weight", "conv.conv_weight"],
                    "conv_bias": ["conv.conv.bias", "conv.conv1d.bias"],
                }
                return [f"{root}.{name}" for name in table[local]]
            if role == "mixer":
                table = {
                    "q_proj": ["self_attn.q_proj.weight"],
                    "k_proj": ["self_attn.k_proj.weight"],
                    "v_proj": ["self_attn.v_proj.weight"],
                    "out_proj": ["self_attn.out_proj.weight", "self_attn.o_proj.weight"],
                    "q_norm": ["self_attn.q_layernorm.weight", "self_attn.q_norm.weight"],
                    "k_norm": ["self_attn.k_layernorm.weight", "self_attn.k_norm.weight"],
                }
                return [f"{root}.{name}" for name in table[local]]
        raise KeyError(f"LFM2 has no tensor {local!r} at {path!r}")

    def checkpoint_shape(self, path: tuple, local: str, shape: tuple[int, ...]) -> tuple[int, ...]:
        """The shape under which a checkpoint stores the tensor (the depthwise convolution is
        ``[dim, 1, taps]`` there, ``lalamo/model_import/loaders/huggingface.py:829-845``)."""
        if local == "conv_weight":
            return (shape[0], 1, shape[1])
        return shape

    def to_json_dict(self) -> dict[str, Any]:
        """A ``config.json`` from which :meth:`from_dict` rebuilds this configuration."""
        return {
            "architectures": ["Lfm2ForCausalLM"],
            "model_type": "lfm2",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "block_auto_adjust_ff_dim": False,
            "block_ff_dim": self.ffn_dim,
            "layer_types": list(self.layer_types),
            "conv_L_cache": self.conv_kernel_size,
            "conv_bias": self.conv_bias,
            "rope_theta": self.rope_theta,
            "block_norm_eps": self.block_norm_eps,
            "norm_eps": self.norm_eps,
            "tie_embedding": self.tie_embedding,
            "max_position_embeddings": self.max_position_embeddings,
            "eos_token_id": self.eos_token_id,
            "bos_token_id": self.bos_token_id,
            "pad_token_id": self.pad_token_id,
        }
