"""A plain, slow LFM2: whole sequences, no cache, one function for each part.

This is the oracle the engine is compared with.  It shares no code with the product path: it
reads ``config.json`` itself, loads tensors with the ``safetensors`` package by their checkpoint
names, and computes in float64 on the CPU.

It rests on the reference's formulas only.  The reference's model code cannot be imported here
(``import lalamo`` needs ``jax`` and ``equinox``, which are not installed and cannot be
installed offline), so no golden outputs of the reference are committed; each function below
cites the reference lines it restates.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch
from safetensors.torch import load_file

DTYPE = torch.float64


def exact(x: torch.Tensor) -> torch.Tensor:
    return x


def to_bfloat16(x: torch.Tensor) -> torch.Tensor:
    """Rounds to bfloat16 and back.  With this as `rnd` the functions below round where the
    reference's default mode rounds its activations (after every product, inside the norm, the
    gated convolution input and output, q/k/v), which measures how much noise bfloat16
    activations put on the logits; the residual stream and the logits stay unrounded."""
    return x.to(torch.bfloat16).to(DTYPE)


def read_config(model_dir: str | Path) -> dict:
    """Derived sizes as the reference derives them
    (lalamo/model_import/model_configs/huggingface/lfm2.py:96-212)."""
    raw = json.loads((Path(model_dir) / "config.json").read_text())
    hidden = raw["hidden_size"]
    heads = raw["num_attention_heads"]
    layers = raw["num_hidden_layers"]
    if raw.get("layer_types") is not None:  # lfm2.py:164-171
        kinds = list(raw["layer_types"])
    else:
        kinds = ["full_attention" if i in raw["full_attn_idxs"] else "conv" for i in range(layers)]
    if not raw.get("block_auto_adjust_ff_dim", False):  # lfm2.py:193-199
        ffn = raw["intermediate_size"] if raw.get("intermediate_size") is not None else raw["block_ff_dim"]
    else:
        adjusted = raw["block_ff_dim"] * raw.get("block_ffn_dim_multiplier", 1.0) * (2 / 3)
        multiple = raw["block_multiple_of"]
        ffn = int((adjusted + multiple - 1) // multiple * multiple)
    nested = (raw.get("rope_parameters") or {}).get("rope_theta")  # lfm2.py:81-94
    theta = nested if nested is not None else raw["rope_theta"]
    return {
        "hidden": hidden,
        "heads": heads,
        "groups": raw["num_key_value_heads"],
        "head_dim": hidden // heads,  # lfm2.py:103
        "layers": layers,
        "kinds": kinds,
        "ffn": ffn,
        "vocab": raw["vocab_size"],
        "taps": raw["conv_L_cache"],
        "conv_bias": raw.get("conv_bias", False),
        "theta": float(theta),
        "block_eps": float(raw.get("block_norm_eps", raw["norm_eps"])),
        "eps": float(raw["norm_eps"]),
        "tied": raw.get("tie_embedding", True),  # lfm2.py:73
    }


def read_weights(model_dir: str | Path) -> dict[str, torch.Tensor]:
    tensors: dict[str, torch.Tensor] = {}
    for path in sorted(Path(model_dir).glob("*.safetensors")):
        tensors.update(load_file(str(path)))
    return {name: tensor.to(DTYPE) for name, tensor in tensors.items()}


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, rnd=exact) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * w over the last axis, no mean subtraction, no offset
    (lalamo/modules/normalization.py:89-126 with the LFM2 settings of lfm2.py:124-129)."""
    variance = x.pow(2).mean(dim=-1, keepdim=True) + eps
    return rnd(rnd(x * torch.rsqrt(variance)) * rnd(weight))


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """x [T, heads, hd]: x * cos + rotate_half(x) * sin with angles pos * theta^(-2i/hd), the
    angle table duplicated over both halves (lalamo/modules/rope.py:94-102, apply at :58-75).
    Frequencies and angles are formed in float32 as the reference forms them."""
    hd = x.shape[-1]
    channel = torch.arange(0, hd, 2, dtype=torch.float32)
    inverse = 1.0 / (torch.tensor(theta, dtype=torch.float32) ** (channel / hd))
    angles = torch.outer(positions.to(torch.float32), inverse)  # float32 product
    angles = torch.cat([angles, angles], dim=-1).to(DTYPE)[:, None, :]
    half = hd // 2
    rotated = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * torch.cos(angles) + rotated * torch.sin(angles)


def attention_mixer(n1: torch.Tensor, w: dict[str, torch.Tensor], prefix: str, cfg: dict, positions: torch.Tensor,
                    window: int | None = None, rnd=exact) -> torch.Tensor:
    """Fused projection order q|k|v, per-head q/k norm, rope, causal softmax attention with
    scale hd^-0.5 and grouped heads g(h) = h // (H/G), out projection
    (lalamo/modules/token_mixers/attention.py:450-473, :511-620; mask kv_cache.py:242-247)."""
    T = n1.shape[0]
    H, G, hd = cfg["heads"], cfg["groups"], cfg["head_dim"]
    q = rnd(n1 @ w[f"{prefix}.q_proj.weight"].T).reshape(T, H, hd)
    k = rnd(n1 @ w[f"{prefix}.k_proj.weight"].T).reshape(T, G, hd)
    v = rnd(n1 @ w[f"{prefix}.v_proj.weight"].T).reshape(T, G, hd)
    q = rnd(rope(rms_norm(q, w[f"{prefix}.q_layernorm.weight"], cfg["block_eps"], rnd), positions, cfg["theta"]))
    k = rnd(rope(rms_norm(k, w[f"{prefix}.k_layernorm.weight"], cfg["block_eps"], rnd), positions, cfg["theta"]))
    out = torch.zeros(T, H, hd, dtype=DTYPE)
    for h in range(H):
        g = h // (H // G)
        scores = (q[:, h, :] @ k[:, g, :].T) / math.sqrt(hd)  # [T, T]
        query_pos = positions[:, None]
        key_pos = positions[None, :]
        visible = query_pos >= key_pos
        if window is not None:
            visible &= query_pos < key_pos + window
        scores = scores.masked_fill(~visible, float("-inf"))
        out[:, h, :] = torch.softmax(scores, dim=-1) @ v[:, g, :]
    return rnd(rnd(out.reshape(T, H * hd)) @ w[f"{prefix}.out_proj.weight"].T)


def short_conv_mixer(n1: torch.Tensor, w: dict[str, torch.Tensor], prefix: str, cfg: dict, rnd=exact) -> torch.Tensor:
    """in_proj rows split in the order (pre-conv gate B, post-conv gate C, x); u = B * x;
    c[t] = sum_k w[:, k] * u[t - (K-1) + k] with zeros before the sequence, so w[:, K-1] multiplies
    the current token; out_proj(C * c)
    (lalamo/modules/token_mixers/short_conv.py:124-145; convolutions.py:154-167;
    restated in tests/unit/modules/test_short_conv.py:71-93)."""
    T, D = n1.shape
    K = cfg["taps"]
    projected = rnd(n1 @ w[f"{prefix}.in_proj.weight"].T)
    pre_gate, post_gate, x = projected[:, :D], projected[:, D : 2 * D], projected[:, 2 * D :]
    u = rnd(pre_gate * x)
    padded = torch.cat([torch.zeros(K - 1, D, dtype=DTYPE), u], dim=0)
    taps = w[f"{prefix}.conv.weight"].reshape(D, K)
    conv = torch.zeros(T, D, dtype=DTYPE)
    for k in range(K):
        conv += padded[k : k + T, :] * taps[:, k]
    if cfg["conv_bias"]:
        conv = conv + w[f"{prefix}.conv.bias"]
    return rnd(rnd(rnd(conv) * post_gate) @ w[f"{prefix}.out_proj.weight"].T)


def swiglu(n2: torch.Tensor, w: dict[str, torch.Tensor], prefix: str, rnd=exact) -> torch.Tensor:
    """down(up * silu(gate)) with up = w3, gate = w1, down = w2
    (lalamo/modules/mlp.py:233-262; names lalamo/model_import/loaders/huggingface.py:1306-1308)."""
    up = rnd(n2 @ w[f"{prefix}.w3.weight"].T)
    gate = rnd(n2 @ w[f"{prefix}.w1.weight"].T)
    return rnd(rnd(up * rnd(gate * torch.sigmoid(gate))) @ w[f"{prefix}.w2.weight"].T)


def block(x: torch.Tensor, w: dict[str, torch.Tensor], index: int, cfg: dict, positions: torch.Tensor, rnd=exact) -> torch.Tensor:
    """h = x + mixer(norm(x)); y = h + ffn(norm(h)) (lalamo/modules/transformer_layer.py:246-344)."""
    root = f"model.layers.{index}"
    n1 = rms_norm(x, w[f"{root}.operator_norm.weight"], cfg["block_eps"], rnd)
    if cfg["kinds"][index] == "full_attention":
        mixed = attention_mixer(n1, w, f"{root}.self_attn", cfg, positions, rnd=rnd)
    else:
        mixed = short_conv_mixer(n1, w, f"{root}.conv", cfg, rnd)
    h = x + mixed
    n2 = rms_norm(h, w[f"{root}.ffn_norm.weight"], cfg["block_eps"], rnd)
    return h + swiglu(n2, w, f"{root}.feed_forward", rnd)


def logits_of(model_dir: str | Path, tokens: list[int], weights: dict[str, torch.Tensor] | None = None, rnd=exact) -> torch.Tensor:
    """Logits [T, vocab] (float64) of the whole sequence at positions 0..T-1
    (lalamo/modules/decoder.py:220-317; final norm lalamo/modules/transformer.py:241-245;
    readout lalamo/modules/embedding.py:125-143, :183-195)."""
    cfg = read_config(model_dir)
    w = weights if weights is not None else read_weights(model_dir)
    positions = torch.arange(len(tokens))
    x = w["model.embed_tokens.weight"][torch.tensor(tokens, dtype=torch.long)]
    for index in range(cfg["layers"]):
        x = block(x, w, index, cfg, positions, rnd)
    normed = rms_norm(x, w["model.embedding_norm.weight"], cfg["eps"], rnd)
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return normed @ head.T


class PlainModel:
    """Caches the weights of one model folder between calls."""

    def __init__(self, model_dir: str | Path) -> None:
        self.model_dir = Path(model_dir)
        self.config = read_config(model_dir)
        self.weights = read_weights(model_dir)

    def logits(self, tokens: list[int], rnd=exact) -> torch.Tensor:
        return logits_of(self.model_dir, tokens, self.weights, rnd)

    def greedy(self, prompt: list[int], new_tokens: int) -> list[int]:
        tokens = list(prompt)
        for _ in range(new_tokens):
            tokens.append(int(torch.argmax(self.logits(tokens)[-1])))
        return tokens[len(prompt) :]
