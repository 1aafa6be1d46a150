"""The tiny LFM2 configurations of the tests (they differ in every size and option) and helpers
that write their model folders with random weights into a temporary directory."""

from __future__ import annotations

from pathlib import Path

from lalamo_b200.weights import write_random_model

# Tiny A: layer kinds by `layer_types`, feed-forward width by `block_ff_dim`, flat `rope_theta`,
# tied embeddings, no convolution bias, 3 taps.
TINY_A = {
    "architectures": ["Lfm2ForCausalLM"],
    "model_type": "lfm2",
    "vocab_size": 512,
    "hidden_size": 64,
    "num_hidden_layers": 4,
    "num_attention_heads": 4,
    "num_heads": 4,
    "num_key_value_heads": 2,
    "layer_types": ["conv", "full_attention", "conv", "full_attention"],
    "block_auto_adjust_ff_dim": False,
    "block_ff_dim": 192,
    "conv_L_cache": 3,
    "conv_bias": False,
    "rope_theta": 10000.0,
    "block_norm_eps": 1e-5,
    "norm_eps": 1e-5,
    "tie_embedding": True,
    "eos_token_id": 7,
}

# Tiny B: starts with attention, two convolutions in a row, one K/V head under three query heads,
# head size 32, vocabulary no power of two, kinds by `full_attn_idxs`, width by auto-adjustment
# (384 * 1.0 * 2/3 = 256 -> 256), nested rope_theta, untied head, convolution bias, 4 taps,
# different eps for block norms and the final norm.
TINY_B = {
    "architectures": ["Lfm2ForCausalLM"],
    "model_type": "lfm2",
    "vocab_size": 1000,
    "hidden_size": 96,
    "num_hidden_layers": 6,
    "num_attention_heads": 3,
    "num_key_value_heads": 1,
    "full_attn_idxs": [0, 3, 5],
    "block_auto_adjust_ff_dim": True,
    "block_ff_dim": 384,
    "block_ffn_dim_multiplier": 1.0,
    "block_multiple_of": 256,
    "conv_L_cache": 4,
    "conv_bias": True,
    "rope_parameters": {"rope_theta": 1000000.0, "rope_type": "default"},
    "block_norm_eps": 1e-6,
    "norm_eps": 3e-6,
    "tie_embedding": False,
    "eos_token_id": 2,
}

# Tiny C: head size 64 (the only one the tcgen05 attention takes, and the one the published checkpoints
# have), two query heads per K/V head, three taps with bias, a width that is a multiple of 128.
TINY_C = {
    "architectures": ["Lfm2ForCausalLM"],
    "model_type": "lfm2",
    "vocab_size": 768,
    "hidden_size": 256,
    "num_hidden_layers": 3,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "layer_types": ["full_attention", "conv", "full_attention"],
    "block_auto_adjust_ff_dim": False,
    "block_ff_dim": 320,
    "conv_L_cache": 3,
    "conv_bias": True,
    "rope_theta": 100000.0,
    "block_norm_eps": 1e-5,
    "norm_eps": 1e-6,
    "tie_embedding": True,
    "eos_token_id": 3,
}

TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2)}

# Random weights of N(0, 0.02) make every sub-block's output tiny beside the embedding, which
# would hide faults in the mixers; the tests use a larger spread so that each part matters.
TEST_STD = 0.08


def make_model(directory: Path, which: str, dtype: str = "bfloat16", std: float = TEST_STD) -> Path:
    config, seed = TINY[which]
    return write_random_model(directory, config, seed=seed, std=std, dtype=dtype)
