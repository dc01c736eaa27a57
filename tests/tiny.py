"""Small configurations and helpers shared by the tests.

TINY_A and TINY_B differ in every size and option: layers, width, heads and groups, head size,
feed-forward width, vocabulary (no power of two in B), rope base and scaling, norm epsilon, tied
or untied output, context.  TINY_C adds what neither has: biases, linear rope scaling, a head size
of 48 and a width that is no multiple of the head count times the head size.
"""

from __future__ import annotations

import json
import tempfile
from pathlib import Path

import numpy as np
import torch

from plain import plain_llama

TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 2,
    "hidden_size": 64,
    "num_attention_heads": 4,
    "num_key_value_heads": 2,
    "head_dim": 16,
    "intermediate_size": 192,
    "vocab_size": 256,
    "rope_theta": 10000.0,
    "rope_scaling": None,
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True,
    "max_position_embeddings": 128,
    "hidden_act": "silu",
    "eos_token_id": 2,
}

TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 3,
    "hidden_size": 96,
    "num_attention_heads": 3,
    "num_key_value_heads": 1,
    "head_dim": 32,
    "intermediate_size": 256,
    "vocab_size": 320,
    "rope_theta": 500000.0,
    "rope_scaling": {
        "rope_type": "llama3",
        "factor": 8.0,
        "low_freq_factor": 1.0,
        "high_freq_factor": 4.0,
        "original_max_position_embeddings": 64,
    },
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False,
    "max_position_embeddings": 256,
    "hidden_act": "silu",
    "eos_token_id": [5, 7],
}

TINY_C = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 2,
    "hidden_size": 80,
    "num_attention_heads": 6,
    "num_key_value_heads": 3,
    "head_dim": 48,
    "intermediate_size": 136,
    "vocab_size": 203,
    "rope_theta": 25000.0,
    "rope_scaling": {"rope_type": "linear", "factor": 2.0},
    "rms_norm_eps": 3e-6,
    "tie_word_embeddings": False,
    "attention_bias": True,
    "mlp_bias": True,
    "max_position_embeddings": 512,
    "hidden_act": "silu",
}

# Not tiny in shape: sizes at which the tensor-core kernels run their real tilings (head size 64 and
# 128, four query heads per kv head, widths of several tiles, K split over clusters), still small
# enough for the plain implementation.
MID_D = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 2,
    "hidden_size": 512,
    "num_attention_heads": 8,
    "num_key_value_heads": 2,
    "head_dim": 64,
    "intermediate_size": 1408,
    "vocab_size": 1000,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 128},
    "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True,
    "max_position_embeddings": 1024,
    "hidden_act": "silu",
}

MID_E = {
    "architectures": ["LlamaForCausalLM"],
    "model_type": "llama",
    "num_hidden_layers": 2,
    "hidden_size": 768,
    "num_attention_heads": 6,
    "num_key_value_heads": 6,
    "head_dim": 128,
    "intermediate_size": 2048,
    "vocab_size": 1203,
    "rope_theta": 10000.0,
    "rope_scaling": None,
    "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False,
    "max_position_embeddings": 512,
    "hidden_act": "silu",
}

TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}
MID = {"D": MID_D, "E": MID_E}


def make_folder(raw_config: dict, seed: int, tmp_path, std: float = 0.02, gain_std: float = 0.1,
                dtype=torch.bfloat16) -> Path:
    """A model folder with random weights, written by the library's random-weights mode."""
    from models_b200.config import config_from_dict
    from models_b200.weights import write_random_model

    folder = Path(tmp_path) / f"model_{seed}"
    write_random_model(folder, config_from_dict(raw_config), seed, std=std, gain_std=gain_std, dtype=dtype)
    return folder


def plain_logits(folder, tokens, dtype=torch.float32):
    config, weights = plain_llama.read_model_folder(folder)
    return plain_llama.forward(config, weights, list(tokens), dtype=dtype)


def random_tokens(vocab: int, n: int, seed: int):
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, vocab, size=n)]


def scaled_error(actual, expected) -> float:
    """Largest absolute difference, as a fraction of the largest expected magnitude."""
    actual = torch.as_tensor(actual, dtype=torch.float64).cpu()
    expected = torch.as_tensor(expected, dtype=torch.float64).cpu()
    assert actual.shape == expected.shape, (actual.shape, expected.shape)
    return float((actual - expected).abs().max() / expected.abs().max().clamp_min(1e-30))


# Largest allowed scaled_error.  float32: both sides compute in float32 and differ in the order of
# additions only.  bfloat16: the engine rounds activations to 8 bits of mantissa (2^-9 relative per
# rounding) between kernels, the plain implementation does not.
TOLERANCE = {"float32": 2e-5, "bfloat16": 3e-2}
