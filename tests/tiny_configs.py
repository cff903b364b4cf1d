"""Two tiny configurations of the architecture that differ in every size and
option, and helpers that write them as model folders with random weights."""
import json
import tempfile
from pathlib import Path

import numpy as np

# A: 2 layers, 4 heads in 2 groups, head size 16, tied head, eps 1e-6, theta 1e4, all keys everywhere
CONFIG_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "intermediate_size": 160, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 1024, "bos_token_id": -1, "eos_token_id": -1,
    "use_sliding_window": False,
}
RANDOM_A = dict(seed=0, std=0.08, bias_std=0.08, gain_std=0.0)

# B: 3 layers, 6 heads in 2 groups of 3, head size 32 given by its own key (6*32 != 80), width and
# vocabulary that are no powers of two, untied head, eps 1e-5, theta 1e6, a window of 24 from layer 1 on
CONFIG_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 80, "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32,
    "intermediate_size": 208, "vocab_size": 391, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 2048, "bos_token_id": -1, "eos_token_id": 7,
    "use_sliding_window": True, "sliding_window": 24, "max_window_layers": 1,
}
RANDOM_B = dict(seed=3, std=0.07, bias_std=0.1, gain_std=0.1)

# C: one KV head, head size 64, no biases at all, window on every layer
CONFIG_C = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 112, "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 64,
    "intermediate_size": 144, "vocab_size": 203, "rope_theta": 50000.0, "rms_norm_eps": 3e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 4096, "attention_bias": False,
    "use_sliding_window": True, "sliding_window": 40, "max_window_layers": 0,
}
RANDOM_C = dict(seed=5, std=0.06, bias_std=0.0, gain_std=0.05)

# D: a head size that is no power of two (48), as many KV heads as query heads (no groups), five of them
CONFIG_D = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 120, "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48,
    "intermediate_size": 176, "vocab_size": 130, "rope_theta": 100000.0, "rms_norm_eps": 2e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 512, "bos_token_id": -1, "eos_token_id": -1,
    "use_sliding_window": False,
}
RANDOM_D = dict(seed=7, std=0.07, bias_std=0.05, gain_std=0.1)

# E: sizes that break every alignment a kernel might lean on: width 100 (rows of 200 bytes), feed-forward
# width 72, vocabulary 77, three query heads on one KV head
CONFIG_E = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 100, "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 16,
    "intermediate_size": 72, "vocab_size": 77, "rope_theta": 20000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 512, "bos_token_id": -1, "eos_token_id": -1,
    "use_sliding_window": False,
}
RANDOM_E = dict(seed=9, std=0.08, bias_std=0.05, gain_std=0.1)

# The two tiny configurations of the benchmark description, word for word.
# Tiny A: 2 layers, hidden 64, 4 query heads, 2 KV heads, head size 16, intermediate 160, vocabulary 256, RoPE base
# 10000, eps 1e-6, QKV bias, tied, max positions 128, no window; weights and biases N(0, 0.02) from seed 0, gains 1.
CONFIG_TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "intermediate_size": 160, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 128, "bos_token_id": -1, "eos_token_id": -1,
    "use_sliding_window": False,
}
RANDOM_TINY_A = dict(seed=0, std=0.02, bias_std=0.02, gain_std=0.0)
# Tiny B: 3 layers, hidden 128, 4 query heads on 1 KV head, head size 32, intermediate 352, vocabulary 384, RoPE base
# 1e6, eps 1e-5, QKV bias, untied head, max positions 256, no window; weights N(0, 0.02), biases N(0, 0.05) from
# seed 3, gains 1 + N(0, 0.1).
CONFIG_TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 128, "num_attention_heads": 4, "num_key_value_heads": 1,
    "intermediate_size": 352, "vocab_size": 384, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 256, "bos_token_id": -1, "eos_token_id": -1,
    "use_sliding_window": False,
}
RANDOM_TINY_B = dict(seed=3, std=0.02, bias_std=0.05, gain_std=0.1)

# F and G: sizes that the fused decode kernel takes (head size 64, widths and vocabularies that are multiples of 16), and
# that differ from each other in everything else: F three layers, two KV heads of two query heads, biases, tied head, all
# keys; G two layers, one KV head of six query heads, no biases, untied head, a window of 40 on every layer
CONFIG_F = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 128, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
    "intermediate_size": 208, "vocab_size": 400, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 4096, "bos_token_id": -1, "eos_token_id": -1,
    "use_sliding_window": False,
}
RANDOM_F = dict(seed=11, std=0.07, bias_std=0.08, gain_std=0.1)
CONFIG_G = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 112, "num_attention_heads": 6, "num_key_value_heads": 1, "head_dim": 64,
    "intermediate_size": 144, "vocab_size": 272, "rope_theta": 500000.0, "rms_norm_eps": 2e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 4096, "attention_bias": False,
    "use_sliding_window": True, "sliding_window": 40, "max_window_layers": 0,
}
RANDOM_G = dict(seed=13, std=0.06, bias_std=0.0, gain_std=0.05)

CONFIGS = {"F": (CONFIG_F, RANDOM_F), "G": (CONFIG_G, RANDOM_G), "TINY_A": (CONFIG_TINY_A, RANDOM_TINY_A), "TINY_B": (CONFIG_TINY_B, RANDOM_TINY_B), "A": (CONFIG_A, RANDOM_A), "B": (CONFIG_B, RANDOM_B), "C": (CONFIG_C, RANDOM_C), "D": (CONFIG_D, RANDOM_D),
           "E": (CONFIG_E, RANDOM_E)}


def write_tiny(name: str, folder=None, store_dtype="float32") -> Path:
    from easy_gpt.cpp_b200.weights.random_init import write_random_model

    cfg, rnd = CONFIGS[name]
    folder = Path(folder or tempfile.mkdtemp(prefix=f"tiny_{name}_"))
    return write_random_model(folder, cfg, store_dtype=store_dtype, **rnd)


def random_tokens(vocab: int, n: int, seed: int):
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()
