"""Tiny configurations of the architecture, differing in every size and option, and helpers that
write them as model folders with random weights."""
import os

import numpy as np

from burn_lm_b200.config import preset

# the two that differ in every size and option; they are the package's presets of the same names
TINY_A = preset("tiny_a")
TINY_B = preset("tiny_b")

# head_dim 48 (not a power of two), 5 query heads on 5 kv heads, a width that is no multiple of 64,
# room for long decoding
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 112, "num_attention_heads": 5, "num_key_value_heads": 5,
    "head_dim": 48, "intermediate_size": 200, "vocab_size": 1000, "rope_theta": 50000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 2.0,
                     "original_max_position_embeddings": 128},
    "rms_norm_eps": 3e-6, "tie_word_embeddings": True, "max_position_embeddings": 2048,
    "hidden_act": "silu",
}

# head_dim 64 and 128: the sizes the tensor-core attention kernels and the skinny product are written for
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 320, "vocab_size": 515, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 256},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 1024, "hidden_act": "silu",
}

TINY_E = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 256, "num_attention_heads": 4, "num_key_value_heads": 1,
    "head_dim": 128, "intermediate_size": 384, "vocab_size": 640, "rope_theta": 10000.0, "rope_scaling": None,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 1024, "hidden_act": "silu",
}

# eight kv heads of size 64 with two query heads each, as many kv heads as the 1B shape: with dozens of
# sequences a decode step offers the attention kernel hundreds of (sequence, kv head) blocks
TINY_F = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 192, "num_attention_heads": 16, "num_key_value_heads": 8,
    "head_dim": 64, "intermediate_size": 448, "vocab_size": 300, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 128},
    "rms_norm_eps": 2e-5, "tie_word_embeddings": False, "max_position_embeddings": 1024, "hidden_act": "silu",
}

CONFIGS = {"tiny_a": TINY_A, "tiny_b": TINY_B, "tiny_c": TINY_C, "tiny_d": TINY_D, "tiny_e": TINY_E}
MORE_CONFIGS = dict(CONFIGS, tiny_f=TINY_F)


def make_folder(tmp_path, name, seed=0, dtype="float32"):
    from burn_lm_b200 import write_random_model

    folder = os.path.join(str(tmp_path), f"{name}-{dtype}-{seed}")
    if not os.path.exists(os.path.join(folder, "model.safetensors")):
        write_random_model(folder, MORE_CONFIGS[name], seed=seed, dtype=dtype)
    return folder


def random_tokens(seed, n, vocab):
    return [int(t) for t in np.random.default_rng(seed).integers(0, vocab, size=n)]


def row_error(got, want):
    """max |got - want| of every row, relative to the row's largest |want|."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return np.abs(got - want).max(axis=-1) / np.abs(want).max(axis=-1)
