"""Named configurations, as config.json dicts.

The reference keeps its models' sizes as constructor presets (crates/burn-lm-llama/src/nn/llama/
base.rs:73-139: llama3_2_1b, llama3_2_3b, llama3_1_8b, ...); here the same sizes are written with the
keys a Llama model folder's config.json carries, so a preset and a folder go through one reader.
Stop ids follow the reference's tokenizer: 256 special tokens after 128,000 ranks, of which
<|end_of_text|> is the 2nd, <|eom_id|> the 9th and <|eot_id|> the 10th
(crates/burn-lm-llama/src/tokenizer/tiktoken.rs:17-30,126-132).

The two tiny ones differ from each other in every size and option (layers, width, heads and groups,
head size, inner size, vocabulary, theta, scaling, eps, tied or untied head, positions); tests and the
smoke run use them with random weights.
"""
from __future__ import annotations

import copy


def _llama3(layers, width, heads, kv_heads, head_dim, inner, factor, tied, positions=131072):
    return {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": layers, "hidden_size": width, "num_attention_heads": heads,
        "num_key_value_heads": kv_heads, "head_dim": head_dim, "intermediate_size": inner,
        "vocab_size": 128256, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": factor, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 8192},
        "rms_norm_eps": 1e-5, "tie_word_embeddings": tied, "max_position_embeddings": positions,
        "hidden_act": "silu", "attention_bias": False, "mlp_bias": False,
        "bos_token_id": 128000, "eos_token_id": [128001, 128008, 128009],
    }


_PRESETS = {
    # base.rs:106-115
    "llama3_2_1b": _llama3(16, 2048, 32, 8, 64, 8192, 32.0, True),
    # base.rs:75-86
    "llama3_2_3b": _llama3(28, 3072, 24, 8, 128, 8192, 32.0, True),
    # base.rs:117-123 (default width 4096, 32 layers, 32 heads: base.rs:43-52; default scaling factor 8)
    "llama3_1_8b": _llama3(32, 4096, 32, 8, 128, 14336, 8.0, False),
    "tiny_a": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
        "head_dim": 16, "intermediate_size": 160, "vocab_size": 256, "rope_theta": 10000.0,
        "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
        "max_position_embeddings": 128, "hidden_act": "silu",
    },
    "tiny_b": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "num_hidden_layers": 3, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 1,
        "head_dim": 32, "intermediate_size": 512, "vocab_size": 384, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 64},
        "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 256,
        "hidden_act": "silu", "eos_token_id": [7, 11],
    },
}


def preset_names() -> list:
    return sorted(_PRESETS)


def preset(name: str) -> dict:
    """The config.json content of a named configuration (a fresh copy)."""
    from .reader import ConfigError
    key = name.lower().replace("-", "_").replace(".", "_")
    if key not in _PRESETS:
        raise ConfigError(f"no preset named {name!r}; presets: {preset_names()}")
    return copy.deepcopy(_PRESETS[key])


def llama3_2_1b() -> dict:
    return preset("llama3_2_1b")


def llama3_2_3b() -> dict:
    return preset("llama3_2_3b")


def llama3_1_8b() -> dict:
    return preset("llama3_1_8b")


def tiny_a() -> dict:
    return preset("tiny_a")


def tiny_b() -> dict:
    return preset("tiny_b")
