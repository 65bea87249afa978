"""The typed configuration of the dense Llama decoder, read from its own config.json keys.

The reference keeps these sizes in `LlamaConfig` / `TransformerConfig` presets
(crates/burn-lm-llama/src/nn/llama/base.rs:40-139, nn/transformer.rs:21-41) and has no config.json;
the keys here are the ones a Llama model folder carries.  Defaults follow the reference: kv heads
default to the heads (base.rs:254), head_dim to width / heads (nn/attention/mha.rs:191), eps 1e-5
(transformer.rs:39-40), theta 10000 (base.rs:61-62).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

from .reader import ConfigError, KeyReader


@dataclass(frozen=True)
class Llama3RopeScaling:
    """The `rope_scaling` block with rope_type "llama3" (reference: RopeFrequencyScaling,
    crates/burn-lm-llama/src/nn/pos_encoding.rs:91-101)."""
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[Llama3RopeScaling]
    max_position_embeddings: int
    tie_word_embeddings: bool
    eos_token_ids: tuple = ()
    bos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None
    architecture: str = "LlamaForCausalLM"
    raw: dict = field(default_factory=dict, compare=False, repr=False)

    @classmethod
    def from_dict(cls, data: dict) -> "LlamaConfig":
        r = KeyReader(data)
        hidden = r.integer("hidden_size", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        kv = r.integer("num_key_value_heads", default=heads, minimum=1)
        head_dim = r.integer("head_dim", default=None, minimum=1)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(f"config key 'head_dim' is absent and 'hidden_size' ({hidden}) is not a "
                                  f"multiple of 'num_attention_heads' ({heads})")
            head_dim = hidden // heads
        if heads % kv:
            raise ConfigError(f"config key 'num_key_value_heads' ({kv}) must divide 'num_attention_heads' ({heads})")
        if head_dim % 2:
            raise ConfigError(f"config key 'head_dim' ({head_dim}) must be even for rotary pairs")
        if r.boolean("attention_bias", default=False):
            raise ConfigError("config key 'attention_bias' is true: biased projections are not part of this decoder")
        if r.boolean("mlp_bias", default=False):
            raise ConfigError("config key 'mlp_bias' is true: biased projections are not part of this decoder")
        act = r.string("hidden_act", default="silu")
        if act != "silu":
            raise ConfigError(f"config key 'hidden_act' must be 'silu', got {act!r}")
        scaling = None
        rs = r.obj("rope_scaling", default=None)
        if rs is not None:
            s = KeyReader(rs, "rope_scaling.")
            kind = s.string("rope_type", default=None) or s.string("type", default=None)
            if kind in (None, "default"):
                scaling = None
            elif kind == "llama3":
                scaling = Llama3RopeScaling(
                    factor=s.number("factor", positive=True),
                    low_freq_factor=s.number("low_freq_factor", positive=True),
                    high_freq_factor=s.number("high_freq_factor", positive=True),
                    original_max_position_embeddings=s.integer("original_max_position_embeddings", minimum=1))
                if scaling.high_freq_factor == scaling.low_freq_factor:
                    raise ConfigError("config keys 'rope_scaling.high_freq_factor' and 'low_freq_factor' must differ")
            else:
                raise ConfigError(f"config key 'rope_scaling.rope_type' is {kind!r}; this decoder knows 'llama3'")
        archs = data.get("architectures")
        arch = archs[0] if isinstance(archs, list) and archs else "LlamaForCausalLM"
        return cls(
            vocab_size=r.integer("vocab_size", minimum=1),
            hidden_size=hidden,
            intermediate_size=r.integer("intermediate_size", minimum=1),
            num_hidden_layers=r.integer("num_hidden_layers", minimum=1),
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=head_dim,
            rms_norm_eps=r.number("rms_norm_eps", default=1e-5, positive=True),
            rope_theta=r.number("rope_theta", default=10000.0, positive=True),
            rope_scaling=scaling,
            max_position_embeddings=r.integer("max_position_embeddings", default=2048, minimum=1),
            tie_word_embeddings=r.boolean("tie_word_embeddings", default=False),
            eos_token_ids=r.int_or_list("eos_token_id", default=()),
            bos_token_id=r.integer("bos_token_id", default=None),
            torch_dtype=r.string("torch_dtype", default=None) or r.string("dtype", default=None),
            architecture=arch,
            raw=dict(data),
        )

    def to_dict(self) -> dict:
        """The config.json content of this configuration."""
        d = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": False,
            "mlp_bias": False,
        }
        if self.rope_scaling is not None:
            s = self.rope_scaling
            d["rope_scaling"] = {
                "rope_type": "llama3", "factor": s.factor, "low_freq_factor": s.low_freq_factor,
                "high_freq_factor": s.high_freq_factor,
                "original_max_position_embeddings": s.original_max_position_embeddings}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.torch_dtype:
            d["torch_dtype"] = self.torch_dtype
        return d
