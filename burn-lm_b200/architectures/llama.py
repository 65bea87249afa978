"""The dense Llama decoder as a plan of parts: the registry entry "LlamaForCausalLM".

Pre-norm blocks of grouped-query attention with rotary positions (Llama-3 scaling when the
configuration has it) and a SwiGLU feed-forward, a final RMS norm and a tied or untied output
projection (crates/burn-lm-llama/src/nn/transformer.rs:45-103,241-256).  Tensor names are the ones
Llama model folders use; the reference's names for the same tensors are listed in its import maps
(crates/burn-lm-llama/src/nn/llama/import.rs:23-88).  Stored q/k projections are in the
half-split rotary layout, so the position part pairs lanes (i, i + head_dim / 2).
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..parts.attention import AttentionSpec
from ..parts.embedding import EmbeddingSpec, HeadSpec
from ..parts.feed_forward import SwiGLUSpec
from ..parts.norm import RMSNormSpec
from ..parts.position import Llama3Scaling, RotarySpec
from ..plan import ModelPlan, PartPlan, ScheduleEntry, prenorm_layer
from ..registry import Architecture, register_architecture


def llama_plan(cfg: LlamaConfig) -> ModelPlan:
    scaling = None
    if cfg.rope_scaling is not None:
        s = cfg.rope_scaling
        scaling = Llama3Scaling(s.factor, s.low_freq_factor, s.high_freq_factor, s.original_max_position_embeddings)
    position = PartPlan("rotary", RotarySpec(head_dim=cfg.head_dim, theta=cfg.rope_theta, interleaved=False,
                                             scaling=scaling))
    norm = RMSNormSpec(cfg.hidden_size, cfg.rms_norm_eps)
    layers = []
    for n in range(cfg.num_hidden_layers):
        p = f"model.layers.{n}."
        layers.append(prenorm_layer(
            mixer_norm=PartPlan("rmsnorm", norm, {"weight": p + "input_layernorm.weight"}),
            mixer=PartPlan("attention",
                           AttentionSpec(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                                         cfg.head_dim, position),
                           {"q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
                            "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight"}),
            feed_forward_norm=PartPlan("rmsnorm", norm, {"weight": p + "post_attention_layernorm.weight"}),
            feed_forward=PartPlan("swiglu", SwiGLUSpec(cfg.hidden_size, cfg.intermediate_size),
                                  {"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
                                   "down": p + "mlp.down_proj.weight"}),
        ))
    table = "model.embed_tokens.weight"
    return ModelPlan(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        embedding=PartPlan("table", EmbeddingSpec(cfg.vocab_size, cfg.hidden_size), {"table": table}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(n) for n in range(cfg.num_hidden_layers)),
        final_norm=PartPlan("rmsnorm", norm, {"weight": "model.norm.weight"}),
        head=PartPlan("linear", HeadSpec(cfg.vocab_size, cfg.hidden_size),
                      {"weight": table if cfg.tie_word_embeddings else "lm_head.weight"}),
        max_positions=cfg.max_position_embeddings,
        stop_ids=tuple(cfg.eos_token_ids),
        ignorable_tensors=(r"model\.layers\.\d+\.self_attn\.rotary_emb\.inv_freq",),
        # some writers store the tied head as well: accepted when it is the table's copy, refused when it differs
        duplicate_tensors=(("lm_head.weight", table),) if cfg.tie_word_embeddings else (),
    )


LLAMA = register_architecture(Architecture(
    name="LlamaForCausalLM", config_class=LlamaConfig, plan=llama_plan, aliases=("llama",),
    description="dense Llama decoder: GQA attention with rotary positions, SwiGLU, RMS norm"))
