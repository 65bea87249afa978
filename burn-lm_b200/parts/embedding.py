"""Token embedding (a row gather, no scale: crates/burn-lm-llama/src/nn/transformer.rs:95) and the
output projection to fp32 logits (transformer.rs:101-102; with tie_word_embeddings the head reads
the embedding table, which the reference leaves as a TODO at :82-84).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.loader import TensorSpec
from .base import Part
from .linear import HandedNorm, Linear


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab_size: int
    hidden_size: int


@register_part("embedding", "table")
class Embedding(Part):
    family = "embedding"
    graph_safe = True
    roles = ("table",)

    def tensor_specs(self):
        return [TensorSpec(self.tensor_names["table"], (self.spec.vocab_size, self.spec.hidden_size))]

    def bind(self, loaded):
        self.table = loaded[self.tensor_names["table"]]

    hands_norm_over = True      # forward() takes the step's handoff and may leave the first norm's input there

    def forward(self, tokens, out, handoff=None):
        """`handoff` (parts.linear.NormHandoff) with a norm expected: for a few tokens the kernel also leaves that
        norm's input (the stream times gamma, the rows' sums of squares), as the products that write the stream do."""
        norm = handoff.wanted if handoff is not None else None
        n = tokens.numel()
        if (norm is not None and n <= K.SQUARES_ROWS and self.runtime.dtype == torch.bfloat16 and out.is_cuda
                and getattr(norm, "gamma", None) is not None and norm.gamma.numel() == out.shape[1]):
            handed = HandedNorm(torch.empty((n, out.shape[1]), dtype=torch.bfloat16, device=out.device),
                                torch.empty((1, K.SQUARES_ROWS), dtype=torch.float32, device=out.device))
            K.embed(tokens, self.table, out, hand_over=(norm.gamma, handed.scaled, handed.squares))
            handoff.leave(out, norm.gamma, handed)
            return
        K.embed(tokens, self.table, out)


@dataclass(frozen=True)
class HeadSpec:
    vocab_size: int
    hidden_size: int


@register_part("head", "linear")
class Head(Part):
    """logits = x W^T in fp32; `weight` may name the embedding table (tied)."""
    family = "head"
    graph_safe = True
    roles = ("weight",)

    def tensor_specs(self):
        return [TensorSpec(self.tensor_names["weight"], (self.spec.vocab_size, self.spec.hidden_size))]

    def bind(self, loaded):
        self.linear = Linear(loaded[self.tensor_names["weight"]])

    takes_pending_norm = True

    def forward(self, x):
        return self.linear(x, out_dtype=torch.float32)
