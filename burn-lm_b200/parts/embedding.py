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
from .linear import Linear


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

    def forward(self, tokens, out):
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
