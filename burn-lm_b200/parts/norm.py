"""RMS norm fused with the residual add.

y = x / sqrt(mean(x^2) + eps) * gamma; it stands before the mixer, before the feed-forward and once
after the last block (crates/burn-lm-llama/src/nn/transformer.rs:248-255,101; eps at :60-62 and
:211-216).  The sum of squares, the root and the product with gamma are fp32 in both paths.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import kernels as K
from ..registry import register_part
from ..weights.loader import TensorSpec
from .base import Part
from .linear import NormedStream


@dataclass(frozen=True)
class RMSNormSpec:
    size: int
    eps: float


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    family = "norm"
    graph_safe = True
    roles = ("weight",)

    def tensor_specs(self):
        return [TensorSpec(self.tensor_names["weight"], (self.spec.size,), init="one_plus_normal:0.1")]

    def bind(self, loaded):
        self.gamma = loaded[self.tensor_names["weight"]]

    takes_handed_norm = True      # a product that writes the stream may leave this norm's input (parts.linear.NormHandoff)

    def add_norm(self, resid, delta, rows=None, lazy=False, handoff=None):
        """`lazy`: the caller can take a norm that is not computed yet (parts.linear.NormedStream);
        it gets one when nothing has to be added into the stream first.  `handoff`: where the writer of
        the stream may have left this norm's input."""
        handed = handoff.claim(resid, self.gamma) if handoff is not None else None
        if lazy and delta is None:
            return NormedStream(resid, self.gamma, self.spec.eps, rows, self.runtime.dtype, handed)
        n = rows.numel() if rows is not None else resid.shape[0]
        out = torch.empty((n, self.spec.size), dtype=self.runtime.dtype, device=resid.device)
        K.add_rmsnorm(resid, delta, self.gamma, self.spec.eps, out, rows)
        return out
