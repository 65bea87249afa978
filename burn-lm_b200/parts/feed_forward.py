"""The dense gated feed-forward: (silu(x Wgate) * (x Wup)) Wdown, no biases
(crates/burn-lm-llama/src/nn/fftn.rs:26-36,44-46).  Gate and up run as one product with a fused
[gate; up] weight; the activation and the product of the two halves are fp32.
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
class SwiGLUSpec:
    hidden_size: int
    intermediate_size: int


@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    family = "feed_forward"
    graph_safe = True
    roles = ("gate", "up", "down")

    def tensor_specs(self):
        s, t = self.spec, self.tensor_names
        return [TensorSpec(t["gate"], (s.intermediate_size, s.hidden_size)),
                TensorSpec(t["up"], (s.intermediate_size, s.hidden_size)),
                TensorSpec(t["down"], (s.hidden_size, s.intermediate_size))]

    def bind(self, loaded):
        t = self.tensor_names
        g, u = loaded[t["gate"]], loaded[t["up"]]
        if g.dtype != u.dtype:
            raise ValueError(f"{t['gate']} and {t['up']} are stored in different dtypes")
        inner = self.spec.intermediate_size
        if g.dtype == torch.bfloat16 and inner % K.GATE_TILE == 0:
            # tiles of 8 gate rows followed by the 8 up rows of the same outputs: the skinny kernel's
            # gated epilogue finds both halves of an output in one 16-row tile
            tile = K.GATE_TILE
            fused = torch.stack([g.view(inner // tile, tile, -1), u.view(inner // tile, tile, -1)], dim=1).reshape(2 * inner, -1)
            self.gate_up = Linear(fused.contiguous(), gate_tile=tile)
        else:
            self.gate_up = Linear(torch.cat([g, u], dim=0).contiguous())
        self.down = Linear(loaded[t["down"]])

    takes_pending_norm = True
    adds_to_stream = True

    def forward(self, x, step, stream=None):
        rt = self.runtime
        act = self.gate_up.gated(x, rt.dtype)
        return self.down.into_stream(act, stream, rt.dtype, handoff=getattr(step, "handoff", None))
