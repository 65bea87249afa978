"""How a layer's parts stand around the residual stream.

Pre-norm: h = x + mixer(norm(x)); out = h + feed_forward(norm(h))
(crates/burn-lm-llama/src/nn/transformer.rs:241-256).  The residual stream is fp32; a part's
output is added into it by the next norm's fused kernel, so a block takes the pending output of
the block before it (`delta`) and returns its own.
"""
from __future__ import annotations

from ..registry import register_part
from .linear import NormHandoff


def _add_norm(norm, resid, delta, lazy, handoff):
    if getattr(norm, "takes_handed_norm", False):
        return norm.add_norm(resid, delta, lazy=lazy, handoff=handoff)
    return norm.add_norm(resid, delta, lazy=lazy)


@register_part("block", "prenorm")
class PreNormBlock:
    family = "block"
    graph_safe = True     # it only calls its parts: a step of graph-safe parts can be captured

    NAMES = ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward")

    def __init__(self, parts: dict):
        if set(parts) != set(self.NAMES):
            raise ValueError(f"the prenorm block arranges parts named {self.NAMES}; the layer has {sorted(parts)}")
        self.mixer_norm, self.mixer = parts["mixer_norm"], parts["mixer"]
        self.feed_forward_norm, self.feed_forward = parts["feed_forward_norm"], parts["feed_forward"]

    def first_norm(self):
        """The norm that reads the stream first in this block: the block before may prepare its input."""
        return self.mixer_norm

    def forward(self, resid, delta, step, cache_view, next_norm=None):
        # Two optional abilities of a mixer or feed-forward shorten the path: `takes_pending_norm`
        # (its first product normalises on the fly) and `adds_to_stream` (its last product adds its
        # result into the residual stream itself and returns None).  A part that adds into the stream
        # is told, through the step's handoff, which norm reads the stream next (`next_norm` after this
        # block), and may leave that norm's input beside its sum.
        mixer, ff = self.mixer, self.feed_forward
        if step.handoff is None:
            step.handoff = NormHandoff()
        handoff = step.handoff
        x = _add_norm(self.mixer_norm, resid, delta, getattr(mixer, "takes_pending_norm", False), handoff)
        if getattr(mixer, "adds_to_stream", False):
            handoff.expect(self.feed_forward_norm)
            a = mixer.forward(x, step, cache_view, stream=resid)
        else:
            a = mixer.forward(x, step, cache_view)
        x = _add_norm(self.feed_forward_norm, resid, a, getattr(ff, "takes_pending_norm", False), handoff)
        if getattr(ff, "adds_to_stream", False):
            handoff.expect(next_norm)
            return ff.forward(x, step, stream=resid)
        return ff.forward(x, step)
