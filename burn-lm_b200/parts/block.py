"""How a layer's parts stand around the residual stream.

Pre-norm: h = x + mixer(norm(x)); out = h + feed_forward(norm(h))
(crates/burn-lm-llama/src/nn/transformer.rs:241-256).  The residual stream is fp32; a part's
output is added into it by the next norm's fused kernel, so a block takes the pending output of
the block before it (`delta`) and returns its own.
"""
from __future__ import annotations

from ..registry import register_part


@register_part("block", "prenorm")
class PreNormBlock:
    family = "block"

    def __init__(self, mixer_norm, mixer, feed_forward_norm, feed_forward):
        self.mixer_norm, self.mixer = mixer_norm, mixer
        self.feed_forward_norm, self.feed_forward = feed_forward_norm, feed_forward

    def parts(self):
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def forward(self, resid, delta, step, cache_view):
        # Two optional abilities of a mixer or feed-forward shorten the path: `takes_pending_norm`
        # (its first product normalises on the fly) and `adds_to_stream` (its last product adds its
        # result into the residual stream itself and returns None).
        mixer, ff = self.mixer, self.feed_forward
        x = self.mixer_norm.add_norm(resid, delta, lazy=getattr(mixer, "takes_pending_norm", False))
        if getattr(mixer, "adds_to_stream", False):
            a = mixer.forward(x, step, cache_view, stream=resid)
        else:
            a = mixer.forward(x, step, cache_view)
        x = self.feed_forward_norm.add_norm(resid, a, lazy=getattr(ff, "takes_pending_norm", False))
        if getattr(ff, "adds_to_stream", False):
            return ff.forward(x, step, stream=resid)
        return ff.forward(x, step)
