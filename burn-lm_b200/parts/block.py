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
        x = self.mixer_norm.add_norm(resid, delta)
        a = self.mixer.forward(x, step, cache_view)
        x = self.feed_forward_norm.add_norm(resid, a)
        return self.feed_forward.forward(x, step)
