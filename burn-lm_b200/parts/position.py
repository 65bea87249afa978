"""Position encodings.  A mixer asks its position part for constants; the rotation itself runs in
the mixer's kernels.

Rotary: pair i of a head is rotated by position * inv_freq[i], inv_freq[i] = theta^(-2i/dim)
(the reference hands theta to burn's RotaryEncoding: crates/burn-lm-llama/src/nn/llama/base.rs:
269-286), applied to q and k after projection and before the cache (nn/attention/mha.rs:91-95).
Llama-3 scaling changes inv_freq by parts (nn/pos_encoding.rs:103-138).  Frequencies are computed
here in float64; the kernel computes angle, sine and cosine in float64 and rotates in float32, so
there is no table to outgrow.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from ..registry import register_part
from .base import Part


@dataclass(frozen=True)
class Llama3Scaling:
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position: int


@dataclass(frozen=True)
class RotarySpec:
    head_dim: int
    theta: float
    rotary_dim: Optional[int] = None      # lanes that rotate; None: all of the head
    interleaved: bool = False             # False: pairs (i, i + dim/2), the layout of weights stored
                                          # under Hugging Face names; True: pairs (2i, 2i + 1), the
                                          # reference's layout (nn/llama/import.rs:95-126 permutes)
    scaling: Optional[Llama3Scaling] = None


def rotary_inverse_frequencies(spec: RotarySpec) -> list:
    dim = spec.rotary_dim or spec.head_dim
    freqs = [spec.theta ** (-(2.0 * i) / dim) for i in range(dim // 2)]
    s = spec.scaling
    if s is None:
        return freqs
    low_wavelen = s.original_max_position / s.low_freq_factor
    high_wavelen = s.original_max_position / s.high_freq_factor
    out = []
    for f in freqs:
        wavelen = 2.0 * math.pi / f
        if wavelen < high_wavelen:
            out.append(f)
        elif wavelen > low_wavelen:
            out.append(f / s.factor)
        else:
            smooth = (s.original_max_position / wavelen - s.low_freq_factor) / (s.high_freq_factor - s.low_freq_factor)
            out.append((1.0 - smooth) * f / s.factor + smooth * f)
    return out


@register_part("position", "rotary")
class Rotary(Part):
    family = "position"
    graph_safe = True

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        dim = spec.rotary_dim or spec.head_dim
        if dim % 2 or dim > spec.head_dim:
            raise ValueError(f"rotary_dim {dim} must be even and at most head_dim {spec.head_dim}")
        self.rotary_dim = dim
        self.inv_freq = torch.tensor(rotary_inverse_frequencies(spec), dtype=torch.float64, device=runtime.device)
        self._table = None

    def rotation(self):
        return self.inv_freq, self.rotary_dim, self.spec.interleaved

    def prepare(self, max_positions: int) -> None:
        """Compute (cos, sin) for positions below max_positions once (on the device, in float64);
        positions beyond the table are still computed per token by the kernel."""
        from .. import kernels as K
        if self.inv_freq.is_cuda and self.rotary_dim and (self._table is None or self._table.shape[0] < max_positions):
            self._table = K.rope_table(self.inv_freq, max_positions)

    def table(self):
        return self._table

    def on_embedding(self, resid, step):
        return None


@dataclass(frozen=True)
class NoPositionSpec:
    pass


@register_part("position", "none")
class NoPosition(Part):
    """No position encoding: the mixer's kernels append k and v unrotated."""
    family = "position"
    graph_safe = True

    def rotation(self):
        return None, 0, False

    def on_embedding(self, resid, step):
        return None
