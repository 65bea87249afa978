"""What every part is, and what a step hands to the parts.

A part is built from its own typed `spec` (sizes and constants), the names of the stored tensors
that feed its roles, and the `Runtime` (compute dtype and device).  It lists the tensors it needs,
takes them when they are loaded, and then runs on the packed tokens of a step.  No part knows which
model it is in.

Interfaces by family (registered with `registry.register_part(family, kind)`):

  norm          add_norm(resid, delta, rows=None) -> normed activations.  `resid` is the fp32 residual
                stream [N, D]; the norm first adds `delta` (the previous part's output, or None) into
                it, in fp32, then normalises.  With `rows` it does so for those rows only, into a
                new tensor, and leaves `resid` alone.
  mixer         cache_need() -> CacheNeed;  forward(x, step, cache_view) -> [N, D] in the compute dtype.
  feed_forward  forward(x, step) -> [N, D].
  position      a constant-holder the mixer asks: rotation() -> (inv_freq float64 tensor or None,
                rotary_dim, interleaved);  on_embedding(resid, step) for encodings added to the stream.
  block         forward(resid, delta, step, cache_view) -> delta: how norms, mixer and feed-forward
                are arranged around the residual stream.
  embedding     forward(tokens, out) fills the fp32 residual stream.
  head          forward(x) -> fp32 logits.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


@dataclass(frozen=True)
class Runtime:
    dtype: torch.dtype           # compute dtype of activations and of the cache: bfloat16 or float32
    device: torch.device

    @property
    def exact(self) -> bool:
        """True in the 32-bit path: every product and sum is fp32, no reduced-precision mode."""
        return self.dtype == torch.float32


@dataclass(frozen=True)
class CacheNeed:
    """What one run of a mixer keeps per sequence.

    kind "kv":    keys and values per position: n_kv_heads x head_dim each; `window` None keeps all
                  positions, a number keeps that many of the latest.
    kind "state": a fixed-size block per sequence of `state_shape` in `state_dtype`, zero when a
                  sequence starts.
    kind "none":  nothing."""
    kind: str
    n_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: tuple = ()
    state_dtype: str = "float32"


@dataclass
class StepContext:
    """One step's packed batch, on the device.  Sequence s owns tokens cu_seqlens[s]..cu_seqlens[s+1];
    its token t sits at position start_pos[s] + t."""
    n_tokens: int
    n_seqs: int
    max_q_len: int               # longest run of new tokens of one sequence in this step
    max_kv_len: int              # longest sequence after this step
    tokens: torch.Tensor         # int32 [N]
    token_seq: torch.Tensor      # int32 [N] index of the token's sequence in this step; -1: a row of no sequence
                                 # (padding up to a captured graph's size), computed like any row but kept out of
                                 # the cache, and outside every sequence's cu_seqlens range
    token_pos: torch.Tensor      # int32 [N] absolute position
    cu_seqlens: torch.Tensor     # int32 [n_seqs + 1]
    slot_of_seq: torch.Tensor    # int32 [n_seqs] cache slot of every sequence
    start_pos: torch.Tensor      # int32 [n_seqs] cached length before the step
    want_rows: Optional[torch.Tensor]   # int32 [W] token rows whose logits are wanted
    n_want: int
    workspace: "object" = None   # the engine's scratch provider: scratch(name, n_floats) -> fp32 tensor
    host: dict = field(default_factory=dict)   # host copies for parts that plan on the CPU
    handoff: "object" = None     # parts.linear.NormHandoff of the step, when the block uses one
    memo: dict = field(default_factory=dict)   # what parts look up once per step and share (emptied when a forward begins)


class Part:
    family = ""
    # True when forward() only launches work on the current stream that depends on the step through
    # the device buffers of the StepContext (never through step.host or Python branches on its
    # values): such a part can be captured in a CUDA graph and replayed for other sequences.  It must also
    # cope with the padding of captured prompt steps: rows whose token_seq is -1 belong to no sequence and
    # must not reach a cache or a state; sequences of no tokens may follow the real ones.
    graph_safe = False

    def __init__(self, spec, tensors: dict, runtime: Runtime):
        self.spec = spec
        self.tensor_names = dict(tensors)
        self.runtime = runtime

    def tensor_specs(self) -> list:
        """The stored tensors this part needs (weights.TensorSpec)."""
        return []

    def bind(self, loaded: dict) -> None:
        """Take the loaded tensors (a dict by stored name)."""
