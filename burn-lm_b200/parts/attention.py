"""The attention mixer: grouped-query causal attention over the paged cache.

q = x Wq, k = x Wk, v = x Wv without bias, feature c of q belonging to head c // head_dim
(crates/burn-lm-llama/src/nn/attention/mha.rs:121-140); q and k are rotated, k and v appended to
the cache (:91-95); query head h reads kv head h // (heads / kv heads) (:174-185); scores are
q.k / sqrt(head_dim), keys after the query's position are hidden, softmax, times v (:157-166);
heads are merged and projected by Wo (:168-170, :118).  The three projections run as one product
with a fused [q; k; v] weight built when the weights are bound.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .. import kernels as K
from ..registry import part_class, register_part
from ..plan import PartPlan
from ..weights.loader import TensorSpec
from .base import CacheNeed, Part
from .linear import Linear

BLOCKS_PER_SM = 2     # blocks a decode step should offer every multiprocessor


@dataclass(frozen=True)
class AttentionSpec:
    hidden_size: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    position: PartPlan                   # family "position"
    window: Optional[int] = None         # None: every earlier key; n: the latest n keys
    softmax_scale: Optional[float] = None  # None: 1 / sqrt(head_dim)


@register_part("mixer", "attention")
class Attention(Part):
    family = "mixer"
    graph_safe = True
    roles = ("q", "k", "v", "o")

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} heads do not divide into {spec.n_kv_heads} kv heads")
        if spec.head_dim % 16 or not 16 <= spec.head_dim <= 256:
            raise ValueError(f"head_dim {spec.head_dim}: the attention kernels take multiples of 16 from 16 to 256")
        self.position = part_class("position", spec.position.kind)(spec.position.spec, spec.position.tensors, runtime)
        if getattr(self.position, "score_bias", None) is not None and self.position.score_bias() is not None:
            # an encoding that adds a per-head bias to the scores (by the distance of key and query, say): the
            # attention kernels of this package compute q.k * scale and the mask only
            raise ValueError(f"position encoding {spec.position.kind!r} asks for a bias on the attention scores, which "
                             f"the attention kernels do not have; it needs a mixer of its own")
        self.scale = spec.softmax_scale if spec.softmax_scale is not None else 1.0 / math.sqrt(spec.head_dim)

    def tensor_specs(self):
        s, t = self.spec, self.tensor_names
        return [TensorSpec(t["q"], (s.n_heads * s.head_dim, s.hidden_size)),
                TensorSpec(t["k"], (s.n_kv_heads * s.head_dim, s.hidden_size)),
                TensorSpec(t["v"], (s.n_kv_heads * s.head_dim, s.hidden_size)),
                TensorSpec(t["o"], (s.hidden_size, s.n_heads * s.head_dim))] + self.position.tensor_specs()

    def bind(self, loaded):
        t = self.tensor_names
        q, k, v = loaded[t["q"]], loaded[t["k"]], loaded[t["v"]]
        if not (q.dtype == k.dtype == v.dtype):
            raise ValueError(f"{t['q']}, {t['k']}, {t['v']} are stored in different dtypes")
        # bfloat16 heads that are rotated whole, in pairs (i, i + head_dim / 2): the rows of every q and k head
        # are dealt out in tiles of eight lanes and their eight partners, so that the skinny product can
        # rotate in its epilogue (kernels.tiled_pair_order).  q and k then carry their lanes in that order
        # everywhere, in the cache too; their dot products do not notice.
        s = self.spec
        _, rot, interleaved = self.position.rotation() if hasattr(self.position, "rotation") else (None, 0, False)
        self.pairs = K.PAIRS_INTERLEAVED if interleaved else K.PAIRS_HALVES
        if q.dtype == torch.bfloat16 and rot == s.head_dim and not interleaved:
            order = torch.tensor(K.tiled_pair_order(s.head_dim), device=q.device)
            q = q.view(s.n_heads, s.head_dim, -1)[:, order].reshape(q.shape)
            k = k.view(s.n_kv_heads, s.head_dim, -1)[:, order].reshape(k.shape)
            self.pairs = K.PAIRS_TILED
        fused = torch.cat([q, k, v], dim=0).contiguous()
        self.qkv = Linear(fused)
        self.q_only = Linear(fused[: self.spec.n_heads * self.spec.head_dim])
        self.o = Linear(loaded[t["o"]])
        self.position.bind(loaded)

    def prepare(self, max_positions: int) -> None:
        if hasattr(self.position, "prepare"):
            self.position.prepare(max_positions)

    def key_layout(self):
        """How this mixer's keys lie in the cache (known once the weights are bound): the order of a head's lanes
        and the rotation they carry.  A run that reads another run's cache line must have the same."""
        return (self.pairs, self.spec.position)

    def cache_need(self) -> CacheNeed:
        s = self.spec
        return CacheNeed("kv", n_kv_heads=s.n_kv_heads, head_dim=s.head_dim, window=s.window)

    def _splits(self, step) -> int:
        if step.max_q_len != 1:
            return 1
        s = self.spec
        group = s.n_heads // s.n_kv_heads
        pages = (step.max_kv_len + K.PAGE - 1) // K.PAGE
        if K.attention_decode_is_specialised(self.runtime.dtype, s.head_dim, group):
            # One block walks all pages of a (sequence, kv head) while they fit its ring of about twelve
            # pages (sixteen still stream well): its groups of warps work on several pages at once and nothing is combined
            # (measured best at batch 1, 8 and 64 with 9 pages).  Longer sequences are cut into a ring's
            # worth per block, as far as that still helps to fill the SMs about twice.
            by_length = (pages + 15) // 16
            want = BLOCKS_PER_SM * K.sm_count(self.runtime.device)
            to_fill = (want + step.n_seqs * s.n_kv_heads - 1) // (step.n_seqs * s.n_kv_heads)
            return max(1, min(by_length, to_fill, pages, 64))
        blocks = step.n_seqs * s.n_kv_heads * ((group + 31) // 32)
        return max(1, min(pages, (BLOCKS_PER_SM * K.sm_count(self.runtime.device) + blocks - 1) // blocks, 64))

    takes_pending_norm = True
    adds_to_stream = True

    def forward(self, x, step, cache, stream=None):
        s, rt = self.spec, self.runtime
        inv_freq, rot, interleaved = self.position.rotation()
        table = self.position.table() if hasattr(self.position, "table") else None
        n = step.n_tokens
        product = self.qkv if cache.writes else self.q_only     # a run that reads another run's cache line needs q only
        qkv = None
        ahead = False
        # the page of every new token and the sequences' rows of the block table: looked up once per step for all
        # the layers that share this block table
        tables = None
        if rt.dtype == torch.bfloat16:
            key = ("step_tables", cache.block_table.data_ptr())
            tables = step.memo.get(key)
            if tables is None:
                tables = step.memo[key] = K.step_tables(step.token_seq, step.token_pos, step.slot_of_seq, cache.block_table, step.n_seqs)
        if self.pairs == K.PAIRS_TILED and table is not None and step.max_kv_len <= table.shape[0]:
            # few tokens: the skinny product rotates and appends in its epilogue and leaves q
            q = torch.empty((n, s.n_heads * s.head_dim), dtype=rt.dtype, device=cache.pool.device)
            rope = dict(token_pos=step.token_pos, token_seq=step.token_seq, slot_of_seq=step.slot_of_seq,
                        block_table=cache.block_table, table=table, pool=cache.pool, n_heads=s.n_heads,
                        n_kv=s.n_kv_heads, head_dim=s.head_dim, write_cache=cache.writes, max_position=step.max_kv_len - 1,
                        token_page=tables[0] if tables is not None else None)
            took = product.with_rotary(x, q, rope)
            if took:
                qkv = q
                ahead = took == "skinny"      # that kernel lets the attention start only after its own wait
        if qkv is None:
            qkv = product(x, out_dtype=rt.dtype)
            K.rope_append(qkv, step.token_seq, step.token_pos, step.slot_of_seq, cache.block_table, inv_freq, rot,
                          self.pairs, cache.pool, s.n_heads, s.n_kv_heads if cache.writes else 0, s.head_dim,
                          write_cache=cache.writes, table=table, max_position=step.max_kv_len - 1)
        out = torch.empty((n, s.n_heads * s.head_dim), dtype=rt.dtype, device=qkv.device)
        n_splits = self._splits(step)
        scratch = None
        if n_splits > 1:
            scratch = step.workspace.scratch("attention", K.attention_scratch_floats(n, s.n_heads, s.head_dim, n_splits))
        K.attention(qkv, qkv.shape[1], cache.pool, cache.block_table, step.cu_seqlens, step.slot_of_seq,
                    step.start_pos, out, n, step.n_seqs, step.max_q_len, s.n_heads, s.n_kv_heads, s.head_dim,
                    self.scale, window=s.window or 0, n_splits=n_splits, scratch=scratch, max_kv_len=step.max_kv_len,
                    seq_table=tables[1] if tables is not None else None, ahead=ahead)
        return self.o.into_stream(out, stream, rt.dtype, handoff=getattr(step, "handoff", None))
