"""Prompt steps as CUDA graphs: a short prompt's step is a hundred small launches, and issuing them
from the interpreter takes longer than the device needs to run them.

A captured graph has fixed sizes, so a step is fitted into a bucket: its token count, its number of
sequences, its longest run of new tokens and its number of wanted rows are rounded up (`bucket_of`: tokens
to 16, then by 64, 128 or 256; sequences and wanted rows to a power of two),
and what the rounding adds changes no result:

  * rows after the last token carry token 0 at position 0 and the sequence index -1.  They belong to no
    sequence: cu_seqlens ends before them, so attention neither reads nor writes them; the kernels that
    append to the cache skip a row of sequence -1; every other kernel works row by row, so whatever
    these rows hold stays in them;
  * sequences after the last are empty (their bounds repeat the packed batch's end): no block of the
    attention kernels finds a query row in them;
  * wanted rows after the last repeat the last one and are cut from the result.

What a step brings goes through one pinned buffer and one copy into device buffers with fixed
addresses, as for the decode graphs.  A bucket's first step runs the same padded launches plainly
(which also loads every kernel it needs); its second step captures them; from then on a step is
one copy and one graph launch.  Plain and captured steps of a bucket launch the same kernels on the
same shapes, so their results are the same bits.
"""
from __future__ import annotations

import weakref
from collections import OrderedDict
from typing import Optional

import torch

from ..parts.base import StepContext
from ..parts.linear import SKINNY_TOKENS
from .decode_graph import _capturing
from .engine import Workspace

MAX_TOKENS = 2048       # longer steps keep the device busy for longer than their launches take
MAX_WANTED = 64
MAX_GRAPHS = 24         # most recently used buckets that keep their graph


def _round_up(n: int, step: int) -> int:
    return -(-n // step) * step


def _pow2(n: int) -> int:
    p = 1
    while p < n:
        p *= 2
    return p


def bucket_of(n_tokens: int, n_seqs: int, max_q_len: int, n_want: int) -> Optional[tuple]:
    """(tokens, sequences, longest run, wanted rows) of the bucket a step falls into, or None for a step
    that runs plainly: a decode step (the decode graphs' business), a long one, one with many wanted rows."""
    if n_tokens == n_seqs or n_tokens > MAX_TOKENS or n_want > MAX_WANTED:
        return None
    if n_tokens <= SKINNY_TOKENS:
        tokens = SKINNY_TOKENS          # a few tokens keep the kernels made for a few tokens
    else:
        tokens = _round_up(n_tokens, 64 if n_tokens <= 512 else 128 if n_tokens <= 1024 else 256)
    longest = min(_round_up(max_q_len, 128), tokens)
    return tokens, _pow2(n_seqs), longest, _pow2(n_want) if n_want else 0


class PrefillGraph:
    """The launches of one bucket's step, with the device buffers they read."""

    def __init__(self, engine, bucket: tuple):
        self._engine = weakref.ref(engine)
        self.bucket = bucket
        t, s, q, w = bucket
        dev = engine.model.runtime.device
        self._sizes = [t, t, t, s + 1, s, s, w]     # tokens | token_seq | token_pos | cu_seqlens | slots | starts | wanted rows
        total = sum(self._sizes)
        self.meta = torch.zeros(total, dtype=torch.int32, device=dev)
        self.host_meta = torch.zeros(total, dtype=torch.int32, pin_memory=True)
        self._host_np = self.host_meta.numpy()
        views, off = [], 0
        for n in self._sizes:
            views.append(self.meta[off: off + n])
            off += n
        self.ctx = StepContext(
            n_tokens=t, n_seqs=s, max_q_len=q, max_kv_len=engine.cache.max_seq_len,
            tokens=views[0], token_seq=views[1], token_pos=views[2], cu_seqlens=views[3], slot_of_seq=views[4],
            start_pos=views[5], want_rows=views[6] if w else None, n_want=w,
            workspace=Workspace(dev),       # its own: a captured graph keeps the addresses it saw
            host={"cu_seqlens": None, "slots": None, "start_pos": None})
        self._graph = None
        self._captured = None
        self._copied = None
        self.steps = 0

    def _load(self, tokens, token_seq, token_pos, cu, slots, starts, want_rows) -> None:
        t, s, _, w = self.bucket
        pad_t, pad_s = t - len(tokens), s - len(slots)
        flat = [*tokens, *([0] * pad_t), *token_seq, *([-1] * pad_t), *token_pos, *([0] * pad_t), *cu, *([cu[-1]] * pad_s), *slots, *([slots[-1]] * pad_s),
                *starts, *([starts[-1]] * pad_s)]
        if w:
            flat += [*want_rows, *([want_rows[-1]] * (w - len(want_rows)))]
        if self._copied is not None:
            self._copied.synchronize()          # the last copy has left the pinned buffer
        self._host_np[:] = flat
        self.meta.copy_(self.host_meta, non_blocking=True)
        self._copied = torch.cuda.Event()
        self._copied.record()
        host = self.ctx.host
        host["cu_seqlens"], host["slots"], host["start_pos"] = flat[3 * t: 3 * t + s + 1], None, None

    def run(self, tokens, token_seq, token_pos, cu, slots, starts, want_rows, pool) -> Optional[torch.Tensor]:
        """The step on the given (unpadded, host) metadata; fp32 logits [wanted, vocab] of its own, or None."""
        engine = self._engine()
        self._load(tokens, token_seq, token_pos, cu, slots, starts, want_rows)
        self.steps += 1
        if self._graph is None and self.steps < 2:
            logits = engine.model.forward(self.ctx, engine.cache)
            return None if logits is None else logits[: len(want_rows)]
        if self._graph is None:
            g = torch.cuda.CUDAGraph()
            with _capturing(g, pool):
                self._captured = engine.model.forward(self.ctx, engine.cache)
            self._graph = g
        self._graph.replay()
        # a copy: the graph's own buffer is written again by the bucket's next step
        return None if self._captured is None else self._captured[: len(want_rows)].clone()


class PrefillGraphs:
    """The engine's buckets, the most recently used of them with their graphs."""

    def __init__(self, engine):
        self._engine = weakref.ref(engine)
        self._graphs: "OrderedDict[tuple, PrefillGraph]" = OrderedDict()
        self._pool = None

    def get(self, bucket: tuple) -> PrefillGraph:
        g = self._graphs.get(bucket)
        if g is None:
            if self._pool is None:
                # one memory pool for all of them: they run one after another and keep nothing between steps
                self._pool = torch.cuda.graph_pool_handle()
            g = self._graphs[bucket] = PrefillGraph(self._engine(), bucket)
            while len(self._graphs) > MAX_GRAPHS:
                self._graphs.popitem(last=False)
        self._graphs.move_to_end(bucket)
        return g

    @property
    def pool(self):
        return self._pool

    def __len__(self):
        return len(self._graphs)
