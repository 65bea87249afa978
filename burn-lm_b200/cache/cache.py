"""The cache of a model: a slot per sequence, keys and values per run of the schedule, each
sequence with its own length, and a fixed-size state per sequence beside it.

Storage is sized in tokens.  Keys and values live in pages of 64 positions; a sequence holds as
many pages as its length needs, listed in its row of the block table, so `max_tokens` bounds the sum
over live sequences of their lengths rounded up to 64, whatever their number.  Runs of the schedule
whose mixers need the same thing (all keys of n heads of size d; a window; a state of some shape)
form a group with storage, page allocator and block table of its own.  A group whose mixers look
back over a window only gives a sequence's pages back as soon as every key in them lies before the
window of every token still to come, so a long sequence holds about window / 64 + 2 of its pages.
Pages and slots are given back when a sequence ends and are used again without being cleared: a
kernel never reads a position at or beyond a sequence's length, nor one before the window.  State
blocks are zeroed when a slot is acquired.

The reference preallocates [max_batch, kv heads, max_seq_len, head_dim] per layer with one length
for the whole batch (crates/burn-lm-llama/src/nn/attention/kv_cache.rs:14-34, nn/transformer.rs:
118-146); slots, pages and per-sequence lengths are this package's own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..kernels import PAGE
from .allocators import CacheError, CacheFull, ContextLengthExceeded, IdAllocator


@dataclass
class CacheView:
    """What one run of the schedule sees of the cache."""
    kind: str                               # "kv", "state" or "none"
    writes: bool                            # False: the line belongs to an earlier run; read only
    pool: Optional[torch.Tensor] = None     # kv: [pages, 2, n_kv_heads, PAGE, head_dim]
    block_table: Optional[torch.Tensor] = None   # kv: int32 [max_seqs, max_pages_per_seq]
    state: Optional[torch.Tensor] = None    # state: [max_seqs, *state_shape]
    window: Optional[int] = None


class _KVGroup:
    def __init__(self, need, runs, n_pages, max_seqs, max_pages_per_seq, dtype, device):
        self.need, self.runs = need, list(runs)
        self.pool = torch.empty((len(runs), n_pages, 2, need.n_kv_heads, PAGE, need.head_dim), dtype=dtype, device=device)
        self.pages = IdAllocator(n_pages, "cache page")
        self.block_table = torch.zeros((max_seqs, max_pages_per_seq), dtype=torch.int32, device=device)
        # pages_of[slot][i]: the page that holds positions 64 i .. 64 i + 63 of the slot's sequence, or None once a
        # windowed group has given it back; dropped[slot]: how many leading pages that is
        self.pages_of: list[list] = [[] for _ in range(max_seqs)]
        self.dropped = [0] * max_seqs

    def live_pages(self, slot: int) -> list:
        return self.pages_of[slot][self.dropped[slot]:]

    def drop_before_window(self, slot: int, length: int) -> None:
        """`length`: how long the slot's sequence is now; the tokens still to come sit at positions >= length and see
        the keys from length - window + 1 on.  Pages that lie wholly before that are given back."""
        if not self.need.window:
            return
        first_needed = max(0, length - self.need.window + 1) // PAGE
        last = min(first_needed, len(self.pages_of[slot]))
        if last > self.dropped[slot]:
            for i in range(self.dropped[slot], last):
                self.pages.release(self.pages_of[slot][i])
                self.pages_of[slot][i] = None
            # the table's entries stay valid page numbers: no kernel reads them, but none may point outside the pool
            self.block_table[slot, self.dropped[slot]:last] = 0
            self.dropped[slot] = last

    def bytes(self):
        return self.pool.numel() * self.pool.element_size()


class _StateGroup:
    def __init__(self, need, runs, max_seqs, compute_dtype, device):
        self.need, self.runs = need, list(runs)
        dt = compute_dtype if need.state_dtype == "compute" else getattr(torch, need.state_dtype)
        self.state = torch.zeros((len(runs), max_seqs, *need.state_shape), dtype=dt, device=device)


class Cache:
    def __init__(self, needs: list, schedule, max_tokens: int, max_seqs: int, max_seq_len: int, dtype, device):
        """needs[run]: CacheNeed of every run of the schedule (None where the run reads another's)."""
        if max_tokens < 1 or max_seqs < 1 or max_seq_len < 1:
            raise CacheError("the cache needs room for at least one token of one sequence")
        self.max_tokens, self.max_seqs, self.max_seq_len = max_tokens, max_seqs, max_seq_len
        self.n_pages = (max_tokens + PAGE - 1) // PAGE
        self.max_pages_per_seq = min((max_seq_len + PAGE - 1) // PAGE, self.n_pages)
        self.dtype, self.device = dtype, device
        self.slots = IdAllocator(max_seqs, "sequence slot")
        self.seq_len = [0] * max_seqs
        self._kv_groups: list[_KVGroup] = []
        self._state_groups: list[_StateGroup] = []
        self._where: dict[int, tuple] = {}      # run -> ("kv" | "state" | "none", group, index in group)
        by_need: dict = {}
        for run, need in enumerate(needs):
            if need is not None:
                by_need.setdefault(need, []).append(run)
        for need, runs in by_need.items():
            if need.kind == "kv":
                # (a windowed group has storage of its own; the window is applied in the kernels, and the
                # group gives the pages before it back as the sequence grows)
                g = _KVGroup(need, runs, self.n_pages, max_seqs, self.max_pages_per_seq, dtype, device)
                self._kv_groups.append(g)
                for i, r in enumerate(runs):
                    self._where[r] = ("kv", g, i)
            elif need.kind == "state":
                g = _StateGroup(need, runs, max_seqs, dtype, device)
                self._state_groups.append(g)
                for i, r in enumerate(runs):
                    self._where[r] = ("state", g, i)
            elif need.kind == "none":
                for r in runs:
                    self._where[r] = ("none", None, 0)
            else:
                raise CacheError(f"unknown cache need {need.kind!r}")
        self._views = []
        for run, entry in enumerate(schedule):
            src = run if entry.cache_of is None else entry.cache_of
            kind, g, i = self._where[src]
            writes = entry.cache_of is None
            if kind == "kv":
                self._views.append(CacheView("kv", writes, pool=g.pool[i], block_table=g.block_table, window=g.need.window))
            elif kind == "state":
                self._views.append(CacheView("state", writes, state=g.state[i]))
            else:
                self._views.append(CacheView("none", writes))

    # -- what the model sees -------------------------------------------------------------------------
    def view(self, run: int) -> CacheView:
        return self._views[run]

    def bytes(self) -> int:
        return sum(g.bytes() for g in self._kv_groups)

    @property
    def free_pages(self) -> int:
        return min((g.pages.free_count for g in self._kv_groups), default=self.n_pages)

    # -- sequences -----------------------------------------------------------------------------------
    def acquire(self) -> int:
        """A free slot for a new sequence of length 0; its state blocks are zeroed."""
        slot = self.slots.acquire()
        self.seq_len[slot] = 0
        for g in self._state_groups:
            g.state[:, slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        """Give the slot and all its pages back."""
        if not self.slots.held(slot):
            raise CacheError(f"sequence slot {slot} is released but not held")
        for g in self._kv_groups:
            for p in g.live_pages(slot):
                g.pages.release(p)
            g.pages_of[slot] = []
            g.dropped[slot] = 0
        self.seq_len[slot] = 0
        self.slots.release(slot)

    def release_all(self) -> None:
        for slot in range(self.max_seqs):
            if self.slots.held(slot):
                self.release(slot)

    def reserve(self, growth: list) -> None:
        """Make room for every (slot, new_length) pair, or acquire nothing and raise."""
        plan = []
        for slot, new_len in growth:
            if not self.slots.held(slot):
                raise CacheError(f"sequence slot {slot} is not held")
            if new_len > self.max_seq_len:
                raise ContextLengthExceeded(new_len, self.max_seq_len)
            plan.append((slot, (new_len + PAGE - 1) // PAGE))
        # what lies before the window of every token still to come goes back first (the sequence's length is that of
        # the steps already run: this step's tokens start there)
        for g in self._kv_groups:
            for slot, _ in plan:
                g.drop_before_window(slot, self.seq_len[slot])
        for g in self._kv_groups:
            extra = sum(max(0, pages - len(g.pages_of[slot])) for slot, pages in plan)
            if extra > g.pages.free_count:
                held = self.n_pages - g.pages.free_count
                raise CacheFull(f"the step needs {extra} more cache pages of {PAGE} tokens; {g.pages.free_count} of "
                                f"{self.n_pages} are free ({held * PAGE} of {self.n_pages * PAGE} token places held)")
        for g in self._kv_groups:
            cells, values = [], []              # all the step's new entries of the block table go over in one piece
            for slot, pages in plan:
                have = len(g.pages_of[slot])
                if pages > have:
                    new = g.pages.acquire_many(pages - have)
                    g.pages_of[slot].extend(new)
                    first = slot * self.max_pages_per_seq + have
                    cells.extend(range(first, first + len(new)))
                    values.extend(new)
            if cells:
                dev = g.block_table.device
                g.block_table.view(-1).index_put_((torch.tensor(cells, dtype=torch.int64).to(dev),),
                                                  torch.tensor(values, dtype=torch.int32).to(dev))

    def set_length(self, slot: int, length: int) -> None:
        self.seq_len[slot] = length
