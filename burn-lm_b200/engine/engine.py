"""The step function: a batch of sequences that start together with unequal lengths, their prompts
in one step, then one token each; only the tokens a step brings are run, as one packed batch, from
the cache, and logits come back for the wanted places only.

The reference's step is `Transformer::forward(input [B, T], cache, pos, mask) -> [B, T, V]` after
`cache.prepare(T)` (crates/burn-lm-llama/src/nn/transformer.rs:88-103, generation/generate.rs:
75-85): rectangular batches of one shared length, logits for every position.  Here tokens of all
sequences are packed without padding, every sequence has its own cached length, and the final norm
and output projection run on the wanted rows only.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from ..cache import Cache, CacheError
from ..model import Model, load_model
from .. import kernels as K
from ..parts.base import StepContext


@dataclass
class StepEntry:
    """One sequence's share of a step: its slot, its next tokens, and the places among these tokens
    whose logits are wanted (may be empty)."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class Workspace:
    """Scratch memory kernels ask for by name; grown when a larger request comes, never shrunk."""

    def __init__(self, device):
        self.device = device
        self._buffers: dict[str, torch.Tensor] = {}

    def scratch(self, name: str, n_floats: int) -> torch.Tensor:
        buf = self._buffers.get(name)
        if buf is None or buf.numel() < n_floats:
            buf = torch.empty(max(n_floats, 1), dtype=torch.float32, device=self.device)
            self._buffers[name] = buf
        return buf


class Engine:
    """A model with its cache.  `acquire()` starts a sequence, `step()` feeds tokens, `release()` ends it."""

    def __init__(self, model: Model, max_tokens: int, max_seqs: Optional[int] = None,
                 max_seq_len: Optional[int] = None, max_step_tokens: Optional[int] = None):
        """`max_tokens`: token places of the cache (rounded up to pages); `max_seqs`: slots; `max_seq_len`: the most
        one sequence may hold; `max_step_tokens`: the most tokens one step may bring (its activations are
        sized by it); None: as many as the cache holds."""
        self.model = model
        rt = model.runtime
        if rt.device.type != "cuda":
            raise RuntimeError("burn-lm_b200 runs on a CUDA device only; there is no CPU path")
        page = K.PAGE
        pages = (max_tokens + page - 1) // page
        if max_seqs is None:
            max_seqs = max(1, min(pages, 1024))
        if max_seq_len is None:
            max_seq_len = model.plan.max_positions
        max_seq_len = min(max_seq_len, pages * page)
        self.cache = Cache(model.cache_needs(), model.plan.schedule, max_tokens, max_seqs, max_seq_len,
                           rt.dtype, rt.device)
        self.workspace = Workspace(rt.device)
        K.prebuild(rt.dtype)
        # tables of positions reach to the end of the last page, as the length buckets of captured steps do
        model.prepare(-(-self.cache.max_seq_len // page) * page)
        self.vocab_size = model.plan.vocab_size
        self.max_step_tokens = max_step_tokens if max_step_tokens is not None else pages * page
        self._staging = None    # pinned int32 staging for the step's metadata
        # decode steps (one token each, its logits wanted) replay a CUDA graph when every part allows it
        self.use_graphs = (all(getattr(p, "graph_safe", False) for p in model.parts())
                           and all(getattr(layer.block, "graph_safe", False) for layer in model.layers))
        self._staging_free = None
        self.decode_ahead = False           # decode_greedy(more=True) may enqueue the following step at once
        self._ahead = None                  # decode_graph.StepInFlight: a greedy step enqueued before it was asked for
        self._decode_graphs: dict = {}      # (batch, length bucket) -> DecodeGraph, least recently used first
        self.max_decode_graphs = 48
        self._last_decode_graph = None      # (batch, lengths above, lengths up to, graph) of the last step
        from .prefill_graph import PrefillGraphs
        self._prefill_graphs = PrefillGraphs(self)

    @classmethod
    def from_folder(cls, folder, dtype="bfloat16", max_tokens=4096, max_seqs=None, max_seq_len=None, device="cuda",
                    max_step_tokens=None):
        return cls(load_model(folder, dtype, device), max_tokens, max_seqs, max_seq_len, max_step_tokens)

    # -- sequences -----------------------------------------------------------------------------------
    def acquire(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.seq_len[slot]

    def verify(self) -> None:
        """Raise if a kernel gave up a bounded wait since the last call (synchronises with the device)."""
        from .. import kernels
        kernels.check_status(self.model.runtime.device)

    def decode_graph(self, batch: int, max_kv_len: int):
        """The captured decode step for `batch` sequences of at most `max_kv_len` tokens (made at first
        use).  Lengths come in buckets (64 tokens times a power of two), because the number of blocks
        that split a sequence's keys is fixed in a captured graph."""
        last = self._last_decode_graph
        if last is not None and last[0] == batch and last[1] < max_kv_len <= last[2]:
            return last[3]                                      # the one of the step before: already the most recently used
        from .decode_graph import DecodeGraph
        pages = 1
        while pages * K.PAGE < max_kv_len:
            pages *= 2
        longest = -(-self.cache.max_seq_len // K.PAGE) * K.PAGE
        bucket = min(pages * K.PAGE, longest)
        graphs = self._decode_graphs
        g = graphs.pop((batch, bucket), None)
        if g is None:
            g = DecodeGraph(self, batch, bucket)
            while len(graphs) >= self.max_decode_graphs:      # the least recently used goes, with its buffers
                del graphs[next(iter(graphs))]
        graphs[(batch, bucket)] = g                             # most recently used last
        # the lengths this graph serves: more than the bucket below it (half of it, unless the bucket was cut to the cache's limit)
        below = pages * K.PAGE // 2 if pages > 1 else 0
        self._last_decode_graph = (batch, below, bucket, g)
        return g

    def decode_run(self, slots, tokens, n_steps: int) -> torch.Tensor:
        """n_steps greedy decode steps for the sequences in `slots`, fed `tokens` first, without the
        host in between.  Returns the sampled tokens, int32 [n_steps, len(slots)], on the device."""
        self._ahead = None
        starts = [self.cache.seq_len[s] for s in slots]
        self.cache.reserve([(s, st + n_steps) for s, st in zip(slots, starts)])
        g = self.decode_graph(len(slots), max(starts) + n_steps)
        g.load(tokens, starts, slots)
        history = g.run(n_steps)
        for s, st in zip(slots, starts):
            self.cache.set_length(s, st + n_steps)
        return history

    def decode_greedy(self, slots, tokens, more: bool = False) -> Optional[list]:
        """One greedy decode step for the sequences in `slots`, each fed its token: the argmax runs in
        the captured graph and the sampled ids come back as a list.  The short way through a step for
        the generation loop; None when this engine does not capture its decode steps.

        `more`: the caller expects to come back with the same sequences and these results as their next
        tokens.  Then (with `decode_ahead` set) the step after this one is enqueued before this one's result is awaited (it is fed on
        the device), so the GPU does not idle while the host looks at the tokens; the next call finds its
        step in flight.  A call that asks for something else (other tokens, fewer sequences) is still served
        from the step in flight where that computed it, and otherwise the step in flight is forgotten: what
        it appended lies beyond its sequences' lengths."""
        if not self.use_graphs:
            return None
        cache = self.cache
        if type(slots) is not list:
            slots = list(slots)
        if type(tokens) is not list:
            tokens = list(tokens)
        more = more and self.decode_ahead
        ahead, self._ahead = self._ahead, None
        cur = None
        if ahead is not None and ahead.tokens_in is not None and len(set(slots)) == len(slots):
            place = {s: i for i, s in enumerate(ahead.slots)}
            if all(s in place and ahead.tokens_in[place[s]] == t and cache.seq_len[s] == ahead.starts[place[s]]
                   for s, t in zip(slots, tokens)):
                if slots == ahead.slots:
                    cur = ahead
                else:
                    # some sequences have left: the others' results are what a step without them gives
                    out = ahead.tokens()
                    for s in slots:
                        cache.seq_len[s] = ahead.starts[place[s]] + 1
                    return [out[place[s]] for s in slots]
        if cur is None:
            starts, grow = self._decode_starts(slots, tokens)
            if grow:
                cache.reserve([(s, n + 1) for s, n in zip(slots, starts)])
            g = self.decode_graph(len(slots), max(starts) + 1)
            if not more:
                out = g.step_greedy_host(tokens, starts, slots)
                for s, n in zip(slots, starts):
                    cache.seq_len[s] = n + 1
                return out
            cur = g.launch_greedy_chained(tokens, starts, slots)
        nxt = self._launch_ahead(cur) if more else None
        out = cur.tokens()
        for s, n in zip(cur.slots, cur.starts):
            cache.seq_len[s] = n + 1
        if nxt is not None:
            nxt.tokens_in = out
            self._ahead = nxt
        return out

    def _decode_starts(self, slots, tokens):
        """The checks of a step for the short ways through a decode step: every slot held and named once, every
        token in the vocabulary.  Returns the sequences' lengths and whether the cache has to make room (a
        new page, or the limit: the careful path decides)."""
        cache = self.cache
        if len(set(slots)) != len(slots):
            raise ValueError(f"a slot appears twice in one step: {sorted(slots)}")
        # (the common case costs a few calls into the interpreter's built-ins, whatever the batch; the loops below only
        # run to name the culprit)
        if slots and not cache.slots.all_held(slots):
            raise CacheError(f"slot {next(s for s in slots if not cache.slots.held(s))} is not held")
        if tokens and not (min(tokens) >= 0 and max(tokens) < self.vocab_size):
            bad = next(t for t in tokens if not 0 <= t < self.vocab_size)
            raise ValueError(f"token id {bad} is outside the vocabulary of {self.vocab_size}")
        starts = list(map(cache.seq_len.__getitem__, slots))
        grow = bool(starts) and (0 in map(K.PAGE.__rmod__, starts) or max(starts) >= cache.max_seq_len)
        return starts, grow

    def _launch_ahead(self, cur):
        """The step after `cur` for the same sequences, enqueued behind it; None where that step needs a
        decision of the careful path (the context limit, no free page) or another graph (a longer bucket)."""
        cache = self.cache
        starts = [n + 1 for n in cur.starts]
        if any(n + 1 > cache.max_seq_len for n in starts):
            return None
        if self.decode_graph(len(cur.slots), max(starts) + 1) is not cur.graph:
            return None
        try:
            cache.reserve([(s, n + 1) for s, n in zip(cur.slots, starts)])
        except CacheError:
            return None
        return cur.graph.launch_greedy_chained(None, starts, cur.slots)

    def decode_sampled(self, slots, tokens, params, stream_ids, counters) -> Optional[list]:
        """One decode step that draws every sequence's next token (temperature, nucleus) inside the captured
        graph; `stream_ids` and `counters` name the draws.  None when this engine does not capture its steps."""
        if not self.use_graphs:
            return None
        self._ahead = None
        cache = self.cache
        slots, tokens = list(slots), list(tokens)
        starts, grow = self._decode_starts(slots, tokens)
        if grow:
            cache.reserve([(s, n + 1) for s, n in zip(slots, starts)])
        g = self.decode_graph(len(slots), max(starts) + 1)
        out = g.step_sampled_host(tokens, starts, slots, params, stream_ids, counters)
        for s, n in zip(slots, starts):
            cache.seq_len[s] = n + 1
        return out

    # -- the step ------------------------------------------------------------------------------------
    def _pack(self, entries):
        """Validate the entries and lay their metadata out in one int32 array (host)."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen = set()
        tokens, token_seq, token_pos, cu, slots, starts, want_rows = [], [], [], [0], [], [], []
        growth = []
        max_q = max_kv = 0
        for s, e in enumerate(entries):
            if e.slot in seen:
                raise ValueError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if not self.cache.slots.held(e.slot):
                raise CacheError(f"slot {e.slot} is not held")
            toks = list(e.tokens)
            if not toks:
                raise ValueError(f"the entry of slot {e.slot} brings no token")
            for t in toks:
                if not 0 <= t < self.vocab_size:
                    raise ValueError(f"token id {t} is outside the vocabulary of {self.vocab_size}")
            start = self.cache.seq_len[e.slot]
            for w in e.want:
                if not 0 <= w < len(toks):
                    raise ValueError(f"wanted place {w} is outside the {len(toks)} tokens of slot {e.slot}")
                want_rows.append(cu[-1] + w)
            tokens.extend(toks)
            token_seq.extend([s] * len(toks))
            token_pos.extend(range(start, start + len(toks)))
            cu.append(cu[-1] + len(toks))
            slots.append(e.slot)
            starts.append(start)
            growth.append((e.slot, start + len(toks)))
            max_q = max(max_q, len(toks))
            max_kv = max(max_kv, start + len(toks))
        if len(tokens) > self.max_step_tokens:
            raise ValueError(f"the step brings {len(tokens)} tokens; this engine takes at most {self.max_step_tokens} in one step")
        return tokens, token_seq, token_pos, cu, slots, starts, want_rows, growth, max_q, max_kv

    def _upload(self, arrays):
        """One pinned staging buffer, one host-to-device copy; returns the device views."""
        total = sum(len(a) for a in arrays)
        if self._staging is None or self._staging.numel() < total:
            self._staging = torch.empty(max(total, 1024), dtype=torch.int32, pin_memory=True)
        if self._staging_free is not None:
            self._staging_free.synchronize()    # the last step's copy has left the staging buffer
        host = self._staging[:total]
        off = 0
        for a in arrays:
            if a:
                host[off: off + len(a)] = torch.tensor(a, dtype=torch.int32)
            off += len(a)
        dev = host.to(self.model.runtime.device, non_blocking=True)
        self._staging_free = torch.cuda.Event()
        self._staging_free.record()
        views, off = [], 0
        for a in arrays:
            views.append(dev[off: off + len(a)])
            off += len(a)
        return views

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the entries' tokens as one batch from the cache.

        Returns fp32 logits [wanted, vocab] in the order of the entries and of their `want`, or None
        when nothing is wanted.  Every sequence's cached length grows by its tokens.  The logits of a
        decode step (one token each) live in a buffer that the next such step overwrites: use or
        copy them before stepping again."""
        self._ahead = None                  # a step enqueued ahead is forgotten: it wrote beyond its sequences' lengths
        (tokens, token_seq, token_pos, cu, slots, starts, want_rows, growth, max_q, max_kv) = self._pack(entries)
        self.cache.reserve(growth)          # raises before anything is launched, changing nothing
        if self.use_graphs and max_q == 1 and want_rows == list(range(len(entries))):
            g = self.decode_graph(len(entries), max_kv)
            g.load(tokens, starts, slots)
            logits = g.step()
            for slot, new_len in growth:
                self.cache.set_length(slot, new_len)
            return logits
        if self.use_graphs:
            # short prompt steps: the same launches at a bucket's sizes, replayed as a graph from its second use
            from .prefill_graph import bucket_of
            bucket = bucket_of(len(tokens), len(entries), max_q, len(want_rows))
            if bucket is not None:
                graphs = self._prefill_graphs
                logits = graphs.get(bucket).run(tokens, token_seq, token_pos, cu, slots, starts, want_rows, graphs.pool)
                for slot, new_len in growth:
                    self.cache.set_length(slot, new_len)
                return logits
        d_tokens, d_seq, d_pos, d_cu, d_slots, d_starts, d_want = self._upload(
            [tokens, token_seq, token_pos, cu, slots, starts, want_rows])
        ctx = StepContext(
            n_tokens=len(tokens), n_seqs=len(entries), max_q_len=max_q, max_kv_len=max_kv,
            tokens=d_tokens, token_seq=d_seq, token_pos=d_pos, cu_seqlens=d_cu, slot_of_seq=d_slots,
            start_pos=d_starts, want_rows=d_want if want_rows else None, n_want=len(want_rows),
            workspace=self.workspace,
            host={"cu_seqlens": cu, "slots": slots, "start_pos": starts})
        logits = self.model.forward(ctx, self.cache)
        for slot, new_len in growth:
            self.cache.set_length(slot, new_len)
        return logits
