"""The generation loop above the step function: batches of unequal prompts, stop tokens, sequences
that end earlier, and as many batches one after another as there are requests.

The reference's loop handles one prompt: reset, tokenize, then per new token prepare the cache,
forward, take the last position's logits, sample, append (crates/burn-lm-llama/src/generation/
generate.rs:37-109); a stop id ends the sequence and is counted but not emitted
(generation/context.rs:142-170).  Here a batch of prompts is prefilled in one step, then every
live sequence gets one token a step; a sequence leaves the batch when it stops, and its slot and
pages go back to the cache.

The loop talks to an engine (acquire / step / release / cache limits) and a sampler through small
interfaces, so its decisions can be tested with stand-ins on the CPU.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

from ..cache.allocators import ContextLengthExceeded
from ..kernels import PAGE
from ..sampling.sampler import SamplingParams
from .engine import StepEntry


@dataclass(frozen=True)
class GenerateOptions:
    """Per-call options, named as the reference names them (Llama3ServerConfig,
    crates/burn-lm-llama/src/server/llama3.rs:14-31): top_p, temperature, sample_len, seed
    (0: a new random seed for the call)."""
    temperature: float = 0.0
    top_p: float = 0.9
    sample_len: int = 4096
    seed: int = 0
    stop_ids: Sequence[int] = ()
    ignore_stop: bool = False        # keep going over stop ids (benchmarks)
    include_stop: bool = False       # the stop id that ends a sequence is part of its output (the reference drops it)
    batch_size: Optional[int] = None  # most sequences decoded together; None: as many as fit


@dataclass
class RequestResult:
    tokens: list = field(default_factory=list)
    finish_reason: str = ""          # "stop", "length", "context" or "error"
    error: Optional[Exception] = None
    prompt_tokens: int = 0


@dataclass
class GenerationStats:
    """Counts and durations; prefill and decode are kept apart (the reference reports one
    tokens / duration figure that mixes them: crates/burn-lm-inference/src/stats.rs:58-67)."""
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    decode_steps: int = 0
    batches: int = 0
    seed: int = 0

    @property
    def inference_seconds(self) -> float:
        return self.prefill_seconds + self.decode_seconds

    @property
    def tokens_per_second(self) -> float:
        return self.generated_tokens / self.inference_seconds if self.inference_seconds > 0 else 0.0


@dataclass
class GenerationOutput:
    results: list
    stats: GenerationStats

    @property
    def tokens(self) -> list:
        return [r.tokens for r in self.results]


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


def plan_batches(prompt_lens, sample_len, free_pages, free_slots, max_seq_len, batch_size=None):
    """Cut the requests, in order, into batches that fit the cache at their longest.

    Returns (batches, rejected): lists of request indices, and {index: exception} for requests that
    can never run (empty, or a prompt with no room for one new token).  A request's worst case is its
    prompt plus sample_len tokens, capped by max_seq_len."""
    batches, rejected, cur, cur_pages = [], {}, [], 0
    limit = min(free_slots, batch_size) if batch_size else free_slots
    for i, n in enumerate(prompt_lens):
        if n == 0:
            rejected[i] = ValueError("empty prompt")
            continue
        if n > max_seq_len or pages_for(n) > free_pages:
            rejected[i] = ContextLengthExceeded(n, min(max_seq_len, free_pages * PAGE))
            continue
        need = min(pages_for(min(n + sample_len, max_seq_len)), free_pages)
        if cur and (len(cur) >= limit or cur_pages + need > free_pages):
            batches.append(cur)
            cur, cur_pages = [], 0
        cur.append(i)
        cur_pages += need
    if cur:
        batches.append(cur)
    return batches, rejected


class GenerationLoop:
    def __init__(self, engine, sampler, default_stop_ids=()):
        self.engine, self.sampler = engine, sampler
        self.default_stop_ids = tuple(default_stop_ids)
        self._next_stream = 0

    def generate(self, prompts: Sequence[Sequence[int]], options: GenerateOptions = GenerateOptions(),
                 on_token: Optional[Callable] = None) -> GenerationOutput:
        seed = options.seed or (time.time_ns() & ((1 << 62) - 1)) or 1
        params = SamplingParams(options.temperature, options.top_p, seed)
        stop = set() if options.ignore_stop else set(self.default_stop_ids) | set(options.stop_ids)
        results = [RequestResult(prompt_tokens=len(p)) for p in prompts]
        stats = GenerationStats(seed=seed)
        cache = self.engine.cache
        batches, rejected = plan_batches([len(p) for p in prompts], options.sample_len, cache.free_pages,
                                         cache.slots.free_count, cache.max_seq_len, options.batch_size)
        for i, err in rejected.items():
            results[i].finish_reason, results[i].error = "error", err
        for batch in batches:
            self._run_batch(batch, prompts, results, params, stop, options.sample_len, stats, on_token, options.include_stop)
            stats.batches += 1
        return GenerationOutput(results, stats)

    def _run_batch(self, batch, prompts, results, params, stop, sample_len, stats, on_token, include_stop=False):
        engine = self.engine
        max_len = engine.cache.max_seq_len
        slots = {i: engine.acquire() for i in batch}
        fused = getattr(engine, "decode_greedy", None)
        fused_draw = getattr(engine, "decode_sampled", None)
        looks_ahead = bool(getattr(engine, "decode_ahead", False))
        # a request's draws are numbered from 0 in a stream of its own: (seed, request index)
        live = list(batch)
        try:
            t0 = time.perf_counter()
            if sample_len <= 0:
                for i in live:
                    results[i].finish_reason = "length"
                return
            entries = [StepEntry(slots[i], prompts[i], [len(prompts[i]) - 1]) for i in live]
            logits = engine.step(entries)
            tokens = self.sampler.sample(logits, params, live, [0] * len(live))
            stats.prompt_tokens += sum(len(prompts[i]) for i in live)
            stats.prefill_seconds += time.perf_counter() - t0
            t0 = time.perf_counter()
            live_slots = None
            while True:
                nxt = []
                for i, tok in zip(live, tokens):
                    r = results[i]
                    stats.generated_tokens += 1           # a stop id is counted, not emitted
                    if tok in stop:
                        r.finish_reason = "stop"
                        if include_stop:
                            r.tokens.append(tok)
                            if on_token is not None:
                                on_token(i, tok)
                    else:
                        r.tokens.append(tok)
                        if on_token is not None:
                            on_token(i, tok)
                        if len(r.tokens) >= sample_len:
                            r.finish_reason = "length"
                        elif len(prompts[i]) + len(r.tokens) > max_len:
                            r.finish_reason = "context"   # no room to feed this token back
                        else:
                            nxt.append(i)
                    if r.finish_reason:
                        engine.release(slots.pop(i))      # its slot and pages are free for others
                if len(nxt) != len(live) or live_slots is None:       # someone left: the others' slots, in their order
                    live_slots = [slots[i] for i in nxt]
                live = nxt
                if not live:
                    break
                tokens = None
                step_fn = fused if params.greedy else fused_draw
                # How many more tokens every live request takes for certain, unless a stop id turns up: until the
                # first of them reaches its length or the context's end.  Steps within that stretch need no look
                # at single requests: the step's tokens are fed back as they came, and they join the requests'
                # lists in one go when the stretch ends (or an error ends it).
                quiet = 0
                if step_fn is not None and on_token is None:
                    quiet = min(min(sample_len - 1 - len(results[i].tokens), max_len - len(prompts[i]) - len(results[i].tokens)) for i in live)
                if quiet > 0:
                    last = [results[i].tokens[-1] for i in live]
                    counts = None if params.greedy else [len(results[i].tokens) for i in live]
                    columns = []
                    try:
                        while quiet > 0:
                            if params.greedy:
                                got = step_fn(live_slots, last, more=looks_ahead)
                            else:
                                got = step_fn(live_slots, last, params, live, counts)
                            if got is None:                    # this engine has no short way: the careful one below
                                break
                            stats.decode_steps += 1
                            if stop and not stop.isdisjoint(got):
                                tokens = got                   # someone stops here: looked at one by one above
                                break
                            stats.generated_tokens += len(got)
                            columns.append(got)
                            last = got
                            if counts is not None:
                                counts = [c + 1 for c in counts]
                            quiet -= 1
                    finally:
                        for j, i in enumerate(live):
                            results[i].tokens.extend([column[j] for column in columns])
                    if tokens is not None:
                        continue
                if params.greedy and fused is not None:      # the engine samples inside its captured step
                    # will anyone need a step after this one (if no stop id turns up)?  Then the engine may enqueue it now.
                    more = looks_ahead and any(len(results[i].tokens) + 1 < sample_len and len(prompts[i]) + len(results[i].tokens) + 1 <= max_len
                                               for i in live)
                    tokens = fused(live_slots, [results[i].tokens[-1] for i in live], more=more)
                elif not params.greedy and fused_draw is not None:
                    tokens = fused_draw(live_slots, [results[i].tokens[-1] for i in live], params, live,
                                        [len(results[i].tokens) for i in live])
                if tokens is None:
                    entries = [StepEntry(slots[i], [results[i].tokens[-1]], [0]) for i in live]
                    logits = engine.step(entries)
                    tokens = self.sampler.sample(logits, params, live, [len(results[i].tokens) for i in live])
                stats.decode_steps += 1
            stats.decode_seconds += time.perf_counter() - t0
            verify = getattr(engine, "verify", None)
            if verify is not None:
                verify()                      # no kernel gave up a bounded wait during this batch
        finally:
            for slot in slots.values():
                engine.release(slot)
