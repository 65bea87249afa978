"""The generation loop's decisions, with stand-ins for the engine and the sampler (no GPU): batches
in order, stop ids, lengths, the context limit, early leavers, release of every slot."""
import pytest
import torch

from burn_lm_b200.cache import Cache, ContextLengthExceeded
from burn_lm_b200.engine.generate import GenerateOptions, GenerationLoop, plan_batches
from burn_lm_b200.parts.base import CacheNeed
from burn_lm_b200.plan import ScheduleEntry

VOCAB = 50


class ScriptedEngine:
    """Keeps a real cache (CPU) and returns logits whose argmax is a function of the sequence so far:
    next = (sum of the sequence's tokens + its length) % VOCAB."""

    def __init__(self, max_tokens=64 * 8, max_seqs=4, max_seq_len=256):
        need = CacheNeed("kv", n_kv_heads=1, head_dim=16)
        self.cache = Cache([need], [ScheduleEntry(0)], max_tokens, max_seqs, max_seq_len, torch.float32, torch.device("cpu"))
        self.history = {}
        self.steps = []

    def acquire(self):
        s = self.cache.acquire()
        self.history[s] = []
        return s

    def release(self, slot):
        self.cache.release(slot)
        del self.history[slot]

    def step(self, entries):
        self.cache.reserve([(e.slot, self.cache.seq_len[e.slot] + len(e.tokens)) for e in entries])
        self.steps.append([(e.slot, len(e.tokens)) for e in entries])
        rows = []
        for e in entries:
            self.history[e.slot].extend(e.tokens)
            self.cache.set_length(e.slot, len(self.history[e.slot]))
            for w in e.want:
                assert w == len(e.tokens) - 1
                h = self.history[e.slot]
                row = torch.zeros(VOCAB)
                row[(sum(h) + len(h)) % VOCAB] = 1.0
                rows.append(row)
        return torch.stack(rows)


class ArgmaxSampler:
    def __init__(self):
        self.calls = []

    def sample(self, logits, params, stream_ids, counters):
        self.calls.append((params, list(stream_ids), list(counters)))
        return logits.argmax(-1).tolist()


def expected(prompt, n, stop=()):
    h, out = list(prompt), []
    for _ in range(n):
        t = (sum(h) + len(h)) % VOCAB
        if t in stop:
            return out, "stop"
        out.append(t)
        h.append(t)
    return out, "length"


def test_unequal_prompts_lengths_and_stops():
    eng, smp = ScriptedEngine(), ArgmaxSampler()
    loop = GenerationLoop(eng, smp, default_stop_ids=(13,))
    prompts = [[1, 2, 3], [4], [5, 6, 7, 8, 9, 10, 11], [2, 2]]
    out = loop.generate(prompts, GenerateOptions(sample_len=12, stop_ids=(29,)))
    for p, r in zip(prompts, out.results):
        toks, why = expected(p, 12, stop=(13, 29))
        assert r.tokens == toks and r.finish_reason == why
    assert {r.finish_reason for r in out.results} == {"stop", "length"}    # the script makes both happen
    # one prefill step with all four, then single tokens for those still alive
    assert [n for _, n in eng.steps[0]] == [3, 1, 7, 2]
    assert all(n == 1 for st in eng.steps[1:] for _, n in st)
    sizes = [len(st) for st in eng.steps]
    assert sizes == sorted(sizes, reverse=True) and sizes[-1] < sizes[0]   # shorter requests left earlier
    assert eng.cache.slots.held_count == 0 and eng.cache.free_pages == eng.cache.n_pages
    assert out.stats.generated_tokens == sum(len(r.tokens) + (r.finish_reason == "stop") for r in out.results)
    assert out.stats.prompt_tokens == 13 and out.stats.batches == 1
    # draw numbers: a request's own stream, counting its own tokens
    assert smp.calls[0][1] == [0, 1, 2, 3] and smp.calls[0][2] == [0, 0, 0, 0]
    assert all(c == k for k, (_, _, cs) in enumerate(smp.calls) for c in cs)


def test_batches_follow_one_another_and_reuse_slots():
    eng, smp = ScriptedEngine(max_seqs=2), ArgmaxSampler()
    loop = GenerationLoop(eng, smp)
    prompts = [[i + 1, i + 2] for i in range(5)]
    out = loop.generate(prompts, GenerateOptions(sample_len=3))
    assert out.stats.batches == 3
    for p, r in zip(prompts, out.results):
        assert r.tokens == expected(p, 3)[0]
    prefills = [st for st in eng.steps if any(n > 1 for _, n in st)]
    assert [len(st) for st in prefills] == [2, 2, 1]
    assert {s for st in eng.steps for s, _ in st} == {0, 1}                # the same two slots again and again


def test_ignore_stop_and_seed():
    eng, smp = ScriptedEngine(), ArgmaxSampler()
    loop = GenerationLoop(eng, smp, default_stop_ids=(13,))
    out = loop.generate([[4]], GenerateOptions(sample_len=20, ignore_stop=True, seed=77, temperature=0.5, top_p=0.8))
    assert out.results[0].tokens == expected([4], 20)[0] and out.results[0].finish_reason == "length"
    p = smp.calls[0][0]
    assert (p.seed, p.temperature, p.top_p) == (77, 0.5, 0.8) and out.stats.seed == 77
    out2 = loop.generate([[4]], GenerateOptions(sample_len=1))
    assert out2.stats.seed != 0                                            # seed 0: a fresh one is drawn


def test_context_limit_and_rejections():
    eng, smp = ScriptedEngine(max_tokens=64 * 8, max_seqs=4, max_seq_len=70), ArgmaxSampler()
    loop = GenerationLoop(eng, smp)
    prompts = [list(range(1, 68)), list(range(80)), [], [3]]
    out = loop.generate(prompts, GenerateOptions(sample_len=10))
    r0, r1, r2, r3 = out.results
    assert r0.finish_reason == "context" and len(r0.tokens) == 4           # 67 + 3 fed = 70 places, one more sampled
    assert r1.finish_reason == "error" and isinstance(r1.error, ContextLengthExceeded) and r1.error.actual == 80
    assert r2.finish_reason == "error" and r3.finish_reason == "length" and len(r3.tokens) == 10
    assert eng.cache.slots.held_count == 0


def test_on_token_streams_in_order():
    eng, smp = ScriptedEngine(), ArgmaxSampler()
    seen = []
    out = GenerationLoop(eng, smp).generate([[1], [2, 3]], GenerateOptions(sample_len=4), on_token=lambda i, t: seen.append((i, t)))
    for i, r in enumerate(out.results):
        assert [t for j, t in seen if j == i] == r.tokens


def test_plan_batches_respects_pages_slots_and_batch_size():
    b, rej = plan_batches([10, 10, 10, 10, 10], sample_len=100, free_pages=4, free_slots=8, max_seq_len=1000)
    assert b == [[0, 1], [2, 3], [4]] and not rej                          # 2 pages each at the longest
    b, _ = plan_batches([10] * 5, sample_len=10, free_pages=100, free_slots=2, max_seq_len=1000)
    assert b == [[0, 1], [2, 3], [4]]
    b, _ = plan_batches([10] * 5, sample_len=10, free_pages=100, free_slots=8, max_seq_len=1000, batch_size=4)
    assert b == [[0, 1, 2, 3], [4]]
    b, rej = plan_batches([10, 500, 0], sample_len=10, free_pages=4, free_slots=8, max_seq_len=1000)
    assert b == [[0]] and set(rej) == {1, 2}


def test_norm_handoff_is_only_claimed_by_the_norm_it_was_left_for():
    """The letterbox between the product that adds into the stream last and the norm that reads it next
    (parts.linear.NormHandoff): what was left is claimed once, by the expected norm's gamma on the same
    stream, and never by another."""
    import torch
    from burn_lm_b200.parts.linear import HandedNorm, NormHandoff

    class Norm:
        takes_handed_norm = True

        def __init__(self):
            self.gamma = torch.ones(4)

    class PlainNorm:
        def __init__(self):
            self.gamma = torch.ones(4)

    h = NormHandoff()
    a, b, plain = Norm(), Norm(), PlainNorm()
    stream, other = torch.zeros(2, 4), torch.zeros(2, 4)
    handed = HandedNorm(torch.zeros(2, 4), torch.zeros(1, 16))
    h.expect(plain)
    assert h.wanted is None                       # a norm that cannot take one is not expected
    h.expect(a)
    assert h.wanted is a
    h.leave(stream, a.gamma, handed)
    assert h.claim(stream, b.gamma) is None       # another norm: nothing, and what was left is gone
    assert h.claim(stream, a.gamma) is None
    h.expect(a)
    h.leave(stream, a.gamma, handed)
    assert h.claim(other, a.gamma) is None        # another stream
    h.expect(a)
    h.leave(stream, a.gamma, handed)
    assert h.claim(stream, a.gamma) is handed
    assert h.claim(stream, a.gamma) is None       # once
    h.expect(a)
    h.leave(stream, a.gamma, handed)
    h.expect(b)                                   # a new expectation forgets what was left for the old one
    assert h.claim(stream, a.gamma) is None


def test_prompt_step_buckets_hold_their_steps():
    """A prompt step's bucket is no smaller than the step in any size, close to it in tokens, and decode
    steps, long steps and steps with many wanted rows have none."""
    from burn_lm_b200.engine.prefill_graph import MAX_TOKENS, MAX_WANTED, bucket_of
    assert bucket_of(8, 8, 1, 8) is None                    # a decode step
    assert bucket_of(MAX_TOKENS + 1, 1, MAX_TOKENS + 1, 1) is None
    assert bucket_of(100, 1, 100, MAX_WANTED + 1) is None
    seen = set()
    for n_seqs in (1, 2, 3, 5, 8, 33):
        for longest in (2, 17, 64, 129, 700, 2048):
            for rest in (0, 1, 63, 500):
                n_tokens = longest + rest + (n_seqs - 1)
                if n_tokens > MAX_TOKENS:
                    continue
                for n_want in (0, 1, n_seqs):
                    t, s, q, w = bucket_of(n_tokens, n_seqs, longest, n_want)
                    assert n_tokens <= t < n_tokens * 1.25 + 64 and t % 16 == 0
                    assert n_seqs <= s < 2 * n_seqs and longest <= q <= t and q % 16 == 0
                    assert (w == 0) == (n_want == 0) and n_want <= w < max(2 * n_want, 1)
                    seen.add((t, s, q, w))
    assert len(seen) < 400


def test_include_stop_emits_the_stop_id_and_still_ends_there():
    """The reference counts the stop id and leaves it out of the answer (generation/context.rs:142-170); with
    include_stop it is the answer's last token, streamed like the others."""
    prompts = [[1, 2, 3], [4], [2, 2]]
    streamed = []
    eng = ScriptedEngine()
    out = GenerationLoop(eng, ArgmaxSampler(), default_stop_ids=(13,)).generate(
        prompts, GenerateOptions(sample_len=12, stop_ids=(29,), include_stop=True), on_token=lambda i, t: streamed.append((i, t)))
    seen_stop = False
    for i, (p, r) in enumerate(zip(prompts, out.results)):
        toks, why = expected(p, 12, stop=(13, 29))
        if why == "stop":
            seen_stop = True
            assert r.finish_reason == "stop" and r.tokens[:-1] == toks and r.tokens[-1] in (13, 29)
        else:
            assert r.tokens == toks
        assert [t for j, t in streamed if j == i] == r.tokens
    assert seen_stop
    assert out.stats.generated_tokens == sum(len(r.tokens) for r in out.results)
    assert eng.cache.slots.held_count == 0


class QuickEngine(ScriptedEngine):
    """The scripted engine with the short ways through a decode step that the real engine has: the loop then takes
    stretches of steps in which nobody can end without looking at single requests."""

    def __init__(self, fail_at=None, **kw):
        super().__init__(**kw)
        self.quick_calls, self.draws, self.fail_at = 0, [], fail_at

    def _quick(self, slots, tokens):
        from burn_lm_b200.engine.engine import StepEntry
        self.quick_calls += 1
        if self.fail_at is not None and self.quick_calls == self.fail_at:
            raise RuntimeError("the device fell over")
        return self.step([StepEntry(s, [t], [0]) for s, t in zip(slots, tokens)]).argmax(-1).tolist()

    def decode_greedy(self, slots, tokens, more=False):
        return self._quick(slots, tokens)

    def decode_sampled(self, slots, tokens, params, stream_ids, counters):
        self.draws.append((params, list(stream_ids), list(counters)))
        return self._quick(slots, tokens)


@pytest.mark.parametrize("temperature", [0.0, 0.7])
def test_stretches_of_quiet_steps_decide_what_single_steps_decide(temperature):
    """With an engine that samples inside its step, the loop runs the steps in which no request can reach its
    length or the context's end without looking at single requests, and hands the tokens out when the stretch
    ends.  Requests, finish reasons, counts and the numbering of the draws are those of the loop that looks at every
    token: over stop ids inside a stretch, unequal lengths, the context's end, batches after one another."""
    prompts = [[1, 2, 3], [4], [5, 6, 7, 8, 9, 10, 11], [2, 2], [9] * 30, [3, 1]]
    reasons = set()
    for kw in (dict(sample_len=12, stop_ids=(29,)), dict(sample_len=40, ignore_stop=True), dict(sample_len=1),
               dict(sample_len=2), dict(sample_len=25, stop_ids=(7, 31), include_stop=True), dict(sample_len=100, ignore_stop=True)):
        opts = GenerateOptions(temperature=temperature, seed=5, **kw)
        slow_eng, slow_smp = ScriptedEngine(max_seqs=3, max_seq_len=48), ArgmaxSampler()
        slow = GenerationLoop(slow_eng, slow_smp, default_stop_ids=(13,)).generate(prompts, opts)
        quick_eng = QuickEngine(max_seqs=3, max_seq_len=48)
        quick = GenerationLoop(quick_eng, ArgmaxSampler(), default_stop_ids=(13,)).generate(prompts, opts)
        assert [r.tokens for r in quick.results] == [r.tokens for r in slow.results], kw
        assert [r.finish_reason for r in quick.results] == [r.finish_reason for r in slow.results], kw
        reasons |= {r.finish_reason for r in slow.results}
        assert quick.stats.generated_tokens == slow.stats.generated_tokens and quick.stats.decode_steps == slow.stats.decode_steps
        assert quick_eng.steps == slow_eng.steps                 # the same steps with the same sequences
        assert quick_eng.cache.slots.held_count == 0
        if kw["sample_len"] > 2:
            assert quick_eng.quick_calls > 0
        if temperature > 0:
            # every draw carries its request's number and how many tokens the request has: as the sampler saw them
            assert quick_eng.draws == [c for c in slow_smp.calls if c[2] != [0] * len(c[2])], kw
    assert reasons == {"stop", "length", "context"}                # the script makes all three happen


def test_an_error_inside_a_stretch_keeps_the_tokens_so_far():
    eng = QuickEngine(fail_at=5)
    loop = GenerationLoop(eng, ArgmaxSampler())
    with pytest.raises(RuntimeError):
        loop.generate([[1, 2, 3], [4]], GenerateOptions(sample_len=30, ignore_stop=True))
    assert eng.cache.slots.held_count == 0


def test_streaming_looks_at_every_token():
    prompts = [[1, 2, 3], [4]]
    seen = []
    eng = QuickEngine()
    out = GenerationLoop(eng, ArgmaxSampler()).generate(prompts, GenerateOptions(sample_len=9, ignore_stop=True),
                                                         on_token=lambda i, t: seen.append((i, t)))
    for i, r in enumerate(out.results):
        assert [t for j, t in seen if j == i] == r.tokens == expected(prompts[i], 9)[0]


def test_quiet_stretches_on_requests_drawn_at_random():
    """Prompts, lengths, stop ids, context limits and batch sizes drawn at random (fixed seeds): the loop over an engine
    with the short ways gives, request by request, what the loop that looks at every token gives."""
    import random
    for case in range(60):
        rng = random.Random(case)
        prompts = [[rng.randrange(VOCAB) for _ in range(rng.choice([1, 2, 5, 17, 40]))] for _ in range(rng.randint(1, 7))]
        max_seq_len = rng.choice([24, 48, 64, 128])
        stops = tuple(rng.sample(range(VOCAB), rng.choice([0, 1, 3, 8])))
        opts = GenerateOptions(temperature=rng.choice([0.0, 0.5]), seed=1 + case, sample_len=rng.choice([1, 2, 3, 10, 50, 200]),
                               stop_ids=stops, ignore_stop=rng.random() < 0.2, include_stop=rng.random() < 0.3,
                               batch_size=rng.choice([None, 1, 2, 3]))
        kw = dict(max_tokens=64 * 8, max_seqs=rng.choice([1, 2, 4]), max_seq_len=max_seq_len)
        slow_eng = ScriptedEngine(**kw)
        slow = GenerationLoop(slow_eng, ArgmaxSampler(), default_stop_ids=(13,)).generate(prompts, opts)
        quick_eng = QuickEngine(**kw)
        quick = GenerationLoop(quick_eng, ArgmaxSampler(), default_stop_ids=(13,)).generate(prompts, opts)
        what = (case, opts, [len(p) for p in prompts], kw)
        assert [r.tokens for r in quick.results] == [r.tokens for r in slow.results], what
        assert [r.finish_reason for r in quick.results] == [r.finish_reason for r in slow.results], what
        assert [type(r.error) for r in quick.results] == [type(r.error) for r in slow.results], what
        assert (quick.stats.generated_tokens, quick.stats.decode_steps, quick.stats.batches) == \
               (slow.stats.generated_tokens, slow.stats.decode_steps, slow.stats.batches), what
        assert quick_eng.steps == slow_eng.steps, what
        assert quick_eng.cache.slots.held_count == 0 and quick_eng.cache.free_pages == quick_eng.cache.n_pages
