"""Generation through the Python entry point, sampling kernels against the plain sampler, long
decoding, and the first tokens of a sequence."""
import math

import numpy as np
import pytest
import torch

import traces
from plain import llama_plain as P
from tiny import CONFIGS, make_folder, random_tokens, row_error

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_greedy_generation_float32_matches_plain(tmp_path, name):
    import burn_lm_b200 as blm
    folder = make_folder(tmp_path, name, seed=8, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    lm = blm.load(folder, dtype="float32", max_seq_len=128, max_batch=3)
    prompts = [random_tokens(20 + n, length, cfg["vocab_size"]) for n, length in enumerate([5, 11, 17, 1, 30])]
    out = lm.generate(prompts, sample_len=8, batch_size=3, ignore_stop=True)
    assert out.stats.batches == 2
    for p, r in zip(prompts, out.results):
        assert r.tokens == P.greedy_generate(cfg, tensors, p, 8) and r.finish_reason == "length"
    assert lm.engine.cache.slots.held_count == 0 and lm.engine.cache.free_pages == lm.engine.cache.n_pages
    # stop ids end a sequence and are not part of the answer
    stop = out.results[1].tokens[3]
    out2 = lm.generate(prompts[:3], sample_len=8, stop_ids=[stop], ignore_stop=False)
    want = P.greedy_generate(cfg, tensors, prompts[1], 8, stop_ids=set(cfg.get("eos_token_id", [])) | {stop})
    assert out2.results[1].tokens == want and out2.results[1].finish_reason == "stop"


def test_greedy_generation_bfloat16_follows_plain_up_to_near_ties(tmp_path):
    import burn_lm_b200 as blm
    folder = make_folder(tmp_path, "tiny_b", seed=9, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    lm = blm.load(folder, dtype="bfloat16", max_seq_len=256, max_batch=4)
    prompts = [random_tokens(40 + n, length, cfg["vocab_size"]) for n, length in enumerate([1, 7, 30, 64])]
    out = lm.generate(prompts, sample_len=16, ignore_stop=True)
    agree = 0
    for p, r in zip(prompts, out.results):
        seq = list(p)
        for tok in r.tokens:
            logits = P.forward(cfg, tensors, seq)[-1]
            best = int(np.argmax(logits))
            if tok != best:      # allowed only where the plain logits nearly tie
                assert logits[best] - logits[tok] < 3e-2 * np.abs(logits).max(), (len(seq), tok, best)
                break
            agree += 1
            seq.append(tok)
    assert agree >= 48       # of 64: ties are rare


def test_sampling_matches_plain_on_the_same_logits():
    from burn_lm_b200 import kernels as K
    from burn_lm_b200.sampling import Sampler, SamplingParams
    g = torch.Generator(device="cuda").manual_seed(0)
    B, V = 64, 1531
    logits = 3.0 * torch.randn(B, V, device="cuda", generator=g)
    smp = Sampler("cuda")
    for temperature, top_p in [(0.8, 0.9), (1.3, 0.5), (0.6, 1.0), (1.0, 0.05)]:
        params = SamplingParams(temperature, top_p, seed=1234)
        streams, counters = list(range(100, 100 + B)), [b % 7 for b in range(B)]
        got = smp.sample(logits, params, streams, counters)
        same = 0
        for b in range(B):
            probs = P.temperature_softmax(logits[b].cpu().numpy(), temperature)
            u = K.uniform32(1234, streams[b], counters[b]) / 2.0 ** 32
            keep = P.top_p_keep(probs, top_p)
            # the boundary of the nucleus may differ by a token or two between fp32 and fp64
            assert keep[got[b]] or probs[got[b]] >= probs[keep].min() * 0.999
            same += int(got[b] == P.top_p_draw(probs, top_p, u))
        assert same >= B - 2, (temperature, top_p, same)
        # a draw is a function of (seed, stream, counter), not of the row or the batch
        perm = torch.randperm(B).tolist()
        again = smp.sample(logits[perm].contiguous(), params, [streams[i] for i in perm], [counters[i] for i in perm])
        assert again == [got[i] for i in perm]
        alone = smp.sample(logits[5:6].contiguous(), params, streams[5:6], counters[5:6])
        assert alone == got[5:6]
    assert smp.sample(logits, SamplingParams(0.0), [0] * B, [0] * B) == logits.argmax(-1).tolist()


@pytest.mark.parametrize("vocab", [5000, 20000, 128256])
def test_a_draw_does_not_depend_on_how_many_blocks_share_a_row(vocab):
    """A row of a large vocabulary is shared by the blocks of a cluster, fewer of them when there are many
    rows: a row sampled alone, among 20 and among 90 rows draws the same token, and the plain draw's."""
    from burn_lm_b200 import kernels as K
    from burn_lm_b200.sampling import Sampler, SamplingParams
    g = torch.Generator(device="cuda").manual_seed(vocab)
    B = 90
    logits = 2.5 * torch.randn(B, vocab, device="cuda", generator=g)
    smp = Sampler("cuda")
    for temperature, top_p in [(0.8, 0.9), (1.2, 1.0), (0.7, 0.3)]:
        params = SamplingParams(temperature, top_p, seed=99)
        streams, counters = list(range(B)), [3 * b for b in range(B)]
        many = smp.sample(logits, params, streams, counters)
        some = smp.sample(logits[:20].contiguous(), params, streams[:20], counters[:20])
        assert some == many[:20]
        for b in (0, 7, 19, 55, 89):
            alone = smp.sample(logits[b:b + 1].contiguous(), params, streams[b:b + 1], counters[b:b + 1])
            assert alone == many[b:b + 1], (vocab, temperature, top_p, b)
        same = 0
        for b in range(0, B, 9):
            probs = P.temperature_softmax(logits[b].cpu().numpy(), temperature)
            u = K.uniform32(99, streams[b], counters[b]) / 2.0 ** 32
            same += int(many[b] == P.top_p_draw(probs, top_p, u))
        assert same >= 9, (vocab, temperature, top_p, same)


def test_sampling_nucleus_far_below_the_largest_probability():
    """One token holds half of the mass and a large vocabulary shares the rest in crumbs 2^-17 of it and
    smaller: the nucleus reaches far below the sixteen exponents under the largest probability that the
    kernel sums in registers, so its general histogram has to find the threshold.  Against the plain
    nucleus: the drawn token is kept, and it is the one (up to fp32 rounding of four hundred thousand
    terms) at which the running kept mass passes u times the kept mass."""
    from burn_lm_b200 import kernels as K
    from burn_lm_b200.sampling import Sampler, SamplingParams
    g = torch.Generator(device="cuda").manual_seed(3)
    B, V = 12, 400000
    logits = 0.1 * torch.randn(B, V, device="cuda", generator=g)
    logits[:, 77] = math.log(V) + 0.05                      # about half of the mass
    smp = Sampler("cuda")
    for top_p in (0.9, 0.6):
        params = SamplingParams(1.0, top_p, seed=99)
        streams, counters = list(range(B)), [3 * b for b in range(B)]
        got = smp.sample(logits, params, streams, counters)
        crumbs = 0
        for b in range(B):
            probs = P.temperature_softmax(logits[b].cpu().numpy(), 1.0)
            assert probs[77] > 0.4 and np.sort(probs)[-2] < probs[77] * 2.0 ** -16
            keep = P.top_p_keep(probs, top_p)
            assert abs(np.where(keep, probs, 0.0).sum() - top_p) < 1e-4          # the nucleus ends among the crumbs
            assert keep[got[b]] or probs[got[b]] >= probs[keep].min() * 0.999
            kept = np.where(keep, probs, 0.0)
            run = np.cumsum(kept)
            target = K.uniform32(99, streams[b], counters[b]) / 2.0 ** 32 * run[-1]
            tol = 2e-5 * run[-1]
            assert run[got[b]] - kept[got[b]] - tol <= target < run[got[b]] + tol, (top_p, b, got[b])
            crumbs += int(got[b] != 77)
        if top_p == 0.9:
            assert crumbs >= 2                                  # some draws do land among the crumbs
    K.check_status("cuda")


def test_sampling_frequencies_follow_the_nucleus():
    from burn_lm_b200.sampling import Sampler, SamplingParams
    logits = torch.tensor([[2.0, 1.0, 0.5, 0.0, -1.0, -2.0, 1.5, -8.0]], device="cuda")
    n = 4000
    rows = logits.repeat(n, 1).contiguous()
    got = Sampler("cuda").sample(rows, SamplingParams(0.7, 0.8, seed=5), [3] * n, list(range(n)))
    probs = P.temperature_softmax(logits[0].cpu().numpy(), 0.7)
    keep = P.top_p_keep(probs, 0.8)
    want = np.where(keep, probs, 0.0)
    want /= want.sum()
    freq = np.bincount(got, minlength=8) / n
    assert (freq[~keep] == 0).all()
    assert np.abs(freq - want).max() < 4 * np.sqrt(0.25 / n)


def test_temperature_generation_is_seeded_and_batch_independent(tmp_path):
    import burn_lm_b200 as blm
    folder = make_folder(tmp_path, "tiny_b", seed=10, dtype="bfloat16")
    lm = blm.load(folder, dtype="float32", max_seq_len=256, max_batch=4)
    cfg = CONFIGS["tiny_b"]
    prompts = [random_tokens(60 + n, length, cfg["vocab_size"]) for n, length in enumerate([1, 7, 30, 64])]
    a = lm.generate(prompts, sample_len=16, temperature=0.8, seed=42, ignore_stop=True).tokens
    b = lm.generate(prompts, sample_len=16, temperature=0.8, seed=42, ignore_stop=True).tokens
    c = lm.generate(prompts, sample_len=16, temperature=0.8, seed=43, ignore_stop=True).tokens
    assert a == b and a != c
    one_by_one = lm.generate(prompts, sample_len=16, temperature=0.8, seed=42, ignore_stop=True, batch_size=1).tokens
    assert one_by_one[0] == a[0]            # request 0 draws the same alone as in the batch


def test_long_decoding(tmp_path):
    """600 tokens one by one after a short prompt: positions cross many pages and the scaled rotary
    frequencies turn many times."""
    from burn_lm_b200 import Engine
    folder = make_folder(tmp_path, "tiny_c", seed=11, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    reqs = {"long": random_tokens(70, 610, cfg["vocab_size"])}
    want = P.forward(cfg, tensors, reqs["long"])
    for dtype, tolerance in (("float32", 1e-4), ("bfloat16", 3e-2)):
        steps = traces.tail(reqs, 600)
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=traces.max_live_tokens(steps))
        got = traces.run_in_process(eng, steps, str(tmp_path / dtype), cfg["vocab_size"])
        err = row_error(got["long"], want)
        assert err.max() < tolerance, (dtype, float(err.max()), int(err.argmax()))


@pytest.mark.parametrize("dtype,tolerance", [("float32", 1e-4), ("bfloat16", 3e-2)])
def test_first_tokens_of_a_sequence(tmp_path, dtype, tolerance):
    """Prompts of one, two and three tokens, then single tokens from the very first position."""
    from burn_lm_b200 import Engine
    folder = make_folder(tmp_path, "tiny_a", seed=12, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    reqs = {f"f{n}": random_tokens(80 + n, n + 1 + 6, cfg["vocab_size"]) for n in range(3)}
    steps = traces.batched(reqs, 3, [6, 6, 6])      # prompts of 1, 2, 3 tokens, then 6 single tokens each
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=traces.max_live_tokens(steps))
    got = traces.run_in_process(eng, steps, str(tmp_path / "o"), cfg["vocab_size"])
    for rid, toks in reqs.items():
        err = row_error(got[rid], P.forward(cfg, tensors, toks))
        assert err.max() < tolerance, (rid, float(err.max()))


@pytest.mark.parametrize("name,dtype,sharpen,tolerance", [("tiny_c", "float32", 12.0, 1e-4), ("tiny_d", "float32", 12.0, 1e-4),
                                                          ("tiny_d", "bfloat16", 5.0, 3e-2)])
def test_a_far_key_decides_the_logits(tmp_path, name, dtype, sharpen, tolerance):
    """Random weights make attention nearly uniform, which would hide a lost key.  Here the
    layers' query and key projections are scaled up so that scores are sharp, on a sequence long
    enough that the keys that matter lie pages away; batched and token-by-token replays must still
    agree with the plain implementation.  In bfloat16 (head size 64: the tensor-core prompt kernels and the
    specialised decode kernel) the weights are stored in bfloat16 after the scaling, so both sides read the
    same numbers."""
    from burn_lm_b200 import Engine
    from burn_lm_b200.weights import SafetensorsFile, write_safetensors
    import os
    import torch
    folder = make_folder(tmp_path, name, seed=13, dtype="float32")
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.get(n).clone() for n in f.names()}
    f.close()
    plain_cfg, plain_t = P.read_model_folder(folder)
    for n in range(2):
        tensors[f"model.layers.{n}.self_attn.q_proj.weight"] *= sharpen
        tensors[f"model.layers.{n}.self_attn.k_proj.weight"] *= sharpen
        tensors[f"model.layers.{n}.self_attn.v_proj.weight"] *= 6.0
        tensors[f"model.layers.{n}.self_attn.o_proj.weight"] *= 6.0
    if dtype == "bfloat16":
        tensors = {n: t.to(torch.bfloat16) for n, t in tensors.items()}
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    cfg, t = P.read_model_folder(folder)
    reqs = {"a": random_tokens(90, 500, cfg["vocab_size"]), "b": random_tokens(91, 200, cfg["vocab_size"]),
            "c": random_tokens(92, 333, cfg["vocab_size"])}
    want = {rid: P.forward(cfg, t, toks) for rid, toks in reqs.items()}
    # the sharpened attention really is far from uniform: logits differ a lot from the unscaled model's
    assert row_error(P.forward(plain_cfg, plain_t, reqs["a"]), want["a"]).max() > 0.3
    for what, steps in (("batched", traces.batched(reqs, 3, [32, 7, 19])), ("tail", traces.tail(reqs, 32))):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=traces.max_live_tokens(steps))
        got = traces.run_in_process(eng, steps, str(tmp_path / what), cfg["vocab_size"])
        for rid in reqs:
            err = row_error(got[rid], want[rid])
            assert err.max() < tolerance, (what, rid, float(err.max()), int(err.argmax()))


def test_repeated_runs_and_captured_steps_give_the_same_tokens(tmp_path):
    """Kernels of a decode step start before the kernel before them has ended (programmatic dependent
    launch): a missing wait would show as tokens that change from run to run, or between the captured
    graph and the same step launched plainly."""
    import burn_lm_b200 as blm
    folder = make_folder(tmp_path, "tiny_c", seed=21, dtype="bfloat16")
    cfg = CONFIGS["tiny_c"]
    lm = blm.load(folder, dtype="bfloat16", max_seq_len=512, max_batch=8)
    prompts = [random_tokens(90 + n, length, cfg["vocab_size"]) for n, length in enumerate([3, 70, 64, 129, 17, 200, 1, 33])]
    runs = [lm.generate(prompts, sample_len=150, ignore_stop=True).tokens for _ in range(3)]
    assert runs[0] == runs[1] == runs[2]
    lm.engine.use_graphs = False
    plain = lm.generate(prompts, sample_len=150, ignore_stop=True).tokens
    lm.engine.use_graphs = True
    assert plain == runs[0]
    sampled = [lm.generate(prompts, sample_len=40, ignore_stop=True, temperature=0.9, seed=8).tokens for _ in range(2)]
    assert sampled[0] == sampled[1]
    lm.engine.verify()


def test_tokens_reach_the_host_by_polling_or_by_copy(tmp_path, monkeypatch):
    """A captured step that samples writes its tokens into pinned memory itself and the native step driver polls for
    them; with that switched off they are copied out and the stream is waited for.  Greedy and drawn tokens are the
    same both ways, over batches that shrink and slots used again; the greedy ones also equal the steps launched
    plainly (a draw may fall on the other side of a boundary when another split of the keys rounds a logit differently)."""
    import burn_lm_b200 as blm
    from burn_lm_b200.engine import decode_graph
    folder = make_folder(tmp_path, "tiny_d", seed=27, dtype="bfloat16")
    cfg = CONFIGS["tiny_d"]
    prompts = [random_tokens(500 + n, length, cfg["vocab_size"]) for n, length in enumerate([9, 70, 33, 128, 1, 64])]

    def run(polling, graphs=True):
        monkeypatch.setattr(decode_graph, "RESULTS_BY_POLLING", polling)
        lm = blm.load(folder, dtype="bfloat16", max_seq_len=256, max_batch=4)
        lm.engine.use_graphs = graphs
        greedy = lm.generate(prompts, sample_len=60, ignore_stop=True).tokens
        drawn = lm.generate(prompts, sample_len=60, ignore_stop=True, temperature=0.8, top_p=0.9, seed=3).tokens
        lm.engine.verify()
        return greedy, drawn

    polled = run(True)
    assert polled == run(False)
    assert polled[0] == run(True, graphs=False)[0]


def test_decode_graphs_are_dropped_and_made_again(tmp_path):
    """The engine keeps a bounded number of captured decode steps; with room for two only, requests that
    alternate between batch sizes and grow through several length buckets generate the same tokens."""
    import burn_lm_b200 as blm
    folder = make_folder(tmp_path, "tiny_d", seed=23, dtype="bfloat16")
    cfg = CONFIGS["tiny_d"]
    prompts = [random_tokens(40 + n, length, cfg["vocab_size"]) for n, length in enumerate([5, 60, 31, 90, 12])]
    lens = [10, 50, 20, 40, 30]

    def run(limit):
        lm = blm.load(folder, dtype="bfloat16", max_seq_len=256, max_batch=8)
        if limit:
            lm.engine.max_decode_graphs = limit
        out = []
        for _ in range(2):
            res = [lm.generate([p], sample_len=n, ignore_stop=True).tokens[0] for p, n in zip(prompts, lens)]
            together = lm.generate(prompts, sample_len=max(lens), ignore_stop=True).tokens
            out.append((res, together))
        assert len(lm.engine._decode_graphs) <= (limit or lm.engine.max_decode_graphs)
        lm.engine.verify()
        return out

    assert run(2) == run(None)


def test_decode_ahead_gives_the_same_tokens(tmp_path):
    """With `decode_ahead` greedy generation enqueues a step before the one before it has been looked at.
    Requests that end at different steps (length limits, stop ids that do turn up) leave a step in flight
    that still holds the others' next tokens; batches follow one another on reused slots; a context limit
    and page boundaries are crossed.  All of it must give the tokens of the plain loop."""
    import burn_lm_b200 as blm
    folder = make_folder(tmp_path, "tiny_d", seed=29, dtype="bfloat16")
    cfg = CONFIGS["tiny_d"]
    prompts = [random_tokens(300 + n, length, cfg["vocab_size"]) for n, length in enumerate([5, 60, 31, 90, 12, 64, 63, 1, 200, 17])]

    def run(ahead):
        lm = blm.load(folder, dtype="bfloat16", max_seq_len=256, max_batch=4, decode_ahead=ahead)
        out = []
        out.append(lm.generate(prompts, sample_len=70, ignore_stop=True).tokens)
        # stop ids that occur in what the model says: requests end where nobody could foresee it
        said = [t for seq in out[0] for t in seq]
        stops = sorted(set(said[5::7]))[:12]
        res = lm.generate(prompts, sample_len=70, stop_ids=stops)
        out.append((res.tokens, [r.finish_reason for r in res.results]))
        out.append(lm.generate(prompts[:3], sample_len=300, ignore_stop=True).tokens)     # runs into the context limit
        one = [lm.generate([p], sample_len=n, ignore_stop=True).tokens[0] for p, n in zip(prompts[:4], [1, 2, 3, 40])]
        out.append(one)
        lm.engine.verify()
        assert lm.engine.cache.slots.free_count == 4
        return out

    plain, ahead = run(False), run(True)
    assert plain == ahead
    assert any(reason == "stop" for reason in plain[1][1])


def test_the_short_ways_through_a_decode_step_check_their_slots(tmp_path):
    """decode_greedy and decode_sampled refuse what step() refuses: a slot named twice, a slot that is not held
    (its block-table row is stale and its pages may be someone else's by now), a token outside the vocabulary,
    and a step of more tokens than the engine was built for; nothing is launched and nothing changes."""
    from burn_lm_b200 import Engine, StepEntry
    from burn_lm_b200.cache import CacheError
    from burn_lm_b200.sampling import SamplingParams
    folder = make_folder(tmp_path, "tiny_d", seed=31, dtype="bfloat16")
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=1024, max_seqs=4)
    a, b = eng.acquire(), eng.acquire()
    eng.step([StepEntry(a, [1, 2, 3], [2]), StepEntry(b, [4, 5], [1])])
    lengths = (eng.length(a), eng.length(b))
    with pytest.raises(ValueError, match="twice"):
        eng.decode_greedy([a, a], [1, 2])
    with pytest.raises(CacheError, match="not held"):
        eng.decode_greedy([a, 3], [1, 2])
    with pytest.raises(ValueError, match="vocabulary"):
        eng.decode_greedy([a, b], [1, 515])
    params = SamplingParams(0.7, 0.9, 5)
    with pytest.raises(ValueError, match="twice"):
        eng.decode_sampled([b, b], [1, 2], params, [0, 1], [0, 0])
    eng.release(b)
    with pytest.raises(CacheError, match="not held"):
        eng.decode_sampled([a, b], [1, 2], params, [0, 1], [0, 0])
    assert (eng.length(a), eng.length(b)) == (lengths[0], 0)
    assert len(eng.decode_greedy([a], [7])) == 1 and eng.length(a) == lengths[0] + 1
    small = Engine.from_folder(folder, dtype="bfloat16", max_tokens=1024, max_seqs=2, max_step_tokens=100)
    s = small.acquire()
    with pytest.raises(ValueError, match="at most 100"):
        small.step([StepEntry(s, [1] * 101, [])])
    assert small.length(s) == 0
    small.step([StepEntry(s, [1] * 100, [])])
    assert small.length(s) == 100


@pytest.mark.parametrize("max_seq_len", [1000, 200])
def test_a_context_limit_that_is_no_multiple_of_a_page(tmp_path, max_seq_len):
    """With a limit of 1,000 (or 200) tokens the longest length bucket of the captured decode steps ends beyond
    the limit, at the end of the last page; generation runs up to the limit on the kernels it always uses
    (the rotary table reaches as far as the bucket) and gives the plain implementation's tokens."""
    import burn_lm_b200 as blm
    folder = make_folder(tmp_path, "tiny_d", seed=33, dtype="float32")
    cfg, tensors = P.read_model_folder(folder)
    lm = blm.load(folder, dtype="float32", max_seq_len=max_seq_len, max_batch=2)
    prompt = random_tokens(3, max_seq_len - 40, cfg["vocab_size"])
    out = lm.generate([prompt], sample_len=100, ignore_stop=True)
    r = out.results[0]
    assert r.finish_reason == "context" and len(prompt) + len(r.tokens) == max_seq_len + 1
    assert r.tokens[:12] == P.greedy_generate(cfg, tensors, prompt, 12)
    lm16 = blm.load(folder, dtype="bfloat16", max_seq_len=max_seq_len, max_batch=2)
    from burn_lm_b200.parts.attention import Attention
    mixer = [p for p in lm16.engine.model.parts() if isinstance(p, Attention)][0]
    assert mixer.position.table().shape[0] >= -(-max_seq_len // 64) * 64
    r16 = lm16.generate([prompt], sample_len=100, ignore_stop=True).results[0]
    assert r16.finish_reason == "context" and len(r16.tokens) == len(r.tokens)
    lm16.engine.verify()
