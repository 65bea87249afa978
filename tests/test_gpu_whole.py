"""The engine against the plain implementation: each request alone and whole, in 32-bit and in
bfloat16, on tiny random models."""
import numpy as np
import pytest

from plain import llama_plain as P
from tiny import CONFIGS, make_folder, random_tokens, row_error

pytestmark = pytest.mark.gpu

# largest error of a logits row relative to the row's largest logit
FP32_TOL = 1e-4
BF16_TOL = 3e-2


def engine_for(folder, dtype, max_tokens=2048):
    from burn_lm_b200 import Engine
    return Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens)


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype,stored,tolerance", [("float32", "float32", FP32_TOL), ("float32", "bfloat16", FP32_TOL),
                                                    ("bfloat16", "bfloat16", BF16_TOL)])
def test_whole_prompts(tmp_path, name, dtype, stored, tolerance):
    from burn_lm_b200 import StepEntry
    folder = make_folder(tmp_path, name, seed=3, dtype=stored)
    cfg, tensors = P.read_model_folder(folder)
    eng = engine_for(folder, dtype)
    for n, length in enumerate([1, 5, 64, 65, 100]):
        if length > cfg["max_position_embeddings"]:
            continue
        toks = random_tokens(10 + n, length, cfg["vocab_size"])
        slot = eng.acquire()
        got = eng.step([StepEntry(slot, toks, list(range(length)))]).cpu().numpy()
        eng.release(slot)
        want = P.forward(cfg, tensors, toks)
        err = row_error(got, want)
        assert err.max() < tolerance, (name, dtype, length, err.max(), int(err.argmax()))


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("few", [None, [[5, 2, 7], [1, 9, 4], [6, 6, 3], [2, 1, 3, 8]]], ids=["dozens", "few"])
@pytest.mark.parametrize("dtype,tolerance", [("float32", FP32_TOL), ("bfloat16", BF16_TOL)])
def test_prompt_steps_of_one_bucket_plain_captured_and_replayed(tmp_path, name, dtype, tolerance, few):
    """Prompt steps are fitted into buckets of sizes and replayed as CUDA graphs from a bucket's second use.
    Batches of different prompts that fall into one bucket: the first runs plainly, the second is captured,
    the third replayed (`few`: steps of at most 16 tokens, which keep the kernels made for a few tokens);
    each against the plain implementation, then the same batch again (replayed) to the
    same bits; and the cache they leave gives the right next token's logits."""
    from burn_lm_b200 import StepEntry
    from burn_lm_b200.engine.prefill_graph import bucket_of
    folder = make_folder(tmp_path, name, seed=5, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    eng = engine_for(folder, dtype)
    assert eng.use_graphs
    limit = cfg["max_position_embeddings"]
    batches = few or [[33, 7, 20], [5, 40, 9], [17, 3, 38], [6, 36, 2, 11]]
    batches = [[min(n, limit - 2) for n in b] for b in batches]
    assert len({bucket_of(sum(b), len(b), max(b), len(b)) for b in batches}) == 1
    first = None
    for rep, lens in enumerate(batches + [batches[0]]):
        prompts = [random_tokens(100 * (rep % len(batches)) + i, n, cfg["vocab_size"]) for i, n in enumerate(lens)]
        slots = [eng.acquire() for _ in prompts]
        got = eng.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]).cpu().numpy()
        for i, p in enumerate(prompts):
            want = P.forward(cfg, tensors, p)[-1:]
            assert row_error(got[i:i + 1], want).max() < tolerance, (rep, i)
        if rep == 0:
            first = got
        if rep == len(batches):
            assert np.array_equal(got, first)       # plain launches and the replayed graph: the same bits
        # one more token each: the cache the step left is the right one
        nxt = [int(np.argmax(got[i])) for i in range(len(prompts))]
        dec = eng.step([StepEntry(s, [t], [0]) for s, t in zip(slots, nxt)]).cpu().numpy()
        for i, p in enumerate(prompts):
            want = P.forward(cfg, tensors, p + [nxt[i]])[-1:]
            assert row_error(dec[i:i + 1], want).max() < tolerance, (rep, i, "decode")
        for s in slots:
            eng.release(s)
    g = eng._prefill_graphs.get(bucket_of(sum(batches[0]), 3, max(batches[0]), 3))
    assert g.steps == len(batches) + 1 and g._graph is not None
    eng.verify()


def test_prompt_step_buckets_are_dropped_and_come_back(tmp_path, monkeypatch):
    """Only the most recently used buckets keep their graph; a bucket that was dropped starts over
    (plain, then captured) and still gives the right logits."""
    from burn_lm_b200 import StepEntry
    from burn_lm_b200.engine import prefill_graph
    monkeypatch.setattr(prefill_graph, "MAX_GRAPHS", 2)
    folder = make_folder(tmp_path, "tiny_d", seed=6, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    eng = engine_for(folder, "bfloat16", max_tokens=4096)
    lengths = [40, 100, 150, 300, 40, 100, 40, 40, 300, 300, 300]
    for n, length in enumerate(lengths):
        toks = random_tokens(50 + n, length, cfg["vocab_size"])
        slot = eng.acquire()
        got = eng.step([StepEntry(slot, toks, [length - 1])]).cpu().numpy()
        eng.release(slot)
        want = P.forward(cfg, tensors, toks)[-1:]
        assert row_error(got, want).max() < BF16_TOL, (n, length)
        assert len(eng._prefill_graphs) <= 2
    eng.verify()


def test_a_step_of_more_than_a_thousand_tokens(tmp_path):
    """From 1,024 tokens in a step the gated product runs the tcgen05 kernel with the activation in its
    epilogue, and the prompts' attention the tcgen05 kernel: two prompts of 600 tokens in one step."""
    from burn_lm_b200 import StepEntry
    from burn_lm_b200.parts.linear import TENSOR_CORE_TOKENS
    folder = make_folder(tmp_path, "tiny_d", seed=8, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    eng = engine_for(folder, "bfloat16", max_tokens=4096)
    prompts = [random_tokens(70 + n, 600, cfg["vocab_size"]) for n in range(2)]
    assert sum(len(p) for p in prompts) >= TENSOR_CORE_TOKENS
    want_at = [0, 63, 64, 300, 599]
    for rep in range(3):        # plain, captured, replayed
        slots = [eng.acquire() for _ in prompts]
        got = eng.step([StepEntry(s, p, want_at) for s, p in zip(slots, prompts)]).cpu().numpy()
        for s in slots:
            eng.release(s)
        for i, p in enumerate(prompts):
            want = P.forward(cfg, tensors, p)[want_at]
            err = row_error(got[i * len(want_at):(i + 1) * len(want_at)], want)
            assert err.max() < BF16_TOL, (rep, i, err)
    eng.verify()


def test_every_prompt_product_on_the_tcgen05_kernel(tmp_path, monkeypatch):
    """With the switch that sends the plain prompt products (qkv, output, down) to this package's tcgen05
    kernel as well (output and down with the epilogue that adds into the fp32 stream), a step of 300 tokens
    agrees with the plain implementation, and the kernel did run."""
    from burn_lm_b200 import StepEntry, kernels
    from burn_lm_b200.parts import linear
    monkeypatch.setattr(linear, "OWN_PRODUCTS", True)
    calls = []
    real = kernels.gemm_tc
    monkeypatch.setattr(kernels, "gemm_tc", lambda *a, **k: (calls.append((a[1].shape, "add_into" in k)), real(*a, **k))[1])
    folder = make_folder(tmp_path, "tiny_e", seed=9, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    eng = engine_for(folder, "bfloat16", max_tokens=1024)
    toks = random_tokens(80, 300, cfg["vocab_size"])
    slot = eng.acquire()
    want_at = [0, 100, 299]
    got = eng.step([StepEntry(slot, toks, want_at)]).cpu().numpy()
    want = P.forward(cfg, tensors, toks)[want_at]
    assert row_error(got, want).max() < BF16_TOL
    assert len(calls) >= 3 * cfg["num_hidden_layers"]
    assert sum(1 for _, adds in calls if adds) == 2 * cfg["num_hidden_layers"]      # output and down add into the stream themselves
    eng.verify()


@pytest.mark.parametrize("name", ["tiny_b", "tiny_d", "tiny_e"])
@pytest.mark.parametrize("dtype,tolerance", [("float32", FP32_TOL), ("bfloat16", BF16_TOL)])
def test_steps_that_hold_decoding_sequences_beside_fresh_prompts(tmp_path, name, dtype, tolerance):
    """`Engine.step` takes any mix: a sequence that goes on by one token beside a prompt that starts, and a
    prompt that goes on by several tokens.  The same mix three times with other tokens (the steps fall into
    prompt buckets: launched plainly, captured, replayed), each against the plain implementation."""
    from burn_lm_b200 import StepEntry
    folder = make_folder(tmp_path, name, seed=11, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    eng = engine_for(folder, dtype)
    vocab = cfg["vocab_size"]
    for rep in range(3):
        a = random_tokens(300 + rep, 70 + 3, vocab)
        b = random_tokens(400 + rep, 40 + 2, vocab)
        c = random_tokens(500 + rep, 33 + 5, vocab)
        sa, sb, sc = eng.acquire(), eng.acquire(), eng.acquire()
        got = {"a": [], "b": [], "c": []}

        def run(entries):
            """entries: (name, slot, tokens); logits are wanted everywhere."""
            out = eng.step([StepEntry(slot, toks, list(range(len(toks)))) for _, slot, toks in entries]).cpu().numpy()
            row = 0
            for who, _, toks in entries:
                got[who].extend(out[row: row + len(toks)])
                row += len(toks)

        run([("a", sa, a[:70])])
        run([("a", sa, a[70:71]), ("b", sb, b[:40])])                            # decoding beside a fresh prompt
        run([("c", sc, c[:33]), ("a", sa, a[71:72]), ("b", sb, b[40:41])])       # the fresh prompt first, two decoding
        run([("b", sb, b[41:42]), ("c", sc, c[33:38]), ("a", sa, a[72:73])])     # a prompt that goes on by five tokens
        for who, toks in (("a", a), ("b", b), ("c", c)):
            err = row_error(np.stack(got[who]), P.forward(cfg, tensors, toks))
            assert err.max() < tolerance, (rep, who, float(err.max()), "first bad place", int(np.argmax(err >= tolerance)))
        for s in (sa, sb, sc):
            eng.release(s)
    eng.verify()
