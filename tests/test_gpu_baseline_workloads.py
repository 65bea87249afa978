"""The two tiny benchmark workloads, literally, and the 1B shape cut down to two layers.

Tiny A: batch of 3 prompts of lengths 5, 11, 17, one prefill step, 8 greedy decode steps, logits at
all positions against the plain implementation.  Tiny B: batch of 4 prompts of lengths 1, 7, 30, 64,
prefill, 16 decode steps at temperature 0.8 with a fixed sampling seed; then the generated tokens are
replayed one by one and compared with whole-prompt logits.  1B shape: the real widths, head size,
groups and vocabulary (so the kernels take the paths they take in production) with two layers.
"""
import numpy as np
import pytest
import torch

import traces
from plain import llama_plain as P
from tiny import TINY_A, TINY_B, make_folder, random_tokens, row_error

pytestmark = pytest.mark.gpu


def test_tiny_a_prefill_and_eight_greedy_steps(tmp_path):
    from burn_lm_b200 import Engine, StepEntry
    from burn_lm_b200 import kernels as K
    folder = make_folder(tmp_path, "tiny_a", seed=0, dtype="float32")
    cfg, tensors = P.read_model_folder(folder)
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=3 * 64)
    prompts = [random_tokens(n, length, 256) for n, length in enumerate([5, 11, 17])]
    slots = [eng.acquire() for _ in prompts]
    got = [[] for _ in prompts]
    logits = eng.step([StepEntry(s, p, list(range(len(p)))) for s, p in zip(slots, prompts)]).cpu().numpy()
    row = 0
    for i, p in enumerate(prompts):
        got[i].extend(logits[row:row + len(p)])
        row += len(p)
    seqs = [list(p) for p in prompts]
    for _ in range(8):
        nxt = [int(np.argmax(g[-1])) for g in got]
        for s, t in zip(seqs, nxt):
            s.append(t)
        logits = eng.step([StepEntry(s, [t], [0]) for s, t in zip(slots, nxt)]).cpu().numpy()
        for i in range(3):
            got[i].append(logits[i])
    for i, s in enumerate(seqs):
        want = P.forward(cfg, tensors, s[:-1] + [s[-1]])[: len(got[i])]
        assert row_error(np.stack(got[i]), want).max() < 1e-4
        assert s[len(prompts[i]):] == P.greedy_generate(cfg, tensors, prompts[i], 8)
    eng.verify()


def test_tiny_b_sampled_generation_then_replay(tmp_path):
    import burn_lm_b200 as blm
    from burn_lm_b200 import Engine
    folder = make_folder(tmp_path, "tiny_b", seed=0, dtype="float32")
    cfg, tensors = P.read_model_folder(folder)
    lm = blm.load(folder, dtype="float32", max_seq_len=256, max_batch=4)
    prompts = [random_tokens(10 + n, length, 384) for n, length in enumerate([1, 7, 30, 64])]
    out = lm.generate(prompts, sample_len=16, temperature=0.8, seed=1234, ignore_stop=True)
    assert all(len(t) == 16 for t in out.tokens)
    assert lm.generate(prompts, sample_len=16, temperature=0.8, seed=1234, ignore_stop=True).tokens == out.tokens
    reqs = {f"r{i}": p + t for i, (p, t) in enumerate(zip(prompts, out.tokens))}
    one_by_one = []
    s = 0
    for rid, toks in reqs.items():        # every token of every sequence alone in its step
        for i, t in enumerate(toks):
            one_by_one.append({"step": s, "entries": [{"id": rid, "tokens": [t], "want": [0]}], "end": [rid] if i == len(toks) - 1 else []})
            s += 1
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=128)
    a = traces.run_in_process(eng, one_by_one, str(tmp_path / "one"), 384)
    eng2 = Engine.from_folder(folder, dtype="float32", max_tokens=traces.max_live_tokens(traces.whole(reqs)))
    b = traces.run_in_process(eng2, traces.whole(reqs), str(tmp_path / "whole"), 384)
    for rid, toks in reqs.items():
        assert row_error(a[rid], b[rid]).max() < 1e-4
        assert row_error(a[rid], P.forward(cfg, tensors, toks)).max() < 1e-4


LLAMA_1B_TWO_LAYERS = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072, "hidden_act": "silu",
}


@pytest.fixture(scope="module")
def one_b(tmp_path_factory):
    from burn_lm_b200 import write_random_model
    folder = write_random_model(str(tmp_path_factory.mktemp("m") / "1b2l"), LLAMA_1B_TWO_LAYERS, seed=2, dtype="bfloat16", device="cuda")
    cfg, tensors = P.read_model_folder(folder)
    reqs = {f"q{n}": random_tokens(30 + n, length, 128256) for n, length in enumerate([70, 9, 33, 100])}
    want = {rid: P.forward(cfg, tensors, toks) for rid, toks in reqs.items()}
    return folder, reqs, want


@pytest.mark.parametrize("dtype,tolerance", [("float32", 1e-4), ("bfloat16", 3e-2)])
def test_one_b_shape_three_ways(tmp_path, one_b, dtype, tolerance):
    from burn_lm_b200 import Engine
    folder, reqs, want = one_b
    for what, steps in (("whole", traces.whole(reqs)), ("tail", traces.tail(reqs, 32)), ("batched", traces.batched(reqs, 4, [32, 3, 17, 0]))):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=traces.max_live_tokens(steps))
        got = traces.run_in_process(eng, steps, str(tmp_path / what), 128256)
        for rid in reqs:
            err = row_error(got[rid], want[rid])
            assert err.max() < tolerance, (what, rid, float(err.max()), int(err.argmax()))
        del eng
        torch.cuda.empty_cache()


# The layer sizes of the 8B model of the same family (width 4096, 32 heads on 8 kv heads of 128, inner 14336),
# one layer, a small vocabulary: wider rows than the 1B shape, a head size of 128 and an inner size whose
# tokens do not fit the skinny kernel's shared memory (that product then goes to the library).
LLAMA_8B_ONE_LAYER = dict(LLAMA_1B_TWO_LAYERS, num_hidden_layers=1, hidden_size=4096, head_dim=128, intermediate_size=14336,
                          vocab_size=3000, tie_word_embeddings=False,
                          rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                        "original_max_position_embeddings": 8192})


@pytest.mark.parametrize("dtype,tolerance", [("float32", 1e-4), ("bfloat16", 3e-2)])
def test_eight_b_layer_shape(tmp_path, dtype, tolerance):
    from burn_lm_b200 import Engine, write_random_model
    folder = write_random_model(str(tmp_path / "8b1l"), LLAMA_8B_ONE_LAYER, seed=4, dtype="bfloat16", device="cuda")
    cfg, tensors = P.read_model_folder(folder)
    reqs = {f"w{n}": random_tokens(50 + n, length, 3000) for n, length in enumerate([80, 5, 140])}
    want = {rid: P.forward(cfg, tensors, toks) for rid, toks in reqs.items()}
    for what, steps in (("whole", traces.whole(reqs)), ("tail", traces.tail(reqs, 32)), ("batched", traces.batched(reqs, 3, [32, 2, 9]))):
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=traces.max_live_tokens(steps))
        got = traces.run_in_process(eng, steps, str(tmp_path / what), 3000)
        for rid in reqs:
            err = row_error(got[rid], want[rid])
            assert err.max() < tolerance, (what, rid, float(err.max()), int(err.argmax()))
        eng.verify()
        del eng
        torch.cuda.empty_cache()
