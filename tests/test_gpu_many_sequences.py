"""Decode steps of dozens of sequences: the paths a batch of 64 takes.

With more than 16 sequences a decode step's products leave the skinny kernel's first form, and with
hundreds of (sequence, kv head) blocks the decode attention plans short rings of pages that a block
walks round several times.  Here 48 requests of 300 to 700 tokens on a model with eight kv heads of
size 64 are fed as prompts in three steps, then one token each for up to 75 steps, the shorter ones
leaving earlier; sequences cross pages and the 512-token length bucket of the captured decode step
meanwhile.  Everything is compared with the plain implementation; the property is the reference's
"token by token equals whole" (crates/burn-lm-llama/src/nn/attention/mha.rs:289-350).
"""
import numpy as np
import pytest
import torch

import traces
from plain import llama_plain as P
from test_gpu_kernels import run_attention_case
from tiny import TINY_F, make_folder, random_tokens, row_error

pytestmark = pytest.mark.gpu


def many_requests(n_requests, seed):
    rng = np.random.default_rng(seed)
    lengths = [int(x) for x in rng.integers(300, 701, size=n_requests)]
    # some that are sure to cross the 512-token bucket and a page while they decode, and the two ends
    lengths[:6] = [540, 515, 577, 700, 300, 449]
    return {f"r{n}": random_tokens(seed * 1000 + n, length, TINY_F["vocab_size"]) for n, length in enumerate(lengths)}


DECODE_COUNTS = [75, 3, 70, 40, 72, 1, 64, 33, 71, 17, 74, 9]


@pytest.mark.parametrize("dtype,tolerance", [("float32", 1e-4), ("bfloat16", 3e-2)])
def test_forty_eight_sequences_prompts_then_token_by_token(tmp_path, dtype, tolerance):
    from burn_lm_b200 import Engine
    folder = make_folder(tmp_path, "tiny_f", seed=9, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    reqs = many_requests(48, 4)
    steps = traces.batched(reqs, 48, DECODE_COUNTS, prompt_steps=3)
    decode_steps = [st for st in steps if all(len(e["tokens"]) == 1 for e in st["entries"])]
    assert len(decode_steps) >= 70 and max(len(st["entries"]) for st in decode_steps) > 40
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=traces.max_live_tokens(steps), max_seqs=48)
    got = traces.run_in_process(eng, steps, str(tmp_path / dtype), cfg["vocab_size"])
    eng.verify()
    for rid, toks in reqs.items():
        err = row_error(got[rid], P.forward(cfg, tensors, toks))
        assert err.max() < tolerance, (rid, len(toks), float(err.max()), "first bad place", int(np.argmax(err >= tolerance)))


def test_forty_eight_sequences_on_the_cluster_product(tmp_path, monkeypatch):
    """The same with the switch that sends steps of 17 to 64 tokens to kernels.gemm_sk (the tcgen05 product with K
    cut over a cluster, with the rotary, gated and stream-adding ends and the handed-over norms): the kernel did
    run, and the logits are the plain implementation's."""
    from burn_lm_b200 import Engine, kernels
    from burn_lm_b200.parts import linear
    monkeypatch.setattr(linear, "SK_TOKENS", 64)
    calls = []
    real = kernels.gemm_sk
    monkeypatch.setattr(kernels, "gemm_sk", lambda *a, **k: (calls.append(sorted(k)), real(*a, **k))[1])
    folder = make_folder(tmp_path, "tiny_f", seed=9, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    reqs = many_requests(48, 4)
    steps = traces.batched(reqs, 48, DECODE_COUNTS, prompt_steps=3)
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=traces.max_live_tokens(steps), max_seqs=48)
    got = traces.run_in_process(eng, steps, str(tmp_path / "sk"), cfg["vocab_size"])
    eng.verify()
    kinds = {tuple(c) for c in calls}
    assert any("rope" in c for c in kinds) and any("swiglu" in c for c in kinds) and any("hand_over" in c for c in kinds) and any("squares" in c for c in kinds)
    for rid, toks in reqs.items():
        err = row_error(got[rid], P.forward(cfg, tensors, toks))
        assert err.max() < 3e-2, (rid, len(toks), float(err.max()), int(err.argmax()))


def test_two_batches_of_forty_through_the_same_slots(tmp_path):
    """A second batch of 40 takes the slots and pages the first one gave back (bfloat16, captured steps)."""
    from burn_lm_b200 import Engine
    folder = make_folder(tmp_path, "tiny_f", seed=10, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    reqs = many_requests(80, 5)
    steps = traces.batched(reqs, 40, [12, 3, 20, 1, 17])
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=traces.max_live_tokens(steps), max_seqs=40)
    got = traces.run_in_process(eng, steps, str(tmp_path / "o"), cfg["vocab_size"])
    eng.verify()
    for rid, toks in reqs.items():
        err = row_error(got[rid], P.forward(cfg, tensors, toks))
        assert err.max() < 3e-2, (rid, float(err.max()), int(err.argmax()))


@pytest.mark.parametrize("H,KV,hd", [(32, 8, 64), (16, 8, 64), (32, 8, 128), (8, 8, 64)])
@pytest.mark.parametrize("window", [0, 200])
def test_decode_attention_with_hundreds_of_blocks(H, KV, hd, window):
    """64 sequences x 8 kv heads in one split: 512 blocks, so every block has a ring of two pages and one
    group of consumer warps, and walks the 5 to 11 pages of its sequence round that ring."""
    rng = np.random.default_rng(H + hd + window)
    before = [int(x) for x in rng.integers(300, 701, size=64)]
    before[:5] = [319, 320, 383, 384, 699]          # the new token opens a page / closes one
    run_attention_case(torch.bfloat16, H, KV, hd, before, [1] * 64, window, 1, seed=60, max_kv_len=max(before) + 1)
    # fewer, longer walks: 40 sequences, two splits
    run_attention_case(torch.bfloat16, H, KV, hd, before[:40], [1] * 40, window, 2, seed=61, max_kv_len=max(before[:40]) + 1)


@pytest.mark.parametrize("H,KV,hd,n_splits", [(24, 8, 128, 3), (32, 8, 64, 5), (8, 8, 128, 4)])
def test_decode_attention_of_very_unequal_lengths_in_many_blocks(H, KV, hd, n_splits):
    """16 to 24 sequences of 1 to 4,200 tokens, cut into several splits: more blocks than fill the SMs twice, so a
    sequence takes blocks in proportion to its length (a short one a single block that writes the output itself, the
    longest all the splits, merged by the combine kernel); with and without a window that leaves a sequence fewer
    pages than its length has."""
    rng = np.random.default_rng(H + hd + n_splits)
    before = [int(x) for x in rng.integers(0, 4200, size=24 if hd == 64 else 16)]
    before[:6] = [0, 63, 64, 4199, 2100, 1400]
    for window in (0, 900):
        run_attention_case(torch.bfloat16, H, KV, hd, before, [1] * len(before), window, n_splits, seed=90 + window,
                           max_kv_len=4224)
