"""Replay of the same requests whole, with the last 32 tokens one by one, and in batches of unequal
lengths whose shorter requests end earlier, one batch after another so that slots and pages are
used again; in 32-bit and in bfloat16; all compared with the plain implementation."""
import os

import numpy as np
import pytest

import traces
from plain import llama_plain as P
from tiny import CONFIGS, make_folder, random_tokens, row_error

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
BF16_TOL = 3e-2


def requests_for(cfg, seed, lengths):
    return {f"r{n}": random_tokens(seed * 100 + n, length, cfg["vocab_size"]) for n, length in enumerate(lengths)}


LENGTHS = {"tiny_a": [5, 11, 17, 64, 65, 128, 33, 100, 2, 97],
           "tiny_b": [1, 7, 30, 64, 200, 129, 256, 40],
           "tiny_c": [300, 45, 640, 64, 129, 33],
           "tiny_d": [200, 16, 333, 64, 65, 40, 7],
           "tiny_e": [129, 48, 260, 17, 64]}


def check(got, want_by_id, tolerance, what):
    for rid, want in want_by_id.items():
        err = row_error(got[rid], want)
        assert err.max() < tolerance, (what, rid, float(err.max()), "first bad place", int(np.argmax(err >= tolerance)))


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype,tolerance", [("float32", FP32_TOL), ("bfloat16", BF16_TOL)])
def test_replay_three_ways(tmp_path, name, dtype, tolerance):
    from burn_lm_b200 import Engine
    folder = make_folder(tmp_path, name, seed=5, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    reqs = requests_for(cfg, 1, LENGTHS[name])
    want = {rid: P.forward(cfg, tensors, toks) for rid, toks in reqs.items()}
    vocab = cfg["vocab_size"]
    ways = {
        "whole": traces.whole(reqs),
        "tail": traces.tail(reqs, 32),
        "batched": traces.batched(reqs, 4, [32, 3, 17, 0, 9]),
        "batched3": traces.batched(reqs, 3, [1, 40, 8]),
    }
    for what, steps in ways.items():
        # the cache is sized for exactly what the trace holds at once: every page gets reused
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=traces.max_live_tokens(steps))
        got = traces.run_in_process(eng, steps, str(tmp_path / f"{what}-{dtype}"), vocab)
        check(got, want, tolerance, what)


@pytest.mark.parametrize("dtype,tolerance", [("float32", FP32_TOL), ("bfloat16", BF16_TOL)])
def test_trace_run_program(tmp_path, dtype, tolerance):
    """The program itself, as a child process fed step by step."""
    folder = make_folder(tmp_path, "tiny_b", seed=6, dtype="bfloat16")
    cfg, tensors = P.read_model_folder(folder)
    reqs = requests_for(cfg, 2, [70, 9, 131, 40, 64])
    want = {rid: P.forward(cfg, tensors, toks) for rid, toks in reqs.items()}
    steps = traces.batched(reqs, 3, [32, 5, 0])
    got = traces.run_program(folder, dtype, steps, str(tmp_path / "out"), cfg["vocab_size"])
    check(got, want, tolerance, "program")


def test_one_engine_many_batches_reuses_slots(tmp_path):
    """One engine, batch after batch through few slots and few pages: what a reused slot or page
    held before does not leak into the next request."""
    from burn_lm_b200 import Engine
    folder = make_folder(tmp_path, "tiny_a", seed=7, dtype="float32")
    cfg, tensors = P.read_model_folder(folder)
    reqs = requests_for(cfg, 3, [100, 3, 64, 17, 128, 5, 90, 65, 1, 31, 77, 12])
    want = {rid: P.forward(cfg, tensors, toks) for rid, toks in reqs.items()}
    steps = traces.batched(reqs, 3, [10, 2, 33])
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=traces.max_live_tokens(steps), max_seqs=3)
    got = traces.run_in_process(eng, steps, str(tmp_path / "o"), cfg["vocab_size"])
    check(got, want, FP32_TOL, "reuse")
