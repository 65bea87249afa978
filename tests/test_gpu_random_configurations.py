"""Configurations, requests and ways of cutting them into steps drawn at random (from fixed seeds): every size
and option of the architecture takes values the hand-made tiny configurations do not, together with request
lengths from one token to several hundred and batches whose members leave at different times.  Each case is the
property the reference states for its cache ("token by token equals whole",
crates/burn-lm-llama/src/nn/attention/mha.rs:289-350), against the plain implementation, in 32-bit or bfloat16.
"""
import os
import random

import numpy as np
import pytest

import traces
from plain import llama_plain as P
from tiny import random_tokens, row_error

pytestmark = pytest.mark.gpu


def draw(case):
    """(config, dtype, requests, steps) of a case."""
    rng = random.Random(case)
    hd = rng.choice([16, 32, 48, 64, 64, 128, 128])
    kv = rng.choice([1, 2, 3, 4, 8])
    group = rng.choice([1, 2, 3, 4, 8]) if hd in (64, 128) else rng.choice([1, 2, 5])
    cfg = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": rng.choice([1, 2, 3]),
           "hidden_size": rng.choice([64, 96, 128, 192, 200, 256]), "num_attention_heads": kv * group,
           "num_key_value_heads": kv, "head_dim": hd, "intermediate_size": rng.choice([64, 136, 200, 320]),
           "vocab_size": rng.choice([97, 300, 515, 1000]), "rope_theta": rng.choice([10000.0, 500000.0]),
           "rope_scaling": rng.choice([None, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                              "high_freq_factor": 4.0, "original_max_position_embeddings": 128}]),
           "rms_norm_eps": rng.choice([1e-5, 1e-6, 3e-5]), "tie_word_embeddings": rng.random() < 0.5,
           "max_position_embeddings": 1024, "hidden_act": "silu"}
    dtype = rng.choice(["bfloat16", "bfloat16", "float32"])
    n_req = rng.randint(1, 7)
    lengths = [rng.choice([rng.randint(1, 40), rng.randint(40, 200), rng.randint(200, 700)]) for _ in range(n_req)]
    reqs = {f"r{i}": random_tokens(case * 100 + i, n, cfg["vocab_size"]) for i, n in enumerate(lengths)}
    way = rng.choice(["whole", "tail", "batched", "batched", "batched"])
    if way == "whole":
        steps = traces.whole(reqs)
    elif way == "tail":
        steps = traces.tail(reqs, rng.choice([1, 5, 32, 70]))
    else:
        steps = traces.batched(reqs, rng.randint(1, min(n_req, 5)), [rng.randint(0, 90) for _ in range(4)],
                               prompt_steps=rng.choice([1, 1, 2, 3]))
    return cfg, dtype, reqs, steps, way


@pytest.mark.parametrize("first_case", [1, 9, 17, 25, 33])
def test_cases_drawn_at_random(tmp_path, first_case):
    from burn_lm_b200 import Engine, write_random_model
    for case in range(first_case, first_case + 8):
        cfg, dtype, reqs, steps, way = draw(case)
        folder = write_random_model(os.path.join(str(tmp_path), f"m{case}"), cfg, seed=case, dtype="bfloat16")
        pcfg, tensors = P.read_model_folder(folder)
        eng = Engine.from_folder(folder, dtype=dtype, max_tokens=traces.max_live_tokens(steps),
                                 max_seqs=max(len(st["entries"]) for st in steps))
        got = traces.run_in_process(eng, steps, os.path.join(str(tmp_path), f"o{case}"), cfg["vocab_size"])
        eng.verify()
        tolerance = 1e-4 if dtype == "float32" else 3e-2
        for rid, toks in reqs.items():
            err = row_error(got[rid], P.forward(pcfg, tensors, toks))
            assert err.max() < tolerance, (case, dtype, way, cfg, [len(t) for t in reqs.values()], rid, float(err.max()),
                                           "first bad row", int(np.argmax(err >= tolerance)))
