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
