"""The command line as a user runs it: `bin/burn-lm random` writes a model folder, `bin/burn-lm run` generates
from it in a child process; the tokens are the plain implementation's.  And a folder of shards generates the
same tokens as the single file it was cut from."""
import json
import os
import subprocess
import sys

import pytest

from plain import llama_plain as P
from tiny import TINY_B, make_folder, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PROGRAM = [sys.executable, os.path.join(ROOT, "bin", "burn-lm")]


def test_random_then_run_as_child_processes(tmp_path):
    folder = str(tmp_path / "b")
    r = subprocess.run(PROGRAM + ["random", folder, "--preset", "tiny_b", "--seed", "4", "--dtype", "float32"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and f"wrote {folder}" in r.stdout, r.stderr
    cfg, tensors = P.read_model_folder(folder)
    prompt = random_tokens(5, 23, cfg["vocab_size"])
    want = P.greedy_generate(cfg, tensors, prompt, 12, stop_ids=TINY_B["eos_token_id"])
    r = subprocess.run(PROGRAM + ["run", folder, "--dtype", "float32", "--sample-len", "12", "--max-seq-len", "128",
                                  ",".join(map(str, prompt))], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert lines[0].split() == [str(t) for t in want], (lines[0], want)
    assert any("tokens per second" in ln for ln in lines) and "model loaded!" in r.stderr
    # a prompt that cannot fit is an error of the request, reported, with the exit code 1
    r = subprocess.run(PROGRAM + ["run", folder, "--dtype", "float32", "--max-seq-len", "16", "--no-stats",
                                  " ".join(["3"] * 40)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 1 and "exceeds the maximum" in r.stderr


def test_a_folder_of_shards_generates_the_same_tokens(tmp_path):
    import burn_lm_b200 as blm
    from burn_lm_b200.weights import SafetensorsFile, write_safetensors
    folder = make_folder(tmp_path, "tiny_d", seed=12, dtype="bfloat16")
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    tensors = {n: f.get(n).clone() for n in f.names()}
    f.close()
    names = sorted(tensors)
    sharded = str(tmp_path / "shards")
    os.makedirs(sharded)
    weight_map = {}
    for k, part in enumerate((names[0::2], names[1::2])):
        fname = f"model-0000{k + 1}-of-00002.safetensors"
        write_safetensors(os.path.join(sharded, fname), {n: tensors[n] for n in part})
        weight_map.update({n: fname for n in part})
    json.dump({"metadata": {}, "weight_map": weight_map}, open(os.path.join(sharded, "model.safetensors.index.json"), "w"))
    json.dump(json.load(open(os.path.join(folder, "config.json"))), open(os.path.join(sharded, "config.json"), "w"))
    prompts = [random_tokens(n, length, 515) for n, length in enumerate([9, 70, 33])]
    a = blm.load(folder, dtype="bfloat16", max_seq_len=256, max_batch=3).generate(prompts, sample_len=20, ignore_stop=True).tokens
    b = blm.load(sharded, dtype="bfloat16", max_seq_len=256, max_batch=3).generate(prompts, sample_len=20, ignore_stop=True).tokens
    assert a == b and all(len(t) == 20 for t in a)
