"""Builds replay traces (the JSON steps `bin/trace_run` reads) from requests, three ways, and reads
the logits files back into per-request arrays."""
import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def whole(requests, first_step=0):
    """Each request alone, all its tokens in one step, logits at every place."""
    steps = []
    for n, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": first_step + n,
                      "entries": [{"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def tail(requests, n_tail=32, first_step=0):
    """Each request alone: all but the last n_tail tokens in one step, then one token a step."""
    steps = []
    s = first_step
    for rid, toks in requests.items():
        toks = list(toks)
        head = max(1, len(toks) - n_tail)
        steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        s += 1
        for i in range(head, len(toks)):
            steps.append({"step": s, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}], "end": []})
            s += 1
        steps[-1]["end"] = [rid]
    return steps


def batched(requests, batch_size, decode_counts, first_step=0, prompt_steps=1):
    """Batches of `batch_size` requests of unequal lengths, one batch after another.  Request i of a
    batch brings all but its last decode_counts[i] tokens in the first step, then one token a step;
    the requests with fewer tokens left end earlier.  With `prompt_steps` > 1 the first part is itself
    cut into that many steps of several tokens per request (the engine takes that; the replay program's
    callers do not ask for it)."""
    steps = []
    s = first_step
    items = list(requests.items())
    for b0 in range(0, len(items), batch_size):
        batch = items[b0: b0 + batch_size]
        heads = {}
        for n, (rid, toks) in enumerate(batch):
            d = decode_counts[(b0 + n) % len(decode_counts)]
            heads[rid] = max(1, len(toks) - d)
        for part in range(prompt_steps):
            cut = lambda rid, k: heads[rid] * k // prompt_steps
            entries = [{"id": rid, "tokens": list(toks[cut(rid, part): cut(rid, part + 1)]),
                        "want": list(range(cut(rid, part + 1) - cut(rid, part)))}
                       for rid, toks in batch if cut(rid, part + 1) > cut(rid, part)]
            done = [rid for rid, toks in batch if heads[rid] == len(toks)] if part == prompt_steps - 1 else []
            steps.append({"step": s, "entries": entries, "end": done})
            s += 1
        pos = dict(heads)
        live = [(rid, toks) for rid, toks in batch if heads[rid] < len(toks)]
        while live:
            entries = [{"id": rid, "tokens": [toks[pos[rid]]], "want": [0]} for rid, toks in live]
            for rid, _ in live:
                pos[rid] += 1
            done = [rid for rid, toks in live if pos[rid] == len(toks)]
            steps.append({"step": s, "entries": entries, "end": done})
            s += 1
            live = [(rid, toks) for rid, toks in live if pos[rid] < len(toks)]
    return steps


def max_live_tokens(steps, unit=64):
    """The --max-tokens a trace needs: the most tokens live requests hold, each rounded up to `unit`."""
    held, most = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum(-(-v // unit) * unit for v in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return most


def gather(steps, read_step, vocab):
    """Per-request [len, vocab] logits from per-step arrays; read_step(step_no) -> float32 [wanted, vocab]."""
    out, at = {}, {}
    for st in steps:
        if not any(e["want"] for e in st["entries"]):
            for e in st["entries"]:
                at[e["id"]] = at.get(e["id"], 0) + len(e["tokens"])
            continue
        data = read_step(st["step"]).reshape(-1, vocab)
        row = 0
        for e in st["entries"]:
            base = at.get(e["id"], 0)
            for w in e["want"]:
                out.setdefault(e["id"], {})[base + w] = data[row]
                row += 1
            at[e["id"]] = base + len(e["tokens"])
        assert row == data.shape[0]
    return {rid: np.stack([rows[i] for i in sorted(rows)]) for rid, rows in out.items()}


def run_in_process(engine, steps, out_dir, vocab):
    from burn_lm_b200.engine.replay import Replayer
    rp = Replayer(engine, out_dir)
    for st in steps:
        rp.run_step(st)
    assert engine.cache.slots.held_count == 0 and engine.cache.free_pages == engine.cache.n_pages
    return gather(steps, lambda n: np.fromfile(os.path.join(out_dir, f"{n}.f32"), dtype="<f4"), vocab)


def run_program(model_dir, dtype, steps, out_dir, vocab, max_tokens=None, env=None):
    """Drive bin/trace_run as a child process, one step at a time, waiting for each `done` line."""
    max_tokens = max_tokens or max_live_tokens(steps)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for st in steps:
            proc.stdin.write(json.dumps(st) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {st['step']}", f"expected 'done {st['step']}', got {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    return gather(steps, lambda n: np.fromfile(os.path.join(out_dir, f"{n}.f32"), dtype="<f4"), vocab)
