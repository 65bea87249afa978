"""Trace replay: feed given token ids through a model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the `Engine`
that generation uses.  A step is one JSON object

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

whose entries bring each request's next tokens and the places among them whose logits are wanted;
`end` lists the requests that are finished after the step (what they hold is given back).  For a
step in which something is wanted the logits go to `<out>/<step>.f32` as little-endian float32
[wanted, vocab], in the order of the entries and of `want`.
"""
from __future__ import annotations

import json
import os
import sys

from .engine import Engine, StepEntry


class Replayer:
    def __init__(self, engine: Engine, out_dir: str):
        self.engine = engine
        self.out_dir = out_dir
        self.slot_of: dict = {}
        os.makedirs(out_dir, exist_ok=True)

    def run_step(self, record: dict):
        step_no = record["step"]
        entries = []
        fresh = []
        try:
            for e in record.get("entries", []):
                rid = e["id"]
                if rid not in self.slot_of:
                    self.slot_of[rid] = self.engine.acquire()
                    fresh.append(rid)
                entries.append(StepEntry(self.slot_of[rid], e["tokens"], e.get("want", ())))
            logits = self.engine.step(entries) if entries else None
            self.engine.verify()
        except Exception:
            for rid in fresh:   # a refused step leaves nothing behind
                self.engine.release(self.slot_of.pop(rid))
            raise
        if logits is not None:
            data = logits.detach().to("cpu").contiguous().numpy().astype("<f4", copy=False)
            tmp = os.path.join(self.out_dir, f".{step_no}.f32.tmp")
            with open(tmp, "wb") as f:
                f.write(data.tobytes())
            os.replace(tmp, os.path.join(self.out_dir, f"{step_no}.f32"))
        for rid in record.get("end", []):
            slot = self.slot_of.pop(rid, None)
            if slot is not None:
                self.engine.release(slot)
        return logits


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to 64")
    args = ap.parse_args(argv)
    engine = Engine.from_folder(args.model, dtype=args.dtype, max_tokens=args.max_tokens)
    rp = Replayer(engine, args.out)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        rp.run_step(record)
        sys.stdout.write(f"done {record['step']}\n")
        sys.stdout.flush()
    return 0
