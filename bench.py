"""Decode and prefill throughput of the Llama-3.2-1B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--config 1b|3b|8b]

A "step" is one decode step of the whole batch.  The default run has the layer sizes of the 1B
configuration (16 layers, width 2048, 32 heads on 8 kv heads of 64, inner 8192, vocabulary 128256,
llama3 rotary scaling, tied head), bfloat16 random weights N(0, 0.02), a batch of 8 sequences with
512-token random prompts in a context of 4096, and prints ONE JSON line:

  value      decoded tokens a second: K steps run back to back on the device (captured CUDA graph,
             greedy token fed back by a kernel), timed with CUDA events
  e2e        the same through the Python entry point `LanguageModel.generate`: every step copies its
             inputs from pinned host memory and reads the sampled tokens back
  prefill    one 2,048-token prompt in one step
  roofline   the decode step against the HBM bandwidth: bytes it has to read / its time
  points     decode at batch 1 and 64

--config 3b: the Llama-3.2-3B shape, 16 prompts of 64 to 4,096 tokens prefilled together, 128 greedy steps,
context 8192.  --config 8b: the Llama-3.1-8B shape, 32 prompts of 128 to 2,048 tokens, 256 steps at temperature
0.7 (the draw runs inside the captured step; the host launches every step), and a 2,048-token prefill.
Models are built with random weights drawn on the device (`load_random`), no folder in between.

Peaks come from MEASURED_PEAKS.json beside this file when it is there.  The weights (2.47 GB) are
far larger than the L2, so nothing is flushed between steps.  For --gpus N > 1 it says that this
library runs on one GPU and exits with 2.  The reference arm is unavailable: tracel-ai/burn-lm is a
Rust workspace and neither cargo nor its git dependency `burn` can be had offline.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# The workloads, by the name --config takes.  "1b" is the headline and the default; "3b" and "8b" are the two
# larger shapes with the batches their configurations state.  `prompts`: ("equal", n) or ("uniform", lo, hi).
WORKLOADS = {
    "1b": {"preset": "llama3_2_1b", "model": "llama-3.2-1b-shape-random", "context": 4096, "batch": 8,
           "prompts": ("equal", 512), "steps": 256, "temperature": 0.0, "prefill": ("one", 2048), "points": (1, 64)},
    "3b": {"preset": "llama3_2_3b", "model": "llama-3.2-3b-shape-random", "context": 8192, "batch": 16,
           "prompts": ("uniform", 64, 4096), "steps": 128, "temperature": 0.0, "prefill": ("batch",), "points": ()},
    "8b": {"preset": "llama3_1_8b", "model": "llama-3.1-8b-shape-random", "context": 8192, "batch": 32,
           "prompts": ("uniform", 128, 2048), "steps": 256, "temperature": 0.7, "prefill": ("one", 2048), "points": ()},
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["source"] = "measured"
        return p
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read only) while a region runs."""

    def __init__(self, period=0.004):
        self.period, self.samples, self.reasons = period, [], set()
        self._stop = threading.Event()
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            idx = int(os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0] or 0)
            try:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    _NAMES = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
              0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
              0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self._NAMES.items():
                    if r & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._t = threading.Thread(target=self._loop, daemon=True)
            self._t.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self.nv is not None:
            self._t.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def weight_bytes(cfg):
    d, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    h, kv, hd, layers = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["num_hidden_layers"]
    per_layer = d * (h + 2 * kv) * hd + h * hd * d + 3 * d * i + 2 * d
    head = v * d if cfg.get("tie_word_embeddings") else 2 * v * d      # untied: the table is stored beside the head
    return 2 * (layers * per_layer + head + d)      # bf16


def decode_step_bytes(cfg, live_tokens):
    """What a decode step has to read: every weight it uses once (the embedding table only as far as it is
    the head: a step gathers a handful of its rows) and the cache of the live sequences."""
    d, v = cfg["hidden_size"], cfg["vocab_size"]
    used = weight_bytes(cfg) - (0 if cfg.get("tie_word_embeddings") else 2 * v * d)
    return used + live_tokens * kv_bytes_per_token(cfg)


def kv_bytes_per_token(cfg):
    return 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg, lengths):
    """Flops of one prompt step over prompts of these lengths: the products over all tokens, attention within
    each prompt (the causal half of QK^T and PV), the head on one row per prompt."""
    d, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    h, kv, hd, layers = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["num_hidden_layers"]
    per_layer = d * (h + 2 * kv) * hd + h * hd * d + 3 * d * i
    total = sum(lengths)
    gemm = 2.0 * total * layers * per_layer + 2.0 * v * d * len(lengths)
    attn = layers * 2.0 * h * hd * sum(t * t for t in lengths)
    return gemm + attn


def make_prompts(spec, n, vocab, seed):
    """`spec`: ("equal", length) or ("uniform", lo, hi); ids uniform over the vocabulary, seeded."""
    import numpy as np
    rng = np.random.default_rng(seed)
    if spec[0] == "equal":
        lengths = [spec[1]] * n
    else:
        lengths = [int(x) for x in rng.integers(spec[1], spec[2] + 1, size=n)]
    return [[int(x) for x in rng.integers(0, vocab, size=length)] for length in lengths]


def prefill_in_parts(engine, slots, prompts, most=8192):
    """Prompts go in a few at a time to keep the prefill's activations small."""
    from burn_lm_b200 import StepEntry
    group, held = [], 0
    for s, p in zip(slots, prompts):
        if group and held + len(p) > most:
            engine.step([StepEntry(a, b, []) for a, b in group])
            group, held = [], 0
        group.append((s, p))
        held += len(p)
    if group:
        engine.step([StepEntry(a, b, []) for a, b in group])


def device_decode(engine, prompts, steps, warmup, sample_clocks=False, temperature=0.0):
    """Prefill the prompts, then time `steps` decode steps.  Greedy: the steps run back to back on the device
    (captured graph, the argmax token fed back by a kernel).  With a temperature: every step is the captured
    graph with the draw inside it, launched by the host with the step's tokens (the draw needs the host's counters)."""
    import torch
    from burn_lm_b200 import kernels
    from burn_lm_b200.sampling import SamplingParams
    batch = len(prompts)
    lengths = [len(p) for p in prompts]
    slots = [engine.acquire() for _ in range(batch)]
    try:
        prefill_in_parts(engine, slots, prompts)
        first = [p[-1] for p in prompts]
        params = SamplingParams(temperature, 0.9, 1234) if temperature > 0 else None

        def run(n):
            if params is None:
                return engine.decode_run(slots, first, n)
            toks = list(first)
            for k in range(n):
                toks = engine.decode_sampled(slots, toks, params, list(range(batch)), [k] * batch)
                assert toks is not None, "this engine does not capture its decode steps"
            return toks

        sampled_per_step = 0
        if params is not None:                                   # the first drawn step runs plainly, then is captured
            count0 = kernels.launch_count()
            run(1)
            sampled_per_step = (kernels.launch_count() - count0) // 2
        run(max(warmup, 3))                                      # warm-up: captures the graph, W steps
        for s, n in zip(slots, lengths):                         # rewind: the timed run decodes from the prompts' ends
            engine.cache.set_length(s, n)
        torch.cuda.synchronize()
        before = kernels.launch_count()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler = ClockSampler() if sample_clocks else None
        if sampler:
            sampler.__enter__()
        torch.cuda.synchronize()
        start.record()
        run(steps)
        stop.record()
        torch.cuda.synchronize()
        if sampler:
            sampler.__exit__()
        ms = start.elapsed_time(stop)
        g = engine.decode_graph(batch, max(lengths) + steps)
        per_step = sampled_per_step or g.launches_per_step or 0
        launches = per_step * steps + (kernels.launch_count() - before)
        engine.verify()        # no kernel gave up a bounded wait
        return {"ms_per_step": ms / steps, "tokens_per_s": batch * steps / (ms / 1e3), "launches": launches,
                "clocks": sampler.summary() if sampler else None, "graph": g}
    finally:
        for s in slots:
            engine.release(s)


def time_prefill(engine, prompts, reps=5):
    """Median time of one prefill step over `prompts`, the last logits of each wanted."""
    import torch
    from burn_lm_b200 import StepEntry
    times = []
    for r in range(reps + 2):
        slots = [engine.acquire() for _ in prompts]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        stop.record()
        torch.cuda.synchronize()
        for s in slots:
            engine.release(s)
        if r >= 2:
            times.append(start.elapsed_time(stop))
    return statistics.median(times)


def sweep(engine, cfg, pk):
    """Decode and prefill at further batch sizes and context lengths, one JSON line each, with the
    fraction of the measured peak (bytes a step has to read, or flops) beside the time."""
    vocab = cfg["vocab_size"]
    for prompt_len in (512, 2048, 3840):
        for b in (1, 8, 64):
            steps = 128
            r = device_decode(engine, make_prompts(("equal", prompt_len), b, vocab, seed=b), steps, 3)
            gbs = decode_step_bytes(cfg, b * (prompt_len + steps / 2.0)) / (r["ms_per_step"] / 1e3) / 1e9
            print(json.dumps({"decode": {"batch": b, "context": prompt_len, "ms_per_step": round(r["ms_per_step"], 4),
                                         "tokens_per_s": round(r["tokens_per_s"], 1), "gb_per_s": round(gbs, 1),
                                         "frac_hbm": round(gbs / pk["hbm_gbs"], 3)}}), flush=True)
    for n_prompts, tokens in ((1, 128), (1, 512), (1, 2048), (1, 4096), (8, 512), (16, 1024)):
        prompts = make_prompts(("equal", tokens), n_prompts, vocab, seed=99)
        ms = time_prefill(engine, prompts, reps=3)
        flops = prefill_flops(cfg, [tokens] * n_prompts)
        print(json.dumps({"prefill": {"prompts": n_prompts, "tokens_each": tokens, "ms": round(ms, 3),
                                      "tokens_per_s": round(n_prompts * tokens / (ms / 1e3), 1),
                                      "frac_bf16": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 3)}}), flush=True)


def run_ours(args):
    import torch
    import burn_lm_b200 as blm
    from burn_lm_b200 import kernels

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: burn-lm_b200 has no CPU path"}))
        return 1
    pk = peaks()
    w = WORKLOADS[args.config]
    cfg = blm.preset(w["preset"])
    full_layers = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = args.layers or full_layers
    context = w["context"]
    batch = args.batch or w["batch"]
    steps, warmup = args.steps or w["steps"], max(args.warmup, 3)
    vocab = cfg["vocab_size"]
    most = max((batch,) + tuple(w["points"]))
    lm = blm.load_random(cfg, seed=0, dtype="bfloat16", max_seq_len=context, max_batch=most, max_tokens=most * context)
    engine = lm.engine
    prompts = make_prompts(w["prompts"], batch, vocab, seed=batch)
    lengths = [len(p) for p in prompts]
    if max(lengths) + steps + 1 > context:
        print(f"--steps {steps} does not fit the context of {context} after a {max(lengths)}-token prompt")
        return 2
    one_prompt = make_prompts(("equal", w["prefill"][1]), 1, vocab, seed=99) if w["prefill"][0] == "one" else None

    if args.only == "decode":      # a short run of one workload, for profilers
        r = device_decode(engine, prompts, steps, warmup, temperature=w["temperature"])
        print(json.dumps({"only": "decode", "batch": batch, "ms_per_step": round(r["ms_per_step"], 4)}))
        return 0
    if args.only == "prefill":
        if args.prompt_tokens:
            one_prompt = make_prompts(("equal", args.prompt_tokens), 1, vocab, seed=99)
        ms = time_prefill(engine, one_prompt or prompts, reps=1)
        print(json.dumps({"only": "prefill", "tokens": sum(len(p) for p in (one_prompt or prompts)), "ms": round(ms, 3)}))
        return 0
    if args.only == "sweep":
        sweep(engine, cfg, pk)
        return 0
    main = device_decode(engine, prompts, steps, warmup, sample_clocks=True, temperature=w["temperature"])
    points = {}
    for b in w["points"]:
        r = device_decode(engine, make_prompts(w["prompts"], b, vocab, seed=b), min(steps, 128), warmup)
        points[f"decode_b{b}"] = round(r["tokens_per_s"], 1)

    # end to end through the Python entry point: host tokens in and out every step
    options = dict(ignore_stop=True, temperature=w["temperature"], seed=1234)
    lm.generate(prompts, sample_len=warmup + 2, **options)                  # warm-up (captures the graph)
    out = lm.generate(prompts, sample_len=steps + 1, **options)             # steps decode steps after the prefill
    st = out.stats
    e2e_value = batch * st.decode_steps / st.decode_seconds
    h2d = main["graph"].bytes_in_per_step() + (8 * batch if w["temperature"] > 0 else 0)      # + the draws' counters

    pre_prompts = one_prompt or prompts
    prefill_ms = time_prefill(engine, pre_prompts, reps=5 if one_prompt else 3)
    pre_tokens = sum(len(p) for p in pre_prompts)
    flops = prefill_flops(cfg, [len(p) for p in pre_prompts])

    live = sum(lengths) + batch * steps / 2.0
    achieved = decode_step_bytes(cfg, live) / (main["ms_per_step"] / 1e3) / 1e9
    rs = cfg["rope_scaling"]
    plen = w["prompts"]
    line = {
        "metric": f"decode tokens/s, {w['model'].replace('-shape-random', '')} shape, bf16, batch {batch} "
                  f"({'%d-token prompts' % plen[1] if plen[0] == 'equal' else 'prompts of %d to %d tokens' % plen[1:]}, context {context})",
        "value": round(main["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {
            "model": w["model"], "layers": cfg["num_hidden_layers"], "layers_full": full_layers,
            "hidden_size": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate_size": cfg["intermediate_size"], "vocab_size": vocab,
            "tied_head": bool(cfg["tie_word_embeddings"]), "rope": f"theta {cfg['rope_theta']:g}, llama3 x{rs['factor']:g}",
            "global_batch": batch, "seq_len": context,
            "prompt_len": plen[1] if plen[0] == "equal" else f"uniform {plen[1]}..{plen[2]} (mean {sum(lengths) // batch})",
            "parallelism": "single-gpu", "weights": "random N(0,0.02) bf16",
            "l2": f"inputs ({weight_bytes(cfg) / 1e9:.2f} GB of weights) exceed the 126 MB L2; no flush",
            "sampling": "greedy" if w["temperature"] == 0 else f"temperature {w['temperature']}, top-p 0.9, host-launched steps",
            "peaks": pk["source"],
        },
        "clocks": main["clocks"],
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4 * batch, "ms_per_step": round(1e3 * st.decode_seconds / st.decode_steps, 4)},
        "gpu_launches": main["launches"],
        "prefill": {"value": round(pre_tokens / (prefill_ms / 1e3), 1), "tokens": pre_tokens,
                    "ms": round(prefill_ms, 3), "frac": round(flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                    "peak_tflops": pk["bf16_tflops"], "prompts": len(pre_prompts)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "impl": "ours",
        "kernel_modules": kernels.loaded_modules(),
    }
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="decode steps to time (default: the workload's: 256, 128, 256)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="1b", choices=sorted(WORKLOADS),
                    help="the workload: 1b (the headline, default), 3b or 8b")
    ap.add_argument("--batch", type=int, default=0, help="sequences decoded together (default: the workload's)")
    ap.add_argument("--only", default=None, choices=["decode", "prefill", "sweep"],
                    help="run one workload briefly (for profilers), or a sweep over batch sizes and context lengths")
    ap.add_argument("--prompt-tokens", type=int, default=0, help="with --only prefill: one prompt of this many tokens instead of the workload's")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (both numbers are named in config)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "tracel-ai/burn-lm is a Rust workspace: no cargo/rustc here, its `burn` dependency is a git "
                          "branch that cannot be fetched offline, and pip finds neither setup.py nor pyproject.toml"}))
        return 0
    if args.gpus != 1:
        print(f"burn-lm_b200 generates on ONE GPU; --gpus {args.gpus} is not built (no multi-GPU path)")
        return 2
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
