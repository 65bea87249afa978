"""Decode and prefill throughput of the Llama-3.2-1B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

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

Peaks come from MEASURED_PEAKS.json beside this file when it is there.  The weights (2.47 GB) are
far larger than the L2, so nothing is flushed between steps.  For --gpus N > 1 it says that this
library runs on one GPU and exits with 2.  The reference arm is unavailable: tracel-ai/burn-lm is a
Rust workspace and neither cargo nor its git dependency `burn` can be had offline.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 16, "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072, "hidden_act": "silu",
}
FULL_LAYERS = 16
CONTEXT = 4096
PROMPT = 512
PREFILL_TOKENS = 2048
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


def model_folder(cfg, seed=0):
    """A folder with the random 1B model, made once per box under the temporary folder."""
    import burn_lm_b200 as blm
    key = hashlib.sha256(json.dumps(cfg, sort_keys=True).encode()).hexdigest()[:12]
    folder = os.path.join(tempfile.gettempdir(), f"burn-lm_b200-bench-{key}-{seed}")
    done = os.path.join(folder, ".complete")
    if not os.path.exists(done):
        t0 = time.time()
        blm.write_random_model(folder, cfg, seed=seed, dtype="bfloat16", device="cuda")
        with open(done, "w") as f:
            f.write("ok")
        print(f"[bench] wrote random model to {folder} in {time.time() - t0:.1f} s", file=sys.stderr)
    return folder


def weight_bytes(cfg):
    d, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    h, kv, hd, layers = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["num_hidden_layers"]
    per_layer = d * (h + 2 * kv) * hd + h * hd * d + 3 * d * i + 2 * d
    return 2 * (layers * per_layer + v * d + d)      # bf16; the tied table is read once, as the head


def kv_bytes_per_token(cfg):
    return 2 * cfg["num_hidden_layers"] * cfg["num_key_value_heads"] * cfg["head_dim"] * 2


def prefill_flops(cfg, t):
    d, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    h, kv, hd, layers = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["num_hidden_layers"]
    per_layer = d * (h + 2 * kv) * hd + h * hd * d + 3 * d * i
    gemm = 2.0 * t * layers * per_layer + 2.0 * v * d          # the head runs on one row
    attn = layers * 2.0 * t * t * h * hd                        # causal half of QK^T and PV
    return gemm + attn


def random_prompts(n, length, vocab, seed):
    import numpy as np
    rng = np.random.default_rng(seed)
    return [[int(x) for x in rng.integers(0, vocab, size=length)] for _ in range(n)]


def device_decode(engine, batch, steps, warmup, cfg, sample_clocks=False, prompt_len=None):
    """Prefill `batch` prompts, then time `steps` decode steps that run back to back on the device."""
    import torch
    from burn_lm_b200 import StepEntry, kernels
    plen = prompt_len or PROMPT
    prompts = random_prompts(batch, plen, cfg["vocab_size"], seed=batch)
    slots = [engine.acquire() for _ in range(batch)]
    try:
        # prompts go in a few at a time to keep the prefill's activations small
        for i in range(0, batch, 8):
            engine.step([StepEntry(s, p, []) for s, p in zip(slots[i:i + 8], prompts[i:i + 8])])
        first = [p[-1] for p in prompts]
        engine.decode_run(slots, first, max(warmup, 3))          # warm-up: captures the graph, W steps
        for s in slots:                                          # rewind: the timed run decodes from the prompt's end
            engine.cache.set_length(s, plen)
        torch.cuda.synchronize()
        before = kernels.launch_count()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler = ClockSampler() if sample_clocks else None
        if sampler:
            sampler.__enter__()
        torch.cuda.synchronize()
        start.record()
        history = engine.decode_run(slots, first, steps)
        stop.record()
        torch.cuda.synchronize()
        if sampler:
            sampler.__exit__()
        ms = start.elapsed_time(stop)
        g = engine.decode_graph(batch, plen + steps)
        launches = g.launches_per_step * steps + (kernels.launch_count() - before)
        assert history.shape == (steps, batch)
        engine.verify()        # no kernel gave up a bounded wait
        return {"ms_per_step": ms / steps, "tokens_per_s": batch * steps / (ms / 1e3), "launches": launches,
                "clocks": sampler.summary() if sampler else None}
    finally:
        for s in slots:
            engine.release(s)


def time_prefill(engine, cfg, reps=5, tokens=PREFILL_TOKENS, n_prompts=1):
    """Median time of one prefill step: `n_prompts` prompts of `tokens` tokens each, the last logits wanted."""
    import torch
    from burn_lm_b200 import StepEntry
    prompts = random_prompts(n_prompts, tokens, cfg["vocab_size"], seed=99)
    times = []
    for r in range(reps + 2):
        slots = [engine.acquire() for _ in prompts]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        engine.step([StepEntry(s, p, [tokens - 1]) for s, p in zip(slots, prompts)])
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
    for prompt_len in (512, 2048, 3840):
        for b in (1, 8, 64):
            steps = 128
            r = device_decode(engine, b, steps, 3, cfg, prompt_len=prompt_len)
            step_bytes = weight_bytes(cfg) + b * (prompt_len + steps / 2.0) * kv_bytes_per_token(cfg)
            gbs = step_bytes / (r["ms_per_step"] / 1e3) / 1e9
            print(json.dumps({"decode": {"batch": b, "context": prompt_len, "ms_per_step": round(r["ms_per_step"], 4),
                                         "tokens_per_s": round(r["tokens_per_s"], 1), "gb_per_s": round(gbs, 1),
                                         "frac_hbm": round(gbs / pk["hbm_gbs"], 3)}}), flush=True)
    h, hd, layers = cfg["num_attention_heads"], cfg["head_dim"], cfg["num_hidden_layers"]
    for n_prompts, tokens in ((1, 128), (1, 512), (1, 2048), (1, 4096), (8, 512), (16, 1024)):
        ms = time_prefill(engine, cfg, reps=3, tokens=tokens, n_prompts=n_prompts)
        total = n_prompts * tokens
        # products over all tokens, attention within each prompt
        flops = prefill_flops(cfg, total) - layers * 2.0 * h * hd * (total * total - n_prompts * tokens * tokens)
        print(json.dumps({"prefill": {"prompts": n_prompts, "tokens_each": tokens, "ms": round(ms, 3),
                                      "tokens_per_s": round(total / (ms / 1e3), 1),
                                      "frac_bf16": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 3)}}), flush=True)


def run_ours(args):
    import torch
    import burn_lm_b200 as blm
    from burn_lm_b200 import kernels

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: burn-lm_b200 has no CPU path"}))
        return 1
    pk = peaks()
    cfg = dict(LLAMA_1B)
    cfg["num_hidden_layers"] = args.layers
    batch, steps, warmup = args.batch, args.steps, max(args.warmup, 3)
    folder = model_folder(cfg)
    lm = blm.LanguageModel(folder, dtype="bfloat16", max_seq_len=CONTEXT, max_batch=64,
                           max_tokens=64 * CONTEXT).load()
    engine = lm.engine

    if args.only == "decode":      # a short run of one workload, for profilers
        r = device_decode(engine, batch, steps, warmup, cfg)
        print(json.dumps({"only": "decode", "batch": batch, "ms_per_step": round(r["ms_per_step"], 4)}))
        return 0
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "tokens": PREFILL_TOKENS, "ms": round(time_prefill(engine, cfg, reps=1), 3)}))
        return 0
    if args.only == "sweep":
        sweep(engine, cfg, pk)
        return 0
    main = device_decode(engine, batch, steps, warmup, cfg, sample_clocks=True)
    points = {}
    for b in (1, 64):
        r = device_decode(engine, b, min(steps, 128), warmup, cfg)
        points[f"decode_b{b}"] = round(r["tokens_per_s"], 1)

    # end to end through the Python entry point: host tokens in and out every step
    prompts = random_prompts(batch, PROMPT, cfg["vocab_size"], seed=batch)
    lm.generate(prompts, sample_len=warmup + 2, ignore_stop=True)                  # warm-up (captures the graph)
    out = lm.generate(prompts, sample_len=steps + 1, ignore_stop=True)             # steps decode steps after the prefill
    st = out.stats
    e2e_value = batch * st.decode_steps / st.decode_seconds
    g = engine.decode_graph(batch, PROMPT + steps)

    prefill_ms = time_prefill(engine, cfg)
    flops = prefill_flops(cfg, PREFILL_TOKENS)

    mean_len = PROMPT + steps / 2.0
    step_bytes = weight_bytes(cfg) + batch * mean_len * kv_bytes_per_token(cfg)
    achieved = step_bytes / (main["ms_per_step"] / 1e3) / 1e9

    line = {
        "metric": "decode tokens/s, Llama-3.2-1B shape, bf16, batch 8 (512-token prompts, context 4096)",
        "value": round(main["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {
            "model": "llama-3.2-1b-shape-random", "layers": cfg["num_hidden_layers"], "layers_full": FULL_LAYERS,
            "hidden_size": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate_size": cfg["intermediate_size"], "vocab_size": cfg["vocab_size"],
            "tied_head": True, "rope": "theta 5e5, llama3 x32", "global_batch": batch, "seq_len": CONTEXT,
            "prompt_len": PROMPT, "parallelism": "single-gpu", "weights": "random N(0,0.02) bf16",
            "l2": "inputs (2.47 GB of weights) exceed the 126 MB L2; no flush", "sampling": "greedy",
            "peaks": pk["source"],
        },
        "clocks": main["clocks"],
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": g.bytes_in_per_step(),
                "d2h_bytes_per_step": 4 * batch, "ms_per_step": round(1e3 * st.decode_seconds / st.decode_steps, 4)},
        "gpu_launches": main["launches"],
        "prefill": {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 3), "frac": round(flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                    "peak_tflops": pk["bf16_tflops"]},
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
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--only", default=None, choices=["decode", "prefill", "sweep"],
                    help="run one workload briefly (for profilers), or a sweep over batch sizes and context lengths")
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the configuration's 16 (named in config)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "tracel-ai/burn-lm is a Rust workspace: no cargo/rustc here, its `burn` dependency is a git "
                          "branch that cannot be fetched offline, and pip finds neither setup.py nor pyproject.toml"}))
        return 0
    if args.gpus != 1:
        print(f"burn-lm_b200 generates on ONE GPU; --gpus {args.gpus} is not built (no multi-GPU path)")
        return 2
    if args.steps + PROMPT > CONTEXT:
        print(f"--steps {args.steps} does not fit the context of {CONTEXT} after a {PROMPT}-token prompt")
        return 2
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
