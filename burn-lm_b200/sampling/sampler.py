"""Sampling the next token from fp32 logits, on the device.

As the reference does (crates/burn-lm-llama/src/server/llama3.rs:453-462, generation/generate.rs:
87-91): temperature 0 takes the argmax of the raw logits; a positive temperature draws from
softmax(logits / temperature) restricted to its top-p nucleus (generation/sampling.rs:44-70: in
descending order a token is kept while the mass before it is below p).  The uniform number of a
draw is a hash of (seed, the sequence's stream id, the index of the draw), so what a sequence
draws does not depend on the batch it is in.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import kernels as K


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 0.9
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0, got {self.temperature}")
        if not 0 < self.top_p <= 1:
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        self._plan = None       # what does not change from step to step, on the device, for the batch last seen

    def sample(self, logits: torch.Tensor, params: SamplingParams, stream_ids, counters) -> list:
        """One token id per row of logits [B, V]; stream_ids[b] and counters[b] name the draw."""
        b = logits.shape[0]
        if params.greedy:
            out = torch.empty(b, dtype=torch.int32, device=logits.device)
            K.argmax(logits, out)
            return out.tolist()
        # temperature, top-p, seed and stream ids stay the same while a batch decodes: they are uploaded once;
        # a step brings its draw counters through pinned memory and takes its tokens back the same way
        mask = (1 << 63) - 1
        key = (b, params, tuple(stream_ids), logits.device)
        plan = self._plan
        if plan is None or plan["key"] != key:
            f = torch.tensor([[params.temperature] * b, [params.top_p] * b], dtype=torch.float32).to(logits.device)
            ids = torch.tensor([[params.seed & mask] * b, [s & mask for s in stream_ids]], dtype=torch.int64).to(logits.device)
            plan = self._plan = {
                "key": key, "f": f, "ids": ids,
                "counters": torch.zeros(b, dtype=torch.int64, device=logits.device),
                "host_counters": torch.zeros(b, dtype=torch.int64, pin_memory=True),
                "out": torch.zeros(b, dtype=torch.int32, device=logits.device),
                "host_out": torch.zeros(b, dtype=torch.int32, pin_memory=True)}
            plan["host_counters_np"] = plan["host_counters"].numpy()
            plan["host_out_np"] = plan["host_out"].numpy()
        plan["host_counters_np"][:] = [c & mask for c in counters]
        plan["counters"].copy_(plan["host_counters"], non_blocking=True)
        K.sample(logits, plan["f"][0], plan["f"][1], plan["ids"][0], plan["ids"][1], plan["counters"], plan["out"])
        plan["host_out"].copy_(plan["out"], non_blocking=True)
        torch.cuda.current_stream(logits.device).synchronize()
        return plan["host_out_np"].tolist()
