"""The generic model: parts built from a `ModelPlan`, weights bound by name, and one forward over
the packed tokens of a step.  It knows no architecture; the plan's schedule says which layer runs
when and whose cache line it reads.
"""
from __future__ import annotations

import torch

from .config.reader import read_config_json
from .parts.base import CacheNeed, Runtime
from .parts.linear import NormHandoff
from .plan import ModelPlan
from .registry import architecture_of, part_class
from .weights.loader import load_tensors

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    try:
        return _DTYPES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"compute dtype must be 'bfloat16' or 'float32', got {dtype!r}") from None


def plan_of(config: dict):
    """(architecture, typed configuration, plan) of a config.json dict."""
    arch = architecture_of(config)
    typed = arch.config_class.from_dict(config)
    return arch, typed, arch.plan(typed)


def _build(plan_part, family, runtime):
    return part_class(family, plan_part.kind)(plan_part.spec, plan_part.tensors, runtime)


class Layer:
    """The parts a layer plan names, built from their families' registries, and the block that arranges them."""

    def __init__(self, lp, runtime):
        self.named = {p.name: (p.family, _build(p.plan, p.family, runtime)) for p in lp.parts}
        if len(self.named) != len(lp.parts):
            raise ValueError(f"a layer names a part twice: {[p.name for p in lp.parts]}")
        self.block = part_class("block", lp.block)({name: part for name, (_, part) in self.named.items()})

    def parts(self):
        return [part for _, part in self.named.values()]

    def cache_need(self):
        """What a run of this layer keeps per sequence: what its block says, else what its one mixer says."""
        if hasattr(self.block, "cache_need"):
            return self.block.cache_need()
        mixers = [part for family, part in self.named.values() if family == "mixer"]
        if not mixers:
            return CacheNeed("none")
        if len(mixers) > 1:
            raise ValueError("a block with several mixers must say itself what a run keeps (cache_need())")
        return mixers[0].cache_need()


class Model:
    def __init__(self, plan: ModelPlan, runtime: Runtime, config=None):
        self.plan, self.runtime, self.config = plan, runtime, config
        self.embedding = _build(plan.embedding, "embedding", runtime)
        self.stream_position = _build(plan.stream_position, "position", runtime) if plan.stream_position is not None else None
        self.layers = [Layer(lp, runtime) for lp in plan.layers]
        self.final_norm = _build(plan.final_norm, "norm", runtime)
        self.head = _build(plan.head, "head", runtime)
        self.bound = False

    # -- weights ---------------------------------------------------------------------------------
    def parts(self):
        out = [self.embedding] + ([self.stream_position] if self.stream_position is not None else [])
        for layer in self.layers:
            out.extend(layer.parts())
        out.extend([self.final_norm, self.head])
        return out

    def tensor_specs(self):
        seen, out = {}, []
        for p in self.parts():
            for s in p.tensor_specs():
                if s.name in seen:
                    if tuple(seen[s.name].shape) != tuple(s.shape):
                        raise ValueError(f"tensor {s.name!r} is wanted with shapes {seen[s.name].shape} and {s.shape}")
                    continue
                seen[s.name] = s
                out.append(s)
        return out

    def bind(self, loaded: dict):
        for p in self.parts():
            p.bind(loaded)
        # a run that reads another run's cache line must agree with its writer on how the entries lie there
        for run, e in enumerate(self.plan.schedule):
            if e.cache_of is not None:
                reader, writer = self._mixer_of(e.layer), self._mixer_of(self.plan.schedule[e.cache_of].layer)
                a = reader.key_layout() if hasattr(reader, "key_layout") else None
                b = writer.key_layout() if hasattr(writer, "key_layout") else None
                if a != b or reader.cache_need() != writer.cache_need():
                    raise ValueError(f"run {run} of the schedule reads the cache line of run {e.cache_of}, whose mixer "
                                     f"keeps its entries in another layout ({b} against {a}) or another size")
        self.bound = True

    def _mixer_of(self, layer: int):
        mixers = [part for family, part in self.layers[layer].named.values() if family == "mixer"]
        if len(mixers) != 1:
            raise ValueError(f"layer {layer} shares a cache line and must have exactly one mixer; it has {len(mixers)}")
        return mixers[0]

    def cache_needs(self):
        """The cache need of every run of the schedule (None for a run that reads another's line)."""
        return [None if e.cache_of is not None else self.layers[e.layer].cache_need()
                for e in self.plan.schedule]

    # -- forward ---------------------------------------------------------------------------------
    def forward(self, step, cache):
        """Logits (fp32 [n_want, vocab]) at the wanted rows of the step, or None when none is wanted."""
        if not self.bound:
            raise RuntimeError("the model has no weights yet")
        step.memo.clear()
        resid = torch.empty((step.n_tokens, self.plan.hidden_size), dtype=torch.float32, device=self.runtime.device)
        schedule = self.plan.schedule
        first = self.layers[schedule[0].layer].block if schedule else None
        if (getattr(self.embedding, "hands_norm_over", False) and self.stream_position is None
                and first is not None and hasattr(first, "first_norm")):
            # the embedding writes the stream: it may leave the input of the norm that reads it first
            if step.handoff is None:
                step.handoff = NormHandoff()
            step.handoff.expect(first.first_norm())
            self.embedding.forward(step.tokens, resid, handoff=step.handoff)
        else:
            self.embedding.forward(step.tokens, resid)
        if self.stream_position is not None:
            self.stream_position.on_embedding(resid, step)      # an encoding that is added to the stream
        delta = None
        for run, entry in enumerate(schedule):
            block = self.layers[entry.layer].block
            if hasattr(block, "first_norm"):
                # the norm that reads the stream after this block: the next run's first, or the last norm
                after = self.layers[schedule[run + 1].layer].block if run + 1 < len(schedule) else None
                next_norm = self.final_norm if after is None else (after.first_norm() if hasattr(after, "first_norm") else None)
                delta = block.forward(resid, delta, step, cache.view(run), next_norm=next_norm)
            else:
                delta = block.forward(resid, delta, step, cache.view(run))
        if step.n_want == 0:
            return None
        lazy = getattr(self.head, "takes_pending_norm", False)
        if getattr(self.final_norm, "takes_handed_norm", False):
            x = self.final_norm.add_norm(resid, delta, rows=step.want_rows, lazy=lazy, handoff=step.handoff)
        else:
            x = self.final_norm.add_norm(resid, delta, rows=step.want_rows, lazy=lazy)
        return self.head.forward(x)

    def prepare(self, max_positions: int) -> None:
        """Let parts precompute what depends on the longest sequence the cache can hold."""
        for p in self.parts():
            if hasattr(p, "prepare"):
                p.prepare(max_positions)


def tensor_specs_of(config: dict):
    """The stored tensors the architecture of `config` needs (no device work)."""
    _, _, plan = plan_of(config)
    return Model(plan, Runtime(torch.bfloat16, torch.device("cpu"))).tensor_specs()


def load_model(folder: str, dtype="bfloat16", device="cuda") -> Model:
    """Build the model a folder's config.json names and bind its safetensors weights."""
    config = read_config_json(folder)
    _, typed, plan = plan_of(config)
    runtime = Runtime(parse_dtype(dtype), torch.device(device))
    model = Model(plan, runtime, typed)
    loaded = load_tensors(folder, model.tensor_specs(), runtime.dtype, runtime.device, plan.ignorable_tensors,
                          plan.duplicate_tensors)
    model.bind(loaded)
    return model


def random_model(config: dict, seed: int = 0, dtype="bfloat16", device="cuda", stored_dtype="bfloat16") -> Model:
    """The model `config` names with random weights drawn on the device, without a folder in between: for
    shapes whose files would take minutes to write and read back.  The numbers are the ones
    `write_random_model(..., device=<the same device>)` stores (every tensor from its own generator, seeded
    by the seed and the tensor's name), kept as a folder stored in `stored_dtype` would be loaded."""
    from .weights.loader import _target_dtype
    from .weights.random_init import _DTYPES, random_tensor
    _, typed, plan = plan_of(config)
    runtime = Runtime(parse_dtype(dtype), torch.device(device))
    model = Model(plan, runtime, typed)
    loaded = {}
    for spec in model.tensor_specs():
        t = random_tensor(spec, seed, _DTYPES[stored_dtype], runtime.device)
        loaded[spec.name] = t.to(_target_dtype(t.dtype, spec.kind, runtime.dtype))
    model.bind(loaded)
    return model
