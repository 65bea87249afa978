"""The architecture-neutral description of a model: which parts stand where, with which sizes,
fed by which stored tensors, and in which order the layers run.

An architecture turns its typed configuration into a `ModelPlan`; the generic `Model` builds the
parts a plan names out of the part registries.  Nothing below this line knows an architecture.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class PartPlan:
    """One part: `kind` is its key in the part registry of its family, `spec` the part's own typed
    sizes and constants, `tensors` maps the part's roles to stored tensor names."""
    kind: str
    spec: Any
    tensors: dict = field(default_factory=dict)


@dataclass(frozen=True)
class NamedPart:
    """A part of a layer under the name its block arrangement knows it by; `family` is the part
    registry it is built from ("mixer", "feed_forward", "norm", ...)."""
    name: str
    family: str
    plan: PartPlan


@dataclass(frozen=True)
class LayerPlan:
    """One layer: a block arrangement (its key in the "block" registry) and the parts it arranges.
    Which parts a layer has is data: a block with one shared norm, with norms behind its parts as well, or
    without a feed-forward lists other names than the pre-norm block of the Llama decoder does."""
    block: str
    parts: tuple          # of NamedPart, in the order their tensors are listed

    def part(self, name: str) -> PartPlan:
        for p in self.parts:
            if p.name == name:
                return p.plan
        raise KeyError(f"the layer has no part named {name!r}; it has {[p.name for p in self.parts]}")

    def with_part(self, name: str, plan: PartPlan) -> "LayerPlan":
        """This layer with the part `name` replaced."""
        self.part(name)
        return LayerPlan(self.block, tuple(NamedPart(p.name, p.family, plan) if p.name == name else p for p in self.parts))


def prenorm_layer(mixer_norm: PartPlan, mixer: PartPlan, feed_forward_norm: PartPlan, feed_forward: PartPlan) -> LayerPlan:
    """The layer of the "prenorm" block: a norm and a mixer, a norm and a feed-forward."""
    return LayerPlan("prenorm", (NamedPart("mixer_norm", "norm", mixer_norm), NamedPart("mixer", "mixer", mixer),
                                 NamedPart("feed_forward_norm", "norm", feed_forward_norm),
                                 NamedPart("feed_forward", "feed_forward", feed_forward)))


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  The order of the runs is data: a layer may be named twice, and a run
    may read the cache line that an earlier run (its index in the schedule) has written, instead
    of writing a line of its own."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding: PartPlan
    layers: tuple
    schedule: tuple
    final_norm: PartPlan
    head: PartPlan
    max_positions: int
    stop_ids: tuple = ()
    ignorable_tensors: tuple = ()   # regular expressions of stored names that may be left unread
    duplicate_tensors: tuple = ()   # (stored name, wanted name) pairs: a stored tensor that may be there as a second copy
                                    # of a wanted one (a tied head written out); it must hold the same values
    stream_position: Optional[PartPlan] = None   # family "position": an encoding added to the stream after the embedding

    def __post_init__(self):
        for n, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {n} names layer {e.layer}; there are {len(self.layers)}")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < n:
                    raise ValueError(f"schedule entry {n} reads the cache of entry {e.cache_of}, "
                                     f"which does not run before it")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {n} reads the cache of entry {e.cache_of}, "
                                     f"which has no cache of its own")
