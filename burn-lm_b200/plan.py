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
class LayerPlan:
    """One layer: a block arrangement around a mixer and a feed-forward with their norms."""
    block: str            # key in the "block" registry, e.g. "prenorm"
    mixer_norm: PartPlan
    mixer: PartPlan
    feed_forward_norm: PartPlan
    feed_forward: PartPlan


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
