"""Weights by tensor name.

A model says which tensors it needs as a list of `TensorSpec`; `load_tensors` reads exactly those
from a model folder and raises ONE `WeightsError` that lists every missing tensor, every unexpected
tensor and every wrong shape together.  Stored dtypes are respected: bfloat16 stays bfloat16 (and
is widened exactly to float32 for the 32-bit path), a tensor stored in 32-bit stays 32-bit, float16
is converted to the compute dtype, integer tables become int32.

The reference loads burn records by module path (crates/burn-lm-llama/src/nn/llama/inference.rs:
54-62) and maps other checkpoints' names with regular expressions (nn/llama/import.rs:23-88).
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightsError(ValueError):
    """Weights that do not fit the model; `missing`, `unexpected`, `wrong_shape` and `differing` (stored
    second copies that do not equal the tensor they should repeat) hold the lists."""

    def __init__(self, message, missing=(), unexpected=(), wrong_shape=(), differing=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.differing = list(differing)


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: tuple
    kind: str = "float"          # "float" or "int"
    init: str = "normal:0.02"    # for the random-weights mode: "normal:<std>" or "one_plus_normal:<std>"


def _open_folder(folder: str) -> list[SafetensorsFile]:
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    if os.path.exists(single):
        return [SafetensorsFile(single)]
    if os.path.exists(index):
        with open(index) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
        return [SafetensorsFile(os.path.join(folder, n)) for n in files]
    raise WeightsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json is there")


def _target_dtype(stored: torch.dtype, kind: str, compute: torch.dtype) -> torch.dtype:
    if kind == "int":
        return torch.int32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    if stored == torch.bfloat16:
        return torch.float32 if compute == torch.float32 else torch.bfloat16
    return compute  # float16 and others


def load_tensors(folder: str, specs: list, compute_dtype: torch.dtype, device, ignorable=(), duplicates=()) -> dict:
    """Read the tensors `specs` name from `folder` onto `device`; see the module text for dtypes.
    `ignorable`: regular expressions of stored names that may be left unread.  `duplicates`: (stored name,
    wanted name) pairs; such a stored tensor is expected when it repeats the wanted one bit for bit."""
    try:
        files = _open_folder(folder)
    except SafetensorsError as e:
        raise WeightsError(str(e)) from None
    try:
        where = {}
        for f in files:
            for n in f.names():
                where[n] = f
        wanted = {}
        for s in specs:
            if s.name in wanted and wanted[s.name].shape != tuple(s.shape):
                raise WeightsError(f"tensor {s.name!r} is asked for with two shapes: "
                                   f"{wanted[s.name].shape} and {tuple(s.shape)}")
            wanted[s.name] = s
        missing = [n for n in wanted if n not in where]
        patterns = [re.compile(p) for p in ignorable]
        copies = {a: b for a, b in duplicates if a in where and a not in wanted and b in where}
        unexpected = [n for n in where if n not in wanted and n not in copies and not any(p.fullmatch(n) for p in patterns)]
        differing = []
        for a, b in copies.items():
            ta, tb = where[a].get(a), where[b].get(b)
            if ta.shape != tb.shape or ta.dtype != tb.dtype or not torch.equal(ta, tb):
                differing.append((a, b))
        wrong = []
        for n, s in wanted.items():
            if n in where:
                f = where[n]
                if tuple(f.shape(n)) != tuple(s.shape):
                    wrong.append((n, tuple(s.shape), tuple(f.shape(n))))
                elif (s.kind == "int") == f.dtype(n).is_floating_point:
                    wrong.append((n, f"{s.kind} table", str(f.dtype(n))))
        if missing or unexpected or wrong or differing:
            lines = [f"{folder}: the stored tensors do not fit the model"]
            if missing:
                lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
            if unexpected:
                lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
            if wrong:
                lines.append(f"  wrong shape ({len(wrong)}): " + "; ".join(
                    f"{n} expected {e} found {g}" for n, e, g in sorted(wrong, key=lambda w: w[0])))
            if differing:
                lines.append(f"  differing ({len(differing)}): " + "; ".join(
                    f"{a} is stored beside {b}, which the model uses for both, and does not equal it" for a, b in sorted(differing)))
            raise WeightsError("\n".join(lines), missing, unexpected, wrong, differing)
        out = {}
        for n, s in wanted.items():
            f = where[n]
            t = f.get(n)
            out[n] = t.to(device=device, dtype=_target_dtype(t.dtype, s.kind, compute_dtype), copy=True)
        return out
    finally:
        for f in files:
            f.close()
