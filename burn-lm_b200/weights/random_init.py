"""The random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed.

Every tensor is drawn from its own generator, seeded by a hash of the seed and the tensor's name,
so a tensor's values do not depend on which other tensors exist or in which order they are made.
Matrices are N(0, std) and norm weights 1 + N(0, std), as each part's `TensorSpec.init` says.  The
reference re-initialises modules for its tests with `Reinitializer` (crates/burn-lm-llama/src/
lib.rs:30-215); the distributions here are the ones the benchmark configurations name.
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

from .safetensors_io import write_safetensors

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & (2**63 - 1)


def random_tensor(spec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    if spec.kind == "int":
        raise ValueError(f"tensor {spec.name!r}: integer tables have no random initialiser")
    kind, _, arg = spec.init.partition(":")
    std = float(arg)
    g = torch.Generator(device=device)
    g.manual_seed(tensor_seed(seed, spec.name))
    t = torch.empty(tuple(spec.shape), dtype=torch.float32, device=device)
    t.normal_(0.0, std, generator=g)
    if kind == "one_plus_normal":
        t += 1.0
    elif kind != "normal":
        raise ValueError(f"tensor {spec.name!r}: unknown initialiser {spec.init!r}")
    return t.to(dtype)


def write_random_model(folder: str, config: dict, seed: int, dtype: str = "bfloat16", device="cpu") -> str:
    """Create `folder` with config.json and model.safetensors for the architecture `config` names.

    `device` is where the numbers are drawn (the values differ between "cpu" and "cuda")."""
    from ..model import tensor_specs_of  # late: model imports the parts, the parts import weights

    if dtype not in _DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {dtype!r}")
    specs = tensor_specs_of(config)
    os.makedirs(folder, exist_ok=True)
    cfg = dict(config)
    cfg["torch_dtype"] = dtype
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    tensors = {s.name: random_tensor(s, seed, _DTYPES[dtype], device).cpu() for s in specs}
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed})
    return folder
