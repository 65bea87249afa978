"""Compiles the CUDA sources of this folder for sm_100a, one shared library per module, on first use.

A module is built when something first asks for one of its kernels, so a program compiles only
what its model needs.  The library's file name carries a hash of its sources and flags: a changed
source is rebuilt, an unchanged one is reused.  Libraries go to `_build/` beside the sources when
that folder can be written, else to a per-user folder under the system's temporary folder.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

# extra compiler flags from the environment, e.g. -DBLM_TRACE for the device-side timeline
NVCC_FLAGS += os.environ.get("BURN_LM_B200_NVCC_FLAGS", "").split()

# module name -> its sources (headers every module includes are hashed too)
MODULES = {
    "elementwise": ["elementwise.cu"],
    "attention": ["attention.cu"],
    "gemm": ["gemm_f32.cu"],
    "gemv": ["gemv.cu"],
    "gemm_tc": ["gemm_tc.cu"],
    "gemm_sk": ["gemm_sk.cu"],
    "sampling": ["sampling.cu"],
    "runtime": ["runtime.cu"],
}
HEADERS = ["common.cuh", "attention_decode.cuh", "attention_prefill.cuh", "attention_prefill_tc.cuh", "sampling_no_alloc.h"]

_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found: the CUDA kernels of burn-lm_b200 cannot be compiled "
                     "(set NVCC or put /usr/local/cuda/bin on PATH)")


def _digest(module: str) -> str:
    h = hashlib.sha256()
    for name in MODULES[module] + HEADERS:
        with open(os.path.join(HERE, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:12]


_dir: str | None = None
_dir_lock = threading.Lock()


def _build_dir() -> str:
    """Where the libraries go: decided once per process (the probe below is not safe to run from two threads)."""
    global _dir
    with _dir_lock:
        if _dir is None:
            _dir = _find_build_dir()
        return _dir


def _find_build_dir() -> str:
    d = os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        uid = os.getuid() if hasattr(os, "getuid") else 0
        d = os.path.join(tempfile.gettempdir(), f"burn-lm_b200-build-{uid}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(module: str) -> str:
    return os.path.join(_build_dir(), f"libblm_{module}_{_digest(module)}.so")


def build(module: str, verbose: bool = True) -> str:
    """Compile one module if its library is not there yet; returns the library's path."""
    if module not in MODULES:
        raise BuildError(f"unknown kernel module {module!r}; known: {sorted(MODULES)}")
    out = library_path(module)
    if os.path.exists(out):
        return out
    srcs = [os.path.join(HERE, s) for s in MODULES[module]]
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", HERE, "-o", tmp, *srcs]
    if verbose:
        print(f"[burn-lm_b200] compiling kernels '{module}' for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            log, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[burn-lm_b200]   still compiling '{module}' ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise BuildError(f"nvcc failed for module {module!r}:\n{log}")
    os.replace(tmp, out)
    for old in os.listdir(os.path.dirname(out)):    # libraries of older sources of this module
        if re.fullmatch(rf"libblm_{module}_[0-9a-f]{{12}}\.so", old) and old != os.path.basename(out):
            try:
                os.remove(os.path.join(os.path.dirname(out), old))
            except OSError:
                pass
    if verbose:
        print(f"[burn-lm_b200] compiled '{module}' in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def build_many(modules, verbose: bool = True) -> list[str]:
    """Compile several modules side by side (a compiler process each); returns their libraries' paths."""
    todo = [m for m in modules if not os.path.exists(library_path(m))]
    if len(todo) > 1:
        threads = [threading.Thread(target=build, args=(m, verbose)) for m in todo]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
    return [build(m, verbose) for m in modules]      # reports a failed build's error; built ones are found


def build_all(verbose: bool = True) -> list[str]:
    return [build(m, verbose) for m in MODULES]


def load(module: str) -> ctypes.CDLL:
    """The module's library, compiled first if need be.  Fails loudly: there is no fallback."""
    with _lock:
        lib = _loaded.get(module)
        if lib is None:
            lib = ctypes.CDLL(build(module))
            _loaded[module] = lib
        return lib
