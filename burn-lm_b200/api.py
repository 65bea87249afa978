"""The Python entry point: load a model folder, generate from token ids, step by hand.

It follows the reference's server interface (trait InferenceServer: load, is_loaded, unload,
run_job, clear_state; crates/burn-lm-inference/src/server.rs:21-52) and its per-request options
(Llama3ServerConfig: top_p 0.9, temperature 0.0, max_seq_len 8192, sample_len 4096, seed 0;
crates/burn-lm-llama/src/server/llama3.rs:14-31).  Text is out of scope: prompts and answers are
token ids.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Optional, Sequence

from .engine.engine import Engine
from .kernels import PAGE
from .engine.generate import GenerateOptions, GenerationLoop, GenerationOutput
from .model import load_model, random_model
from .sampling.sampler import Sampler


class LanguageModel:
    """A loaded model with its cache, generation loop and sampler."""

    def __init__(self, folder: Optional[str], dtype: str = "bfloat16", max_seq_len: int = 8192, max_batch: int = 8,
                 max_tokens: Optional[int] = None, device: str = "cuda:0", decode_ahead: bool = False,
                 random_config: Optional[dict] = None, random_seed: int = 0):
        """`folder`: a model folder; or None with `random_config` (a config.json dict) and `random_seed`: the model
        is then built with random weights drawn on the device (see model.random_model).
        `decode_ahead`: greedy generation enqueues the step after the one it waits for (fed on the device), so
        the GPU does not idle while the host looks at a step's tokens; off, every step brings its tokens from
        the host.  The tokens are the same either way."""
        self.folder, self.dtype, self.device = folder, dtype, device
        self.decode_ahead = decode_ahead
        if (folder is None) == (random_config is None):
            raise ValueError("a LanguageModel takes a folder, or a configuration to fill with random weights")
        self.random_config, self.random_seed = random_config, random_seed
        self.max_seq_len, self.max_batch, self.max_tokens = max_seq_len, max_batch, max_tokens
        self.engine: Optional[Engine] = None
        self.loop: Optional[GenerationLoop] = None
        self.load_seconds = 0.0
        # one job at a time, as the reference's channel to a server holds a mutex around every call
        # (crates/burn-lm-inference/src/channels/mutex.rs:27-77)
        self._lock = threading.RLock()

    # -- the reference's server interface --------------------------------------------------------
    def load(self) -> "LanguageModel":
        with self._lock:
            return self._load()

    def _load(self) -> "LanguageModel":
        if self.engine is None:
            t0 = time.perf_counter()
            if self.folder is not None:
                model = load_model(self.folder, self.dtype, self.device)
            else:
                model = random_model(self.random_config, self.random_seed, self.dtype, self.device)
            seq = min(self.max_seq_len, model.plan.max_positions)
            tokens = self.max_tokens or -(-seq // PAGE) * PAGE * self.max_batch
            self.engine = Engine(model, max_tokens=tokens, max_seqs=max(self.max_batch, 1), max_seq_len=seq)
            self.engine.decode_ahead = self.decode_ahead
            self.loop = GenerationLoop(self.engine, Sampler(model.runtime.device), model.plan.stop_ids)
            self.load_seconds = time.perf_counter() - t0
        return self

    def is_loaded(self) -> bool:
        return self.engine is not None

    def unload(self) -> None:
        with self._lock:
            self.engine = self.loop = None
        import torch
        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    def clear_state(self) -> None:
        """Give every slot and page back (every request re-reads its whole prompt anyway)."""
        with self._lock:
            if self.engine is not None:
                self.engine.cache.release_all()

    def run_job(self, prompts, **options) -> GenerationOutput:
        return self.generate(prompts, **options)

    # -- generation ------------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], temperature: float = 0.0, top_p: float = 0.9,
                 sample_len: int = 4096, seed: int = 0, stop_ids: Sequence[int] = (), ignore_stop: bool = False,
                 include_stop: bool = False, batch_size: Optional[int] = None, on_token: Optional[Callable] = None) -> GenerationOutput:
        """Generate up to sample_len tokens for every prompt (lists of token ids).

        temperature 0 is greedy; otherwise tokens are drawn from the top_p nucleus of
        softmax(logits / temperature).  seed 0 takes a new random seed.  Prompts run in batches of
        unequal lengths, batch after batch; a sequence ends at a stop id (the model's eos ids and
        `stop_ids`), at sample_len or at the context limit; the stop id is counted but left out of the
        output unless `include_stop`.  One call runs at a time; a second thread waits."""
        single = bool(prompts) and isinstance(prompts[0], int)
        if single:
            prompts = [prompts]
        opts = GenerateOptions(temperature=temperature, top_p=top_p, sample_len=sample_len, seed=seed,
                               stop_ids=tuple(stop_ids), ignore_stop=ignore_stop, include_stop=include_stop,
                               batch_size=batch_size)
        with self._lock:
            self._load()
            return self.loop.generate(prompts, opts, on_token)


def load(folder: str, dtype: str = "bfloat16", max_seq_len: int = 8192, max_batch: int = 8,
         max_tokens: Optional[int] = None, device: str = "cuda:0", decode_ahead: bool = False) -> LanguageModel:
    """Load the model a folder's config.json names; see LanguageModel."""
    return LanguageModel(folder, dtype, max_seq_len, max_batch, max_tokens, device, decode_ahead).load()


def load_random(config: dict, seed: int = 0, dtype: str = "bfloat16", max_seq_len: int = 8192, max_batch: int = 8,
                max_tokens: Optional[int] = None, device: str = "cuda:0") -> LanguageModel:
    """A model of the configuration `config` (a config.json dict, e.g. config.preset("llama3_2_3b")) with random
    weights drawn on the device from `seed`."""
    return LanguageModel(None, dtype, max_seq_len, max_batch, max_tokens, device, random_config=config, random_seed=seed).load()
