"""Decode steps as CUDA graphs: one token for each of B sequences, with every launch of the step
captured once and replayed.

What changes from step to step (tokens, positions, slots, block tables, lengths) lives in device
buffers with fixed addresses, so one graph per batch size serves every step and every set of
sequences.  `DecodeGraph.step` takes a step's tokens from pinned host memory and leaves the logits
in a fixed buffer; `DecodeGraph.run` goes on for many steps without the host in between: the greedy
token of a step is written back as the next step's input by a kernel inside the graph.
"""
from __future__ import annotations

import contextlib
import gc
import weakref

import torch

from .. import kernels as K
from ..parts.base import StepContext
from .engine import Workspace

# A captured step that samples hands its tokens to the host through pinned memory that its last kernel writes and the
# native step driver polls (no copy out, no wait for the stream: 14 us of a 0.79 ms step at batch 8).  False: the
# tokens are copied out and the stream is waited for.
RESULTS_BY_POLLING = True


@contextlib.contextmanager
def _capturing(graph, pool=None):
    """Capture with the garbage collector held back: a collection in the middle of a capture may
    destroy an older CUDA graph, which CUDA does not permit while a stream is capturing.  `pool`: the
    memory pool of graphs that run one after another and may share their buffers."""
    gc.collect()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph, pool=pool):
            yield
    finally:
        if was_enabled:
            gc.enable()


class StepInFlight:
    """A greedy decode step that has been enqueued: the sequences' slots, their lengths before it, the tokens
    it was fed (None until known: a chained step is fed on the device) and where its result will be."""

    def __init__(self, graph, slots, starts, tokens_in, done, host):
        self.graph, self.slots, self.starts, self.tokens_in = graph, slots, starts, tokens_in
        self._done, self._host = done, host

    def tokens(self) -> list:
        """The sampled tokens, in the order of `slots` (waits for the step)."""
        self._done.synchronize()
        return self._host.numpy().tolist()


class DecodeGraph:
    def __init__(self, engine, batch: int, max_kv_len: int):
        self._engine = weakref.ref(engine)      # the engine owns its graphs, not the other way round
        self.batch, self.max_kv_len = batch, max_kv_len
        dev = engine.model.runtime.device
        b = batch
        # tokens | positions | slots: what a step brings, in one buffer, one copy
        self.meta = torch.zeros(3 * b, dtype=torch.int32, device=dev)
        self.host_meta = torch.zeros(3 * b, dtype=torch.int32, pin_memory=True)
        self._host_meta_np = self.host_meta.numpy()             # the same pinned bytes, filled without a tensor in between
        self.host_sampled = torch.zeros(b, dtype=torch.int32, pin_memory=True)
        self._host_sampled_np = self.host_sampled.numpy()
        # the buffer a sampling kernel writes the tokens to as well, where the device can address pinned host memory
        try:
            self.mirror = self.host_sampled if K.host_device_pointer(self.host_sampled) else None
        except K.KernelError:
            self.mirror = None
        self.tokens, self.pos, self.slots = self.meta[:b], self.meta[b:2 * b], self.meta[2 * b:]
        ar = torch.arange(b + 1, dtype=torch.int32, device=dev)
        self.ctx = StepContext(
            n_tokens=b, n_seqs=b, max_q_len=1, max_kv_len=max_kv_len,
            tokens=self.tokens, token_seq=ar[:b], token_pos=self.pos, cu_seqlens=ar, slot_of_seq=self.slots,
            start_pos=self.pos, want_rows=ar[:b], n_want=b,
            workspace=Workspace(dev),     # its own: a captured graph keeps the addresses it saw
           
            host={"cu_seqlens": list(range(b + 1)), "slots": None, "start_pos": None})
        self.sampled = torch.zeros(b, dtype=torch.int32, device=dev)
        self.step_no = torch.zeros(1, dtype=torch.int32, device=dev)
        self.tickets = torch.zeros(b + 1, dtype=torch.int32, device=dev)     # the argmax kernel's, zero between launches
        self.history = None
        self.logits = None
        self._graph = None          # forward only
        self._loop_graph = None     # forward + argmax + advance
        self._greedy_graph = None   # forward + argmax
        self._greedy_exec = None    # its cudaGraphExec_t (an integer) once known; False when torch does not give it out
        self._greedy_again = None   # (stream, the native call for one more step on it)
        self._sample_again = None
        self._chain_graph = None    # forward + argmax + advance: a step whose successor needs nothing from the host
        self._chain_out = None      # two pinned buffers for its results, used in turn
        self._chain_launches = 0
        self._sample_graph = None   # forward + temperature / nucleus draw
        self._sample_exec = None
        self._sample_key = None     # (sampling parameters, stream ids) now in the graph's buffers
        self._sample_f = self._sample_ids = self._sample_counters = None
        self._loop_history_steps = 0
        self._copied = None
        self.launches_per_step = 0

    @property
    def engine(self):
        return self._engine()

    def bytes_in_per_step(self) -> int:
        return self.host_meta.numel() * 4

    def load(self, tokens, positions, slots) -> None:
        """Bring a step's inputs from (pinned) host memory to the graph's buffers."""
        if self._copied is not None:
            self._copied.synchronize()       # the last copy has left the pinned buffer
        self._host_meta_np[:] = [*tokens, *positions, *slots]
        self.meta.copy_(self.host_meta, non_blocking=True)
        self._copied = torch.cuda.Event()
        self._copied.record()
        self.ctx.host["slots"], self.ctx.host["start_pos"] = list(slots), list(positions)

    def _forward(self):
        return self.engine.model.forward(self.ctx, self.engine.cache)

    def step(self) -> torch.Tensor:
        """One decode step on the loaded inputs; fp32 logits [B, vocab] in a buffer that the next
        step overwrites."""
        if self._graph is None:
            self.logits = self._forward()            # the first step runs plainly and warms everything up
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with _capturing(g):
                self._captured_logits = self._forward()
            self._graph = g
            return self.logits
        self._graph.replay()
        return self._captured_logits

    def step_greedy(self) -> torch.Tensor:
        """One decode step on the loaded inputs with the argmax inside the captured graph; the
        sampled tokens, int32 [B], in a buffer that the next step overwrites."""
        if self._greedy_graph is None:
            K.argmax(self._forward(), self.sampled, tickets=self.tickets)  # the first step runs plainly and warms everything up
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with _capturing(g):
                K.argmax(self._forward(), self.sampled, mirror=self.mirror, tickets=self.tickets)
            self._greedy_graph = g
            return self.sampled
        self._greedy_graph.replay()
        return self.sampled

    def step_greedy_host(self, tokens, positions, slots) -> list:
        """A greedy step from host inputs to host outputs: the inputs go from pinned memory to the graph's
        buffers, the captured step runs, the sampled tokens come back through pinned memory as a list.
        Once the graph exists, native code issues the copies, the launch and the wait in one call."""
        if self._greedy_exec:
            self._host_meta_np[:] = [*tokens, *positions, *slots]
            self.ctx.host["slots"], self.ctx.host["start_pos"] = list(slots), list(positions)
            stream = K.stream_handle()
            if self._greedy_again is None or self._greedy_again[0] != stream:
                # the captured argmax writes the pinned buffer itself (its `mirror`): nothing to copy out
                self._greedy_again = (stream, K.graph_step(self._greedy_exec, self.meta, self.host_meta, self.host_sampled,
                                                           self.sampled, written_by_graph=RESULTS_BY_POLLING and self.mirror is not None))
            else:
                self._greedy_again[1]()
            return self._host_sampled_np.tolist()
        self.load(tokens, positions, slots)
        sampled = self.step_greedy()
        self.host_sampled.copy_(sampled, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        if self._greedy_graph is not None and self._greedy_exec is None:
            try:        # the instantiated graph's handle, where this torch gives it out
                self._greedy_exec = int(self._greedy_graph.raw_cuda_graph_exec()) or None
            except Exception:
                self._greedy_exec = None
            if self._greedy_exec is None:
                self._greedy_exec = False      # asked once; stay on the interpreter's path
        return self._host_sampled_np.tolist()

    def launch_greedy_chained(self, tokens, positions, slots) -> "StepInFlight":
        """Enqueue one greedy step and the copy of its sampled tokens to pinned memory, and come back without
        waiting.  The captured step ends by feeding itself: tokens = sampled, positions += 1 on the device, so
        the step after it can be enqueued with `tokens=None` before this one's result has reached the host.
        The result is in `StepInFlight.tokens()` once its event has passed."""
        if tokens is not None:
            self.load(tokens, positions, slots)
        else:
            self.ctx.host["slots"], self.ctx.host["start_pos"] = list(slots), list(positions)
        if self._chain_out is None:
            self._chain_out = [torch.zeros(self.batch, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        if self._chain_graph is None:
            self._one_chained_step()                 # the first step runs plainly and warms everything up
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with _capturing(g):
                self._one_chained_step()
            self._chain_graph = g
        else:
            self._chain_graph.replay()
        host = self._chain_out[self._chain_launches % 2]
        self._chain_launches += 1
        host.copy_(self.sampled, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return StepInFlight(self, list(slots), list(positions), None if tokens is None else list(tokens), done, host)

    def _one_chained_step(self):
        K.argmax(self._forward(), self.sampled, tickets=self.tickets, advance=(self.tokens, self.pos, None, self.step_no))

    def step_sampled_host(self, tokens, positions, slots, params, stream_ids, counters) -> list:
        """A step that draws its tokens by temperature and nucleus inside the captured graph, from host
        inputs to host outputs.  temperature, top-p, seed and the sequences' stream ids sit in device
        buffers of the graph (rewritten when they change); a step brings its draw counters beside its
        tokens, positions and slots."""
        mask = (1 << 63) - 1
        b = self.batch
        key = (params, tuple(stream_ids))
        if self._sample_key != key:
            if self._sample_f is None:
                dev = self.meta.device
                self._sample_f = torch.zeros((2, b), dtype=torch.float32, device=dev)
                self._sample_ids = torch.zeros((2, b), dtype=torch.int64, device=dev)
                self._sample_counters = torch.zeros(b, dtype=torch.int64, device=dev)
                self._host_counters = torch.zeros(b, dtype=torch.int64, pin_memory=True)
                self._host_counters_np = self._host_counters.numpy()
            self._sample_f.copy_(torch.tensor([[params.temperature] * b, [params.top_p] * b], dtype=torch.float32))
            self._sample_ids.copy_(torch.tensor([[params.seed & mask] * b, [s & mask for s in stream_ids]], dtype=torch.int64))
            self._sample_key = key
        self._host_counters_np[:] = [c & mask for c in counters]
        self.ctx.host["slots"], self.ctx.host["start_pos"] = list(slots), list(positions)

        def draw():
            K.sample(self._forward(), self._sample_f[0], self._sample_f[1], self._sample_ids[0], self._sample_ids[1],
                     self._sample_counters, self.sampled, mirror=self.mirror)

        if self._sample_exec:
            self._host_meta_np[:] = [*tokens, *positions, *slots]
            stream = K.stream_handle()
            if self._sample_again is None or self._sample_again[0] != stream:
                self._sample_again = (stream, K.graph_step(self._sample_exec, self.meta, self.host_meta, self.host_sampled, self.sampled,
                                                           dev_in2=self._sample_counters, host_in2=self._host_counters,
                                                           written_by_graph=RESULTS_BY_POLLING and self.mirror is not None))
            else:
                self._sample_again[1]()
            return self._host_sampled_np.tolist()
        self.load(tokens, positions, slots)
        self._sample_counters.copy_(self._host_counters, non_blocking=True)
        if self._sample_graph is None:
            draw()                                   # the first step runs plainly and warms everything up
            torch.cuda.synchronize()
            result = self.sampled.tolist()
            g = torch.cuda.CUDAGraph()
            with _capturing(g):
                draw()
            self._sample_graph = g
            try:
                self._sample_exec = int(g.raw_cuda_graph_exec()) or False
            except Exception:
                self._sample_exec = False            # stay on the interpreter's path
            return result
        self._sample_graph.replay()
        self.host_sampled.copy_(self.sampled, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._host_sampled_np.tolist()

    def run(self, n_steps: int, keep_history: bool = True) -> torch.Tensor:
        """n_steps greedy decode steps without the host in between, starting from the loaded inputs.
        Pages for positions up to (loaded position + n_steps) must be reserved.  Returns the sampled
        tokens int32 [n_steps, B] (on the device)."""
        if self._loop_graph is None or (keep_history and self._loop_history_steps < n_steps):
            self._loop_history_steps = max(n_steps, 256)
            self.history = torch.zeros((self._loop_history_steps, self.batch), dtype=torch.int32, device=self.meta.device)
            saved = self.meta.clone()
            self._one_loop_step()                    # warm-up, undone below
            torch.cuda.synchronize()
            self.meta.copy_(saved)
            g = torch.cuda.CUDAGraph()
            before = K.launch_count()
            with _capturing(g):
                self._one_loop_step()
            self.launches_per_step = K.launch_count() - before   # this package's kernels in one replay
            self._loop_graph = g
        self.step_no.zero_()
        for _ in range(n_steps):
            self._loop_graph.replay()
        return self.history[:n_steps]

    def _one_loop_step(self):
        logits = self._forward()
        K.argmax(logits, self.sampled, tickets=self.tickets, advance=(self.tokens, self.pos, self.history, self.step_no))
