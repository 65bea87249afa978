"""Python faces of the CUDA kernels in `csrc/`.

Each function checks what it is given, hands raw device pointers to the C entry point of the same
name, and raises `KernelError` with the kernel's own message when that refuses.  Kernels run on
torch's current CUDA stream, so they can be captured in a CUDA graph with the matrix products
around them.  There is no fallback: without a CUDA device or without the compiled library these
functions raise.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_size_t, c_uint, c_ulonglong, c_void_p

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
PAGE = 64  # positions per cache page; the attention kernels are written for this size


class KernelError(RuntimeError):
    pass


_sm_counts: dict = {}


def sm_count(device=None) -> int:
    """How many multiprocessors the device has (asked once per device)."""
    index = torch.device(device).index if device is not None else None
    if index is None:
        index = torch.cuda.current_device()
    n = _sm_counts.get(index)
    if n is None:
        n = _sm_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return n


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dtype}")


def _ptr(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """torch's current stream on the current device, as a raw handle.  Asked once per launch: the short way
    (two calls into torch's C module) costs a tenth of building a torch.cuda.Stream object each time."""
    if _raw_stream is not None and _current_device is not None:
        return c_void_p(_raw_stream(_current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("burn-lm_b200 kernels run on a CUDA device only; got a CPU tensor")
        if t is not None and not t.is_contiguous():
            raise KernelError("kernel arguments must be contiguous")


_protos = {
    "elementwise": {
        "blm_embed": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p],
        "blm_add_rmsnorm": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int,
                            c_float, c_void_p],
        "blm_rope_append": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                            c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p],
        "blm_rope_table": [c_void_p, c_void_p, c_int, c_int, c_void_p],
        "blm_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "blm_convert": [c_void_p, c_int, c_void_p, c_int, c_size_t, c_void_p],
        "blm_decode_advance": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "blm_step_tables": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
    },
    "attention": {
        "blm_attention": [c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
                          c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                          c_int, c_int, c_float, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p],
    },
    "gemm": {
        "blm_gemm_f32": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong,
                         c_longlong, c_void_p],
    },
    "gemv": {
        "blm_gemv": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int,
                     c_float, c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p, c_int,
                     c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "blm_gemv_supported": [c_int, c_int, c_int, c_int],
    },
    "runtime": {
        "blm_graph_step": [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong,
                           c_int, c_void_p],
        "blm_host_device_pointer": [c_void_p, c_void_p],
    },
    "gemm_tc": {
        "blm_gemm_tc": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_int,
                        c_void_p, c_void_p],
        "blm_gemm_tc_supported": [c_int, c_int, c_int],
    },
    "gemm_sk": {
        "blm_gemm_sk": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_longlong, c_int, c_void_p, c_longlong, c_int, c_void_p, c_int,
                        c_void_p, c_int, c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "blm_gemm_sk_supported": [c_int, c_int, c_int],
        "blm_gemm_sk_squares_row": [],
    },
    "sampling": {
        "blm_argmax": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_int, c_void_p],
        "blm_argmax_advances": [c_int],
        "blm_argmax_scratch_floats": [c_int, c_int],
        "blm_sample": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_void_p, c_void_p],
    },
}
_bound: dict[str, ctypes.CDLL] = {}


def _lib(module: str) -> ctypes.CDLL:
    lib = _bound.get(module)
    if lib is None:
        lib = _build.load(module)
        for name, argtypes in _protos.get(module, {}).items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        err = getattr(lib, f"blm_{module}_last_error")
        err.restype = ctypes.c_char_p
        err.argtypes = []
        _bound[module] = lib
    return lib


def prebuild(dtype) -> None:
    """Compile, side by side, the modules that every step of a model of this dtype uses, so that a first
    call waits for the slowest of them instead of for their sum.  The others are still built when first used."""
    _build.build_many(["elementwise", "attention", "gemv" if dtype == torch.bfloat16 else "gemm"])


_launches = 0


def launch_count() -> int:
    """How many kernels of this package have been launched (or captured) by this process."""
    return _launches


def stream_handle() -> int:
    """torch's current stream as an integer."""
    return _stream().value or 0


def _call(module: str, name: str, *args, kernels: int = 1):
    global _launches
    lib = _lib(module)
    rc = getattr(lib, name)(*args)
    _launches += kernels
    if rc != 0:
        msg = getattr(lib, f"blm_{module}_last_error")().decode(errors="replace")
        raise KernelError(f"{name}: {msg}")


def loaded_modules():
    return sorted(_bound)


# ------------------------------------------------------------------------------------------------
def embed(tokens, table, out, hand_over=None):
    """out[n, :] = table[tokens[n], :] as fp32.  tokens int32 [N]; table [V, D]; out fp32 [N, D].
    `hand_over` = (gamma [D], scaled bfloat16 [N, D], squares float32 [1, SQUARES_ROWS]) for up to SQUARES_ROWS
    tokens: the kernel also leaves the input of the norm that reads the stream first, scaled = out * gamma and the
    rows' sums of squares in one part, as gemv's `hand_over` does."""
    _need_cuda(tokens, table, out)
    n, (v, d) = tokens.numel(), table.shape
    if tokens.dtype != torch.int32 or out.dtype != torch.float32 or tuple(out.shape) != (n, d):
        raise KernelError("embed: tokens int32 [N], out float32 [N, D]")
    gamma = scaled = squares = None
    if hand_over is not None:
        gamma, scaled, squares = hand_over
        _need_cuda(gamma, scaled, squares)
        if (n > SQUARES_ROWS or gamma.numel() != d or scaled.dtype != torch.bfloat16 or tuple(scaled.shape) != (n, d)
                or not scaled.is_contiguous() or squares.dtype != torch.float32 or tuple(squares.shape) != (1, SQUARES_ROWS)):
            raise KernelError("embed: hand_over = (gamma [D], scaled bfloat16 [N, D], squares float32 [1, 16]) for up to 16 tokens")
    _call("elementwise", "blm_embed", _ptr(tokens), _ptr(table), _code(table.dtype), _ptr(out), n, d, v,
          _ptr(gamma), 1 if (gamma is not None and gamma.dtype == torch.float32) else 0, _ptr(scaled), _ptr(squares),
          SQUARES_ROWS, _stream())


def add_rmsnorm(resid, delta, gamma, eps, out, rows=None):
    """Residual add fused with the RMS norm, in fp32.

    rows is None: resid[n] += delta[n] (stored), out[n] = norm(resid[n]) * gamma for every row.
    rows given (int32 [R]): out[i] = norm(resid[rows[i]] + delta[rows[i]]) * gamma; resid unchanged.
    delta may be None.  resid is fp32 [N, D]; delta and out have the activation dtype."""
    _need_cuda(resid, delta, gamma, out, rows)
    d = resid.shape[-1]
    n_out = rows.numel() if rows is not None else resid.shape[0]
    if resid.dtype != torch.float32 or gamma.numel() != d or tuple(out.shape) != (n_out, d):
        raise KernelError("add_rmsnorm: resid float32 [N, D], gamma [D], out [rows, D]")
    if delta is not None and (delta.dtype != out.dtype or delta.shape != resid.shape):
        raise KernelError("add_rmsnorm: delta must match resid's shape and out's dtype")
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("add_rmsnorm: rows must be int32")
    _call("elementwise", "blm_add_rmsnorm", _ptr(resid), _ptr(delta), _ptr(gamma), _code(gamma.dtype), _ptr(out),
          _code(out.dtype), _ptr(rows), n_out, d, c_float(eps), _stream())


def rope_table(inv_freq, n_positions):
    """(cos, sin) of position * inv_freq for positions below n_positions: float32 [n_positions, half, 2],
    computed in float64 on the device; rope_append reads it instead of computing angles per token."""
    _need_cuda(inv_freq)
    half = inv_freq.numel()
    table = torch.empty((n_positions, half, 2), dtype=torch.float32, device=inv_freq.device)
    _call("elementwise", "blm_rope_table", _ptr(inv_freq), _ptr(table), n_positions, half, _stream())
    return table


PAIRS_HALVES, PAIRS_INTERLEAVED, PAIRS_TILED = 0, 1, 2


def rope_append(qkv, token_seq, token_pos, slot_of_seq, block_table, inv_freq, rotary_dim, interleaved,
                pool, n_heads, n_kv, head_dim, write_cache=True, table=None, max_position=None):
    """Rotate q (in place) and k of every token by its position, and append k, v to the paged cache.

    `interleaved`: False or PAIRS_HALVES: pair i is lanes (i, i + rotary_dim / 2); True or
    PAIRS_INTERLEAVED: lanes (2i, 2i + 1); PAIRS_TILED: lanes (16 (i // 8) + i % 8, that + 8), the order
    of a head whose weight rows were dealt out with tiled_pair_order().

    qkv [N, (n_heads + 2 n_kv) * head_dim]; pool [pages, 2, n_kv, PAGE, head_dim] of one cache line;
    inv_freq float64 [rotary_dim / 2] or None when rotary_dim == 0; `table` (from rope_table) spares
    the per-token angles for positions it covers.  `max_position`: an upper bound of the step's
    positions known on the host; when the table covers it, the vector kernel may run."""
    _need_cuda(qkv, token_seq, token_pos, slot_of_seq, block_table, inv_freq, pool, table)
    if table is not None and (table.dtype != torch.float32 or tuple(table.shape[1:]) != (rotary_dim // 2, 2)):
        raise KernelError("rope_append: table must be float32 [positions, rotary_dim / 2, 2]")
    n = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv) * head_dim:
        raise KernelError("rope_append: qkv width does not match the head counts")
    if write_cache:
        if pool.dtype != qkv.dtype or tuple(pool.shape[1:]) != (2, n_kv, PAGE, head_dim):
            raise KernelError(f"rope_append: pool must be [pages, 2, {n_kv}, {PAGE}, {head_dim}] of {qkv.dtype}")
    if rotary_dim:
        if inv_freq.dtype != torch.float64 or inv_freq.numel() != rotary_dim // 2:
            raise KernelError("rope_append: inv_freq must be float64 [rotary_dim / 2]")
    _call("elementwise", "blm_rope_append", _ptr(qkv), _code(qkv.dtype), _ptr(token_seq), _ptr(token_pos),
          _ptr(slot_of_seq), _ptr(block_table), block_table.shape[1], _ptr(inv_freq), rotary_dim,
          int(interleaved), _ptr(pool), n, n_heads, n_kv, head_dim, PAGE, 1 if write_cache else 0,
          _ptr(table), table.shape[0] if table is not None else 0,
          1 if (table is not None and max_position is not None and max_position < table.shape[0]) else 0, _stream())


def tiled_pair_order(head_dim: int) -> list:
    """For PAIRS_TILED: which lane of a head (in the stored order, pairs (i, i + head_dim / 2)) goes to each
    place: every 16 places hold lanes 8j .. 8j + 7 and then their partners."""
    half = head_dim // 2
    return [(8 * (p // 16) + p % 16) if p % 16 < 8 else (half + 8 * (p // 16) + p % 16 - 8) for p in range(head_dim)]


GATE_TILE = 8   # a fused [gate; up] weight for the skinny kernel: tiles of 8 gate rows, then their 8 up rows


def swiglu(gate_up, out, tile=0):
    """out[n, i] = silu(gate_i) * up_i.  gate_up [N, 2 I] holds all gates then all ups (tile 0), or
    tiles of `tile` gates followed by the ups of the same outputs."""
    _need_cuda(gate_up, out)
    n, two_i = gate_up.shape
    if tuple(out.shape) != (n, two_i // 2) or out.dtype != gate_up.dtype or two_i % 2:
        raise KernelError("swiglu: out must be [N, I] for gate_up [N, 2 I], same dtype")
    _call("elementwise", "blm_swiglu", _ptr(gate_up), _ptr(out), _code(out.dtype), n, two_i // 2, tile, _stream())


def convert(src, dst):
    """dst = src in the other of float32 / bfloat16."""
    _need_cuda(src, dst)
    if src.numel() != dst.numel():
        raise KernelError("convert: sizes differ")
    _call("elementwise", "blm_convert", _ptr(src), _code(src.dtype), _ptr(dst), _code(dst.dtype),
          c_size_t(src.numel()), _stream())


def decode_advance(tokens, pos, sampled, history, step_no, counters=None):
    """Between two decode steps that run without the host: tokens = sampled, pos += 1 (and counters += 1),
    history[step_no] = sampled, step_no += 1.  All int32 on the device (counters int64)."""
    _need_cuda(tokens, pos, sampled, history, step_no, counters)
    b = tokens.numel()
    steps = history.shape[0] if history is not None else 0
    _call("elementwise", "blm_decode_advance", _ptr(tokens), _ptr(pos), _ptr(sampled), _ptr(history), _ptr(step_no),
          _ptr(counters), b, steps, _stream(), kernels=2)


def step_tables(token_seq, token_pos, slot_of_seq, block_table, n_seqs):
    """Looked up once per step for all layers that share a block table: (token_page int32 [N], the page every new
    token goes to, -1 for a row of no sequence; seq_table int32 [n_seqs, pages per sequence], the block table's
    rows in the order of the step's sequences)."""
    _need_cuda(token_seq, token_pos, slot_of_seq, block_table)
    n = token_seq.numel()
    token_page = torch.empty(n, dtype=torch.int32, device=block_table.device)
    seq_table = torch.empty((n_seqs, block_table.shape[1]), dtype=torch.int32, device=block_table.device)
    _call("elementwise", "blm_step_tables", _ptr(token_seq), _ptr(token_pos), _ptr(slot_of_seq), _ptr(block_table),
          block_table.shape[1], PAGE, n, n_seqs, _ptr(token_page), _ptr(seq_table), _stream())
    return token_page, seq_table


def attention_decode_is_specialised(dtype, head_dim, group) -> bool:
    """Whether a step of one token per sequence runs the specialised decode kernel (whose blocks
    split the keys by pages and skip splits a sequence does not need)."""
    return dtype == torch.bfloat16 and head_dim in (64, 128) and 1 <= group <= 8


def attention_scratch_floats(n_tokens, n_heads, head_dim, n_splits):
    return 0 if n_splits <= 1 else n_tokens * n_heads * n_splits * (head_dim + 2)


def attention(q, q_stride, pool, block_table, cu_seqlens, slot_of_seq, start_pos, out, n_tokens, n_seqs,
              max_q_len, n_heads, n_kv, head_dim, scale, window=0, n_splits=1, scratch=None, general_only=False,
              max_kv_len=0, seq_table=None, ahead=False):
    """Causal grouped-query attention of the step's tokens over the paged cache (after the append).

    q: tensor whose token n, head h starts at element n * q_stride + h * head_dim (the qkv buffer).
    Token t of sequence s sits at position start_pos[s] + t and sees keys 0..that position (the last
    `window` of them when window > 0).  n_splits > 1 cuts every sequence's keys over that many
    blocks and combines the partial results; it needs `scratch` (float32,
    attention_scratch_floats(...) elements).  bfloat16 steps of one token per sequence with a head
    size of 64 or 128 and up to 8 query heads per kv head run a specialised kernel unless
    `general_only`; `max_kv_len` (the longest sequence after the step, when known) lets it size its
    rings of pages; `seq_table` (from step_tables) spares it the way through the slots.  `ahead`: the kernel
    launched just before this one was gemv() with `rope`, which lets its successor start only after its own wait;
    the specialised kernel then reads the step's tables and fetches the pages of earlier tokens before it waits
    for that kernel itself (for q and the page of the new token).  Say so only when it is so."""
    _need_cuda(q, pool, block_table, cu_seqlens, slot_of_seq, start_pos, out, scratch, seq_table)
    if seq_table is not None and (seq_table.dtype != torch.int32 or tuple(seq_table.shape) != (n_seqs, block_table.shape[1])):
        raise KernelError("attention: seq_table must be int32 [n_seqs, pages per sequence]")
    if tuple(out.shape) != (n_tokens, n_heads * head_dim) or out.dtype != q.dtype or pool.dtype != q.dtype:
        raise KernelError("attention: out must be [N, heads * head_dim] in q's dtype, as the pool")
    if tuple(pool.shape[1:]) != (2, n_kv, PAGE, head_dim):
        raise KernelError(f"attention: pool must be [pages, 2, {n_kv}, {PAGE}, {head_dim}]")
    if n_splits > 1:
        need = attention_scratch_floats(n_tokens, n_heads, head_dim, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention: {n_splits} splits need {need} float32 of scratch")
    _call("attention", "blm_attention", _ptr(q), q_stride, _ptr(pool), _code(q.dtype), _ptr(block_table),
          block_table.shape[1], _ptr(cu_seqlens), _ptr(slot_of_seq), _ptr(start_pos), _ptr(out), _ptr(scratch),
          n_tokens, n_seqs, max_q_len, n_heads, n_kv, head_dim, PAGE, int(window or 0), n_splits,
          c_float(scale), 1 if general_only else 0, _ptr(status_word(q.device)), pool.shape[0], int(max_kv_len), _ptr(seq_table),
          1 if ahead else 0, _stream(), kernels=2 if n_splits > 1 else 1)


def gemm_f32(x, w, out=None):
    """x [N, K] times w [M, K] transposed, in true fp32 (no tensor-core mode)."""
    _need_cuda(x, w, out)
    if x.dtype != torch.float32 or w.dtype != torch.float32 or x.shape[1] != w.shape[1]:
        raise KernelError("gemm_f32: float32 x [N, K] and w [M, K]")
    n, k = x.shape
    m = w.shape[0]
    if out is None:
        out = torch.empty((n, m), dtype=torch.float32, device=x.device)
    elif tuple(out.shape) != (n, m) or out.dtype != torch.float32:
        raise KernelError("gemm_f32: out must be float32 [N, M]")
    _call("gemm", "blm_gemm_f32", _ptr(x), _ptr(w), _ptr(out), n, m, k, k, k, m, _stream())
    return out


EPI_STORE, EPI_SWIGLU, EPI_RESID_ADD, EPI_ROPE = 0, 1, 2, 3


class _GemvRope(ctypes.Structure):
    _fields_ = [("token_pos", c_void_p), ("token_seq", c_void_p), ("slot_of_seq", c_void_p), ("block_table", c_void_p),
                ("table", c_void_p), ("pool", c_void_p), ("table_stride", c_int), ("n_heads", c_int), ("n_kv", c_int),
                ("hd", c_int), ("page_size", c_int), ("write_cache", c_int), ("token_page", c_void_p)]


def gemv_supported(n_tokens, m, k, plain_tokens=False) -> bool:
    """Whether gemv() takes the shape.  `plain_tokens`: the input is a bfloat16 [N, K] tensor used row by row
    (no stream to normalise, no gathered rows): then a very wide K is taken too."""
    return bool(_lib("gemv").blm_gemv_supported(n_tokens, m, k, 1 if plain_tokens else 0))


def gemm_tc_supported(m, n, k) -> bool:
    return bool(_lib("gemm_tc").blm_gemm_tc_supported(m, n, k))


def gemm_tc(x, w, out=None, swiglu=False, add_into=None):
    """x [M, K] times w [N, K] transposed on the tcgen05 tensor cores (bfloat16, fp32 accumulation in
    tensor memory).  out [M, N]; with `swiglu`, w is a fused gate/up weight in tiles of GATE_TILE gate
    rows followed by their up rows and out [M, N / 2] = silu(gate) * up, formed in the epilogue; with
    `add_into` (float32 [M, N], the residual stream) the product is added into it in the epilogue and
    nothing else is written."""
    _need_cuda(x, w, out, add_into)
    m, k = x.shape
    n = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.shape[1] != k:
        raise KernelError("gemm_tc: bfloat16 x [M, K] and w [N, K]")
    if add_into is not None:
        if swiglu or out is not None or add_into.dtype != torch.float32 or tuple(add_into.shape) != (m, n) or add_into.stride(1) != 1:
            raise KernelError("gemm_tc: add_into must be float32 [M, N], alone")
        _call("gemm_tc", "blm_gemm_tc", _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(add_into), add_into.stride(0), m, n, k,
              2, _ptr(status_word(x.device)), _stream())
        return
    if out is None or out.dtype != torch.bfloat16 or tuple(out.shape) != (m, n // 2 if swiglu else n):
        raise KernelError("gemm_tc: out must be bfloat16 [M, N] (or [M, N / 2] with the gated epilogue)")
    _call("gemm_tc", "blm_gemm_tc", _ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), m, n, k,
          1 if swiglu else 0, _ptr(status_word(x.device)), _stream())


SK_SQUARES_ROWS = 64     # row length of the sums of squares that go with a norm handed over between gemm_sk products
SK_TOKENS = 128          # gemm_sk takes up to this many tokens


def gemm_sk_supported(n_tokens, m, k) -> bool:
    return bool(_lib("gemm_sk").blm_gemm_sk_supported(n_tokens, m, k))


def gemm_sk(w, x, out=None, add_into=None, swiglu=False, squares=None, eps=0.0, hand_over=None, rope=None):
    """x [N, K] times w [M, K] transposed for up to 128 tokens on the tcgen05 tensor cores, the weight rows as the
    wide operand, K cut over the blocks of a cluster where the weight has few rows; bfloat16 operands, fp32 sums.

    Ends, one at a time: `out` [N, M] bfloat16 or float32; `swiglu`: w is [2 I, K] in tiles of GATE_TILE gate rows
    followed by their up rows and out [N, I] = silu(gate) * up; `add_into` (fp32 [N, M]) += the product, with
    `hand_over` = (gamma, scaled bfloat16 [N, M], squares float32 [ceil(M / 16), SK_SQUARES_ROWS]) also the next
    norm's input; `rope` (as for gemv): w is a step's [q; k; v] with q and k rows in tiled_pair_order(), q goes
    to `out`, the rotated k and the v to the cache.  `squares` (+ `eps`): x is a handed-over norm,
    bfloat16(stream * gamma), and the results' rows are divided by the stream rows' root mean square."""
    _need_cuda(w, x, out, add_into, squares)
    if w.dtype != torch.bfloat16 or x.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise KernelError("gemm_sk: bfloat16 x [N, K] and w [M, K]")
    n, k = x.shape
    m_rows = w.shape[0]
    m = m_rows // 2 if swiglu else m_rows
    epi = EPI_SWIGLU if swiglu else (EPI_RESID_ADD if add_into is not None else (EPI_ROPE if rope is not None else EPI_STORE))
    if sum(v is not None and v is not False for v in (add_into, rope, swiglu or None)) > 1:
        raise KernelError("gemm_sk: one epilogue at a time")
    rope_arg = None
    if rope is not None:
        r = rope
        hd, table, pool = r["head_dim"], r["table"], r["pool"]
        _need_cuda(r["token_pos"], r["token_seq"], r["slot_of_seq"], r["block_table"], table, pool)
        if table is None or table.dtype != torch.float32 or tuple(table.shape[1:]) != (hd // 2, 2) \
                or r.get("max_position") is None or r["max_position"] >= table.shape[0]:
            raise KernelError("gemm_sk: the rotary epilogue needs a table [positions, head_dim / 2, 2] that covers the step")
        if r["write_cache"] and (pool.dtype != torch.bfloat16 or tuple(pool.shape[1:]) != (2, r["n_kv"], PAGE, hd)):
            raise KernelError(f"gemm_sk: pool must be bfloat16 [pages, 2, {r['n_kv']}, {PAGE}, {hd}]")
        if out is None or out.dtype != torch.bfloat16 or tuple(out.shape) != (n, r["n_heads"] * hd):
            raise KernelError("gemm_sk: the rotary epilogue writes q to a bfloat16 out [N, n_heads * head_dim]")
        rope_arg = _GemvRope(r["token_pos"].data_ptr(), r["token_seq"].data_ptr(), r["slot_of_seq"].data_ptr(),
                             r["block_table"].data_ptr(), table.data_ptr(), pool.data_ptr() if pool is not None else 0,
                             r["block_table"].shape[1], r["n_heads"], r["n_kv"], hd, PAGE, 1 if r["write_cache"] else 0,
                             r["token_page"].data_ptr() if r.get("token_page") is not None else 0)
    if squares is not None and (squares.dtype != torch.float32 or squares.dim() != 2 or squares.shape[1] != SK_SQUARES_ROWS
                                or n > SK_SQUARES_ROWS):
        raise KernelError(f"gemm_sk: squares are float32 [parts, {SK_SQUARES_ROWS}] for up to {SK_SQUARES_ROWS} tokens")
    next_gamma = scaled = squares_out = None
    if hand_over is not None:
        next_gamma, scaled, squares_out = hand_over
        _need_cuda(next_gamma, scaled, squares_out)
        if (epi != EPI_RESID_ADD or scaled.dtype != torch.bfloat16 or tuple(scaled.shape) != (n, m) or squares_out.dtype != torch.float32
                or tuple(squares_out.shape) != ((m + 15) // 16, SK_SQUARES_ROWS) or next_gamma.numel() != m or n > SK_SQUARES_ROWS):
            raise KernelError(f"gemm_sk: hand_over = (gamma [M], scaled bfloat16 [N, M], squares float32 [ceil(M / 16), {SK_SQUARES_ROWS}]) "
                              "with add_into")
    if epi == EPI_RESID_ADD:
        if add_into.dtype != torch.float32 or tuple(add_into.shape) != (n, m):
            raise KernelError("gemm_sk: add_into must be float32 [N, M]")
    elif epi != EPI_ROPE and (out is None or tuple(out.shape) != (n, m) or out.dtype not in (torch.bfloat16, torch.float32)
                              or (swiglu and out.dtype != torch.bfloat16)):
        raise KernelError("gemm_sk: out must be [N, M] bfloat16 (or float32 for a plain store)")
    _call("gemm_sk", "blm_gemm_sk", _ptr(w), w.stride(0), m_rows, k, _ptr(x), x.stride(0), n, _ptr(out),
          out.stride(0) if out is not None else 0, 1 if (out is not None and out.dtype == torch.float32) else 0, _ptr(add_into), epi,
          _ptr(squares), squares.shape[0] if squares is not None else 0, c_float(eps), _ptr(next_gamma),
          1 if (next_gamma is not None and next_gamma.dtype == torch.float32) else 0, _ptr(scaled), _ptr(squares_out),
          ctypes.byref(rope_arg) if rope_arg is not None else None, _ptr(status_word(w.device)), _stream())


def graph_step(graph_exec: int, dev_in, host_in, host_out, dev_out, dev_in2=None, host_in2=None, written_by_graph=False):
    """One captured step driven from native code: host_in (pinned) -> dev_in (and host_in2 -> dev_in2), the
    instantiated graph `graph_exec` (a cudaGraphExec_t as an integer), dev_out -> host_out (pinned), and the
    wait, on the current stream.  `written_by_graph`: the graph's last kernel writes host_out itself (int32 >= 0,
    see `argmax`'s `mirror`); then nothing is copied out and the call returns as soon as every entry is there.

    Returns a function of no arguments that does the same again (same buffers, same stream) at the cost of one
    foreign call: every argument is converted once, here."""
    nbytes = lambda t: t.numel() * t.element_size() if t is not None else 0
    fn = getattr(_lib("runtime"), "blm_graph_step")
    args = (c_void_p(graph_exec), _ptr(dev_in), c_void_p(host_in.data_ptr()), nbytes(host_in),
            _ptr(dev_in2), c_void_p(host_in2.data_ptr()) if host_in2 is not None else c_void_p(0), nbytes(host_in2),
            c_void_p(host_out.data_ptr()), _ptr(dev_out), nbytes(host_out), 1 if written_by_graph else 0, _stream())

    def again():
        if fn(*args) != 0:
            raise KernelError("graph_step: " + _lib("runtime").blm_runtime_last_error().decode(errors="replace"))
    again()
    return again


def host_device_pointer(pinned) -> int:
    """The address under which kernels see a pinned host tensor."""
    if not pinned.is_pinned():
        raise KernelError("host_device_pointer: the tensor is not in pinned host memory")
    dev = c_void_p(0)
    _call("runtime", "blm_host_device_pointer", c_void_p(pinned.data_ptr()), ctypes.byref(dev), kernels=0)
    return int(dev.value or 0)


_status: dict = {}


def status_word(device) -> torch.Tensor:
    """The device word in which kernels with bounded waits record that a wait ran out (0: all well)."""
    dev = torch.device(device)
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    w = _status.get(key)
    if w is None:
        w = _status[key] = torch.zeros(1, dtype=torch.int32, device=dev)
    return w


def check_status(device) -> None:
    """Raise if a kernel gave up a bounded wait since the last check (reads one word from the device)."""
    w = status_word(device)
    code = int(w.item())
    if code:
        w.zero_()
        what = {21: "decode attention: a consumer waited in vain for a page", 22: "decode attention: the producer waited in vain for a free stage",
                1: "gemv: a consumer waited in vain for a weight stage", 2: "gemv: the producer waited in vain for a free stage",
                31: "prompt attention: the query tile did not arrive", 32: "prompt attention: a key tile did not arrive",
                33: "prompt attention: a value tile did not arrive", 34: "prompt attention: the scores did not arrive",
                35: "prompt attention: the probabilities were not written", 36: "prompt attention: the product with the values did not arrive",
                37: "prompt attention: the producer waited in vain for a free stage",
                11: "gemm_tc: the tensor-core thread waited in vain for a stage", 12: "gemm_tc: the producer waited in vain for a free stage",
                13: "gemm_tc: the epilogue waited in vain for the accumulator",
                41: "gemm_sk: the tensor-core thread waited in vain for a stage", 42: "gemm_sk: the producer waited in vain for a free stage",
                43: "gemm_sk: the epilogue waited in vain for the accumulator"}
        raise KernelError(f"{what.get(code, 'status ' + str(code))}; the step's results are not valid")


SQUARES_ROWS = 16     # row length of the sums of squares that go with a handed-over norm


def gemv(w, n_tokens, x=None, stream_rows=None, gamma=None, eps=0.0, rows=None, out=None, add_into=None, swiglu=False,
         squares=None, hand_over=None, rope=None):
    """Skinny product of n_tokens <= 16 tokens with a bfloat16 weight [M, K], with fused ends.

    Input: `x` bfloat16 [N, K], or the fp32 residual stream `stream_rows` [*, K] to be RMS-normalised
    with `gamma`, `eps` (optionally gathering `rows`), or a norm that the writer of the stream handed
    over: `x` = bfloat16(stream * gamma) with `squares` (fp32 [parts, SQUARES_ROWS], the stream rows'
    sums of squares in parts) and `eps`; the result is then divided by the rows' root mean square.
    Output: `out` [N, M] bfloat16 or float32;
    with `swiglu` the weight is [2 I, K] in tiles of GATE_TILE gate rows followed by the up rows of the
    same outputs, and out [N, I] = silu(gate) * up; with
    `add_into` (fp32 [N, M]) the product is added into it and nothing else is written, unless
    `hand_over` = (gamma, scaled, squares) asks for the next norm's input as well: scaled
    (bfloat16 [N, M]) = the new stream times gamma, squares (fp32 [ceil(M / 16), SQUARES_ROWS]) its
    sums of squares by tiles of 16 lanes.
    With `rope` (a dict: token_pos, token_seq, slot_of_seq, block_table, table from rope_table, pool,
    n_heads, n_kv, head_dim, write_cache, max_position) the weight is a step's [q; k; v] (or q alone without
    write_cache) whose q and k heads have their rows in tiled_pair_order(): q and k are rotated by their
    token's position, q goes to `out` [N, n_heads * head_dim] (lanes in that order), the rotated k and the
    v to the token's place in `pool`."""
    _need_cuda(w, x, stream_rows, gamma, rows, out, add_into, squares)
    m_rows, k = w.shape
    if w.dtype != torch.bfloat16:
        raise KernelError("gemv: the weight must be bfloat16")
    m = m_rows // 2 if swiglu else m_rows
    epi = EPI_SWIGLU if swiglu else (EPI_RESID_ADD if add_into is not None else (EPI_ROPE if rope is not None else EPI_STORE))
    rope_arg = None
    if rope is not None:
        if swiglu or add_into is not None:
            raise KernelError("gemv: one epilogue at a time")
        r = rope
        hd, table, pool = r["head_dim"], r["table"], r["pool"]
        _need_cuda(r["token_pos"], r["token_seq"], r["slot_of_seq"], r["block_table"], table, pool)
        if table is None or table.dtype != torch.float32 or tuple(table.shape[1:]) != (hd // 2, 2) \
                or r.get("max_position") is None or r["max_position"] >= table.shape[0]:
            raise KernelError("gemv: the rotary epilogue needs a table [positions, head_dim / 2, 2] that covers the step")
        if r["write_cache"] and (pool.dtype != torch.bfloat16 or tuple(pool.shape[1:]) != (2, r["n_kv"], PAGE, hd)):
            raise KernelError(f"gemv: pool must be bfloat16 [pages, 2, {r['n_kv']}, {PAGE}, {hd}]")
        if out is None or out.dtype != torch.bfloat16 or tuple(out.shape) != (n_tokens, r["n_heads"] * hd):
            raise KernelError("gemv: the rotary epilogue writes q to a bfloat16 out [N, n_heads * head_dim]")
        rope_arg = _GemvRope(r["token_pos"].data_ptr(), r["token_seq"].data_ptr(), r["slot_of_seq"].data_ptr(),
                             r["block_table"].data_ptr(), table.data_ptr(), pool.data_ptr() if pool is not None else 0,
                             r["block_table"].shape[1], r["n_heads"], r["n_kv"], hd, PAGE, 1 if r["write_cache"] else 0,
                             r["token_page"].data_ptr() if r.get("token_page") is not None else 0)
    if x is not None and (x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != k
                          or (rows is None and x.shape[0] != n_tokens)):
        raise KernelError("gemv: x must be bfloat16 [N, K]")
    if rows is not None and rows.numel() != n_tokens:
        raise KernelError("gemv: one row index per token")
    if squares is not None and (x is None or squares.dtype != torch.float32 or squares.dim() != 2
                                or squares.shape[1] != SQUARES_ROWS or not squares.is_contiguous()
                                or x.shape[0] > SQUARES_ROWS):
        raise KernelError("gemv: squares go with x and are float32 [parts, 16]")
    next_gamma = scaled = squares_out = None
    if hand_over is not None:
        next_gamma, scaled, squares_out = hand_over
        _need_cuda(next_gamma, scaled, squares_out)
        if (epi != EPI_RESID_ADD or scaled.dtype != torch.bfloat16 or tuple(scaled.shape) != (n_tokens, m)
                or not scaled.is_contiguous() or squares_out.dtype != torch.float32 or not squares_out.is_contiguous()
                or tuple(squares_out.shape) != ((m + 15) // 16, SQUARES_ROWS) or next_gamma.numel() != m):
            raise KernelError("gemv: hand_over = (gamma [M], scaled bfloat16 [N, M], squares float32 [ceil(M / 16), 16]) "
                              "with add_into")
    if stream_rows is not None and (stream_rows.dtype != torch.float32 or stream_rows.shape[1] != k or gamma is None):
        raise KernelError("gemv: the stream must be float32 [*, K] with a gamma")
    if epi == EPI_RESID_ADD:
        if add_into.dtype != torch.float32 or tuple(add_into.shape) != (n_tokens, m):
            raise KernelError("gemv: add_into must be float32 [N, M]")
    elif epi == EPI_ROPE:
        pass
    elif out is None or tuple(out.shape) != (n_tokens, m) or out.dtype not in (torch.bfloat16, torch.float32) \
            or (swiglu and out.dtype != torch.bfloat16):
        raise KernelError("gemv: out must be [N, M] bfloat16 (or float32 for a plain store)")
    _call("gemv", "blm_gemv", _ptr(w), w.stride(0), m, k, _ptr(x), x.stride(0) if x is not None else 0,
          _ptr(stream_rows), _ptr(gamma), 1 if (gamma is not None and gamma.dtype == torch.float32) else 0, c_float(eps),
          _ptr(rows), n_tokens, _ptr(out), out.stride(0) if out is not None else 0,
          1 if (out is not None and out.dtype == torch.float32) else 0, _ptr(add_into), epi,
          _ptr(squares), squares.shape[0] if squares is not None else 0,
          _ptr(next_gamma), 1 if (next_gamma is not None and next_gamma.dtype == torch.float32) else 0,
          _ptr(scaled), _ptr(squares_out), ctypes.byref(rope_arg) if rope_arg is not None else None,
          _ptr(status_word(w.device)), _stream())


def argmax(logits, out, mirror=None, tickets=None, advance=None):
    """out[b] = index of the largest logit of row b (the lowest index on a tie).  `mirror`: a pinned host int32
    tensor that the kernel fills as well, through the address the device sees it under, so that a host which
    polls it has the result without a copy (`graph_step`).  `tickets`: B + 1 zeroed int32 on the device that belong
    to the caller and to no other launch in flight (the kernel leaves them zero): a large vocabulary then takes one
    launch instead of two.  `advance` = (tokens, positions, history or None, step counter): the step feeds itself
    as `decode_advance` says, in that same launch where there is one."""
    _need_cuda(logits, out)
    if logits.dtype != torch.float32 or out.dtype != torch.int32 or out.numel() < logits.shape[0]:
        raise KernelError("argmax: float32 logits [B, V], int32 out [B]")
    b, v = logits.shape
    if mirror is not None and (mirror.dtype != torch.int32 or mirror.numel() < b or not mirror.is_contiguous()):
        raise KernelError("argmax: the mirror is a pinned int32 tensor of at least B entries")
    lib = _lib("sampling")
    need = lib.blm_argmax_scratch_floats(b, v)
    scratch = torch.empty(need, dtype=torch.float32, device=logits.device) if need else None
    if tickets is not None:
        _need_cuda(tickets)
        if tickets.dtype != torch.int32 or tickets.numel() < b + 1 or not tickets.is_contiguous():
            raise KernelError("argmax: the tickets are B + 1 int32")
        if not need:
            tickets = None
    fed = None
    if advance is not None and tickets is not None and lib.blm_argmax_advances(v):
        fed = advance
        tokens, pos, history, step_no = fed
        _need_cuda(tokens, pos, step_no)
        if tokens.dtype != torch.int32 or pos.dtype != torch.int32 or tokens.numel() != b or pos.numel() != b:
            raise KernelError("argmax: a step that feeds itself has int32 tokens and positions [B]")
        if history is not None and (history.dtype != torch.int32 or history.shape[1] != b or not history.is_contiguous()):
            raise KernelError("argmax: the history is int32 [steps, B]")
    tokens, pos, history, step_no = fed if fed is not None else (None, None, None, None)
    _call("sampling", "blm_argmax", _ptr(logits), logits.stride(0), b, v, _ptr(out),
          c_void_p(host_device_pointer(mirror) if mirror is not None else 0), _ptr(scratch), _ptr(tickets),
          _ptr(tokens), _ptr(pos), _ptr(history), _ptr(step_no), c_void_p(0), history.shape[0] if history is not None else 0,
          _stream(), kernels=(1 if tickets is not None else 2) if need else 1)
    if advance is not None and fed is None:
        decode_advance(advance[0], advance[1], out, advance[2], advance[3])


def sample(logits, temperature, top_p, seeds, stream_ids, counters, out, mirror=None):
    """Draw out[b] from softmax(logits[b] / temperature[b]) restricted to its top-p nucleus.

    temperature, top_p float32 [B]; seeds, stream_ids, counters int64 [B] (read as unsigned): the
    uniform number of a draw is a hash of the three, so it does not depend on the batch.
    `mirror`: as `argmax`'s."""
    _need_cuda(logits, temperature, top_p, seeds, stream_ids, counters, out)
    b = logits.shape[0]
    if logits.dtype != torch.float32 or out.dtype != torch.int32:
        raise KernelError("sample: float32 logits, int32 out")
    if mirror is not None and (mirror.dtype != torch.int32 or mirror.numel() < b or not mirror.is_contiguous()):
        raise KernelError("sample: the mirror is a pinned int32 tensor of at least B entries")
    for t, dt in ((temperature, torch.float32), (top_p, torch.float32), (seeds, torch.int64),
                  (stream_ids, torch.int64), (counters, torch.int64)):
        if t.dtype != dt or t.numel() < b:
            raise KernelError("sample: per-row arguments must be float32/int64 of length B")
    work = torch.empty((b, logits.shape[1]), dtype=torch.float32, device=logits.device)     # the rows' exponentials
    _call("sampling", "blm_sample", _ptr(logits), logits.stride(0), b, logits.shape[1], _ptr(temperature),
          _ptr(top_p), _ptr(seeds), _ptr(stream_ids), _ptr(counters), _ptr(out),
          c_void_p(host_device_pointer(mirror) if mirror is not None else 0), _ptr(work), _stream())


def uniform32(seed, stream_id, counter) -> int:
    """The 32-bit uniform number the sampling kernel uses for (seed, stream, counter); host side."""
    lib = _lib("sampling")
    fn = lib.blm_sampling_uniform32
    fn.argtypes = [c_ulonglong, c_ulonglong, c_ulonglong]
    fn.restype = c_uint
    return int(fn(seed & (2**64 - 1), stream_id & (2**64 - 1), counter & (2**64 - 1)))
