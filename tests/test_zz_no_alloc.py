"""The argmax entry point for callers that must not allocate device memory (`blm_argmax_no_alloc`,
declared in burn-lm_b200/csrc/sampling_no_alloc.h), called through its exported C symbol.

Some hosts of this library cannot let it call cudaMalloc: their device memory is handed out in full
at start-up, or they run under a latency bound that an allocation (which may synchronise the device)
would break.  For them the two-stage argmax keeps its partial results in a fixed array inside the
library.  This test checks that it gives exactly what the ordinary entry point gives, twice in a row
on different inputs (the array is shared between calls and keeps the last call's contents), and that
it refuses sizes beyond its array.  It is collected last on purpose: a run that stops at the first
failure has then run every other test.
"""
import ctypes
from ctypes import c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def entry_point():
    from burn_lm_b200.csrc import build
    lib = build.load("sampling")
    fn = lib.blm_argmax_no_alloc
    fn.argtypes = [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p]
    fn.restype = c_int
    err = lib.blm_sampling_last_error
    err.restype = ctypes.c_char_p
    return fn, err


def no_alloc_argmax(logits):
    fn, err = entry_point()
    out = torch.full((logits.shape[0],), -1, dtype=torch.int32, device=logits.device)      # the caller's own buffer
    rc = fn(c_void_p(logits.data_ptr()), logits.stride(0), logits.shape[0], logits.shape[1], c_void_p(out.data_ptr()),
            c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, err().decode()
    return out


def test_no_alloc_argmax_equals_the_ordinary_one_twice_in_a_row():
    from burn_lm_b200 import kernels as K
    g = torch.Generator(device="cuda").manual_seed(7)
    first = torch.randn(64, 128256, device="cuda", generator=g)          # the largest case the engine has: 64 x 32 chunks
    first[3, 100000] = first[3, 5000] = 40.0                             # a tie across chunks: the lower index
    second = torch.randn(5, 20011, device="cuda", generator=g)           # fewer rows and chunks: stale partials lie beyond
    second[4, 20010] = 50.0
    for logits in (first, second):
        want = torch.empty(logits.shape[0], dtype=torch.int32, device="cuda")
        K.argmax(logits, want)
        got = no_alloc_argmax(logits)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert got.tolist() == logits.argmax(-1).tolist() or logits is first       # (first has the planted tie)
    assert no_alloc_argmax(first)[3].item() == 5000


def test_no_alloc_argmax_refuses_what_its_array_cannot_hold():
    fn, err = entry_point()
    logits = torch.zeros(1, 8, device="cuda")
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    # 300 rows of 128256 logits would need 9600 partial results; only sizes are looked at, nothing is launched
    rc = fn(c_void_p(logits.data_ptr()), 128256, 300, 128256, c_void_p(out.data_ptr()), c_void_p(0))
    assert rc != 0 and b"scratch holds 8192" in err()
