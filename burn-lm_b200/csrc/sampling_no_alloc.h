// An entry point of the sampling library for callers that must not allocate device memory.
//
// It has no counterpart in tracel-ai/burn-lm: the reference takes its argmax through its tensor
// library, which allocates as it pleases.  It is offered for host programs in which this library is
// a guest: a serving process whose device memory was handed out in full at start-up (a cudaMalloc
// there fails, or fragments what an arena carefully laid out), a control loop with a latency bound
// (cudaMalloc and cudaFree may synchronise the whole device and take an unbounded time), or a
// runtime that forbids allocation calls outside its own allocator.  Such a caller owns the input
// and output buffers; the kernel's scratch memory lives inside the library.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Most (row, chunk) partial results one call may need: n_rows * ceil(vocab / 4096) must not exceed it.
// The scratch array is 8 bytes per partial result (64 KB); every device that loads the library holds
// it until the process exits.
#define BLM_ARGMAX_NO_ALLOC_MAX_PARTIALS 8192

// out[b] = index of the largest of logits[b * row_stride .. + vocab) for b < n_rows (the lowest index
// wins a tie), the same result as blm_argmax, computed with the same two kernels, but with the
// partial results of the first kernel kept in a fixed array inside the library instead of in memory
// the caller allocates.
//
// Returns 0, or a non-zero code with a message in blm_sampling_last_error(): sizes beyond
// BLM_ARGMAX_NO_ALLOC_MAX_PARTIALS are refused, nothing is launched.  It calls no cudaMalloc, no
// cudaFree and no allocating library routine.
//
// The first call on a device looks up the device address of the scratch array (once per device, with
// that device current): make that first call outside any stream capture.  All calls share the one
// array, which keeps what the last call left in it (a call overwrites every partial result it reads,
// so nothing has to be cleared); two calls that overlap on the GPU (different streams, different host
// threads) race on it: order them.
int blm_argmax_no_alloc(const float* logits, long long row_stride, int n_rows, int vocab, int* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
