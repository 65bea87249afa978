// Shared helpers of the sm_100a kernels: element types, error reporting, small reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define BLM_API extern "C" __attribute__((visibility("default")))

// Codes returned by every entry point.  0 is success; the message of the last failure of the
// calling thread is kept for blm_*_last_error().
enum { BLM_OK = 0, BLM_BAD_ARGUMENT = 1, BLM_CUDA_ERROR = 2 };

static thread_local char g_blm_error[512] = "";

static inline int blm_fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
#include <stdarg.h>
static inline int blm_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_blm_error, sizeof(g_blm_error), fmt, ap);
    va_end(ap);
    return code;
}

static inline int blm_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "%s: %s", what, cudaGetErrorString(e));
    return BLM_OK;
}

#define BLM_REQUIRE(cond, ...)                                    \
    do {                                                          \
        if (!(cond)) return blm_fail(BLM_BAD_ARGUMENT, __VA_ARGS__); \
    } while (0)

// Programmatic dependent launch: a kernel launched through blm_launch_dependent may start while the kernel
// before it on the stream is still running.  What it does before pdl_wait() must touch nothing that an
// earlier kernel writes (barrier setup, prefetching weights); pdl_wait() returns when the earlier kernels
// are complete and their writes visible.  pdl_launch_dependents() lets the kernel after this one start its
// own preamble.  Without the launch attribute both are no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t blm_launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                               Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// dtype tags shared with the Python side
enum { BLM_F32 = 0, BLM_BF16 = 1 };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    float r = red[32];
    __syncthreads();
    return r;
}
