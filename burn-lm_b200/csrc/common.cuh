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

// How many multiprocessors the current device has: asked once per device, never written down as a number.
static inline int blm_sm_count() {
    static int counts[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (counts[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 1;
        counts[dev] = n;
    }
    return counts[dev];
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

// Device-side timeline, compiled in with -DBLM_TRACE only: thread 0 of a block records (globaltimer, tag,
// block) at the places that call blm_trace(); blm_trace_dump copies the records of this library to the host.
#ifdef BLM_TRACE
constexpr unsigned kTraceCapacity = 1u << 18;
__device__ unsigned long long g_blm_trace[kTraceCapacity][2];
__device__ unsigned g_blm_trace_n;
__device__ __forceinline__ void blm_trace_here(unsigned tag);
__device__ __forceinline__ void blm_trace(unsigned tag) {
    if (threadIdx.x == 0) blm_trace_here(tag);
}
// for the one thread the caller picked
__device__ __forceinline__ void blm_trace_here(unsigned tag) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    const unsigned i = atomicAdd(&g_blm_trace_n, 1u);
    if (i < kTraceCapacity) {
        g_blm_trace[i][0] = t;
        g_blm_trace[i][1] = ((unsigned long long)tag << 32) | (blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
    }
}
// copies up to `capacity` records (two 64-bit words each) to `host`, returns how many there were, and clears them
BLM_API long long blm_trace_dump(unsigned long long* host, long long capacity) {
    unsigned n = 0;
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(&n, g_blm_trace_n, sizeof(n));
    const long long have = n < kTraceCapacity ? n : kTraceCapacity;
    const long long take = have < capacity ? have : capacity;
    if (take > 0) cudaMemcpyFromSymbol(host, g_blm_trace, (size_t)take * 16);
    n = 0;
    cudaMemcpyToSymbol(g_blm_trace_n, &n, sizeof(n));
    return have;
}
#else
#define blm_trace(tag) ((void)0)
#define blm_trace_here(tag) ((void)0)
#endif

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
