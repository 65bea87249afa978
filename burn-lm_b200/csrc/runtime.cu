// The host side of a captured decode step in one call: the step's inputs (one or two buffers) from pinned host
// memory to the device, the captured graph, and the step's result in pinned host memory: copied back and waited for, or
// written there by the graph's own last kernel and polled for.  The driver calls are issued back to back from native
// code instead of from the interpreter, which otherwise costs the GPU tens of microseconds of idling per step.
#include "common.cuh"
#include <time.h>

BLM_API const char* blm_runtime_last_error() { return g_blm_error; }

// The address under which the device sees a piece of pinned host memory.
BLM_API int blm_host_device_pointer(void* host, void** device) {
    BLM_REQUIRE(host != nullptr && device != nullptr, "host_device_pointer: null argument");
    cudaError_t e = cudaHostGetDevicePointer(device, host, 0);
    if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "host_device_pointer: %s", cudaGetErrorString(e));
    return BLM_OK;
}

// `written_by_graph` != 0: host_out is an array of int32 that the graph's own last kernel writes through the
// pointer above, every entry >= 0.  Then there is no copy out and no wait for the stream: the entries are set to -1
// before the launch and the call comes back when none of them is -1 any more, which is a few microseconds before the
// driver would have said so.  Should that take seconds, the stream is waited for in the ordinary way.
BLM_API int blm_graph_step(void* graph_exec, void* dev_in, const void* host_in, long long bytes_in, void* dev_in2, const void* host_in2,
                           long long bytes_in2, void* host_out, const void* dev_out, long long bytes_out, int written_by_graph,
                           cudaStream_t stream) {
    BLM_REQUIRE(graph_exec != nullptr, "graph_step: no instantiated graph");
    volatile int* result = static_cast<volatile int*>(host_out);
    const long long n_result = bytes_out / 4;
    if (written_by_graph) {
        BLM_REQUIRE(host_out != nullptr && bytes_out > 0 && bytes_out % 4 == 0, "graph_step: a graph writes int32 results to pinned memory");
        for (long long i = 0; i < n_result; ++i) result[i] = -1;
    }
    cudaError_t e = cudaSuccess;
    if (bytes_in > 0) e = cudaMemcpyAsync(dev_in, host_in, (size_t)bytes_in, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess && bytes_in2 > 0) e = cudaMemcpyAsync(dev_in2, host_in2, (size_t)bytes_in2, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaGraphLaunch((cudaGraphExec_t)graph_exec, stream);
    if (e == cudaSuccess && written_by_graph) {
        timespec t0;
        clock_gettime(CLOCK_MONOTONIC, &t0);
        bool there = false;
        for (unsigned long long spins = 1; !there; ++spins) {
            long long i = 0;
            while (i < n_result && result[i] >= 0) ++i;
            there = i == n_result;
            if (there) break;
            __builtin_ia32_pause();
            if ((spins & 0x3fff) == 0) {
                timespec t;
                clock_gettime(CLOCK_MONOTONIC, &t);
                if (t.tv_sec - t0.tv_sec >= 2) break;
            }
        }
        if (!there) {
            e = cudaStreamSynchronize(stream);
            if (e == cudaSuccess)
                for (long long i = 0; i < n_result; ++i)
                    if (result[i] < 0) return blm_fail(BLM_CUDA_ERROR, "graph_step: the step ended without result %lld", i);
        }
    } else {
        if (e == cudaSuccess && bytes_out > 0) e = cudaMemcpyAsync(host_out, dev_out, (size_t)bytes_out, cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    }
    if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "graph_step: %s", cudaGetErrorString(e));
    return BLM_OK;
}
