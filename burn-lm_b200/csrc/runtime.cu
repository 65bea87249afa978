// The host side of a captured decode step in one call: the step's inputs (one or two buffers) from pinned host
// memory to the device, the captured graph, the step's result back to pinned host memory, and the wait for it.  Four
// driver calls issued back to back from native code instead of from the interpreter, which otherwise
// costs the GPU tens of microseconds of idling per step.
#include "common.cuh"

BLM_API const char* blm_runtime_last_error() { return g_blm_error; }

BLM_API int blm_graph_step(void* graph_exec, void* dev_in, const void* host_in, long long bytes_in, void* dev_in2, const void* host_in2,
                           long long bytes_in2, void* host_out, const void* dev_out, long long bytes_out, cudaStream_t stream) {
    BLM_REQUIRE(graph_exec != nullptr, "graph_step: no instantiated graph");
    cudaError_t e = cudaSuccess;
    if (bytes_in > 0) e = cudaMemcpyAsync(dev_in, host_in, (size_t)bytes_in, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess && bytes_in2 > 0) e = cudaMemcpyAsync(dev_in2, host_in2, (size_t)bytes_in2, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaGraphLaunch((cudaGraphExec_t)graph_exec, stream);
    if (e == cudaSuccess && bytes_out > 0) e = cudaMemcpyAsync(host_out, dev_out, (size_t)bytes_out, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "graph_step: %s", cudaGetErrorString(e));
    return BLM_OK;
}
