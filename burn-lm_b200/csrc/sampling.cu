// Sampling from fp32 logits on the device: greedy, and temperature with an optional nucleus
// (top-p).  One block per sequence, or a cluster of blocks for a large vocabulary.  Every decision of the nucleus and of the draw is made on
// probabilities quantised to 2^-40, in integer arithmetic, so the result does not depend on the
// order in which threads add things up.
#include "common.cuh"
#include "sampling_no_alloc.h"

BLM_API const char* blm_sampling_last_error() { return g_blm_error; }

constexpr int kSampleThreads = 1024;

// ---------------------------------------------------------------------------------------------
// greedy: the largest logit; the lowest index wins a tie
// ---------------------------------------------------------------------------------------------
// A row's result; `mirror`, where given, is pinned host memory as the device sees it: the host may be polling it
// (blm_graph_step), so the value is pushed out at once.
__device__ __forceinline__ void blm_store_result(int* out, int* mirror, int row, int value) {
    out[row] = value;
    if (mirror != nullptr) {
        *reinterpret_cast<volatile int*>(mirror + row) = value;
        __threadfence_system();
    }
}

__global__ void __launch_bounds__(kSampleThreads) argmax_kernel(const float* __restrict__ logits, long long row_stride,
                                                                int vocab, int* __restrict__ out, int* __restrict__ mirror) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const float* row = logits + (size_t)blockIdx.x * row_stride;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v > best || (v == best && i < idx)) { best = v; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        const int nwarp = blockDim.x >> 5;
        best = lane < nwarp ? bv[lane] : -INFINITY;
        idx = lane < nwarp ? bi[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
        }
        if (lane == 0) blm_store_result(out, mirror, blockIdx.x, idx == 0x7fffffff ? 0 : idx);
    }
}

// Large vocabularies: many blocks per row find the best of their chunk, one block per row merges.
constexpr int kArgmaxChunk = 4096;

// What a step that feeds itself does with a row's token (see decode_advance_kernel in elementwise.cu, which does the
// same as a launch of its own): the token becomes the row's next input, its position moves on, the token joins the
// history of the run; when every row has done so, the run's step counter moves on.
struct ArgmaxAdvance {
    int* tokens;            // null: nothing of this
    int* pos;
    int* history;           // [history_steps, rows] or null
    int* step_no;
    long long* counters;    // per row, or null
    int history_steps;
};

// `tickets` (rows + 1 ints, zero before and after): null, and the chunks' results wait for argmax_merge_kernel; else
// the block that finishes a row's last chunk merges the row itself, so the row's result needs no second launch.
__global__ void __launch_bounds__(256) argmax_chunk_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
                                                           float* __restrict__ part_val, int* __restrict__ part_idx,
                                                           int* __restrict__ tickets, int* __restrict__ out, int* __restrict__ mirror,
                                                           ArgmaxAdvance adv) {
    pdl_launch_dependents();
    pdl_wait();
    blm_trace(0x310);
    __shared__ float bv[8];
    __shared__ int bi[8];
    __shared__ int s_last;
    const float* row = logits + (size_t)blockIdx.y * row_stride;
    const int lo = blockIdx.x * kArgmaxChunk, hi = min(vocab, lo + kArgmaxChunk);
    float best = -INFINITY;
    int idx = 0x7fffffff;
    if (hi - lo == kArgmaxChunk && ((size_t)(row + lo) & 15) == 0) {
        // a whole chunk, 16-byte aligned: a thread's four loads of four values are all asked for before any is looked at
        float4 v[kArgmaxChunk / (4 * 256)];
#pragma unroll
        for (int q = 0; q < kArgmaxChunk / (4 * 256); ++q) v[q] = reinterpret_cast<const float4*>(row + lo)[q * 256 + threadIdx.x];
#pragma unroll
        for (int q = 0; q < kArgmaxChunk / (4 * 256); ++q) {
            const int i = lo + 4 * (q * 256 + (int)threadIdx.x);      // ascending in q, so a tie keeps the lower index
            if (v[q].x > best) { best = v[q].x; idx = i; }
            if (v[q].y > best) { best = v[q].y; idx = i + 1; }
            if (v[q].z > best) { best = v[q].z; idx = i + 2; }
            if (v[q].w > best) { best = v[q].w; idx = i + 3; }
        }
    } else {
        for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
            const float v = row[i];
            if (v > best || (v == best && i < idx)) { best = v; idx = i; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    if ((threadIdx.x & 31) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (bv[w] > best || (bv[w] == best && bi[w] < idx)) { best = bv[w]; idx = bi[w]; }
        part_val[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = best;
        part_idx[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = idx;
        if (tickets != nullptr) {
            __threadfence();
            s_last = atomicAdd(&tickets[blockIdx.y], 1) == (int)gridDim.x - 1;
        }
    }
    if (tickets == nullptr) return;
    __syncthreads();
    if (!s_last || threadIdx.x >= 32) return;
    // the row's last block: every chunk's result is written (the fences around the ticket); the lowest index among the
    // largest values does not depend on which block this is
    __threadfence();
    const int chunks = gridDim.x, r = blockIdx.y, rows = gridDim.y;
    best = -INFINITY;
    idx = 0x7fffffff;
    for (int i = threadIdx.x; i < chunks; i += 32) {
        const float v = __ldcg(part_val + (size_t)r * chunks + i);
        const int vi = __ldcg(part_idx + (size_t)r * chunks + i);
        if (v > best || (v == best && vi < idx)) { best = v; idx = vi; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    if (threadIdx.x != 0) return;
    blm_trace(0x320);
    const int token = idx == 0x7fffffff ? 0 : idx;
    tickets[r] = 0;
    blm_store_result(out, mirror, r, token);
    if (adv.tokens != nullptr) {
        const int s = *reinterpret_cast<volatile int*>(adv.step_no);     // read before this row's ticket below
        adv.tokens[r] = token;
        adv.pos[r] += 1;
        if (adv.counters != nullptr) adv.counters[r] += 1;
        if (adv.history != nullptr && s < adv.history_steps) adv.history[(size_t)s * rows + r] = token;
        __threadfence();
        if (atomicAdd(&tickets[rows], 1) == rows - 1) {      // every row has read the counter: it may move on
            tickets[rows] = 0;
            *adv.step_no = s + 1;
        }
    }
}

__global__ void argmax_merge_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx, int chunks,
                                    int* __restrict__ out, int* __restrict__ mirror) {
    pdl_launch_dependents();
    pdl_wait();
    blm_trace(0x320);
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < chunks; i += 32) {
        const float v = part_val[(size_t)blockIdx.x * chunks + i];
        const int vi = part_idx[(size_t)blockIdx.x * chunks + i];
        if (v > best || (v == best && vi < idx)) { best = v; idx = vi; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    if (threadIdx.x == 0) blm_store_result(out, mirror, blockIdx.x, idx == 0x7fffffff ? 0 : idx);
}

// How many floats of scratch blm_argmax wants for a vocabulary (0: none).
BLM_API int blm_argmax_scratch_floats(int n_rows, int vocab) {
    if (vocab <= 2 * kArgmaxChunk) return 0;
    return 2 * n_rows * ((vocab + kArgmaxChunk - 1) / kArgmaxChunk);
}

// `mirror`: null, or pinned host memory (its device address) that gets the results as well.
// `tickets`: null, or rows + 1 ints that are zero (and are zero again afterwards), used by no other launch in flight:
// then a large vocabulary takes one launch instead of two.  tokens .. history_steps: null / 0, or the step feeds itself
// (ArgmaxAdvance; needs the tickets and a large vocabulary: ask blm_argmax_advances).
BLM_API int blm_argmax_advances(int vocab) { return vocab > 2 * kArgmaxChunk ? 1 : 0; }

BLM_API int blm_argmax(const float* logits, long long row_stride, int n_rows, int vocab, int* out, int* mirror, float* scratch,
                       int* tickets, int* tokens, int* pos, int* history, int* step_no, long long* counters, int history_steps,
                       cudaStream_t stream) {
    if (n_rows == 0) return BLM_OK;
    BLM_REQUIRE(vocab > 0, "argmax: empty vocabulary");
    ArgmaxAdvance adv = {tokens, pos, history, step_no, counters, history_steps};
    if (vocab <= 2 * kArgmaxChunk || scratch == nullptr) {
        BLM_REQUIRE(tokens == nullptr, "argmax: a step feeds itself only from the chunked kernel (a vocabulary above %d, scratch and tickets)", 2 * kArgmaxChunk);
        argmax_kernel<<<n_rows, kSampleThreads, 0, stream>>>(logits, row_stride, vocab, out, mirror);
        return blm_check_launch("argmax");
    }
    BLM_REQUIRE(tokens == nullptr || (tickets != nullptr && pos != nullptr && step_no != nullptr), "argmax: a step that feeds itself needs tickets, positions and a step counter");
    const int chunks = (vocab + kArgmaxChunk - 1) / kArgmaxChunk;
    float* part_val = scratch;
    int* part_idx = reinterpret_cast<int*>(scratch + (size_t)n_rows * chunks);
    blm_launch_dependent(argmax_chunk_kernel, dim3(chunks, n_rows), dim3(256), 0, stream, logits, row_stride, vocab, part_val, part_idx,
                         tickets, out, mirror, adv);
    if (tickets == nullptr)
        blm_launch_dependent(argmax_merge_kernel, dim3(n_rows), dim3(32), 0, stream, (const float*)part_val, (const int*)part_idx, chunks, out, mirror);
    return blm_check_launch("argmax");
}

// ---------------------------------------------------------------------------------------------
// temperature + nucleus
// ---------------------------------------------------------------------------------------------
// The uniform number of sequence stream `stream_id` at its `counter`-th draw: a splitmix64 hash.
__host__ __device__ inline unsigned long long blm_mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__host__ __device__ inline unsigned int blm_uniform32(unsigned long long seed, unsigned long long stream_id,
                                                     unsigned long long counter) {
    unsigned long long k = blm_mix64(seed + 0x9E3779B97F4A7C15ull);
    k = blm_mix64(k ^ (stream_id * 0xD1342543DE82EF95ull + 0x2545F4914F6CDD1Dull));
    k = blm_mix64(k + counter * 0x9E3779B97F4A7C15ull);
    return (unsigned int)(k >> 32);
}
BLM_API unsigned int blm_sampling_uniform32(unsigned long long seed, unsigned long long stream_id, unsigned long long counter) {
    return blm_uniform32(seed, stream_id, counter);
}

__device__ __forceinline__ unsigned long long block_sum_u64(unsigned long long v, unsigned long long* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        unsigned long long t = lane < nwarp ? red[lane] : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    const unsigned long long r = red[32];
    __syncthreads();
    return r;
}

// exclusive prefix over the threads of a block; `total` gets the sum
__device__ __forceinline__ unsigned long long block_exclusive_scan_u64(unsigned long long v, unsigned long long* red,
                                                                       unsigned long long* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    unsigned long long inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) red[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        unsigned long long w = lane < nwarp ? red[lane] : 0ull;
        unsigned long long winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        red[lane] = winc - w;  // exclusive prefix of the warps
        if (lane == 31) red[32] = winc;
    }
    __syncthreads();
    const unsigned long long r = red[warp] + inc - v;
    *total = red[32];
    __syncthreads();
    return r;
}

constexpr double kQuant = 1099511627776.0;  // 2^40

// A 64-bit add into a histogram in shared memory out of two native 32-bit atomic adds (a 64-bit atomic add
// to shared memory is a compare-and-swap loop): the low word's add returns what it found, which tells
// whether it carried; the carry goes with the high word.
__device__ __forceinline__ void hist_add(unsigned int* lo, unsigned int* hi, int bin, unsigned long long v) {
    const unsigned int vl = (unsigned int)v;
    const unsigned int old = atomicAdd(lo + bin, vl);
    const unsigned int carry = old + vl < old ? 1u : 0u;
    const unsigned int vh = (unsigned int)(v >> 32) + carry;
    if (vh) atomicAdd(hi + bin, vh);
}

// The probability of token i: its exponential, computed once and kept in the row of `work`, times 1 / Z.
// Every pass below goes through this one function, so that all passes see the same bits.
__device__ __forceinline__ float prob_of(const float* __restrict__ e, int i, float inv_z) { return __fmul_rn(e[i], inv_z); }

// Calls f(i, probability of token i) for i = lo .. hi - 1 in order.  A thread's chunk is contiguous (the
// order of the vocabulary matters to the draw), so its loads do not coalesce with its neighbours'; sixteen
// are asked for at once, so that the round trips to L2 overlap instead of following one another.
// Calls f(probability of token i) for every token, in no particular order: the threads stride through the
// row together, 16 bytes each, so the loads coalesce.  For the passes whose sums do not care for the order.
template <typename F>
__device__ __forceinline__ void for_all(const float* __restrict__ e, int vocab, float inv_z, F f) {
    if ((vocab & 3) == 0 && ((size_t)e & 15) == 0) {
        const float4* e4 = reinterpret_cast<const float4*>(e);
        for (int i = threadIdx.x; i < (vocab >> 2); i += blockDim.x) {
            const float4 v = e4[i];
            f(__fmul_rn(v.x, inv_z));
            f(__fmul_rn(v.y, inv_z));
            f(__fmul_rn(v.z, inv_z));
            f(__fmul_rn(v.w, inv_z));
        }
    } else {
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) f(__fmul_rn(e[i], inv_z));
    }
}

template <typename F>
__device__ __forceinline__ void for_chunk(const float* __restrict__ e, int lo, int hi, float inv_z, F f) {
    constexpr int kBatch = 16;
    for (int i0 = lo; i0 < hi; i0 += kBatch) {
        float v[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) v[u] = i0 + u < hi ? e[i0 + u] : 0.f;
#pragma unroll
        for (int u = 0; u < kBatch; ++u)
            if (i0 + u < hi) f(i0 + u, __fmul_rn(v[u], inv_z));
    }
}
// floor(p * 2^40): scaling a float by a power of two is exact, so this needs no double
__device__ __forceinline__ unsigned long long quantise(float p) { return __float2ull_rz(__fmul_rn(p, (float)kQuant)); }

// ---- a row over the blocks of a cluster ----
// The blocks of a cluster share a row: block r takes the r-th piece of the vocabulary in every pass.  What
// a block-wide sum was becomes: the block's sum into a word of its shared memory, a cluster barrier, every
// block reads all the words (distributed shared memory) and adds them in the order of the ranks.  The
// words are used in turn (two sets), so one barrier per sum is enough: a block can only overwrite a word
// after the barrier of the sum in between, which every block passes after it has read.
__device__ __forceinline__ unsigned cl_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned cl_size() { unsigned r; asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(r)); return r; }
__device__ __forceinline__ void cl_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ unsigned long long cl_ld_u64(const unsigned long long* local, unsigned rank) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"((unsigned)__cvta_generic_to_shared(local)), "r"(rank));
    unsigned long long v;
    asm volatile("ld.shared::cluster.u64 %0, [%1];\n" : "=l"(v) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ unsigned cl_ld_u32(const unsigned* local, unsigned rank) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"((unsigned)__cvta_generic_to_shared(local)), "r"(rank));
    unsigned v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];\n" : "=r"(v) : "r"(remote) : "memory");
    return v;
}

struct ClusterWords {
    unsigned long long word[2];     // used in turn
    int turn;
};
// every thread of every block of the cluster calls these with its block's value (the same in all its threads)
__device__ __forceinline__ unsigned long long cl_sum_u64(unsigned long long block_value, ClusterWords* w, unsigned long long* before) {
    const int t = w->turn;
    __syncthreads();
    if (threadIdx.x == 0) { w->word[t] = block_value; w->turn = t ^ 1; }
    cl_sync();
    unsigned long long total = 0, pre = 0;
    const unsigned me = cl_rank(), n = cl_size();
    for (unsigned r = 0; r < n; ++r) {
        const unsigned long long v = cl_ld_u64(&w->word[t], r);
        if (r < me) pre += v;
        total += v;
    }
    if (before) *before = pre;
    return total;
}
__device__ __forceinline__ float cl_max_f32(float block_value, ClusterWords* w) {
    const int t = w->turn;
    __syncthreads();
    if (threadIdx.x == 0) { w->word[t] = (unsigned long long)__float_as_uint(block_value); w->turn = t ^ 1; }
    cl_sync();
    float m = -INFINITY;
    for (unsigned r = 0, n = cl_size(); r < n; ++r) m = fmaxf(m, __uint_as_float((unsigned)cl_ld_u64(&w->word[t], r)));
    return m;
}
// sums of floats across blocks are taken in the order of the ranks, from the blocks' own sums
__device__ __forceinline__ float cl_sum_f32(float block_value, ClusterWords* w) {
    const int t = w->turn;
    __syncthreads();
    if (threadIdx.x == 0) { w->word[t] = (unsigned long long)__float_as_uint(block_value); w->turn = t ^ 1; }
    cl_sync();
    float sum = 0.f;
    for (unsigned r = 0, n = cl_size(); r < n; ++r) sum += __uint_as_float((unsigned)cl_ld_u64(&w->word[t], r));
    return sum;
}

__global__ void __launch_bounds__(kSampleThreads) sample_kernel(
    const float* __restrict__ logits, long long row_stride, int vocab, const float* __restrict__ temperature,
    const float* __restrict__ top_p, const unsigned long long* __restrict__ seeds,
    const unsigned long long* __restrict__ stream_ids, const unsigned long long* __restrict__ counters,
    int* __restrict__ out, int* __restrict__ mirror, float* __restrict__ work, int n_pieces) {
    __shared__ float redf[33];
    __shared__ float piece_z[8];                              // the normaliser's sums over this block's pieces
    __shared__ unsigned long long red[33];
    __shared__ unsigned int hist_lo[256], hist_hi[256];      // a bin's 64-bit sum in two words (see hist_add)
    __shared__ unsigned int s_prefix;
    __shared__ unsigned long long s_above;
    __shared__ int s_result;
    __shared__ ClusterWords words;

    const unsigned rank = cl_rank(), n_blocks = cl_size();
    const int b = blockIdx.x / n_blocks;             // the cluster's row
    const float* row = logits + (size_t)b * row_stride;
    float* e = work + (size_t)b * vocab;             // exp(logit / temperature - max), written once below
    const float inv_t = 1.0f / temperature[b];
    const int tid = threadIdx.x;
    if (tid == 0) words.turn = 0;
    // The vocabulary is cut into n_pieces pieces (a multiple of 4 tokens each, so that 16-byte loads stay
    // aligned) whatever the number of blocks: a block takes n_pieces / n_blocks of them, one after another.
    // The only sum here that depends on its order, the normaliser, is taken piece by piece, so that a row's
    // draw does not depend on how many blocks shared it (fewer when there are many rows).
    const int piece = ((vocab + n_pieces - 1) / n_pieces + 3) & ~3;
    const int per_block = n_pieces / (int)n_blocks;
    const int p_lo = min(vocab, (int)rank * per_block * piece), p_hi = min(vocab, p_lo + per_block * piece), p_len = p_hi - p_lo;
    const float* ep = e + p_lo;

    // max and normaliser of softmax(logits / temperature)
    float mx = -INFINITY;
    for (int i = p_lo + tid; i < p_hi; i += blockDim.x) mx = fmaxf(mx, __fmul_rn(row[i], inv_t));
    mx = warp_max(mx);
    if ((tid & 31) == 0) redf[tid >> 5] = mx;
    __syncthreads();
    if (tid < 32) {
        float t = tid < (blockDim.x >> 5) ? redf[tid] : -INFINITY;
        t = warp_max(t);
        if (tid == 0) redf[32] = t;
    }
    __syncthreads();
    mx = cl_max_f32(redf[32], &words);
    for (int k = 0; k < per_block; ++k) {
        const int k_lo = min(p_hi, p_lo + k * piece), k_hi = min(p_hi, k_lo + piece);
        float zk = 0.f;
        for (int i = k_lo + tid; i < k_hi; i += blockDim.x) {
            const float ei = expf(__fsub_rn(__fmul_rn(row[i], inv_t), mx));
            e[i] = ei;
            zk += ei;
        }
        zk = block_sum(zk, redf);    // (its barriers also make every thread's e visible to the others of the block)
        if (tid == 0) piece_z[k] = zk;
    }
    // the pieces' sums in the order of the pieces: the blocks in the order of their ranks, each one's in turn
    cl_sync();
    float z = 0.f;
    for (unsigned r = 0; r < n_blocks; ++r)
        for (int k = 0; k < per_block; ++k) z += __uint_as_float(cl_ld_u32(reinterpret_cast<const unsigned*>(piece_z + k), r));
    const float inv_z = 1.0f / z;

    // contiguous chunk of the block's piece per thread (index order matters below)
    const int per = (p_len + blockDim.x - 1) / blockDim.x;
    const int lo = min(p_hi, p_lo + tid * per), hi = min(p_hi, lo + per);

    unsigned long long total = 0;
    for_all(ep, p_len, inv_z, [&](float p) { total += quantise(p); });
    total = cl_sum_u64(block_sum_u64(total, red), &words, nullptr);

    // nucleus: the key tau (float bits of a probability) with mass(> tau) < target <= mass(>= tau)
    const float pp = top_p[b];
    unsigned int tau = 0;                 // 0: keep everything
    unsigned long long above = 0;         // mass strictly above tau
    unsigned long long tie_w = 0;         // quantised mass of one token at tau
    unsigned long long ties_kept = ~0ull; // how many tokens at tau are kept, in index order
    // after a block has filled its histogram: every block adds the blocks' histograms up for itself (thread t
    // takes bin t, in the order of the ranks) and then all of them scan the same numbers
    auto merge_hist = [&]() {
        cl_sync();
        unsigned long long h = 0;
        if (tid < 256)
            for (unsigned r = 0; r < n_blocks; ++r)
                h += ((unsigned long long)cl_ld_u32(hist_hi + tid, r) << 32) | cl_ld_u32(hist_lo + tid, r);
        cl_sync();                        // everybody has read everybody's bins
        if (tid < 256) { hist_lo[tid] = (unsigned int)h; hist_hi[tid] = (unsigned int)(h >> 32); }
        __syncthreads();
    };
    if (pp < 1.0f) {
        unsigned long long target = (unsigned long long)((double)pp * (double)total);
        if (target < 1) target = 1;
        if (tid == 0) { s_prefix = 0; s_above = 0; }
        __syncthreads();
        // The digits of a probability's bits, from the top: its exponent (the sign is 0), then its mantissa in
        // pieces of 8, 8 and 7 bits.
        //
        // First digit.  The whole vocabulary takes part and shares a dozen exponents, so a histogram in shared
        // memory would have a thousand threads adding to the same few words.  Instead every thread sums, in
        // registers, the sixteen exponents from the largest probability's down (that one is 1 / Z exactly)
        // and what lies below them; the block adds the threads' sums up.  Only if the nucleus reaches below
        // those sixteen exponents (2^-16 of the largest probability) does the general histogram run.
        int first_round = 0;
        {
            constexpr int kTop = 16;
            const int top = (int)((__float_as_uint(inv_z) >> 23) & 255u), base = top - (kTop - 1);
            unsigned long long wacc[kTop + 1];          // [kTop]: everything below the window
#pragma unroll
            for (int k = 0; k <= kTop; ++k) wacc[k] = 0ull;
            for_all(ep, p_len, inv_z, [&](float p) {
                const int d = (int)(__float_as_uint(p) >> 23) - base;
                const unsigned long long w = quantise(p);
#pragma unroll
                for (int k = 0; k < kTop; ++k) wacc[k] += d == k ? w : 0ull;
                wacc[kTop] += d < 0 ? w : 0ull;
            });
            for (int i = tid; i < 256; i += blockDim.x) { hist_lo[i] = 0u; hist_hi[i] = 0u; }
            __syncthreads();
#pragma unroll
            for (int k = 0; k <= kTop; ++k) {
                unsigned long long v = wacc[k];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if ((tid & 31) == 0 && v) hist_add(hist_lo, hist_hi, k, v);       // 32 adds a word
            }
            merge_hist();
            if (tid == 0) {
                unsigned long long run = 0;
                int k = kTop - 1;
                for (; k >= 0; --k) {
                    const unsigned long long h = ((unsigned long long)hist_hi[k] << 32) | hist_lo[k];
                    if (run + h >= target) break;
                    run += h;
                }
                if (k >= 0 && base + k >= 0) {       // found inside the window
                    s_above = run;
                    s_prefix = (unsigned int)(base + k) << 23;
                    s_result = 1;
                } else {
                    s_result = 0;
                }
            }
            __syncthreads();
            first_round = s_result;                   // 1: the exponent is known, go on with the mantissa
            __syncthreads();
        }
        for (int round = first_round; round < 4; ++round) {
            const int shift = round == 0 ? 23 : (round == 1 ? 15 : (round == 2 ? 7 : 0));
            const int width = round == 3 ? 7 : 8;
            for (int i = tid; i < 256; i += blockDim.x) { hist_lo[i] = 0u; hist_hi[i] = 0u; }
            __syncthreads();
            const unsigned int prefix = s_prefix;
            const unsigned int mask = round == 0 ? 0u : (0xffffffffu << (shift + width));
            const unsigned int digit = (1u << width) - 1u;
            // the tokens that share the digits found so far, spread over the bins of the next one (integer sums:
            // the order does not matter)
            for_all(ep, p_len, inv_z, [&](float p) {
                const unsigned int bits = __float_as_uint(p);
                if ((bits & mask) == prefix) hist_add(hist_lo, hist_hi, (int)((bits >> shift) & digit), quantise(p));
            });
            __syncthreads();
            merge_hist();
            if (tid < 32) {
                // The first bin from the top at which the mass reaches the target (bin 0 if none does).  Lane l
                // takes the eight bins 255 - 8 l downwards; the lanes' sums are prefixed from lane 0 up; the
                // lowest lane whose bins reach the target walks them.
                const unsigned long long above0 = s_above;
                unsigned long long h8[8], mine = 0;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int bin = 255 - 8 * tid - k;
                    h8[k] = ((unsigned long long)hist_hi[bin] << 32) | hist_lo[bin];
                    mine += h8[k];
                }
                unsigned long long incl = mine;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
                    if (tid >= o) incl += up;
                }
                const unsigned long long before_me = above0 + incl - mine;
                const bool reaches = before_me + mine >= target;
                const unsigned ballot = __ballot_sync(0xffffffffu, reaches);
                const int owner = ballot ? __ffs(ballot) - 1 : 31;      // nobody: the last lane ends at bin 0
                __syncwarp();                                           // every lane has read s_above
                if (tid == owner) {
                    unsigned long long run = before_me;
                    int k = 0;
                    for (; k < 8; ++k) {
                        const int bin = 255 - 8 * tid - k;
                        if (bin == 0 || run + h8[k] >= target) break;
                        run += h8[k];
                    }
                    s_above = run;
                    s_prefix = prefix | ((unsigned int)(255 - 8 * tid - k) << shift);
                }
            }
            __syncthreads();
        }
        tau = s_prefix;
        above = s_above;
        tie_w = quantise(__uint_as_float(tau));
        // ties are kept while the mass before them is below the target
        if (tie_w == 0) ties_kept = ~0ull;
        else ties_kept = (target - above + tie_w - 1) / tie_w;  // smallest j with above + j * w >= target
    }

    // Tokens at tau.  How many there are is a sum in any order; only when not all of them are kept does their
    // order in the vocabulary matter, and the rank of this thread's first one is counted over its chunk.
    unsigned long long ties_before = 0;
    if (pp < 1.0f) {
        unsigned long long n_ties = 0;
        for_all(ep, p_len, inv_z, [&](float p) {
            if (__float_as_uint(p) == tau) ++n_ties;
        });
        n_ties = cl_sum_u64(block_sum_u64(n_ties, red), &words, nullptr);
        if (n_ties <= ties_kept) {
            ties_kept = ~0ull;          // all of them: no ranks needed
        } else {
            unsigned long long my_ties = 0;
            for_chunk(e, lo, hi, inv_z, [&](int, float p) {
                if (__float_as_uint(p) == tau) ++my_ties;
            });
            unsigned long long block_ties, blocks_before;
            ties_before = block_exclusive_scan_u64(my_ties, red, &block_ties);
            cl_sum_u64(block_ties, &words, &blocks_before);
            ties_before += blocks_before;
        }
    }

    // kept mass of the chunk, then its prefix over the threads of the block and the blocks of the cluster
    unsigned long long mass = 0, t_rank = ties_before;
    for_chunk(e, lo, hi, inv_z, [&](int, float p) {
        const unsigned int bits = __float_as_uint(p);
        const unsigned long long w = quantise(p);
        if (pp >= 1.0f || bits > tau) mass += w;
        else if (bits == tau) { if (t_rank < ties_kept) mass += w; ++t_rank; }
    });
    unsigned long long block_mass, blocks_before;
    unsigned long long before = block_exclusive_scan_u64(mass, red, &block_mass);
    const unsigned long long kept_total = cl_sum_u64(block_mass, &words, &blocks_before);
    before += blocks_before;

    // draw: the first kept token, in vocabulary order, whose running kept mass exceeds u * kept_total
    const unsigned int u = blm_uniform32(seeds[b], stream_ids[b], counters[b]);
    const unsigned long long pick = __umul64hi(kept_total, (unsigned long long)u << 32);
    if (tid == 0) s_result = -1;
    __syncthreads();
    if (kept_total > 0 && pick >= before && pick < before + mass) {
        unsigned long long run = before;
        t_rank = ties_before;
        for (int i = lo; i < hi; ++i) {
            const float p = prob_of(e, i, inv_z);
            const unsigned int bits = __float_as_uint(p);
            const unsigned long long w = quantise(p);
            bool kept = false;
            if (pp >= 1.0f || bits > tau) kept = true;
            else if (bits == tau) { kept = t_rank < ties_kept; ++t_rank; }
            if (kept) {
                run += w;
                if (run > pick) { s_result = i; break; }
            }
        }
    }
    __syncthreads();
    // exactly one thread of the cluster can have found the token; the blocks tell one another
    const unsigned long long found = cl_sum_u64(s_result >= 0 ? (unsigned long long)(s_result + 1) : 0ull, &words, nullptr);
    if (rank == 0 && tid == 0) {
        int r = (int)found - 1;
        if (r < 0) {  // every probability underflowed the quantum: fall back to the largest logit
            float best = -INFINITY; r = 0;
            for (int i = 0; i < vocab; ++i) if (row[i] > best) { best = row[i]; r = i; }
        }
        blm_store_result(out, mirror, b, r);
    }
    cl_sync();       // nobody leaves while its shared memory may still be read
}

BLM_API int blm_sample(const float* logits, long long row_stride, int n_rows, int vocab, const float* temperature,
                       const float* top_p, const unsigned long long* seeds, const unsigned long long* stream_ids,
                       const unsigned long long* counters, int* out, int* mirror, float* work, cudaStream_t stream) {
    if (n_rows == 0) return BLM_OK;
    BLM_REQUIRE(vocab > 0, "sample: empty vocabulary");
    BLM_REQUIRE(work != nullptr, "sample: no room for the rows' exponentials (n_rows x vocab floats)");
    // a row is cut into pieces by the size of the vocabulary (eight for a large one) and shared by the blocks
    // of a cluster: one per piece while all the rows' blocks fit the SMs at once, fewer when there are many rows
    const unsigned pieces = vocab >= 65536 ? 8u : (vocab >= 16384 ? 4u : (vocab >= 4096 ? 2u : 1u));
    unsigned blocks = pieces;
    while (blocks > 1 && blocks * (unsigned)n_rows > (unsigned)blm_sm_count()) blocks >>= 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks * (unsigned)n_rows);
    cfg.blockDim = dim3(kSampleThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = blocks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t err = cudaLaunchKernelEx(&cfg, sample_kernel, logits, row_stride, vocab, temperature, top_p, seeds, stream_ids, counters, out, mirror, work, (int)pieces);
    if (err != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "sample: %s", cudaGetErrorString(err));
    return blm_check_launch("sample");
}

// ---------------------------------------------------------------------------------------------
// argmax for callers that must not allocate (see sampling_no_alloc.h; no counterpart in the reference)
// ---------------------------------------------------------------------------------------------
// The partial results of argmax_chunk_kernel: values first, then indices.  In host code this name is
// only a stand-in for the array; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) float g_argmax_no_alloc_scratch[2 * BLM_ARGMAX_NO_ALLOC_MAX_PARTIALS];

constexpr int kNoAllocMaxDevices = 64;
static float* g_argmax_no_alloc_ptr[kNoAllocMaxDevices] = {};   // per device, found at the first call there

BLM_API int blm_argmax_no_alloc(const float* logits, long long row_stride, int n_rows, int vocab, int* out,
                                cudaStream_t stream) {
    if (n_rows == 0) return BLM_OK;
    BLM_REQUIRE(n_rows > 0 && vocab > 0, "argmax_no_alloc: bad sizes");
    const int chunks = (vocab + kArgmaxChunk - 1) / kArgmaxChunk;
    BLM_REQUIRE((long long)n_rows * chunks <= BLM_ARGMAX_NO_ALLOC_MAX_PARTIALS,
                "argmax_no_alloc: %d rows of %d logits need %lld partial results, the built-in scratch holds %d",
                n_rows, vocab, (long long)n_rows * chunks, BLM_ARGMAX_NO_ALLOC_MAX_PARTIALS);
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "argmax_no_alloc: %s", cudaGetErrorString(e));
    BLM_REQUIRE(device >= 0 && device < kNoAllocMaxDevices, "argmax_no_alloc: device %d", device);
    if (g_argmax_no_alloc_ptr[device] == nullptr) {
        // set-up, once per device, with that device current
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_argmax_no_alloc_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return blm_fail(BLM_CUDA_ERROR, "argmax_no_alloc: no device address for the scratch array: %s", cudaGetErrorString(e));
        g_argmax_no_alloc_ptr[device] = ptr;
    }
    float* part_val = g_argmax_no_alloc_ptr[device];
    int* part_idx = reinterpret_cast<int*>(part_val + BLM_ARGMAX_NO_ALLOC_MAX_PARTIALS);
    argmax_chunk_kernel<<<dim3(chunks, n_rows), 256, 0, stream>>>(logits, row_stride, vocab, part_val, part_idx, (int*)nullptr, (int*)nullptr, (int*)nullptr, ArgmaxAdvance{});
    argmax_merge_kernel<<<n_rows, 32, 0, stream>>>(part_val, part_idx, chunks, out, (int*)nullptr);
    return blm_check_launch("argmax_no_alloc");
}
