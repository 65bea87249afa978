// Attention over the paged cache: causal, grouped-query, optional window, online softmax in fp32.
//
// attn_tile_kernel is the general kernel (fp32 and bf16, any head size that is a multiple of 16 up
// to 256, any number of heads and groups, prompts and single tokens, optional split of the keys
// over several blocks).  One block owns up to 32 "rows": `qp` consecutive query positions of one
// sequence times `gs` query heads that share one kv head, so a page of keys and values is read
// once for all of them.  Pages (64 positions) go through shared memory; rows of a page that lie
// beyond the sequence are zero-filled, because the pool is never cleared and a reused page may
// hold anything.
#include <math.h>

#include "attention_decode.cuh"
#include "attention_prefill.cuh"
#include "attention_prefill_tc.cuh"
#include "common.cuh"

BLM_API const char* blm_attention_last_error() { return g_blm_error; }

constexpr int kPage = 64;       // positions per cache page
constexpr int kRowsMax = 32;    // rows (positions x heads) per block
constexpr int kThreads = 128;
constexpr int kRowGroups = 16;  // PV: thread = (row group, column group)
constexpr int kColGroups = 8;
constexpr int kAccRows = kRowsMax / kRowGroups;  // 2
constexpr int kChunksMax = 4;                    // 8-lane chunks per thread: head size <= 256

template <typename T> struct Pad;  // 16 bytes of padding per shared row: conflict-free 16-byte loads
template <> struct Pad<float> { static constexpr int n = 4; };
template <> struct Pad<__nv_bfloat16> { static constexpr int n = 8; };

__device__ __forceinline__ void load8(const float* p, float* o) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* o) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        o[2 * i] = f.x;
        o[2 * i + 1] = f.y;
    }
}

struct AttnArgs {
    const void* q;            // token n, head h at q + (n * q_stride + h * hd)
    long long q_stride;       // elements between tokens
    const void* pool;         // [pages][2][n_kv][kPage][hd] of one cache line
    const int* block_table;   // [slots][table_stride] page ids
    int table_stride;
    const int* cu_seqlens;    // [n_seqs + 1] first token of every sequence in the packed step
    const int* slot_of_seq;   // [n_seqs]
    const int* start_pos;     // [n_seqs] cached length before this step
    void* out;                // [N, n_heads * hd]
    float* part_acc;          // [N, n_heads, n_splits, hd] when n_splits > 1
    float* part_ml;           // [N, n_heads, n_splits, 2]
    int n_heads, n_kv, hd, window, n_splits, qp, gs, subgroups;
    float scale;
};

template <typename T>
__global__ void __launch_bounds__(kThreads) attn_tile_kernel(const AttnArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int hd = a.hd;
    const int kstride = hd + Pad<T>::n;
    float* qs = reinterpret_cast<float*>(smem_raw);                       // [kRowsMax][hd]
    float* S = qs + kRowsMax * hd;                                        // [kRowsMax][kPage + 1]
    float* row_m = S + kRowsMax * (kPage + 1);                            // [kRowsMax]
    float* row_l = row_m + kRowsMax;
    float* row_alpha = row_l + kRowsMax;
    T* Ks = reinterpret_cast<T*>(row_alpha + kRowsMax);                   // [kPage][kstride]
    T* Vs = Ks + kPage * kstride;

    const int tid = threadIdx.x;
    const int seq = blockIdx.z / a.n_splits, split = blockIdx.z % a.n_splits;
    const int tok0 = a.cu_seqlens[seq];
    const int q_len = a.cu_seqlens[seq + 1] - tok0;
    const int q0 = blockIdx.x * a.qp;
    if (q0 >= q_len) return;
    const int qn = min(a.qp, q_len - q0);          // positions of this block
    const int kvh = blockIdx.y / a.subgroups, sub = blockIdx.y % a.subgroups;
    const int group = a.n_heads / a.n_kv;
    const int g0 = sub * a.gs;
    const int gn = min(a.gs, group - g0);          // heads of this block
    const int R = qn * gn;
    const int start = a.start_pos[seq];
    const int kv_len = start + q_len;
    const int p_first = start + q0, p_last = p_first + qn - 1;
    const int slot = a.slot_of_seq[seq];
    const int* pages = a.block_table + (size_t)slot * a.table_stride;
    const T* pool = reinterpret_cast<const T*>(a.pool);
    const size_t page_elems = (size_t)a.n_kv * kPage * hd;

    // queries, scaled, as fp32
    const T* qbase = reinterpret_cast<const T*>(a.q);
    for (int idx = tid; idx < R * hd; idx += kThreads) {
        const int r = idx / hd, d = idx % hd;
        const int qi = r / gn, g = r % gn;
        const int head = kvh * group + g0 + g;
        qs[r * hd + d] = to_f32(qbase[(size_t)(tok0 + q0 + qi) * a.q_stride + (size_t)head * hd + d]) * a.scale;
    }
    if (tid < kRowsMax) {
        row_m[tid] = -INFINITY;
        row_l[tid] = 0.f;
    }

    float acc[kAccRows][kChunksMax][8];
#pragma unroll
    for (int i = 0; i < kAccRows; ++i)
#pragma unroll
        for (int c = 0; c < kChunksMax; ++c)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[i][c][e] = 0.f;

    const int rg = tid / kColGroups, cg = tid % kColGroups;
    const int n_chunks = hd / 8;

    // pages this block walks
    int key_lo = 0;
    if (a.window > 0) key_lo = max(0, p_first - a.window + 1);
    int pg_lo = key_lo / kPage, pg_hi = p_last / kPage;  // inclusive
    if (a.n_splits > 1) {
        const int n_pg = pg_hi - pg_lo + 1;
        const int per = (n_pg + a.n_splits - 1) / a.n_splits;
        const int lo = pg_lo + split * per;
        pg_hi = min(pg_hi, lo + per - 1);
        pg_lo = lo;
    }

    for (int pg = pg_lo; pg <= pg_hi; ++pg) {
        __syncthreads();  // previous page fully consumed (and qs / row stats visible the first time)
        const int page = pages[pg];
        const T* kp = pool + (size_t)page * 2 * page_elems + (size_t)kvh * kPage * hd;
        const T* vp = kp + page_elems;
        const int key0 = pg * kPage;
        const int valid = min(kPage, kv_len - key0);  // rows of the page that belong to the sequence
        const int vec_per_row = hd / 8;
        for (int idx = tid; idx < kPage * vec_per_row; idx += kThreads) {
            const int j = idx / vec_per_row, c = idx % vec_per_row;
            T* kd = Ks + j * kstride + c * 8;
            T* vd = Vs + j * kstride + c * 8;
            if (j < valid) {
                if (sizeof(T) == 2) {
                    *reinterpret_cast<uint4*>(kd) = *reinterpret_cast<const uint4*>(kp + (size_t)j * hd + c * 8);
                    *reinterpret_cast<uint4*>(vd) = *reinterpret_cast<const uint4*>(vp + (size_t)j * hd + c * 8);
                } else {
                    const float4* ks4 = reinterpret_cast<const float4*>(kp + (size_t)j * hd + c * 8);
                    const float4* vs4 = reinterpret_cast<const float4*>(vp + (size_t)j * hd + c * 8);
                    reinterpret_cast<float4*>(kd)[0] = ks4[0];
                    reinterpret_cast<float4*>(kd)[1] = ks4[1];
                    reinterpret_cast<float4*>(vd)[0] = vs4[0];
                    reinterpret_cast<float4*>(vd)[1] = vs4[1];
                }
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    kd[e] = from_f32<T>(0.f);
                    vd[e] = from_f32<T>(0.f);
                }
            }
        }
        __syncthreads();

        // scores: thread = (key, rows r0, r0 + 2, ...)
        {
            const int j = tid % kPage;
            const int key = key0 + j;
            const T* krow = Ks + j * kstride;
            for (int r = tid / kPage; r < R; r += kThreads / kPage) {
                const int p = p_first + r / gn;
                float s;
                const bool visible = key <= p && (a.window <= 0 || key > p - a.window);
                if (visible) {
                    const float* qrow = qs + r * hd;
                    float sum = 0.f;
                    for (int c = 0; c < n_chunks; ++c) {
                        float kv[8];
                        load8(krow + c * 8, kv);
                        const float4 qa = *reinterpret_cast<const float4*>(qrow + c * 8);
                        const float4 qb = *reinterpret_cast<const float4*>(qrow + c * 8 + 4);
                        sum += qa.x * kv[0] + qa.y * kv[1] + qa.z * kv[2] + qa.w * kv[3] +
                               qb.x * kv[4] + qb.y * kv[5] + qb.z * kv[6] + qb.w * kv[7];
                    }
                    s = sum;
                } else {
                    s = -INFINITY;
                }
                S[r * (kPage + 1) + j] = s;
            }
        }
        __syncthreads();

        // online softmax: 4 threads per row
        {
            const int r = tid / 4, part = tid % 4;
            float mx = -INFINITY;
            if (r < R)
                for (int j = part * 16; j < part * 16 + 16; ++j) mx = fmaxf(mx, S[r * (kPage + 1) + j]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            float m_old = 0.f, m_new = 0.f, sum = 0.f;
            if (r < R) {
                m_old = row_m[r];
                m_new = fmaxf(m_old, mx);
                for (int j = part * 16; j < part * 16 + 16; ++j) {
                    const float s = S[r * (kPage + 1) + j];
                    const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
                    S[r * (kPage + 1) + j] = p;
                    sum += p;
                }
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            if (r < R && part == 0) {
                const float alpha = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
                row_alpha[r] = alpha;
                row_l[r] = row_l[r] * alpha + sum;
                row_m[r] = m_new;
            }
        }
        __syncthreads();

        // acc = acc * alpha + P V
#pragma unroll
        for (int i = 0; i < kAccRows; ++i) {
            const int r = rg + i * kRowGroups;
            if (r >= R) continue;
            const float alpha = row_alpha[r];
#pragma unroll
            for (int c = 0; c < kChunksMax; ++c)
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[i][c][e] *= alpha;
        }
        const int jmax = min(valid, kPage);
        for (int j = 0; j < jmax; ++j) {
            float p[kAccRows];
#pragma unroll
            for (int i = 0; i < kAccRows; ++i) {
                const int r = rg + i * kRowGroups;
                p[i] = r < R ? S[r * (kPage + 1) + j] : 0.f;
            }
#pragma unroll
            for (int c = 0; c < kChunksMax; ++c) {
                const int chunk = cg + c * kColGroups;
                if (chunk < n_chunks) {
                    float v[8];
                    load8(Vs + j * kstride + chunk * 8, v);
#pragma unroll
                    for (int i = 0; i < kAccRows; ++i)
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[i][c][e] += p[i] * v[e];
                }
            }
        }
    }
    __syncthreads();

    // write: normalised output, or the partial of this split
#pragma unroll
    for (int i = 0; i < kAccRows; ++i) {
        const int r = rg + i * kRowGroups;
        if (r >= R) continue;
        const int qi = r / gn, g = r % gn;
        const int head = kvh * group + g0 + g;
        const size_t tok = (size_t)(tok0 + q0 + qi);
        const float l = row_l[r];
        if (a.n_splits == 1) {
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            T* o = reinterpret_cast<T*>(a.out) + tok * (size_t)a.n_heads * hd + (size_t)head * hd;
#pragma unroll
            for (int c = 0; c < kChunksMax; ++c) {
                const int chunk = cg + c * kColGroups;
                if (chunk < n_chunks)
#pragma unroll
                    for (int e = 0; e < 8; ++e) o[chunk * 8 + e] = from_f32<T>(acc[i][c][e] * inv);
            }
        } else {
            const size_t pi = (tok * a.n_heads + head) * a.n_splits + split;
            float* o = a.part_acc + pi * hd;
#pragma unroll
            for (int c = 0; c < kChunksMax; ++c) {
                const int chunk = cg + c * kColGroups;
                if (chunk < n_chunks)
#pragma unroll
                    for (int e = 0; e < 8; ++e) o[chunk * 8 + e] = acc[i][c][e];
            }
            if (cg == 0) {
                a.part_ml[pi * 2] = row_m[r];
                a.part_ml[pi * 2 + 1] = l;
            }
        }
    }
}

// out[tok, head, :] = sum_z acc_z e^(m_z - M) / sum_z l_z e^(m_z - M)
template <typename T>
__global__ void attn_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                    T* __restrict__ out, int n_splits, int hd) {
    const size_t row = blockIdx.x;  // tok * n_heads + head
    float M = -INFINITY;
    for (int z = 0; z < n_splits; ++z) M = fmaxf(M, part_ml[(row * n_splits + z) * 2]);
    float L = 0.f;
    for (int z = 0; z < n_splits; ++z) {
        const float m = part_ml[(row * n_splits + z) * 2];
        if (m != -INFINITY) L += part_ml[(row * n_splits + z) * 2 + 1] * expf(m - M);
    }
    const float inv = L > 0.f ? 1.0f / L : 0.f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float s = 0.f;
        for (int z = 0; z < n_splits; ++z) {
            const float m = part_ml[(row * n_splits + z) * 2];
            if (m != -INFINITY) s += part_acc[(row * n_splits + z) * hd + d] * expf(m - M);
        }
        out[row * hd + d] = from_f32<T>(s * inv);
    }
}

static size_t attn_smem_bytes(int hd, int elem) {
    const int pad = elem == 2 ? 8 : 4;
    return (size_t)kRowsMax * hd * 4 + (size_t)kRowsMax * (kPage + 1) * 4 + 3 * kRowsMax * 4 +
           2 * (size_t)kPage * (hd + pad) * elem;
}

// Bytes of scratch the split path needs for n_tokens tokens (0 when n_splits == 1).
BLM_API size_t blm_attention_scratch_bytes(int n_tokens, int n_heads, int hd, int n_splits) {
    if (n_splits <= 1) return 0;
    return (size_t)n_tokens * n_heads * n_splits * (hd + 2) * sizeof(float);
}

BLM_API int blm_attention(const void* q, long long q_stride, const void* pool, int dtype,
                          const int* block_table, int table_stride, const int* cu_seqlens,
                          const int* slot_of_seq, const int* start_pos, void* out, float* scratch,
                          int n_tokens, int n_seqs, int max_q_len, int n_heads, int n_kv, int hd,
                          int page_size, int window, int n_splits, float scale, int general_only, int* status,
                          int n_pages, int max_kv_len, const int* seq_table, int ahead, cudaStream_t stream) {
    if (n_tokens == 0 || n_seqs == 0) return BLM_OK;
    BLM_REQUIRE(page_size == kPage, "attention: the cache page holds %d positions, the kernel wants %d", page_size, kPage);
    BLM_REQUIRE(hd >= 16 && hd <= 8 * kColGroups * kChunksMax && hd % 16 == 0,
                "attention: head size %d is not a multiple of 16 between 16 and %d", hd, 8 * kColGroups * kChunksMax);
    BLM_REQUIRE(n_kv > 0 && n_heads % n_kv == 0, "attention: %d heads do not divide into %d kv heads", n_heads, n_kv);
    BLM_REQUIRE(n_splits >= 1 && (n_splits == 1 || scratch != nullptr), "attention: split without scratch");
    BLM_REQUIRE(max_q_len >= 1, "attention: empty step");
    const int group = n_heads / n_kv;
    if (dtype == BLM_BF16 && max_q_len == 1 && n_tokens == n_seqs && !general_only) {
        // one new token per sequence: the specialised kernel, where it has the shape
        AttnDecodeArgs d;
        d.q = (const __nv_bfloat16*)q; d.q_stride = q_stride; d.pool = (const __nv_bfloat16*)pool;
        d.block_table = block_table; d.table_stride = table_stride; d.seq_table = seq_table; d.cu_seqlens = cu_seqlens;
        d.slot_of_seq = slot_of_seq; d.start_pos = start_pos; d.out = (__nv_bfloat16*)out;
        d.part_acc = scratch;
        d.part_ml = scratch ? scratch + (size_t)n_tokens * n_heads * n_splits * hd : nullptr;
        d.n_heads = n_heads; d.n_kv = n_kv; d.window = window; d.n_splits = n_splits;
        d.scale_log2e = scale * 1.4426950408889634f;
        d.status = status;
        d.ahead = ahead ? 1 : 0;
        BLM_REQUIRE(status != nullptr, "attention: no status word");
        BLM_REQUIRE(n_splits <= 64, "attention: at most 64 splits, got %d", n_splits);
        BLM_REQUIRE(n_pages > 0 && ((size_t)pool & 15) == 0, "attention: the pool's page count is needed");
        if (launch_attn_decode(d, hd, group, n_seqs, n_pages, max_kv_len, stream)) return blm_check_launch("attention decode");
    }
    if (dtype == BLM_BF16 && max_q_len >= 16 && (hd == 64 || hd == 128) && !general_only) {
        // prompts: the tensor-core kernel
        AttnPrefillArgs f;
        f.q = (const __nv_bfloat16*)q; f.q_stride = q_stride; f.pool = (const __nv_bfloat16*)pool;
        f.block_table = block_table; f.table_stride = table_stride; f.cu_seqlens = cu_seqlens;
        f.slot_of_seq = slot_of_seq; f.start_pos = start_pos; f.out = (__nv_bfloat16*)out;
        f.n_heads = n_heads; f.n_kv = n_kv; f.window = window; f.scale_log2e = scale * 1.4426950408889634f;
        BLM_REQUIRE(q_stride % 8 == 0 && ((size_t)q & 15) == 0, "attention: q rows must be 16-byte aligned");
        if (max_q_len >= 64 && status != nullptr && n_pages > 0 && ((size_t)pool & 15) == 0) {
            // long prompts: the products on tcgen05, accumulators in tensor memory
            AttnPrefillTcArgs t;
            t.block_table = block_table; t.table_stride = table_stride; t.cu_seqlens = cu_seqlens; t.slot_of_seq = slot_of_seq;
            t.start_pos = start_pos; t.out = (__nv_bfloat16*)out; t.n_heads = n_heads; t.n_kv = n_kv; t.window = window;
            t.scale_log2e = f.scale_log2e; t.status = status;
            const int rc = launch_attn_prefill_tc(t, q, q_stride, pool, n_pages, hd, n_tokens, n_seqs, max_q_len, stream);
            if (rc == BLM_OK) return blm_check_launch("attention prefill (tcgen05)");
            if (rc > 0) return rc;
        }
        if (launch_attn_prefill(f, hd, n_seqs, max_q_len, stream)) return blm_check_launch("attention prefill");
    }
    AttnArgs a;
    a.q = q; a.q_stride = q_stride; a.pool = pool; a.block_table = block_table; a.table_stride = table_stride;
    a.cu_seqlens = cu_seqlens; a.slot_of_seq = slot_of_seq; a.start_pos = start_pos; a.out = out;
    a.n_heads = n_heads; a.n_kv = n_kv; a.hd = hd; a.window = window; a.n_splits = n_splits; a.scale = scale;
    a.gs = group < kRowsMax ? group : kRowsMax;
    a.subgroups = (group + a.gs - 1) / a.gs;
    a.qp = kRowsMax / a.gs;
    if (a.qp > max_q_len) a.qp = max_q_len;
    a.part_acc = scratch;
    a.part_ml = scratch ? scratch + (size_t)n_tokens * n_heads * n_splits * hd : nullptr;
    const dim3 grid((max_q_len + a.qp - 1) / a.qp, n_kv * a.subgroups, n_seqs * n_splits);
    BLM_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "attention: grid %u x %u too large", grid.y, grid.z);
    const size_t smem = attn_smem_bytes(hd, dtype == BLM_BF16 ? 2 : 4);
    // the opt-in to large shared memory is set once per kernel (for the largest head size)
    static bool opted_in[2] = {false, false};
    if (dtype != BLM_F32 && dtype != BLM_BF16) return blm_fail(BLM_BAD_ARGUMENT, "attention: dtype %d", dtype);
    if (!opted_in[dtype]) {
        const int most = (int)attn_smem_bytes(8 * kColGroups * kChunksMax, dtype == BLM_BF16 ? 2 : 4);
        cudaError_t e = dtype == BLM_F32
            ? cudaFuncSetAttribute(attn_tile_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, most)
            : cudaFuncSetAttribute(attn_tile_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
        if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "attention: %s", cudaGetErrorString(e));
        opted_in[dtype] = true;
    }
    if (dtype == BLM_F32)
        attn_tile_kernel<float><<<grid, kThreads, smem, stream>>>(a);
    else
        attn_tile_kernel<__nv_bfloat16><<<grid, kThreads, smem, stream>>>(a);
    int rc = blm_check_launch("attention");
    if (rc != BLM_OK || n_splits == 1) return rc;
    const int cthreads = hd >= 128 ? 128 : 64;
    if (dtype == BLM_F32)
        attn_combine_kernel<float><<<n_tokens * n_heads, cthreads, 0, stream>>>(a.part_acc, a.part_ml, (float*)out, n_splits, hd);
    else
        attn_combine_kernel<__nv_bfloat16><<<n_tokens * n_heads, cthreads, 0, stream>>>(a.part_acc, a.part_ml, (__nv_bfloat16*)out, n_splits, hd);
    return blm_check_launch("attention combine");
}
