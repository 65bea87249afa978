// Matrix product for steps of a few dozen tokens (17 to 64: a decode step of that many sequences, a short
// prompt) on the 5th-generation tensor cores: y[N, M] = x[N, K] . W[M, K]^T with the WEIGHT rows as the
// 128-row operand of tcgen05.mma and the tokens as its narrow one, so a weight that is read once from HBM
// fills the tensor core's rows whatever the number of tokens.
//
// A tile is 128 weight rows x all tokens.  A weight of a few thousand rows has only a few dozen tiles, far
// fewer than there are SMs, so the K range of a tile is cut over the S blocks of a thread-block cluster
// (S = 1, 2, 4 or 8): block r of a cluster multiplies its slice of K into its own accumulator in tensor
// memory, writes it to its shared memory, and after a cluster barrier every block sums one S-th of the
// tile's rows over all S blocks through distributed shared memory, in the order of the ranks, and runs the
// epilogue on them.  Nothing partial ever goes to global memory and every sum has one fixed order.
//
// Per block: warp 0 (one thread) streams tiles by TMA (cp.async.bulk.tensor.2d, 128-byte swizzle): 128 x 64
// of W and NP x 64 of x per stage, into a ring as deep as shared memory allows; the weights of the first
// stages go out before griddepcontrol.wait (the kernel is a programmatic dependent: they are nobody's
// output), the tokens after it.  Warp 1 allocates tensor memory and (one thread) issues
// tcgen05.mma.cta_group::1.kind::f16 M 128, N NP, K 16, four per stage; tcgen05.commit frees the stage.
// Warps 2..5 read the accumulator (tcgen05.ld), and after the cluster's meeting apply one of the ends:
//   store (bf16 or fp32) | silu(gate) * up for a weight in tiles of 8 gate rows and their 8 up rows
//   | stream += y, optionally leaving the next norm's input (bf16(stream * gamma) and the rows' sums of
//     squares by tiles of 16 lanes) | rotary embedding of q and k and the append of k and v to the cache.
// A norm handed over by the writer of the stream (x = bf16(stream * gamma) with the sums of squares) is
// finished by scaling every token's results by 1 / rms.
//
// Every mbarrier wait is bounded; one that runs out records a code in the status word, and the block still
// goes to both cluster barriers and gives its tensor memory back.
#include <cuda.h>

#include <map>
#include <tuple>

#include "common.cuh"

BLM_API const char* blm_gemm_sk_last_error() { return g_blm_error; }

namespace {

constexpr int TM = 128, BK = 64;                 // weight rows per tile; k per stage (128 bytes: one swizzle row)
constexpr int kThreads = 192;                    // producer warp, mma warp, 4 epilogue warps
constexpr unsigned kWBytes = TM * BK * 2;
constexpr unsigned kSpinLimit = 1u << 22;
constexpr int kSquaresRow = 64;                  // row length of the sums of squares that go with a handed-over norm

enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_RESID_ADD = 2, EPI_ROPE = 3 };
enum { SK_OK = 0, SK_TIMEOUT_FULL = 41, SK_TIMEOUT_EMPTY = 42, SK_TIMEOUT_ACCUM = 43 };

struct SkRope {
    const int* token_pos;        // [N] position of every token
    const int* token_seq;        // [N] the token's sequence in the step (-1: a row of no sequence)
    const int* slot_of_seq;
    const int* block_table;      // [slots][table_stride]
    const float2* table;         // (cos, sin) [positions][hd / 2]
    __nv_bfloat16* pool;         // [pages][2][n_kv][page_size][hd]
    int table_stride, n_heads, n_kv, hd, page_size, write_cache;
};

struct SkArgs {
    int M, K, N;                 // weight rows (for EPI_SWIGLU: 2 x the inner size), reduction length, tokens
    int S;                       // blocks of a cluster = slices of K
    void* y;                     // EPI_STORE / EPI_SWIGLU / EPI_ROPE (q): [N, ldy]
    long long ldy;
    int y_f32;
    float* acc;                  // EPI_RESID_ADD: fp32 stream [N, M]
    int epi;
    const float* ssq_in;         // a handed-over norm: [ssq_parts][kSquaresRow] sums of squares of the stream's rows
    int ssq_parts;
    float eps;
    const void* next_gamma;      // EPI_RESID_ADD may hand the next norm over: gamma [M], xg_out [N, M], ssq_out [M / 16][kSquaresRow]
    int next_gamma_f32;
    __nv_bfloat16* xg_out;
    float* ssq_out;
    SkRope rope;
    int* status;
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    const unsigned addr = smem_u32(bar);
    for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
        unsigned done;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
// shared-memory operand descriptor: K-major rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ unsigned long long umma_desc(const void* tile) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(tile) >> 4) & 0x3fff);
    d |= (unsigned long long)1 << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
__device__ __forceinline__ void umma(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc, unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(unsigned taddr, float (&v)[16]) {
    unsigned r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// every thread of every block of the cluster; what was written to shared memory before is visible after
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// a float of block `rank`'s shared memory, at the place `local` has in this block's
__device__ __forceinline__ float ld_peer(const float* local, unsigned rank) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

template <int NP>
__global__ void __launch_bounds__(kThreads, 1) gemm_sk_kernel(const SkArgs a, const __grid_constant__ CUtensorMap wmap,
                                                              const __grid_constant__ CUtensorMap xmap, const int n_stages) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr unsigned kXBytes = NP * BK * 2;
    constexpr unsigned kStage = kWBytes + kXBytes;
    constexpr int kTmemCols = NP < 32 ? 32 : NP;
    constexpr unsigned kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(NP >> 3) << 17) | ((unsigned)(TM >> 4) << 24);
    unsigned char* ring = smem;                                                  // [n_stages][W tile | x tile]
    float* part = reinterpret_cast<float*>(ring + (size_t)n_stages * kStage);    // [NP][TM]: this block's sums over its slice of K
    float* row_scale = part + NP * TM;                                           // [NP] 1 / rms of a handed-over norm's rows
    long long* rope_where = reinterpret_cast<long long*>(row_scale + NP);        // [NP] where a token's k row of kv head 0 starts in the pool
    int* rope_pos = reinterpret_cast<int*>(rope_where + NP);                     // [NP]
    unsigned long long* full = reinterpret_cast<unsigned long long*>(rope_pos + NP);
    unsigned long long* empty = full + n_stages;
    unsigned long long* acc_full = empty + n_stages;
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = a.S;
    const int rank = (int)cluster_rank();
    const int tile = (int)blockIdx.x / S, m0 = tile * TM;
    const int k_iters = (a.K + BK - 1) / BK, k_per = (k_iters + S - 1) / S;
    const int k_lo = rank * k_per;
    const int my_iters = max(0, min(k_iters, k_lo + k_per) - k_lo);

    if (threadIdx.x == 0) {
        for (int s = 0; s < n_stages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = *tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- producer ----------------
            const int pre = min(n_stages, my_iters);
            for (int i = 0; i < pre; ++i) {           // weights are nobody's output: they go out at once
                mbar_expect_tx(full + i, kStage);
                tma_load_2d(ring + (size_t)i * kStage, &wmap, (k_lo + i) * BK, m0, full + i);
            }
            pdl_wait();                               // the tokens are the work of the kernel before
            for (int i = 0; i < pre; ++i) tma_load_2d(ring + (size_t)i * kStage + kWBytes, &xmap, (k_lo + i) * BK, 0, full + i);
            for (int it = pre; it < my_iters; ++it) {
                const int s = it % n_stages;
                if (!mbar_wait(empty + s, ((it / n_stages) - 1) & 1)) {
                    atomicCAS(a.status, SK_OK, SK_TIMEOUT_EMPTY);
                    break;
                }
                mbar_expect_tx(full + s, kStage);
                tma_load_2d(ring + (size_t)s * kStage, &wmap, (k_lo + it) * BK, m0, full + s);
                tma_load_2d(ring + (size_t)s * kStage + kWBytes, &xmap, (k_lo + it) * BK, 0, full + s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- tensor core ----------------
            bool ok = true;
            for (int it = 0; it < my_iters; ++it) {
                const int s = it % n_stages;
                if (!mbar_wait(full + s, (it / n_stages) & 1)) {
                    atomicCAS(a.status, SK_OK, SK_TIMEOUT_FULL);
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned long long ad = umma_desc(ring + (size_t)s * kStage), bd = umma_desc(ring + (size_t)s * kStage + kWBytes);
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk) umma(tmem_base, ad + 2 * kk, bd + 2 * kk, kIdesc, (it > 0 || kk > 0) ? 1u : 0u);
                umma_commit(empty + s);
            }
            if (ok && my_iters > 0) umma_commit(acc_full);
        }
    } else {
        // ---------------- epilogue, first half: this block's sums to its shared memory ----------------
        const int e = (int)threadIdx.x - 64;          // 0 .. 127
        const int quarter = warp & 3;                 // the 32 lanes of tensor memory this warp may read
        pdl_wait();
        if (e < NP) {
            float sc = 1.0f;
            if (a.ssq_in != nullptr && e < a.N) {
                float ssq = 0.f;
                for (int p = 0; p < a.ssq_parts; ++p) ssq += a.ssq_in[(size_t)p * kSquaresRow + e];      // one fixed order
                sc = 1.0f / sqrtf(ssq / (float)a.K + a.eps);
            }
            row_scale[e] = sc;
            if (a.epi == EPI_ROPE && e < a.N) {
                const SkRope& r = a.rope;
                const int pos = r.token_pos[e];
                rope_pos[e] = pos;
                long long where = -1;                  // a row of no sequence: nothing of it reaches the cache
                if (r.write_cache) {
                    const int seq = r.token_seq[e];
                    if (seq >= 0) {
                        const int page = r.block_table[(size_t)r.slot_of_seq[seq] * r.table_stride + pos / r.page_size];
                        where = ((long long)page * 2 * r.n_kv * r.page_size + pos % r.page_size) * r.hd;
                    }
                }
                rope_where[e] = where;
            }
        }
        const int ml = quarter * 32 + lane;           // the tile's row this thread reads
        bool have = my_iters > 0;
        if (have && !mbar_wait(acc_full, 0)) {
            if (lane == 0) atomicCAS(a.status, SK_OK, SK_TIMEOUT_ACCUM);
            have = false;
        }
        have = __all_sync(0xffffffffu, have);         // tcgen05.ld is a warp's instruction: all lanes or none
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16);
#pragma unroll 1
        for (int j = 0; j < NP / 16; ++j) {
            float v[16];
            if (have) {
                tmem_ld16(taddr + j * 16, v);
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) part[(j * 16 + i) * TM + ml] = v[i];
        }
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    }
    __syncthreads();
    cluster_sync();          // every block's sums are in its shared memory

    if (warp >= 2) {
        // ---------------- epilogue, second half: this block's share of the tile's rows, summed over the cluster ----------------
        const int e = (int)threadIdx.x - 64;
        const int R = TM / S;                         // rows per block: 128, 64, 32 or 16 (16 lanes are always 16 rows of one tile of 16)
        const int mr = rank * R + e % R;              // row of the tile
        const int m = m0 + mr;
        const bool m_ok = m < a.M;
        const int half16 = lane & 8;                  // 0: rows 0..7 of a tile of 16; 8: rows 8..15
        for (int t = e / R; t < NP; t += S) {
            float v = 0.f;
            for (int c = 0; c < S; ++c) v += ld_peer(part + t * TM + mr, (unsigned)c);      // in the order of the ranks
            v *= row_scale[t];
            const bool ok = m_ok && t < a.N;
            if (a.epi == EPI_STORE) {
                if (ok) {
                    if (a.y_f32) reinterpret_cast<float*>(a.y)[(size_t)t * a.ldy + m] = v;
                    else reinterpret_cast<__nv_bfloat16*>(a.y)[(size_t)t * a.ldy + m] = __float2bfloat16_rn(v);
                }
            } else if (a.epi == EPI_RESID_ADD) {
                float nv = 0.f;
                if (ok) {
                    nv = a.acc[(size_t)t * a.M + m] + v;
                    a.acc[(size_t)t * a.M + m] = nv;
                }
                if (a.xg_out != nullptr) {
                    if (ok) {
                        const float gm = a.next_gamma_f32 ? reinterpret_cast<const float*>(a.next_gamma)[m]
                                                          : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.next_gamma)[m]);
                        a.xg_out[(size_t)t * a.M + m] = __float2bfloat16_rn(nv * gm);
                    }
                    float sq = nv * nv;               // over the tile of 16 rows: the lanes of a group of 16, in a fixed order
                    sq += __shfl_xor_sync(0xffffffffu, sq, 1);
                    sq += __shfl_xor_sync(0xffffffffu, sq, 2);
                    sq += __shfl_xor_sync(0xffffffffu, sq, 4);
                    sq += __shfl_xor_sync(0xffffffffu, sq, 8);
                    if ((lane & 15) == 0 && ok) a.ssq_out[(size_t)(m >> 4) * kSquaresRow + t] = sq;
                }
            } else if (a.epi == EPI_SWIGLU) {
                const float other = __shfl_xor_sync(0xffffffffu, v, 8);      // rows 0..7 of a tile are gates, rows 8..15 their ups
                const int i = (m >> 4) * 8 + (m & 7);
                if (half16 == 0 && t < a.N && i < (a.M >> 1))
                    reinterpret_cast<__nv_bfloat16*>(a.y)[(size_t)t * a.ldy + i] = __float2bfloat16_rn(v / (1.0f + expf(-v)) * other);
            } else {
                // EPI_ROPE: rows 0..7 of a tile of 16 are lanes 8j..8j+7 of a head (in its dealt order), rows 8..15 their partners
                const SkRope& r = a.rope;
                const float other = __shfl_xor_sync(0xffffffffu, v, 8);
                if (ok) {
                    const int head = m / r.hd, lane_of_head = m % r.hd;
                    float res = v;
                    if (head < r.n_heads + r.n_kv) {
                        const float2 cs = r.table[(size_t)rope_pos[t] * (r.hd >> 1) + 8 * (lane_of_head >> 4) + (m & 7)];
                        res = half16 == 0 ? v * cs.x - other * cs.y : other * cs.y + v * cs.x;
                    }
                    if (head < r.n_heads) {
                        reinterpret_cast<__nv_bfloat16*>(a.y)[(size_t)t * a.ldy + m] = __float2bfloat16_rn(res);
                    } else if (rope_where[t] >= 0) {
                        const int kvh = head - r.n_heads;          // k heads, then v heads
                        const size_t head_stride = (size_t)r.page_size * r.hd, page_elems = (size_t)r.n_kv * head_stride;
                        __nv_bfloat16* dst = r.pool + rope_where[t] +
                                             (kvh < r.n_kv ? (size_t)kvh * head_stride : page_elems + (size_t)(kvh - r.n_kv) * head_stride);
                        dst[lane_of_head] = __float2bfloat16_rn(res);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    cluster_sync();          // nobody leaves while a peer may still read its shared memory
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols));
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The TMA's view of a K-major bf16 matrix [rows, K] (row stride ld): boxes of box_rows x 64, 128-byte swizzle;
// what lies outside the matrix arrives as zeros.
int make_map(const void* base, long long ld, int rows, int K, int box_rows, CUtensorMap* out) {
    static EncodeTiledFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
            return blm_fail(BLM_CUDA_ERROR, "gemm_sk: the driver has no cuTensorMapEncodeTiled");
        encode = (EncodeTiledFn)fn;
    }
    static std::map<std::tuple<const void*, long long, int, int, int>, CUtensorMap> maps;
    const auto key = std::make_tuple(base, ld, rows, K, box_rows);
    auto it = maps.find(key);
    if (it != maps.end()) {
        *out = it->second;
        return BLM_OK;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return blm_fail(BLM_CUDA_ERROR, "gemm_sk: cuTensorMapEncodeTiled failed (%d)", (int)r);
    if (maps.size() > 8192) maps.clear();
    maps.emplace(key, *out);
    return BLM_OK;
}

int padded_tokens(int N) { return N <= 16 ? 16 : (N <= 32 ? 32 : (N <= 64 ? 64 : 128)); }

// bytes of shared memory beside the ring, and the ring's depth that fits with it
size_t fixed_bytes(int NP) { return (size_t)NP * TM * 4 + (size_t)NP * 16 + 1024 + 512; }
int ring_depth(int NP, int k_per) {
    const size_t stage = kWBytes + (size_t)NP * BK * 2;
    int n = (int)((220 * 1024 - fixed_bytes(NP)) / (stage + 16));
    if (n > k_per) n = k_per;
    if (n > 32) n = 32;
    return n < 2 ? 2 : n;
}

template <int NP>
int launch(const SkArgs& a, const CUtensorMap& wmap, const CUtensorMap& xmap, int tiles, cudaStream_t stream) {
    const int k_iters = (a.K + BK - 1) / BK, k_per = (k_iters + a.S - 1) / a.S;
    const int n_stages = ring_depth(NP, k_per);
    const size_t smem = (size_t)n_stages * (kWBytes + (size_t)NP * BK * 2 + 16) + fixed_bytes(NP);
    static bool opted_in = false;
    if (!opted_in) {
        cudaError_t e = cudaFuncSetAttribute(gemm_sk_kernel<NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "gemm_sk: %s", cudaGetErrorString(e));
        opted_in = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles * a.S));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)a.S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_sk_kernel<NP>, a, wmap, xmap, n_stages);
    if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "gemm_sk: %s", cudaGetErrorString(e));
    return blm_check_launch("gemm_sk");
}

}  // namespace

// 1 when blm_gemm_sk takes the shape: up to 128 tokens, K a multiple of 8 (rows 16-byte aligned) and at least 64
BLM_API int blm_gemm_sk_supported(int N, int M, int K) { return N >= 1 && N <= 128 && M >= 1 && K >= 64 && K % 8 == 0; }

BLM_API int blm_gemm_sk_squares_row() { return kSquaresRow; }

// y = x . w^T for N <= 128 tokens with one of the fused ends; see the head of this file.  x [N, K] bfloat16 (row
// stride ldx), w [M, K] bfloat16 (ldw).  epi 0: y [N, M] bfloat16 or fp32 (y_f32).  epi 1: w is [2 I, K] in tiles
// of 8 gate rows and their 8 up rows, M = 2 I, y [N, I] bfloat16.  epi 2: acc [N, M] fp32 += the product; with
// next_gamma also xg_out and ssq_out.  epi 3: q, k and v with the rotary embedding; q to y, k and v to the cache.
BLM_API int blm_gemm_sk(const void* w, long long ldw, int M, int K, const void* x, long long ldx, int N, void* y, long long ldy,
                        int y_f32, float* acc, int epi, const float* ssq_in, int ssq_parts, float eps, const void* next_gamma,
                        int next_gamma_f32, void* xg_out, float* ssq_out, const SkRope* rope, int* status, cudaStream_t stream) {
    if (N == 0 || M == 0) return BLM_OK;
    BLM_REQUIRE(blm_gemm_sk_supported(N, M, K), "gemm_sk: %d tokens x %d outputs x K %d (1..128 tokens, K a multiple of 8, at least 64)", N, M, K);
    BLM_REQUIRE(ldx % 8 == 0 && ldw % 8 == 0 && ((size_t)x & 15) == 0 && ((size_t)w & 15) == 0, "gemm_sk: operand rows must be 16-byte aligned");
    BLM_REQUIRE(epi >= EPI_STORE && epi <= EPI_ROPE, "gemm_sk: epilogue %d", epi);
    BLM_REQUIRE(status != nullptr, "gemm_sk: no status word");
    BLM_REQUIRE(epi != EPI_SWIGLU || (M % 16 == 0 && y != nullptr && !y_f32), "gemm_sk: the gated epilogue needs weight rows in tiles of 16 and a bfloat16 output");
    BLM_REQUIRE(epi != EPI_RESID_ADD || acc != nullptr, "gemm_sk: no stream to add into");
    BLM_REQUIRE(epi == EPI_RESID_ADD || y != nullptr, "gemm_sk: no output");
    BLM_REQUIRE(ssq_in == nullptr || (ssq_parts >= 1 && N <= kSquaresRow), "gemm_sk: a handed-over norm serves up to %d tokens", kSquaresRow);
    BLM_REQUIRE(xg_out == nullptr || (epi == EPI_RESID_ADD && next_gamma != nullptr && ssq_out != nullptr && N <= kSquaresRow),
                "gemm_sk: only the product that adds into the stream can hand a norm over (up to %d tokens), with gamma and room for the sums", kSquaresRow);
    SkArgs a = {};
    a.M = M; a.K = K; a.N = N; a.y = y; a.ldy = ldy; a.y_f32 = y_f32; a.acc = acc; a.epi = epi; a.ssq_in = ssq_in;
    a.ssq_parts = ssq_parts; a.eps = eps; a.next_gamma = next_gamma; a.next_gamma_f32 = next_gamma_f32;
    a.xg_out = (__nv_bfloat16*)xg_out; a.ssq_out = ssq_out; a.status = status;
    if (epi == EPI_ROPE) {
        BLM_REQUIRE(rope != nullptr && rope->token_pos && rope->table && !y_f32, "gemm_sk: the rotary epilogue needs positions, a table and a bfloat16 q");
        BLM_REQUIRE(rope->hd % 16 == 0 && rope->hd >= 16, "gemm_sk: the rotary epilogue takes head sizes in steps of 16, got %d", rope->hd);
        BLM_REQUIRE(M == (rope->n_heads + (rope->write_cache ? 2 * rope->n_kv : 0)) * rope->hd, "gemm_sk: %d outputs are not %d q heads%s of %d lanes",
                    M, rope->n_heads, rope->write_cache ? " and the k and v heads" : "", rope->hd);
        BLM_REQUIRE(!rope->write_cache || (rope->pool && rope->token_seq && rope->slot_of_seq && rope->block_table && rope->page_size > 0),
                    "gemm_sk: the rotary epilogue writes the cache and needs its pool and tables");
        a.rope = *rope;
    }
    const int tiles = (M + TM - 1) / TM, k_iters = (K + BK - 1) / BK, sms = blm_sm_count();
    int S = 8;
    while (S > 1 && (tiles * S > sms || k_iters < 2 * S)) S >>= 1;
    a.S = S;
    const int NP = padded_tokens(N);
    CUtensorMap wmap, xmap;
    int rc = make_map(w, ldw, M, K, TM, &wmap);
    if (rc != BLM_OK) return rc;
    rc = make_map(x, ldx, N, K, NP, &xmap);
    if (rc != BLM_OK) return rc;
    switch (NP) {
        case 16: return launch<16>(a, wmap, xmap, tiles, stream);
        case 32: return launch<32>(a, wmap, xmap, tiles, stream);
        case 64: return launch<64>(a, wmap, xmap, tiles, stream);
        default: return launch<128>(a, wmap, xmap, tiles, stream);
    }
}
