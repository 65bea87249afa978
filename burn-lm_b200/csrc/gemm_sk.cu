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
    const int* token_page;       // optional [N]: the page every token goes to (-1: a row of no sequence)
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
    int vec;                     // 1: rows of the outputs are 16-byte aligned, eight results leave as one store
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
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    const __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
    return make_uint4(*reinterpret_cast<const unsigned*>(&a), *reinterpret_cast<const unsigned*>(&b),
                      *reinterpret_cast<const unsigned*>(&c), *reinterpret_cast<const unsigned*>(&d));
}
// four floats of block `rank`'s shared memory, at the place `local` has in this block's (read after the cluster's
// barrier, which orders it; no memory clobber, so that several of these loads are in flight together)
__device__ __forceinline__ float4 ld_peer4(const float* local, unsigned rank) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];\n" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote));
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
    // [NP][TM]: this block's sums over its slice of K, token by token.  It lies over the ring: it is written when the
    // accumulator is complete, and by then the tensor core has read every stage and no copy is in flight.
    float* part = reinterpret_cast<float*>(ring);
    const size_t ring_bytes = max((size_t)n_stages * kStage, (size_t)NP * TM * 4);
    float* row_scale = reinterpret_cast<float*>(ring + ring_bytes);                                         // [NP] 1 / rms of a handed-over norm's rows
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
    // The blocks that run together start at different places of their K range: requests that go out at the same
    // moment then differ in the address bits that pick the memory channel (rows of W lie a multiple of K apart).
    // A tile's order of summation depends on the tile only, never on the tokens.
    const int skew = my_iters > 0 ? (tile * 5 + rank * 3) % my_iters : 0;
    auto k_of = [&](int it) { const int j = it + skew; return k_lo + (j >= my_iters ? j - my_iters : j); };

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&wmap) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&xmap) : "memory");
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
    blm_trace(0x500);

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- producer ----------------
            const int pre = min(n_stages, my_iters);
            for (int i = 0; i < pre; ++i) {           // weights are nobody's output: they go out at once
                mbar_expect_tx(full + i, kStage);
                tma_load_2d(ring + (size_t)i * kStage, &wmap, k_of(i) * BK, m0, full + i);
            }
            pdl_wait();                               // the tokens are the work of the kernel before
            blm_trace_here(0x510);
            for (int i = 0; i < pre; ++i) tma_load_2d(ring + (size_t)i * kStage + kWBytes, &xmap, k_of(i) * BK, 0, full + i);
            for (int it = pre; it < my_iters; ++it) {
                const int s = it % n_stages;
                if (!mbar_wait(empty + s, ((it / n_stages) - 1) & 1)) {
                    atomicCAS(a.status, SK_OK, SK_TIMEOUT_EMPTY);
                    break;
                }
                mbar_expect_tx(full + s, kStage);
                tma_load_2d(ring + (size_t)s * kStage, &wmap, k_of(it) * BK, m0, full + s);
                tma_load_2d(ring + (size_t)s * kStage + kWBytes, &xmap, k_of(it) * BK, 0, full + s);
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
                if (it == 0) blm_trace_here(0x520);
                const unsigned long long ad = umma_desc(ring + (size_t)s * kStage), bd = umma_desc(ring + (size_t)s * kStage + kWBytes);
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk) umma(tmem_base, ad + 2 * kk, bd + 2 * kk, kIdesc, (it > 0 || kk > 0) ? 1u : 0u);
                umma_commit(empty + s);
            }
            if (ok && my_iters > 0) umma_commit(acc_full);
            blm_trace_here(0x530);
        }
    } else {
        // ---------------- epilogue, first half: this block's sums to its shared memory ----------------
        const int e = (int)threadIdx.x - 64;          // 0 .. 127
        const int quarter = warp & 3;                 // the 32 lanes of tensor memory this warp may read
        pdl_wait();
        if (NP <= kSquaresRow && a.ssq_in != nullptr) {
            // A handed-over norm: warp w sums the parts for its quarter of the tokens.  The lanes go over the parts
            // (lane, lane + 32, ...), each reading its tokens 16 bytes at a time, four parts in flight together (one
            // round trip for up to 128 parts); then the butterfly over the lanes: one fixed order.
            constexpr int TQ = NP / 4;                // tokens of a warp
            constexpr int V4 = TQ / 4;                // 16-byte loads per part
            const int t0 = (warp - 2) * TQ;
            float ssq[TQ];
#pragma unroll
            for (int u = 0; u < TQ; ++u) ssq[u] = 0.f;
            if (t0 < kSquaresRow) {
                for (int p0 = lane; p0 < a.ssq_parts; p0 += 128) {
                    float4 got[4][V4];
#pragma unroll
                    for (int q = 0; q < 4; ++q)
#pragma unroll
                        for (int x = 0; x < V4; ++x)
                            got[q][x] = (p0 + 32 * q < a.ssq_parts && t0 + 4 * x < kSquaresRow)
                                            ? *reinterpret_cast<const float4*>(a.ssq_in + (size_t)(p0 + 32 * q) * kSquaresRow + t0 + 4 * x)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int q = 0; q < 4; ++q)
#pragma unroll
                        for (int x = 0; x < V4; ++x) {      // what lies beyond the step's tokens was never written: it is not added
                            if (t0 + 4 * x + 0 < a.N) ssq[4 * x + 0] += got[q][x].x;
                            if (t0 + 4 * x + 1 < a.N) ssq[4 * x + 1] += got[q][x].y;
                            if (t0 + 4 * x + 2 < a.N) ssq[4 * x + 2] += got[q][x].z;
                            if (t0 + 4 * x + 3 < a.N) ssq[4 * x + 3] += got[q][x].w;
                        }
                }
            }
#pragma unroll
            for (int u = 0; u < TQ; ++u) {
                const float total = warp_sum(ssq[u]);
                if (lane == 0) row_scale[t0 + u] = (t0 + u < a.N) ? 1.0f / sqrtf(total / (float)a.K + a.eps) : 1.0f;
            }
        } else if (e < NP) {
            row_scale[e] = 1.0f;
        }
        if (e < NP) {
            if (a.epi == EPI_ROPE && e < a.N) {
                const SkRope& r = a.rope;
                const int pos = r.token_pos[e];
                rope_pos[e] = pos;
                long long where = -1;                  // a row of no sequence: nothing of it reaches the cache
                if (r.write_cache) {
                    int page = -1;
                    if (r.token_page != nullptr) {
                        page = r.token_page[e];
                    } else {
                        const int seq = r.token_seq[e];
                        if (seq >= 0) page = r.block_table[(size_t)r.slot_of_seq[seq] * r.table_stride + pos / r.page_size];
                    }
                    if (page >= 0) where = ((long long)page * 2 * r.n_kv * r.page_size + pos % r.page_size) * r.hd;
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
        if (e == 0) blm_trace_here(0x540);
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
    blm_trace(0x550);
    cluster_sync();          // every block's sums are in its shared memory
    blm_trace(0x560);

    if (warp >= 2) {
        // ---------------- epilogue, second half: this block's share of the tile's rows, summed over the cluster ----------------
        // A unit of work is (eight consecutive rows, one token): the sums of the S blocks are read 16 bytes at a time
        // and added in the order of the ranks; the eight results leave as one 16-byte store.  Neighbouring lanes
        // hold the two halves of a tile of 16 rows (gates | ups, or the two halves of eight rotary pairs).
        const int e = (int)threadIdx.x - 64;
        const int R = TM / S, G8 = R / 8;             // rows per block, groups of eight rows per block
        const int items = G8 * NP;
        const bool vec = a.vec != 0;
        for (int it = e; it < items; it += 128) {     // a warp's lanes are all inside or all outside
            const int t = it / G8, mr0 = rank * R + 8 * (it % G8);
            const int m = m0 + mr0;
            const bool odd = (it & 1) != 0;           // rows 8..15 of a tile of 16
            const float* mine = part + t * TM + mr0;
            float v[8];
            {
                float4 lo[8], hi[8];
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    if (c < S) {
                        if (S == 1) { lo[c] = *reinterpret_cast<const float4*>(mine); hi[c] = *reinterpret_cast<const float4*>(mine + 4); }
                        else { lo[c] = ld_peer4(mine, (unsigned)c); hi[c] = ld_peer4(mine + 4, (unsigned)c); }
                    }
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = 0.f;
#pragma unroll
                for (int c = 0; c < 8; ++c)           // in the order of the ranks
                    if (c < S) {
                        v[0] += lo[c].x; v[1] += lo[c].y; v[2] += lo[c].z; v[3] += lo[c].w;
                        v[4] += hi[c].x; v[5] += hi[c].y; v[6] += hi[c].z; v[7] += hi[c].w;
                    }
            }
            const float sc = row_scale[t];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] *= sc;
            const bool t_ok = t < a.N;
            const bool whole = vec && m + 8 <= a.M;   // all eight rows exist and 16-byte stores are aligned
            if (a.epi == EPI_STORE) {
                if (!t_ok || m >= a.M) continue;
                if (a.y_f32) {
                    float* dst = reinterpret_cast<float*>(a.y) + (size_t)t * a.ldy + m;
                    if (whole) {
                        reinterpret_cast<float4*>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
                        reinterpret_cast<float4*>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
                    } else {
                        for (int i = 0; i < 8 && m + i < a.M; ++i) dst[i] = v[i];
                    }
                } else {
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.y) + (size_t)t * a.ldy + m;
                    if (whole) *reinterpret_cast<uint4*>(dst) = pack8(v);
                    else for (int i = 0; i < 8 && m + i < a.M; ++i) dst[i] = __float2bfloat16_rn(v[i]);
                }
            } else if (a.epi == EPI_RESID_ADD) {
                float nv[8], sq = 0.f;
                float* dst = a.acc + (size_t)t * a.M + m;
                const bool live = t_ok && m < a.M;
                if (live && whole) {
                    const float4 o0 = reinterpret_cast<const float4*>(dst)[0], o1 = reinterpret_cast<const float4*>(dst)[1];
                    nv[0] = o0.x + v[0]; nv[1] = o0.y + v[1]; nv[2] = o0.z + v[2]; nv[3] = o0.w + v[3];
                    nv[4] = o1.x + v[4]; nv[5] = o1.y + v[5]; nv[6] = o1.z + v[6]; nv[7] = o1.w + v[7];
                    reinterpret_cast<float4*>(dst)[0] = make_float4(nv[0], nv[1], nv[2], nv[3]);
                    reinterpret_cast<float4*>(dst)[1] = make_float4(nv[4], nv[5], nv[6], nv[7]);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        nv[i] = 0.f;
                        if (live && m + i < a.M) { nv[i] = dst[i] + v[i]; dst[i] = nv[i]; }
                    }
                }
                if (a.xg_out != nullptr) {
                    float gm[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        gm[i] = (live && m + i < a.M) ? (a.next_gamma_f32 ? reinterpret_cast<const float*>(a.next_gamma)[m + i]
                                                                          : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.next_gamma)[m + i]))
                                                      : 0.f;
                    float xg[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) { xg[i] = nv[i] * gm[i]; sq += nv[i] * nv[i]; }       // the eight rows in order
                    if (live) {
                        __nv_bfloat16* xd = a.xg_out + (size_t)t * a.M + m;
                        if (whole) *reinterpret_cast<uint4*>(xd) = pack8(xg);
                        else for (int i = 0; i < 8 && m + i < a.M; ++i) xd[i] = __float2bfloat16_rn(xg[i]);
                    }
                    const float other = __shfl_xor_sync(0xffffffffu, sq, 1);
                    if (!odd && live) a.ssq_out[(size_t)(m >> 4) * kSquaresRow + t] = sq + other;        // rows 0..7, then rows 8..15
                }
            } else if (a.epi == EPI_SWIGLU) {
                float up[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) up[i] = __shfl_xor_sync(0xffffffffu, v[i], 1);       // the odd lane holds the ups of these gates
                const int i0 = (m >> 4) * 8, inner = a.M >> 1;
                if (odd || !t_ok || i0 >= inner) continue;
                float r8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) r8[i] = v[i] / (1.0f + expf(-v[i])) * up[i];
                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.y) + (size_t)t * a.ldy + i0;
                if (vec && i0 + 8 <= inner) *reinterpret_cast<uint4*>(dst) = pack8(r8);
                else for (int i = 0; i < 8 && i0 + i < inner; ++i) dst[i] = __float2bfloat16_rn(r8[i]);
            } else {
                // EPI_ROPE: the even lane holds lanes 8j..8j+7 of a head (in its dealt order), the odd lane their partners
                const SkRope& r = a.rope;
                float other[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) other[i] = __shfl_xor_sync(0xffffffffu, v[i], 1);
                if (!t_ok || m >= a.M) continue;
                const int head = m / r.hd, lane_of_head = m % r.hd;
                if (head < r.n_heads + r.n_kv) {
                    const float2* cs = r.table + (size_t)rope_pos[t] * (r.hd >> 1) + 8 * (lane_of_head >> 4);
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        const float4 c2 = *reinterpret_cast<const float4*>(cs + i);      // (cos, sin) of pairs i and i + 1
                        if (!odd) { v[i] = v[i] * c2.x - other[i] * c2.y; v[i + 1] = v[i + 1] * c2.z - other[i + 1] * c2.w; }
                        else { v[i] = other[i] * c2.y + v[i] * c2.x; v[i + 1] = other[i + 1] * c2.w + v[i + 1] * c2.z; }
                    }
                }
                __nv_bfloat16* dst;
                if (head < r.n_heads) {
                    dst = reinterpret_cast<__nv_bfloat16*>(a.y) + (size_t)t * a.ldy + m;
                } else {
                    if (rope_where[t] < 0) continue;
                    const int kvh = head - r.n_heads;          // k heads, then v heads
                    const size_t head_stride = (size_t)r.page_size * r.hd, page_elems = (size_t)r.n_kv * head_stride;
                    dst = r.pool + rope_where[t] + (kvh < r.n_kv ? (size_t)kvh * head_stride : page_elems + (size_t)(kvh - r.n_kv) * head_stride) + lane_of_head;
                }
                if (vec) *reinterpret_cast<uint4*>(dst) = pack8(v);
                else for (int i = 0; i < 8; ++i) dst[i] = __float2bfloat16_rn(v[i]);
            }
        }
    }
    if (threadIdx.x == 64) blm_trace_here(0x570);
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

// bytes of shared memory beside the ring (which also holds the block's sums once it is drained), and the ring's
// depth that fits with it
size_t fixed_bytes(int NP) { return (size_t)NP * 16 + 1024 + 512; }
size_t ring_bytes_of(int NP, int n_stages) {
    const size_t ring = (size_t)n_stages * (kWBytes + (size_t)NP * BK * 2), sums = (size_t)NP * TM * 4;
    return ring > sums ? ring : sums;
}
// `room`: what a block may take: all of an SM's shared memory, or half of it when the blocks come in more than
// one wave, so that a second block streams while the first one is in its epilogue
int ring_depth(int NP, int k_per, size_t room) {
    const size_t stage = kWBytes + (size_t)NP * BK * 2;
    int n = room > fixed_bytes(NP) ? (int)((room - fixed_bytes(NP)) / (stage + 16)) : 0;
    if (n > k_per) n = k_per;
    if (n > 32) n = 32;
    return n < 2 ? 2 : n;
}

template <int NP>
int launch(const SkArgs& a, const CUtensorMap& wmap, const CUtensorMap& xmap, int tiles, cudaStream_t stream) {
    const int k_iters = (a.K + BK - 1) / BK, k_per = (k_iters + a.S - 1) / a.S;
    // A block that allocates tensor memory has its SM to itself (cudaOccupancyMaxActiveBlocksPerMultiprocessor
    // answers 1 for such a kernel whatever its size), so the ring takes what shared memory there is; measured, a ring
    // of four stages streams as fast as one of seven.
    int n_stages = ring_depth(NP, k_per, 220 * 1024);
    const size_t smem = ring_bytes_of(NP, n_stages) + (size_t)n_stages * 16 + fixed_bytes(NP);
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
    if (a.S > 1) {
        // all clusters at once, or smaller ones: a cluster that has to wait for SMs of one GPC to come free starts a
        // second wave (how many fit is asked once per cluster size and shared-memory size)
        static std::map<std::pair<int, size_t>, int> fits;
        const auto key = std::make_pair(a.S, smem);
        auto it = fits.find(key);
        if (it == fits.end()) {
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_sk_kernel<NP>, &cfg) != cudaSuccess) n = 0;
            it = fits.emplace(key, n).first;
        }
        if (it->second > 0 && it->second < tiles) return -1;       // the caller halves the clusters
    }
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
    auto aligned = [](const void* p) { return ((size_t)p & 15) == 0; };
    if (epi == EPI_STORE) a.vec = aligned(y) && ldy % (y_f32 ? 4 : 8) == 0;
    else if (epi == EPI_SWIGLU) a.vec = aligned(y) && ldy % 8 == 0;
    else if (epi == EPI_RESID_ADD) a.vec = M % 8 == 0 && aligned(acc) && (xg_out == nullptr || aligned(xg_out));
    else a.vec = aligned(y) && ldy % 8 == 0 && (!rope->write_cache || aligned(rope->pool)) && aligned(rope->table);
    const int tiles = (M + TM - 1) / TM, k_iters = (K + BK - 1) / BK, sms = blm_sm_count();
    const int NP = padded_tokens(N);
    int S = 8;
    while (S > 1 && (tiles * S > sms || k_iters < 2 * S)) S >>= 1;
    a.S = S;
    CUtensorMap wmap, xmap;
    int rc = make_map(w, ldw, M, K, TM, &wmap);
    if (rc != BLM_OK) return rc;
    rc = make_map(x, ldx, N, K, NP, &xmap);
    if (rc != BLM_OK) return rc;
    for (;;) {
        switch (NP) {
            case 16: rc = launch<16>(a, wmap, xmap, tiles, stream); break;
            case 32: rc = launch<32>(a, wmap, xmap, tiles, stream); break;
            case 64: rc = launch<64>(a, wmap, xmap, tiles, stream); break;
            default: rc = launch<128>(a, wmap, xmap, tiles, stream); break;
        }
        if (rc != -1 || a.S == 1) return rc == -1 ? blm_fail(BLM_CUDA_ERROR, "gemm_sk: no room for a block") : rc;
        a.S >>= 1;       // the clusters did not all fit at once
    }
}
