// Skinny matrix products for decode steps: y[N, M] = x[N, K] . W[M, K]^T with N <= 16 tokens, bf16
// weights streamed once from HBM, fp32 accumulation on the tensor cores.
//
// One persistent block per SM.  A producer warp feeds a ring of shared-memory stages with TMA tile copies
// (cp.async.bulk.tensor, one 8 KB box of 16 weight rows by 256 k per stage, 128-byte swizzle, completion
// counted on mbarriers), eight of its lanes each polling the barriers of one consumer warp, so ~100 KB of
// weights are in flight per SM whatever the consumers do.  Each of the eight consumer warps owns a tile
// of 16 weight rows at a time (or a slice of its K, when the block has few tiles) and walks it stage after
// stage through a part of the ring that is its own (so that it sees every phase of its barriers, which a
// parity wait needs), multiplying with mma.sync.m16n8k16: the weight rows are the "A" operand, the tokens
// the "B" operand.  A thread reads 16 contiguous bytes of a weight row; the k index inside an instruction
// is permuted the same way for both operands, which a dot product does not notice, so the rows need no
// transpose.  Sums are taken in one fixed order; slices of K meet in shared memory.
// The weight is seen by the TMA as [K / 64][rows][64]: a box is 4 chunks of 64 k for 16 rows, which
// lands in shared memory as [chunk][row][128 bytes].
//
// The tokens reach shared memory in one of three ways: with the weights, a box behind every stage's
// weight box (one tile per block, or tokens too wide to keep); fetched once by TMA in chunks of 256 k with
// a barrier each, so that the first weights are worked on while later tokens are on their way; or staged
// by the consumers, which then also compute the RMS norm of the fp32 stream.
//
// Fused around the product, to save launches and activation traffic:
//   prologue  x = rmsnorm(resid[rows]) * gamma from the fp32 residual stream, or a norm handed over by the
//             product that wrote the stream (x = stream * gamma in bf16 and the rows' sums of squares in
//             parts): the result's rows are then scaled by 1 / rms
//   epilogue  store (bf16 or fp32) | silu(gate) * up (a fused weight whose 16-row tiles hold 8 gate
//             rows, then the 8 up rows of the same outputs)
//             | resid += y (exactly one writer per element), optionally handing the next norm over
//             | rotary embedding of q and k and the append of k and v to the paged cache
// The kernel is launched as a programmatic dependent: its blocks start while the kernel before still
// runs, set up and prefetch weights, and wait (griddepcontrol.wait) only where they first touch its output.
// Every wait on an mbarrier is bounded: after kSpinLimit polls the thread records the failure in
// the status word the caller gave and leaves the kernel.
#include <cuda.h>

#include <map>
#include <tuple>

#include "common.cuh"

BLM_API const char* blm_gemv_last_error() { return g_blm_error; }

constexpr int kConsumerWarps = 8;
constexpr int kGemvThreads = (kConsumerWarps + 1) * 32;   // + the producer warp
// k elements per stage, a parameter of the kernel: 256 (8 KB of weights a stage), or 128 (4 KB) where many wide
// tokens leave the ring too little room for two stages of 256 per warp; a stage is [SK / 64 chunks][16 rows][128
// bytes], swizzled
constexpr unsigned kSpinLimit = 1u << 20;   // polls of a wait before it gives up (seconds; a real wait is microseconds)

enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_RESID_ADD = 2, EPI_ROPE = 3 };

// EPI_ROPE: the product is a step's q, k and v (heads in that order); q and k are rotated by their token's
// position and the rotated k and the v go straight to the token's place in the paged cache, q to y.  The
// rows of every q and k head are dealt out so that a 16-row tile holds eight pairs: rows 0..7 the lanes
// 8j .. 8j + 7 of the head, rows 8..15 their partners (lanes + hd / 2); a thread then has both halves of
// its pairs in registers.  q and k keep that order of lanes (a dot product does not mind), v the stored one.
struct GemvRope {
    const int* token_pos;        // [N] position of every token
    const int* token_seq;        // [N] the token's sequence in the step
    const int* slot_of_seq;      // cache slot of every sequence
    const int* block_table;      // [slots][table_stride] pages of every slot
    const float2* table;         // (cos, sin) [positions][hd / 2]; covers every position of the step
    __nv_bfloat16* pool;         // [pages][2][n_kv][page_size][hd] of this cache line
    int table_stride, n_heads, n_kv, hd, page_size, write_cache;
    const int* token_page;       // optional [N]: the page every token goes to (-1: a row of no sequence), looked up once per step
};
enum { GEMV_OK = 0, GEMV_TIMEOUT_FULL = 1, GEMV_TIMEOUT_EMPTY = 2 };
enum { X_STAGED = 0, X_IN_RING = 1, X_BY_TMA = 2 };

struct GemvArgs {
    const __nv_bfloat16* w;
    long long ldw;
    int M;              // outputs (for EPI_SWIGLU: the inner size I; W has 2 I rows in tiles of 8 gate + 8 up)
    int K;
    const __nv_bfloat16* x;  // plain input [N, K] (ldx), or null when the norm prologue is used
    long long ldx;
    const float* resid;      // norm prologue: fp32 stream [*, K]
    const void* gamma;
    int gamma_f32;
    float eps;
    const int* rows;         // optional gather of stream rows
    int N;
    void* y;                 // EPI_STORE / EPI_SWIGLU output [N, M]
    long long ldy;
    int y_f32;
    float* acc;              // EPI_RESID_ADD: fp32 [N, M] (ld = M)
    int epi;
    int n_stages;            // ring depth
    // A norm handed over by the kernel that wrote the stream: x is bf16(stream * gamma), not yet divided by
    // the root mean square; ssq_in[part][16] holds, for each stream row, sums of squares whose total over
    // the parts is the row's; the result is scaled by 1 / sqrt(total / K + eps) per row.
    const float* ssq_in;
    int ssq_parts;
    // EPI_RESID_ADD can hand such a norm over: besides the sum it leaves bf16(stream * next_gamma) in
    // xg_out [N, M] and its tile's sums of squares in ssq_out[tile][16].
    const void* next_gamma;
    int next_gamma_f32;
    __nv_bfloat16* xg_out;
    float* ssq_out;
    // How plain tokens reach shared memory.  X_STAGED: the consumers copy them (or normalise the stream)
    // before they start.  X_IN_RING: every block has one tile, so a token lane is used once per block and
    // the tokens travel with the weights, a box of [token rows x 256 k] behind the weight box of every
    // stage.  X_BY_TMA: the producer fetches them once, in chunks of 256 k with a barrier each, and a
    // consumer only waits for the chunk it is about to use: the first weights are worked on while the
    // later tokens are still on their way.
    int x_mode;
    GemvRope rope;           // EPI_ROPE
    int* status;             // device word: 0, or the first failure (a bounded wait ran out)
};

__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// false when the phase did not complete within the poll limit
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
// one box of the weight: chunks [chunk0, chunk0 + 4) of rows [row0, row0 + 16); what lies outside the
// matrix arrives as zeros
__device__ __forceinline__ void tma_load_box(void* dst, const CUtensorMap* map, int row0, int chunk0, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(0), "r"(row0), "r"(chunk0), "r"(smem_u32(bar))
        : "memory");
}
// the tokens' part of a stage: chunks [chunk0, chunk0 + 4) of all token rows (rows beyond N arrive as zeros)
__device__ __forceinline__ void tma_load_tokens(void* dst, const CUtensorMap* map, int chunk0, unsigned long long* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(0), "r"(0), "r"(chunk0), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;\n" ::"n"(kConsumerWarps * 32) : "memory"); }

// Stages all tokens in shared memory as bf16 (zero beyond K and N); run by the consumer warps.
template <int NBT>
__device__ __forceinline__ void gemv_stage_tokens(const GemvArgs& a, __nv_bfloat16* xs, int xstride, int kpad,
                                                  int tid, int lane, int warp) {
    constexpr int nrows = NBT * 8;
    constexpr int n_threads = kConsumerWarps * 32;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    if (a.resid == nullptr) {
        // plain tokens: asynchronous 16-byte copies straight into shared memory
        const int vec = kpad / 8;
        for (int idx = tid; idx < nrows * vec; idx += n_threads) {
            const int r = idx / vec, k = (idx % vec) * 8;
            __nv_bfloat16* dst = xs + (size_t)r * xstride + k;
            if (r < a.N && k < a.K) {
                const size_t src_row = a.rows ? a.rows[r] : r;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(dst)), "l"(a.x + src_row * a.ldx + k));
            } else {
                *reinterpret_cast<uint4*>(dst) = zero4;
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
        asm volatile("cp.async.wait_group 0;\n" ::);
        return;
    }
    // norm prologue: a warp takes a stream row through registers in passes of 2048 lanes: sixteen
    // independent 16-byte loads of the row per lane and the matching gamma, all through the read-only
    // path and all issued before anything is stored, so that they overlap instead of queueing behind
    // the stores; first for the sum of squares, then to scale and store
    for (int r = warp; r < nrows; r += kConsumerWarps) {
        const bool live = r < a.N;
        const float* src = a.resid + (size_t)(live ? (a.rows ? a.rows[r] : r) : 0) * a.K;
        float4 v[16];
        auto load_pass = [&](int k0) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int k = k0 + (i * 32 + lane) * 4;
                v[i] = (live && k < a.K) ? __ldg(reinterpret_cast<const float4*>(src + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        };
        auto gamma_at = [&](int k) -> float4 {
            if (k >= a.K) return make_float4(0.f, 0.f, 0.f, 0.f);
            if (a.gamma_f32) return __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.gamma) + k));
            const uint2 raw = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.gamma) + k));
            const float2 ga = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
            const float2 gb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
            return make_float4(ga.x, ga.y, gb.x, gb.y);
        };
        float ss = 0.f;
        for (int k0 = 0; k0 < a.K; k0 += 2048) {
            load_pass(k0);
#pragma unroll
            for (int i = 0; i < 16; ++i) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
        }
        float4 gm[16];
        if (a.K <= 2048) {
#pragma unroll
            for (int i = 0; i < 16; ++i) gm[i] = gamma_at((i * 32 + lane) * 4);     // in flight during the reduction
        }
        ss = warp_sum(ss);
        const float sc = 1.0f / sqrtf(ss / (float)a.K + a.eps);
        for (int k0 = 0; k0 < kpad; k0 += 2048) {
            if (a.K > 2048) {      // a single pass is still in registers
                load_pass(k0);
#pragma unroll
                for (int i = 0; i < 16; ++i) gm[i] = gamma_at(k0 + (i * 32 + lane) * 4);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int k = k0 + (i * 32 + lane) * 4;
                if (k < kpad) {
                    __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(xs + (size_t)r * xstride + k);
                    dst[0] = __floats2bfloat162_rn(v[i].x * sc * gm[i].x, v[i].y * sc * gm[i].y);
                    dst[1] = __floats2bfloat162_rn(v[i].z * sc * gm[i].z, v[i].w * sc * gm[i].w);
                }
            }
        }
    }
}

template <int NBT, int SK>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_kernel(const GemvArgs a, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap) {
    extern __shared__ __align__(1024) unsigned char smem[];
    constexpr int nrows = NBT * 8;
    constexpr int kStageK = SK;
    constexpr int kStageBytes = 16 * SK * 2;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kpad = (a.K + kStageK - 1) / kStageK * kStageK;
    const int xstride = kpad + 8;                                   // bf16 elements; 16 bytes of padding
    // layout: ring | tokens | partial sums of warps that share a tile | barriers
    unsigned char* ring = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);   // the swizzle wants 1024-byte alignment
    constexpr int kTokenBytes = nrows * kStageK * 2;                 // the tokens' part of a stage: [4 chunks][nrows][128 bytes]
    const int stage_bytes = kStageBytes + (a.x_mode == X_IN_RING ? kTokenBytes : 0);
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(ring + (size_t)a.n_stages * stage_bytes);
    // X_STAGED: [nrows][xstride]; X_BY_TMA: [chunks of 256 k][4][nrows][128 bytes], swizzled like a stage
    const size_t xs_bytes = a.x_mode == X_IN_RING ? 0 : (a.x_mode == X_BY_TMA ? (size_t)nrows * kpad * 2 : (size_t)nrows * xstride * 2);
    float* red = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(xs) + xs_bytes);   // [warp][16][nrows]
    unsigned long long* full = reinterpret_cast<unsigned long long*>(red + kConsumerWarps * 16 * nrows);
    unsigned long long* empty = full + a.n_stages;
    unsigned long long* meet = empty + a.n_stages;     // where warps that share a tile meet (a bounded wait, like all)
    float* row_scale = reinterpret_cast<float*>(meet + 1);          // [16]: 1 / rms of a handed-over norm's rows
    unsigned long long* xfull = reinterpret_cast<unsigned long long*>(row_scale + 16);   // X_BY_TMA: one per chunk of 256 k
    long long* rope_cache = reinterpret_cast<long long*>(xfull + kpad / kStageK);          // EPI_ROPE [16]: where a token's k row of kv head 0 starts in the pool
    int* rope_pos = reinterpret_cast<int*>(rope_cache + 16);                              // EPI_ROPE [16]: the tokens' positions

    const int out_per_tile = a.epi == EPI_SWIGLU ? 8 : 16;
    const int n_tiles = (a.M + out_per_tile - 1) / out_per_tile;
    const int stages_per_tile = kpad / kStageK;
    // A unit of work is (tile, slice of K): `ks` warps share a tile when a block has few tiles.
    // This block's tiles are blockIdx.x, blockIdx.x + gridDim.x, ...; its work units go to the warps
    // in turn, in rounds of eight.
    const int my_tiles = n_tiles > (int)blockIdx.x ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    // few tiles in this block: several warps share a tile, each on a slice of K (1, 2, 4 or 8 of them)
    // The slices are cut in units of 256 k whatever the stage size: where a sum is cut, and so its rounding, then
    // does not depend on the stage size, which follows the number of tokens.
    const int units_per_tile = (a.K + 255) / 256;
    int ks = 1;
    while (ks * 2 * my_tiles <= kConsumerWarps && ks * 2 <= units_per_tile) ks *= 2;
    const int stages_per_slice = (units_per_tile + ks - 1) / ks * (256 / kStageK);
    const int my_units = my_tiles * ks;
    const int n_rounds = (my_units + kConsumerWarps - 1) / kConsumerWarps;
    // the ring is dealt out to the warps that work (fewer units than warps: fewer, deeper parts); a warp
    // sees every phase of the barriers of its part, which a parity wait needs
    const int depth = a.n_stages / max(1, min(kConsumerWarps, my_units));

    if (tid == 0) {
        for (int s = 0; s < a.n_stages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        mbar_init(meet, kConsumerWarps);
        if (a.x_mode == X_BY_TMA)
            for (int ch = 0; ch < kpad / kStageK; ++ch) mbar_init(xfull + ch, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    // The weights are nobody's output: the producer streams them at once, also while the kernel before this
    // one still runs; the consumers wait for it before they touch the tokens.  The rotary product lets its
    // dependent start only after its own wait: that kernel (the attention) may then take everything but this
    // product's output as written, the cache pages of earlier tokens among it, and fetch them before its own wait.
    if (a.epi != EPI_ROPE) pdl_launch_dependents();

    if (warp == kConsumerWarps) {
        // ---------------- producer: lane w of this warp feeds consumer warp w's part of the ring ----------------
        // Eight lanes poll their own barriers without blocking one another (test_wait, not try_wait), so a
        // stage is re-issued as soon as its warp has let go of it, whatever the other warps do.
        const int w = lane;
        int round = 0, st = 0;            // the next stage of warp w: stage `st` of its unit in `round`
        unsigned q = 0;                   // how many stages warp w has been dealt
        bool more = w < kConsumerWarps && w < my_units;
        unsigned idle = 0;
        if (a.x_mode != X_STAGED) {
            // The weights of the first stages (of the warps' first units) go out at once; the tokens
            // are the work of the kernel before, so they follow after the wait: with the weights, onto
            // the same barriers, or in chunks of their own, one lane a chunk.
            int pre = 0;
            if (more) {
                for (; pre < depth && pre < stages_per_slice; ++pre) {
                    const int stage_of_tile = (w % ks) * stages_per_slice + pre;
                    if (stage_of_tile >= stages_per_tile) break;
                    const int slot = w * depth + pre;
                    mbar_expect_tx(full + slot, stage_bytes);
                    tma_load_box(ring + (size_t)slot * stage_bytes, &wmap, ((int)blockIdx.x + (w / ks) * (int)gridDim.x) * 16,
                                 stage_of_tile * (kStageK / 64), full + slot);
                }
            }
            pdl_wait();
            if (a.x_mode == X_IN_RING) {
                for (int i = 0; i < pre; ++i) {
                    const int slot = w * depth + i;
                    tma_load_tokens(ring + (size_t)slot * stage_bytes + kStageBytes, &xmap,
                                    ((w % ks) * stages_per_slice + i) * (kStageK / 64), full + slot);
                }
            } else if (my_units > 0) {
                for (int ch = lane; ch < stages_per_tile; ch += 32) {
                    mbar_expect_tx(xfull + ch, kTokenBytes);
                    tma_load_tokens(reinterpret_cast<unsigned char*>(xs) + (size_t)ch * kTokenBytes, &xmap, ch * (kStageK / 64), xfull + ch);
                }
            }
            q = pre;
            st = pre;
            if (more && (st == stages_per_slice || (w % ks) * stages_per_slice + st >= stages_per_tile)) { st = 0; ++round; }
        }
        while (__any_sync(0xffffffffu, more)) {
            bool progressed = false;
            if (more) {
                const int unit = round * kConsumerWarps + w;
                const int stage_of_tile = (unit % ks) * stages_per_slice + st;
                if (unit >= my_units) {
                    more = false;
                } else if (stage_of_tile >= stages_per_tile) {      // a short last slice: on to the next round
                    ++round;
                    st = 0;
                    progressed = true;
                } else {
                    const int slot = w * depth + (int)(q % depth);
                    bool free_slot = q < (unsigned)depth;
                    if (!free_slot) {
                        unsigned done;
                        asm volatile(
                            "{\n.reg .pred p;\n"
                            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
                            "selp.u32 %0, 1, 0, p;\n}\n"
                            : "=r"(done)
                            : "r"(smem_u32(empty + slot)), "r"(((q / depth) - 1) & 1)
                            : "memory");
                        free_slot = done != 0;
                    }
                    if (free_slot) {
                        const int tile = blockIdx.x + (unit / ks) * gridDim.x;
                        mbar_expect_tx(full + slot, stage_bytes);
                        tma_load_box(ring + (size_t)slot * stage_bytes, &wmap, tile * 16, stage_of_tile * (kStageK / 64), full + slot);
                        if (a.x_mode == X_IN_RING)
                            tma_load_tokens(ring + (size_t)slot * stage_bytes + kStageBytes, &xmap, stage_of_tile * (kStageK / 64), full + slot);
                        ++q;
                        if (++st == stages_per_slice) { st = 0; ++round; }
                        progressed = true;
                    }
                }
            }
            if (__any_sync(0xffffffffu, progressed)) {
                idle = 0;
            } else {
                __nanosleep(128);      // leave the shared-memory pipe to the consumers while there is nothing to issue
            }
            if (++idle > (kSpinLimit << 2)) {             // nobody could issue for seconds
                if (lane == 0) atomicCAS(a.status, GEMV_OK, GEMV_TIMEOUT_EMPTY);
                return;
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    blm_trace(0x100 | a.epi);
    pdl_wait();
    if (a.epi == EPI_ROPE) pdl_launch_dependents();
    blm_trace(0x110 | a.epi);
    if (a.x_mode == X_STAGED) gemv_stage_tokens<NBT>(a, xs, xstride, kpad, tid, lane, warp);
    if (a.ssq_in != nullptr) {
        // a warp per row: the parts in a fixed order (lane p, p + 32, ..., then the butterfly)
        for (int r = warp; r < nrows; r += kConsumerWarps) {
            float ssq = 0.f;
            if (r < a.N) {
                const int src_row = a.rows ? a.rows[r] : r;
                for (int part = lane; part < a.ssq_parts; part += 32) ssq += a.ssq_in[(size_t)part * 16 + src_row];
            }
            ssq = warp_sum(ssq);
            if (lane == 0) row_scale[r] = r < a.N ? 1.0f / sqrtf(ssq / (float)a.K + a.eps) : 0.f;
        }
    }
    if (a.epi == EPI_ROPE && tid < a.N) {
        // the chain token -> sequence -> slot -> page, walked once here instead of by every thread of the epilogue
        const GemvRope& r = a.rope;
        const int pos = r.token_pos[tid];
        rope_pos[tid] = pos;
        if (r.write_cache) {
            long long where = -1;       // a row of no sequence (padding): nothing of it reaches the cache
            if (r.token_page != nullptr) {
                const int page = r.token_page[tid];          // read beside the position: one round trip, not three
                if (page >= 0) where = ((long long)page * 2 * r.n_kv * r.page_size + pos % r.page_size) * r.hd;
            } else {
                const int seq = r.token_seq[tid];
                if (seq >= 0) {
                    const int slot = r.slot_of_seq[seq];
                    const int page = r.block_table[(size_t)slot * r.table_stride + pos / r.page_size];
                    where = ((long long)page * 2 * r.n_kv * r.page_size + pos % r.page_size) * r.hd;
                }
            }
            rope_cache[tid] = where;
        }
    }
    consumer_barrier();
    blm_trace(0x120 | a.epi);

    const int g = lane >> 2, t = lane & 3;
    for (int round = 0; round < n_rounds; ++round) {
        const int live = min(kConsumerWarps, my_units - round * kConsumerWarps);
        const int unit = round * kConsumerWarps + warp;
        const int tile = blockIdx.x + (unit / ks) * gridDim.x;
        float c[2][NBT][4];     // two sets, used in turn: two chains of dependent instructions instead of one
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int j = 0; j < NBT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) c[h][j][e] = 0.f;
        bool failed = false;
        if (warp < live) {
            for (int st = 0; st < stages_per_slice; ++st) {
                const int stage_of_tile = (unit % ks) * stages_per_slice + st;
                if (stage_of_tile >= stages_per_tile) break;
                const unsigned q = (unsigned)(round * stages_per_slice + st);      // this warp's q-th stage
                const int slot = warp * depth + (int)(q % depth);
                if (!mbar_wait(full + slot, (q / depth) & 1)) {
                    if (lane == 0) atomicCAS(a.status, GEMV_OK, GEMV_TIMEOUT_FULL);
                    failed = true;       // the status word says so; go on to where the others wait for this warp
                    break;
                }
                const unsigned char* stage = ring + (size_t)slot * stage_bytes;
                if (a.x_mode == X_BY_TMA && !mbar_wait(xfull + stage_of_tile, 0)) {      // this chunk of the tokens (it arrives once)
                    if (lane == 0) atomicCAS(a.status, GEMV_OK, GEMV_TIMEOUT_FULL);
                    failed = true;
                    break;
                }
                // where this stage's tokens lie when they are swizzled boxes [4][nrows][128 bytes]
                const unsigned char* xbox = a.x_mode == X_IN_RING ? stage + kStageBytes
                                                                  : reinterpret_cast<const unsigned char*>(xs) + (size_t)stage_of_tile * kTokenBytes;
                // The stage is 8 units of 32 k: chunk u / 2, 64-byte half u % 2; the 16-byte slot of a line is
                // XORed with the line's number mod 8 (the 128-byte swizzle), here the row's.
#pragma unroll
                for (int u = 0; u < kStageK / 32; ++u) {
                    const int k = stage_of_tile * kStageK + u * 32;
                    if (k < a.K) {
                        const unsigned char* chunk = stage + (u >> 1) * (16 * 128);
                        const int s16 = (u & 1) * 4 + t;
                        const uint4 lo = *reinterpret_cast<const uint4*>(chunk + g * 128 + ((s16 ^ g) << 4));
                        const uint4 hi = *reinterpret_cast<const uint4*>(chunk + (g + 8) * 128 + ((s16 ^ g) << 4));
#pragma unroll
                        for (int j = 0; j < NBT; ++j) {
                            // tokens: staged rows, or the stage's own box [chunk][token row][128 bytes], swizzled like the weights
                            const uint4 xv = a.x_mode != X_STAGED
                                ? *reinterpret_cast<const uint4*>(xbox + (u >> 1) * (nrows * 128) + (j * 8 + g) * 128 + ((s16 ^ g) << 4))
                                : *reinterpret_cast<const uint4*>(xs + (size_t)(j * 8 + g) * xstride + k + 8 * t);
                            mma16816(c[0][j], lo.x, hi.x, lo.y, hi.y, xv.x, xv.y);
                            mma16816(c[1][j], lo.z, hi.z, lo.w, hi.w, xv.z, xv.w);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty + slot);          // the stage is read: the producer may refill it
            }
        }
        if (ks > 1) {
            // warps that share a tile: the partial sums meet in shared memory; the warp of slice 0 adds them
            // in a fixed order.  With a split there is a single round (a block has at most 8 / ks tiles).
            float* mine = red + (size_t)warp * 16 * nrows;
#pragma unroll
            for (int j = 0; j < NBT; ++j) {
                mine[(size_t)g * nrows + j * 8 + 2 * t] = c[0][j][0] + c[1][j][0];
                mine[(size_t)g * nrows + j * 8 + 2 * t + 1] = c[0][j][1] + c[1][j][1];
                mine[(size_t)(g + 8) * nrows + j * 8 + 2 * t] = c[0][j][2] + c[1][j][2];
                mine[(size_t)(g + 8) * nrows + j * 8 + 2 * t + 1] = c[0][j][3] + c[1][j][3];
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(meet);
            if (!mbar_wait(meet, 0)) {
                if (lane == 0) atomicCAS(a.status, GEMV_OK, GEMV_TIMEOUT_FULL);
                return;
            }
            if (failed || warp >= live || unit % ks != 0) return;
#pragma unroll
            for (int j = 0; j < NBT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) { c[0][j][e] = 0.f; c[1][j][e] = 0.f; }
            for (int z = 0; z < ks; ++z) {
                const float* part = red + (size_t)(warp + z) * 16 * nrows;
#pragma unroll
                for (int j = 0; j < NBT; ++j) {
                    c[0][j][0] += part[(size_t)g * nrows + j * 8 + 2 * t];
                    c[0][j][1] += part[(size_t)g * nrows + j * 8 + 2 * t + 1];
                    c[0][j][2] += part[(size_t)(g + 8) * nrows + j * 8 + 2 * t];
                    c[0][j][3] += part[(size_t)(g + 8) * nrows + j * 8 + 2 * t + 1];
                }
            }
        } else if (failed) {
            return;
        } else if (warp >= live) {
            continue;
        }
        // the tile is done: rows g and g + 8, tokens 2t and 2t + 1 of every token tile
        if (a.ssq_in != nullptr) {
#pragma unroll
            for (int j = 0; j < NBT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    c[0][j][e] = (c[0][j][e] + c[1][j][e]) * row_scale[j * 8 + 2 * t + (e & 1)];
                    c[1][j][e] = 0.f;
                }
        }
        if (a.epi == EPI_RESID_ADD) {
            // all loads of the stream first, then the sums: the round trips overlap
            float old[NBT][4];
#pragma unroll
            for (int j = 0; j < NBT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int m = tile * 16 + g + 8 * (e >> 1), b = j * 8 + 2 * t + (e & 1);
                    old[j][e] = (m < a.M && b < a.N) ? a.acc[(size_t)b * a.M + m] : 0.f;
                }
            float gm[2] = {0.f, 0.f};          // the next norm's gamma of rows g and g + 8
            if (a.xg_out != nullptr) {
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const int m = tile * 16 + g + 8 * rr;
                    if (m < a.M)
                        gm[rr] = a.next_gamma_f32 ? reinterpret_cast<const float*>(a.next_gamma)[m]
                                                  : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.next_gamma)[m]);
                }
            }
            float sq[NBT][2];                  // this thread's share of the sums of squares of tokens 2t, 2t + 1
#pragma unroll
            for (int j = 0; j < NBT; ++j) {
                sq[j][0] = 0.f;
                sq[j][1] = 0.f;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int m = tile * 16 + g + 8 * (e >> 1), b = j * 8 + 2 * t + (e & 1);
                    if (m < a.M && b < a.N) {
                        const float v = old[j][e] + (c[0][j][e] + c[1][j][e]);
                        a.acc[(size_t)b * a.M + m] = v;
                        if (a.xg_out != nullptr) {
                            a.xg_out[(size_t)b * a.M + m] = __float2bfloat16_rn(v * gm[e >> 1]);
                            sq[j][e & 1] += v * v;
                        }
                    }
                }
            }
            if (a.xg_out != nullptr) {
                // over the tile's 16 rows: the lanes of equal t, in a fixed order
#pragma unroll
                for (int j = 0; j < NBT; ++j)
#pragma unroll
                    for (int bb = 0; bb < 2; ++bb) {
                        float v = sq[j][bb];
                        v += __shfl_xor_sync(0xffffffffu, v, 4);
                        v += __shfl_xor_sync(0xffffffffu, v, 8);
                        v += __shfl_xor_sync(0xffffffffu, v, 16);
                        const int b = j * 8 + 2 * t + bb;
                        if (g == 0 && b < a.N) a.ssq_out[(size_t)tile * 16 + b] = v;
                    }
            }
            continue;
        }
        if (a.epi == EPI_ROPE) {
            const GemvRope& r = a.rope;
            const int tiles_per_head = r.hd >> 4, head = tile / tiles_per_head, jt = tile % tiles_per_head;
            const int half = r.hd >> 1;
            const size_t head_stride_cache = (size_t)r.page_size * r.hd, page_elems = (size_t)r.n_kv * head_stride_cache;
#pragma unroll
            for (int j = 0; j < NBT; ++j)
#pragma unroll
                for (int bb = 0; bb < 2; ++bb) {
                    const int b = j * 8 + 2 * t + bb;
                    if (b >= a.N || tile * 16 >= a.M) continue;
                    float lo = c[0][j][bb] + c[1][j][bb], hi = c[0][j][2 + bb] + c[1][j][2 + bb];   // rows g and g + 8
                    const int pos = rope_pos[b];
                    if (head < r.n_heads + r.n_kv) {
                        const float2 cs = r.table[(size_t)pos * half + 8 * jt + g];
                        const float rl = lo * cs.x - hi * cs.y, rh = lo * cs.y + hi * cs.x;
                        lo = rl;
                        hi = rh;
                    }
                    __nv_bfloat16* dst;
                    if (head < r.n_heads) {
                        dst = reinterpret_cast<__nv_bfloat16*>(a.y) + (size_t)b * a.ldy + (size_t)head * r.hd;
                    } else {
                        const int kvh = head - r.n_heads;          // k heads, then v heads
                        if (rope_cache[b] < 0) continue;
                        dst = r.pool + rope_cache[b] +
                              (kvh < r.n_kv ? (size_t)kvh * head_stride_cache : page_elems + (size_t)(kvh - r.n_kv) * head_stride_cache);
                    }
                    dst[16 * jt + g] = __float2bfloat16_rn(lo);
                    dst[16 * jt + g + 8] = __float2bfloat16_rn(hi);
                }
            continue;
        }
#pragma unroll
        for (int j = 0; j < NBT; ++j) {
            const float v00 = c[0][j][0] + c[1][j][0], v01 = c[0][j][1] + c[1][j][1];   // row g
            const float v10 = c[0][j][2] + c[1][j][2], v11 = c[0][j][3] + c[1][j][3];   // row g + 8
            const int b0 = j * 8 + 2 * t, b1 = b0 + 1;
            if (a.epi == EPI_SWIGLU) {
                const int i = tile * 8 + g;      // rows 0..7 of the tile are gates, rows 8..15 their ups
                if (i < a.M) {
                    __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(a.y);
                    if (b0 < a.N) y[(size_t)b0 * a.ldy + i] = __float2bfloat16_rn(v00 / (1.0f + expf(-v00)) * v10);
                    if (b1 < a.N) y[(size_t)b1 * a.ldy + i] = __float2bfloat16_rn(v01 / (1.0f + expf(-v01)) * v11);
                }
            } else {
                const float v[2][2] = {{v00, v01}, {v10, v11}};
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const int m = tile * 16 + g + 8 * rr;
                    if (m >= a.M) continue;
#pragma unroll
                    for (int bb = 0; bb < 2; ++bb) {
                        const int b = b0 + bb;
                        if (b >= a.N) continue;
                        if (a.y_f32) reinterpret_cast<float*>(a.y)[(size_t)b * a.ldy + m] = v[rr][bb];
                        else reinterpret_cast<__nv_bfloat16*>(a.y)[(size_t)b * a.ldy + m] = __float2bfloat16_rn(v[rr][bb]);
                    }
                }
            }
        }
    }
    blm_trace(0x130 | a.epi);
}

// Shared memory for a shape and the ring depth it leaves room for; 0 when the tokens do not fit.  `stage_k`: k per
// stage.  The ring has a whole number of stages for each of the eight warps where that is possible.
static size_t gemv_plan(int N, int K, int x_mode, int stage_k, int* n_stages_out, int* nbt_out) {
    int nbt = 1;
    while (nbt * 8 < N) nbt *= 2;
    if (nbt > 2) return 0;
    const int nrows = nbt * 8;
    const int kpad = (K + stage_k - 1) / stage_k * stage_k;
    const size_t tokens = x_mode == X_IN_RING ? 0 : (x_mode == X_BY_TMA ? (size_t)nrows * kpad * 2 : (size_t)nrows * (kpad + 8) * 2);
    const size_t stage = (size_t)16 * stage_k * 2 + (x_mode == X_IN_RING ? (size_t)nrows * stage_k * 2 : 0);
    const size_t fixed = 128 + 1024 + (size_t)(kpad / stage_k) * 8 + 256;      // the other barriers, the row scales, the rotary epilogue's tables, alignment
    const size_t red = (size_t)kConsumerWarps * 16 * nrows * 4;
    const size_t limit = 220 * 1024;
    int stages = stage_k == 256 ? 16 : 32;
    while (stages > 8 && (size_t)stages * stage + tokens + red + (size_t)stages * 16 + fixed > limit) --stages;
    if (stages > 8) stages -= stages % 8;
    const size_t total = (size_t)stages * stage + tokens + red + (size_t)stages * 16 + fixed;
    if (total > limit) return 0;
    *n_stages_out = stages;
    *nbt_out = nbt;
    return total;
}
// The plan with stages of 256 k, or, where that leaves a warp a single stage (it could then not fetch one stage
// while it works on another), the plan with stages of 128 k when that gives it at least two.
static size_t gemv_plan_best(int N, int K, int x_mode, int* stage_k_out, int* n_stages_out, int* nbt_out) {
    int st = 0, nbt = 0;
    size_t smem = gemv_plan(N, K, x_mode, 256, &st, &nbt);
    *stage_k_out = 256;
    if (smem > 0 && st < 2 * kConsumerWarps) {
        int st2 = 0, nbt2 = 0;
        const size_t smem2 = gemv_plan(N, K, x_mode, 128, &st2, &nbt2);
        if (smem2 > 0 && st2 >= 2 * kConsumerWarps) {
            *stage_k_out = 128;
            st = st2;
            nbt = nbt2;
            smem = smem2;
        }
    }
    *n_stages_out = st;
    *nbt_out = nbt;
    return smem;
}

// 1 when blm_gemv takes the shape, else 0 (the caller then uses the library product).  `plain_tokens`: the
// input is a bfloat16 matrix used row by row (not a stream to normalise, no gathered rows); such tokens
// can travel with the weights, so their K is not bounded by shared memory.
BLM_API int blm_gemv_supported(int N, int M, int K, int plain_tokens) {
    int st, nbt;
    if (!(N >= 1 && N <= 16 && K % 64 == 0 && M >= 1)) return 0;
    if (gemv_plan(N, K, X_STAGED, 256, &st, &nbt) > 0) return 1;
    return plain_tokens && gemv_plan(N, K, X_IN_RING, 256, &st, &nbt) > 0;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The TMA's view of a weight [rows, K] (row stride ldw): dims (64 k, rows, K / 64); box (64, 16, 4).
static int weight_map(const void* w, long long ldw, int rows, int K, int stage_k, CUtensorMap* out) {
    static EncodeTiledFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
            return blm_fail(BLM_CUDA_ERROR, "gemv: the driver has no cuTensorMapEncodeTiled");
        encode = (EncodeTiledFn)fn;
    }
    static std::map<std::tuple<const void*, long long, int, int, int>, CUtensorMap> cache;
    const auto key = std::make_tuple(w, ldw, rows, K, stage_k);
    auto it = cache.find(key);
    if (it == cache.end()) {
        CUtensorMap m;
        const cuuint64_t dims[3] = {64, (cuuint64_t)rows, (cuuint64_t)(K / 64)};
        const cuuint64_t strides[2] = {(cuuint64_t)ldw * 2, 128};     // bytes: between rows, between chunks
        const cuuint32_t box[3] = {64, 16, (cuuint32_t)(stage_k / 64)};
        const cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(w), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return blm_fail(BLM_CUDA_ERROR, "gemv: cuTensorMapEncodeTiled failed (%d)", (int)r);
        if (cache.size() > 4096) cache.clear();
        it = cache.emplace(key, m).first;
    }
    *out = it->second;
    return BLM_OK;
}

// The TMA's view of the tokens [N, K] (row stride ldx): dims (64 k, N, K / 64); box (64, token rows, 4).
static int token_map(const void* x, long long ldx, int N, int K, int nrows, int stage_k, CUtensorMap* out) {
    static EncodeTiledFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
            return blm_fail(BLM_CUDA_ERROR, "gemv: the driver has no cuTensorMapEncodeTiled");
        encode = (EncodeTiledFn)fn;
    }
    static std::map<std::tuple<const void*, long long, int, int, int, int>, CUtensorMap> cache;
    const auto key = std::make_tuple(x, ldx, N, K, nrows, stage_k);
    auto it = cache.find(key);
    if (it == cache.end()) {
        CUtensorMap m;
        const cuuint64_t dims[3] = {64, (cuuint64_t)N, (cuuint64_t)(K / 64)};
        const cuuint64_t strides[2] = {(cuuint64_t)ldx * 2, 128};
        const cuuint32_t box[3] = {64, (cuuint32_t)nrows, (cuuint32_t)(stage_k / 64)};
        const cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(x), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return blm_fail(BLM_CUDA_ERROR, "gemv: cuTensorMapEncodeTiled failed for the tokens (%d)", (int)r);
        if (cache.size() > 4096) cache.clear();
        it = cache.emplace(key, m).first;
    }
    *out = it->second;
    return BLM_OK;
}

BLM_API int blm_gemv(const void* w, long long ldw, int M, int K, const void* x, long long ldx,
                     const float* resid, const void* gamma, int gamma_f32, float eps, const int* rows, int N,
                     void* y, long long ldy, int y_f32, float* acc, int epi, const float* ssq_in, int ssq_parts,
                     const void* next_gamma, int next_gamma_f32, void* xg_out, float* ssq_out, const GemvRope* rope,
                     int* status, cudaStream_t stream) {
    if (N == 0 || M == 0) return BLM_OK;
    BLM_REQUIRE(N >= 1 && N <= 16, "gemv: %d tokens (1..16)", N);
    BLM_REQUIRE(K % 64 == 0 && K >= 64, "gemv: K = %d must be a multiple of 64", K);
    BLM_REQUIRE((x != nullptr) != (resid != nullptr), "gemv: give either x or the stream to normalise");
    BLM_REQUIRE(x == nullptr || (ldx % 8 == 0 && ((size_t)x & 15) == 0), "gemv: x rows must be 16-byte aligned");
    BLM_REQUIRE(ldw % 8 == 0 && ((size_t)w & 15) == 0, "gemv: weight rows must be 16-byte aligned");
    BLM_REQUIRE(epi == EPI_STORE || epi == EPI_SWIGLU || epi == EPI_RESID_ADD || epi == EPI_ROPE, "gemv: epilogue %d", epi);
    if (epi == EPI_ROPE) {
        BLM_REQUIRE(rope != nullptr && rope->token_pos && rope->table && y_f32 == 0, "gemv: the rotary epilogue needs positions, a table and a bfloat16 q");
        BLM_REQUIRE(rope->hd % 16 == 0 && rope->hd >= 16, "gemv: the rotary epilogue takes head sizes in steps of 16, got %d", rope->hd);
        BLM_REQUIRE(M == (rope->n_heads + (rope->write_cache ? 2 * rope->n_kv : 0)) * rope->hd,
                    "gemv: %d outputs are not %d q heads%s of %d lanes", M, rope->n_heads, rope->write_cache ? " and the k and v heads" : "", rope->hd);
        BLM_REQUIRE(!rope->write_cache || (rope->pool && rope->token_seq && rope->slot_of_seq && rope->block_table && rope->page_size > 0),
                    "gemv: the rotary epilogue writes the cache and needs its pool and tables");
    }
    BLM_REQUIRE(epi != EPI_SWIGLU || M % 8 == 0, "gemv: the gated epilogue needs an inner size that is a multiple of 8, got %d", M);
    BLM_REQUIRE(epi != EPI_RESID_ADD || acc != nullptr, "gemv: no stream to add into");
    BLM_REQUIRE(epi == EPI_RESID_ADD || y != nullptr, "gemv: no output");
    BLM_REQUIRE(resid == nullptr || ((size_t)resid & 15) == 0, "gemv: the stream must be 16-byte aligned");
    BLM_REQUIRE(status != nullptr, "gemv: no status word");
    BLM_REQUIRE(ssq_in == nullptr || (x != nullptr && ssq_parts >= 1), "gemv: a handed-over norm comes with x and its sums of squares");
    BLM_REQUIRE(xg_out == nullptr || (epi == EPI_RESID_ADD && next_gamma != nullptr && ssq_out != nullptr),
                "gemv: only the product that adds into the stream can hand a norm over, with gamma and room for the sums");
    GemvArgs a;
    a.w = (const __nv_bfloat16*)w; a.ldw = ldw; a.M = M; a.K = K;
    a.x = (const __nv_bfloat16*)x; a.ldx = ldx; a.resid = resid; a.gamma = gamma; a.gamma_f32 = gamma_f32; a.eps = eps;
    a.rows = rows; a.N = N; a.y = y; a.ldy = ldy; a.y_f32 = y_f32; a.acc = acc; a.epi = epi; a.status = status;
    a.ssq_in = ssq_in; a.ssq_parts = ssq_parts; a.next_gamma = next_gamma; a.next_gamma_f32 = next_gamma_f32;
    a.xg_out = (__nv_bfloat16*)xg_out; a.ssq_out = ssq_out;
    if (epi == EPI_ROPE) a.rope = *rope;
    else a.rope = GemvRope{};
    const int out_per_tile = epi == EPI_SWIGLU ? 8 : 16;
    const int tiles = (M + out_per_tile - 1) / out_per_tile;
    const int sms = blm_sm_count();
    // One block per SM, or per tile when there are fewer.  The rotary product takes no more blocks than its longest
    // block's load needs (192 tiles are two tiles each for 96 blocks, not two for 44 and one for 104 of 148) when
    // the decode attention that follows it, with a block or more per token and kv head, would mostly find room on
    // the SMs that leaves free: its blocks then start while the product runs, read their tables and ask for the pages
    // of earlier tokens.  Measured: batch 8 0.772 to 0.766 ms, batch 1 0.725 to 0.719 ms; with more attention blocks
    // than that (16 tokens x 8 kv heads on the 3B shape) or for the other products the evener grid gains nothing or
    // loses (3.11 to 3.13 ms), so they keep the full grid.
    int grid = tiles < sms ? tiles : sms;
    if (epi == EPI_ROPE && tiles > sms) {
        const int per_block = (tiles + sms - 1) / sms, even = (tiles + per_block - 1) / per_block;
        if (N * rope->n_kv <= 2 * (sms - even)) grid = even;
    }
    // Plain tokens: with one tile per block they travel with the weights; else they are fetched once by TMA;
    // and when they are too many for that (a very wide input) they travel with the weights after all, once
    // per tile.  A stream to normalise or gathered rows are staged by the consumers.
    a.x_mode = X_STAGED;
    int nbt, stage_k = 256;
    size_t smem = 0;
    if (x != nullptr && rows == nullptr) {
        a.x_mode = (tiles <= sms && ssq_in == nullptr && K >= 2 * 256) ? X_IN_RING : X_BY_TMA;
        smem = gemv_plan_best(N, K, a.x_mode, &stage_k, &a.n_stages, &nbt);
        if (smem == 0 && a.x_mode == X_BY_TMA) {
            a.x_mode = X_IN_RING;
            smem = gemv_plan_best(N, K, X_IN_RING, &stage_k, &a.n_stages, &nbt);
        }
    }
    if (smem == 0) {
        a.x_mode = X_STAGED;
        smem = gemv_plan_best(N, K, X_STAGED, &stage_k, &a.n_stages, &nbt);
    }
    BLM_REQUIRE(smem > 0, "gemv: the shape N=%d K=%d does not fit shared memory", N, K);
    CUtensorMap wmap, xmap;
    int rc = weight_map(w, ldw, epi == EPI_SWIGLU ? 2 * M : M, K, stage_k, &wmap);
    if (rc != BLM_OK) return rc;
    if (a.x_mode != X_STAGED) {
        rc = token_map(x, ldx, N, K, nbt * 8, stage_k, &xmap);
        if (rc != BLM_OK) return rc;
    } else {
        xmap = wmap;      // not used
    }
    static bool opted_in[3][2] = {};     // per variant of the kernel
    auto launch = [&](auto kernel) -> int {
        bool& done = opted_in[nbt][stage_k == 128];
        if (!done) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
            if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "gemv: %s", cudaGetErrorString(e));
            done = true;
        }
        cudaError_t e = blm_launch_dependent(kernel, dim3(grid), dim3(kGemvThreads), smem, stream, a, wmap, xmap);
        if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "gemv: %s", cudaGetErrorString(e));
        return blm_check_launch("gemv");
    };
    if (stage_k == 128) return nbt == 1 ? launch(gemv_kernel<1, 128>) : launch(gemv_kernel<2, 128>);
    return nbt == 1 ? launch(gemv_kernel<1, 256>) : launch(gemv_kernel<2, 256>);
}
