// Prompt attention on the 5th-generation tensor cores (bf16, head size 64 or 128): causal grouped-query
// attention of a step's new tokens over the paged cache, the products on tcgen05 with their accumulators
// in tensor memory.
//
// A block owns 128 query rows of one head of one sequence and walks the keys a cache page (64 keys) a
// step.  Seven warps:
//   warp 0 (one thread), the producer: TMA tile loads with the 128-byte swizzle of the query tile (once,
//     from the step's q rows), of the pages' keys (a ring of four; two at head size 128) and values (a ring
//     of two), completion on mbarriers;
//   warp 1 (one thread), the scores: S(j) = Q K(j)^T (M 128, N 64, both operands K-major in shared memory)
//     into a ring of three 64-column tiles of tensor memory (two at head size 128), so that a step's scores
//     are formed two steps (one) before the softmax warps come for them;
//   warp 2 (one thread), the values: O += P(j) V(j), with A = P read from tensor memory and B = V as it
//     lies in the cache (keys by lanes, read MN-major);
//   warps 3..6, the softmax: a thread owns one query row (its lane of tensor memory), reads the row of S
//     with tcgen05.ld, keeps the row's reference maximum and sum in registers, and writes the
//     probabilities as bf16 pairs over the first 32 columns of the same S tile (tcgen05.st), from where
//     the values warp's product takes them: they never pass through shared memory.
// tcgen05.commit frees stages and tells the next warp.  Two issuing warps, because one thread that issues
// both products is the longest chain of a step (each instruction it issues costs it some fifty cycles).
// O accumulates in tensor memory over the steps; a row of it is rescaled there (tcgen05.ld, multiply,
// tcgen05.st) only when a step's maximum exceeds the row's reference by more than 2^8, which after the
// first steps is rare.  Either head size: 256 columns of tensor memory a block (3 x 64 for the scores and 64
// for O; 2 x 64 and 128) and 66 or 99 KB of shared memory, two blocks to an SM, one's softmax under the other's.
//
// Rows of a value page that no key of the sequence has written (the page's tail) are cleared by the
// softmax threads before the product: a probability of zero does not silence a NaN.  Every mbarrier wait
// is bounded; one that runs out records a code in the status word and the block goes to its end, where
// the tensor memory is given back.
#pragma once
#include <cuda.h>

#include <map>
#include <tuple>

#include "common.cuh"

struct AttnPrefillTcArgs {
    const int* block_table;
    int table_stride;
    const int* cu_seqlens;
    const int* slot_of_seq;
    const int* start_pos;
    __nv_bfloat16* out;          // [N, n_heads * HD]
    int n_heads, n_kv, window;
    float scale_log2e;
    int* status;                 // 0, or 31..37 when a bounded wait ran out
};

namespace attn_tc {
constexpr unsigned kSpinLimit = 1u << 22;
constexpr int kThreads = 224;        // producer warp, two tensor-core warps (scores; values), four softmax warps
constexpr int BQ = 128, BKV = 64;    // query rows of a block, keys of a step (one cache page)
constexpr int kVStages = 2;          // pages of values in shared memory
// pages of keys in shared memory and score tiles in tensor memory: what lets two blocks share an SM
__host__ __device__ constexpr int key_stages(int hd) { return hd == 64 ? 4 : 2; }
__host__ __device__ constexpr int score_ring(int hd) { return hd == 64 ? 3 : 2; }
enum { TC_ATTN_Q = 31, TC_ATTN_K = 32, TC_ATTN_V = 33, TC_ATTN_S = 34, TC_ATTN_P = 35, TC_ATTN_PV = 36, TC_ATTN_FREE = 37 };

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    const unsigned addr = smem_u32(bar);
    {   // a phase that is over already answers at once
        unsigned done;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
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
// Shared-memory operand descriptors; tiles are rows of 128 bytes with the 128-byte swizzle, eight rows
// 1024 bytes apart.  K-major (Q, K, P): the rows are the operand's M or N index, a row holds 64 of its k.
// MN-major (V): the rows are the k index (keys), a row holds 64 of the operand's N (lanes of the head);
// groups of eight k rows are 1024 bytes apart (the stride offset), the next 64 lanes `lanes_step` bytes
// further (the leading offset).
__device__ __forceinline__ unsigned long long desc_k_major(const void* tile) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(tile) >> 4) & 0x3fff);
    d |= (unsigned long long)1 << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
__device__ __forceinline__ unsigned long long desc_mn_major(const void* tile, unsigned lanes_step) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(tile) >> 4) & 0x3fff);
    d |= (unsigned long long)((lanes_step >> 4) & 0x3fff) << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
// instruction descriptor of kind::f16: fp32 accumulator, bf16 x bf16, M 128
__host__ __device__ constexpr unsigned idesc(int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((unsigned)(n >> 3) << 17) | ((unsigned)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc, unsigned id, unsigned accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(id), "r"(accumulate)
        : "memory");
}
// the same with the A operand read from tensor memory (row m in lane m, two bf16 of k a column)
__device__ __forceinline__ void umma_a_tmem(unsigned tmem_d, unsigned tmem_a, unsigned long long b_desc, unsigned id, unsigned accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(b_desc), "r"(id), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// 2^x on the special-function unit (x = -inf gives 0)
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// The same in two halves, so that a load is in flight while the columns before it are worked on: issue, and
// later wait; the wait names the registers, so nothing that uses them is moved before it.
__device__ __forceinline__ void tmem_ld32_issue(unsigned taddr, unsigned (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld32_wait(unsigned (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;\n"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]),
                   "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]),
                   "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]),
                   "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :
                 : "memory");
}
__device__ __forceinline__ void tmem_st32(unsigned taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_st32_bits(unsigned taddr, const unsigned (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
        "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]),
        "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]),
        "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}
constexpr float kLazy = 8.0f;     // the reference maximum of a row moves only when a block exceeds it by more than 2^kLazy
}  // namespace attn_tc

template <int HD>
__global__ void __launch_bounds__(attn_tc::kThreads, 2) attn_prefill_tc_kernel(const AttnPrefillTcArgs a, const __grid_constant__ CUtensorMap qmap,
                                                                            const __grid_constant__ CUtensorMap pool_map) {
    using namespace attn_tc;
    constexpr int SUB = HD / 64;                         // 64-lane sub-tiles of a row
    constexpr int kKStages = key_stages(HD), kSRing = score_ring(HD);
    constexpr unsigned kTile = 128 * 128;                // bytes of a sub-tile: 128 rows of 128 bytes
    constexpr unsigned kPage = 64 * 128;                 // bytes of a page's sub-tile: 64 keys of 128 bytes
    constexpr unsigned kQBytes = SUB * kTile, kKBytes = SUB * kPage, kVBytes = SUB * kPage;
    constexpr int kOCol = kSRing * BKV;                  // S of step j: columns 64 (j % kSRing) ..; O: the columns behind the ring
    constexpr int kTmemCols = kOCol + HD <= 256 ? 256 : 512;
    extern __shared__ __align__(1024) unsigned char smem_tc_raw[];
    unsigned char* smem = smem_tc_raw + ((1024u - (smem_u32(smem_tc_raw) & 1023u)) & 1023u);
    unsigned char* Qs = smem;                            // [SUB][128 rows][128 bytes]
    unsigned char* Ks = Qs + kQBytes;                    // [kKStages][SUB][64 keys][128 bytes]
    unsigned char* Vs = Ks + kKStages * kKBytes;         // [kVStages][SUB][64 keys][128 bytes]
    unsigned long long* q_full = reinterpret_cast<unsigned long long*>(Vs + kVStages * kVBytes);
    unsigned long long* k_full = q_full + 1;             // [kKStages] a page's keys have landed
    unsigned long long* k_empty = k_full + kKStages;     // [kKStages] the scores that read them are formed
    unsigned long long* v_full = k_empty + kKStages;     // [kVStages] a page's values have landed
    unsigned long long* s_full = v_full + kVStages;      // [kSRing] the scores of a step are in tensor memory
    unsigned long long* p_full = s_full + kSRing;        // [kSRing] its probabilities are written and its scores read
    unsigned long long* pv_done = p_full + kSRing;       // [kSRing] its product into O is over: its columns of tensor memory and the value stage are free
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(pv_done + kSRing);

    pdl_wait();          // q and the keys are the work of the kernels before
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // blocks start in the order x, y, z: all heads of the longest query tile first, then the next tile, so
    // that the long walks begin early and the short ones fill the end
    const int head = blockIdx.x, seq = blockIdx.z;
    const int qt = (int)gridDim.y - 1 - (int)blockIdx.y;
    const int tok0 = a.cu_seqlens[seq], q_len = a.cu_seqlens[seq + 1] - tok0;
    const int q0 = qt * BQ;
    if (q0 >= q_len) return;                                      // the whole block: nothing was set up yet
    pdl_launch_dependents();
    const int start = a.start_pos[seq];
    const int kv_total = start + q_len;                           // keys of this sequence in the cache after the step's append
    const int rows = min(BQ, q_len - q0);
    const int key_hi = start + q0 + rows - 1;                     // the last key any row of the block sees
    const int key_lo = a.window > 0 ? max(0, start + q0 - a.window + 1) : 0;
    const int kb_lo = key_lo / BKV, kb_hi = key_hi / BKV, n_blocks = kb_hi - kb_lo + 1;
    const int kvh = head / (a.n_heads / a.n_kv);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < kKStages; ++s) { mbar_init(k_full + s, 1); mbar_init(k_empty + s, 1); }
        for (int s = 0; s < kVStages; ++s) mbar_init(v_full + s, 1);
        for (int s = 0; s < kSRing; ++s) {
            mbar_init(s_full + s, 1);
            mbar_init(p_full + s, 4);    // one arrival per softmax warp
            mbar_init(pv_done + s, 1);
        }
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

    // Who waits for whom, step j (a page of 64 keys; t = j % kSRing, b = j & 1):
    //   scores warp:  pv_done[t] of step j - kSRing (its columns were read), k_full  ->  S(j)  ->  s_full[t], k_empty
    //   softmax:      s_full[t]                                            ->  P(j) over S(j)'s first columns  ->  p_full[t]
    //   values warp:  p_full[t], v_full[b]                                  ->  O += P V  ->  pv_done[t]
    //   producer:     pv_done of step j - 2  ->  the values of step j;  k_empty  ->  the keys of step j + kKStages - 1
    // so the scores of a step are formed kSRing - 1 steps before the softmax warps come for them.
    if (warp == 0) {
        if (lane == 0) {
            // ---------------- producer ----------------
            const int* pages = a.block_table + (size_t)a.slot_of_seq[seq] * a.table_stride;
            mbar_expect_tx(q_full, kQBytes);
#pragma unroll
            for (int h = 0; h < SUB; ++h) tma_load_2d(Qs + h * kTile, &qmap, head * HD + h * 64, tok0 + q0, q_full);
            auto row_of = [&](int step) { return ((pages[kb_lo + step] * 2) * a.n_kv + kvh) * 64; };      // the page's keys of this kv head
            auto load_keys = [&](int step) -> bool {
                const int ks = step % kKStages;
                if (step >= kKStages && !mbar_wait(k_empty + ks, ((step / kKStages) - 1) & 1)) { atomicCAS(a.status, 0, TC_ATTN_FREE); return false; }
                mbar_expect_tx(k_full + ks, kKBytes);
                const int krow = row_of(step);
#pragma unroll
                for (int h = 0; h < SUB; ++h) tma_load_2d(Ks + ks * kKBytes + h * kPage, &pool_map, h * 64, krow, k_full + ks);
                return true;
            };
            for (int j = 0; j < kKStages - 1 && j < n_blocks; ++j) load_keys(j);
            for (int j = 0; j < n_blocks; ++j) {
                const int b = j & 1;
                if (j >= 2 && !mbar_wait(pv_done + (j - 2) % kSRing, ((j - 2) / kSRing) & 1)) { atomicCAS(a.status, 0, TC_ATTN_FREE); break; }
                mbar_expect_tx(v_full + b, kVBytes);
                const int vrow = row_of(j) + a.n_kv * 64;                    // the values lie n_kv * 64 rows after the keys
#pragma unroll
                for (int h = 0; h < SUB; ++h) tma_load_2d(Vs + b * kVBytes + h * kPage, &pool_map, h * 64, vrow, v_full + b);
                if (j + kKStages - 1 < n_blocks && !load_keys(j + kKStages - 1)) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- tensor core, scores: S(j) = Q K(j)^T into columns 64 (j % 3) .. ----------------
            constexpr unsigned kIdescS = idesc(BKV, false);
            // operand descriptors: the address field counts 16 bytes, so a stage or a sub-tile further is an addition
            const unsigned long long q_desc = desc_k_major(Qs), k_desc = desc_k_major(Ks);
            bool ok = mbar_wait(q_full, 0);
            if (!ok) atomicCAS(a.status, 0, TC_ATTN_Q);
            for (int j = 0; j < n_blocks && ok; ++j) {
                const int t = j % kSRing, ks = j % kKStages;
                if (j >= kSRing && !mbar_wait(pv_done + t, ((j / kSRing) - 1) & 1)) { atomicCAS(a.status, 0, TC_ATTN_PV); break; }
                if (!mbar_wait(k_full + ks, (j / kKStages) & 1)) { atomicCAS(a.status, 0, TC_ATTN_K); break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                // HD / 16 steps of k; a step is 32 bytes along the swizzled row (+2 in the address field), the
                // second half of a 128-lane head lies in the next sub-tile
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const unsigned long long ad = q_desc + (unsigned)((kk >> 2) * (kTile >> 4) + 2 * (kk & 3));
                    const unsigned long long bd = k_desc + (unsigned)(ks * (kKBytes >> 4) + (kk >> 2) * (kPage >> 4) + 2 * (kk & 3));
                    umma(tmem_base + (unsigned)(t * BKV), ad, bd, kIdescS, kk > 0 ? 1u : 0u);
                }
                umma_commit(k_empty + ks);
                umma_commit(s_full + t);
            }
        }
    } else if (warp == 2) {
        if (lane == 0) {
            // ---------------- tensor core, values: O += P(j) V(j) ----------------
            constexpr unsigned kIdescPV = idesc(HD, true);
            const unsigned long long v_desc = desc_mn_major(Vs, kPage);
            for (int j = 0; j < n_blocks; ++j) {
                const int b = j & 1, t = j % kSRing;
                if (!mbar_wait(p_full + t, (j / kSRing) & 1)) { atomicCAS(a.status, 0, TC_ATTN_P); break; }
                if (!mbar_wait(v_full + b, (j >> 1) & 1)) { atomicCAS(a.status, 0, TC_ATTN_V); break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
                for (int kk = 0; kk < BKV / 16; ++kk) {
                    // A: the probabilities in tensor memory, 16 keys = 8 columns of two bf16 a step; B: 16 keys further
                    // are two groups of eight rows, 2048 bytes
                    const unsigned long long bd = v_desc + (unsigned)(b * (kVBytes >> 4) + kk * (2048 >> 4));
                    umma_a_tmem(tmem_base + kOCol, tmem_base + (unsigned)(t * BKV + 8 * kk), bd, kIdescPV, (j > 0 || kk > 0) ? 1u : 0u);      // O accumulates over the steps
                }
                umma_commit(pv_done + t);
            }
        }
    } else {
        // ---------------- softmax: thread <-> query row ----------------
        const int quarter = warp & 3;                            // the lanes of tensor memory this warp may read
        const int r = quarter * 32 + lane;                       // row of the tile, lane of tensor memory
        const bool live = r < rows;
        const int pos = start + q0 + r;                          // this row's position: it sees keys lo .. pos
        const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
        const unsigned trow = tmem_base + ((unsigned)(quarter * 32) << 16);
        // O accumulates in tensor memory over the blocks, against a reference maximum m_run per row that only
        // moves when a block's maximum exceeds it by more than 2^kLazy: then the row of O is rescaled in tensor
        // memory (read, multiply, write back).  Otherwise probabilities may exceed one, by at most that factor.
        float m_run = -INFINITY, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < n_blocks && ok; ++j) {
            const int key0 = (kb_lo + j) * BKV;
            const int b = j & 1, t = j % kSRing;                 // which V stage, which score tile this step has
            if (!mbar_wait(s_full + t, (j / kSRing) & 1)) { if (lane == 0) atomicCAS(a.status, 0, TC_ATTN_S); ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            // Decided by warp (32 rows): a page whose every key every row of the warp sees needs no masks (all but
            // the diagonal and the window's edge); one of which no row of the warp sees a key gives probabilities
            // of zero without a look at the scores.
            const unsigned taddr = trow + (unsigned)(t * BKV);
            const int wpos_lo = start + q0 + quarter * 32, wpos_hi = wpos_lo + 31;
            const bool open_block = key0 + BKV - 1 <= wpos_lo && (a.window <= 0 || key0 >= wpos_hi - a.window + 1);
            const bool dead = key0 > wpos_hi || (a.window > 0 && key0 + BKV - 1 < wpos_lo - a.window + 1);
            unsigned buf[2][32];           // two loads of 32 columns: one in flight, one being worked on
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};
            // An open block of a row that has its reference maximum already: ONE pass over the scores.  The
            // exponentials are taken against the reference as it stands while the same pass finds the block's
            // maximum; only if some row of the warp has outgrown its reference by more than 2^kLazy (rare after
            // the first blocks) is the step done again the long way, maximum first.  The numbers are the same
            // either way: the same reference, the same operations.
            // the row's probabilities as bf16 pairs: kept in registers until the scores need not be read again, then
            // written over the first 32 of their columns
            unsigned packed[BKV / 2];
            bool done = dead;
            if (dead) {
#pragma unroll
                for (int i = 0; i < BKV / 2; ++i) packed[i] = 0u;
            } else if (open_block && __all_sync(0xffffffffu, m_run != -INFINITY)) {
                const float neg_ref = -m_run;
                float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
                tmem_ld32_issue(taddr, buf[0]);
#pragma unroll
                for (int c = 0; c < BKV / 32; ++c) {
                    tmem_ld32_wait(buf[c & 1]);
                    if (c + 1 < BKV / 32) tmem_ld32_issue(taddr + (c + 1) * 32, buf[(c + 1) & 1]);
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float s0 = __uint_as_float(buf[c & 1][i]), s1 = __uint_as_float(buf[c & 1][i + 1]);
                        m4[(i >> 1) & 3] = fmaxf(m4[(i >> 1) & 3], fmaxf(s0, s1));
                        const float p0 = ex2(fmaf(s0, a.scale_log2e, neg_ref)), p1 = ex2(fmaf(s1, a.scale_log2e, neg_ref));
                        rs4[(i >> 1) & 3] += p0 + p1;
                        const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                        packed[c * 16 + (i >> 1)] = *reinterpret_cast<const unsigned*>(&pk);
                    }
                }
                const float m_one = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * a.scale_log2e;
                done = !__any_sync(0xffffffffu, m_one > m_run + kLazy);
                if (!done) { rs4[0] = 0.f; rs4[1] = 0.f; rs4[2] = 0.f; rs4[3] = 0.f; }
            }
            if (!done) {
                // the row's maximum (of the raw scores: the scale is positive)
                float mx = -INFINITY;
                tmem_ld32_issue(taddr, buf[0]);
#pragma unroll
                for (int c = 0; c < BKV / 32; ++c) {
                    tmem_ld32_wait(buf[c & 1]);
                    // the next columns of this pass, or the first of the next pass
                    tmem_ld32_issue(taddr + ((c + 1) % (BKV / 32)) * 32, buf[(c + 1) & 1]);
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(buf[c & 1][i]);
                    if (open_block) {
                        float m4[4] = {v[0], v[1], v[2], v[3]};
#pragma unroll
                        for (int i = 4; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], v[i]);
                        mx = fmaxf(mx, fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])));
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int key = key0 + c * 32 + i;
                            if (live && key >= lo && key <= pos) mx = fmaxf(mx, v[i]);
                        }
                    }
                }
                const float m_blk = mx * a.scale_log2e;
                const bool move = m_blk > m_run + kLazy;                     // also the first block that shows the row a key
                if (__any_sync(0xffffffffu, move)) {
                    const float alpha = move ? (m_run == -INFINITY ? 0.f : ex2(m_run - m_blk)) : 1.0f;
                    if (j > 0) {
                        // the last product into O must have landed before its rows are touched
                        if (!mbar_wait(pv_done + (j - 1) % kSRing, ((j - 1) / kSRing) & 1)) { if (lane == 0) atomicCAS(a.status, 0, TC_ATTN_PV); ok = false; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
                        for (int c = 0; c < HD / 32; ++c) {
                            float v[32];
                            tmem_ld32(trow + kOCol + c * 32, v);
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] *= alpha;
                            tmem_st32(trow + kOCol + c * 32, v);
                        }
                    }
                    if (move) {
                        l_run *= alpha;
                        m_run = m_blk;
                    }
                }
                const float neg_m = m_run == -INFINITY ? 0.f : -m_run;      // a row without a visible key: every probability is masked anyway
                // the probabilities, as bf16 pairs
#pragma unroll
                for (int c = 0; c < BKV / 32; ++c) {
                    tmem_ld32_wait(buf[c & 1]);
                    if (c + 1 < BKV / 32) tmem_ld32_issue(taddr + (c + 1) * 32, buf[(c + 1) & 1]);
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(buf[c & 1][i]);
                    if (open_block) {
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const float p0 = ex2(fmaf(v[i], a.scale_log2e, neg_m)), p1 = ex2(fmaf(v[i + 1], a.scale_log2e, neg_m));
                            rs4[(i >> 1) & 3] += p0 + p1;
                            const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                            packed[c * 16 + (i >> 1)] = *reinterpret_cast<const unsigned*>(&pk);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            const int key = key0 + c * 32 + i;
                            const float p0 = (live && key >= lo && key <= pos) ? ex2(fmaf(v[i], a.scale_log2e, neg_m)) : 0.f;
                            const float p1 = (live && key + 1 >= lo && key + 1 <= pos) ? ex2(fmaf(v[i + 1], a.scale_log2e, neg_m)) : 0.f;
                            rs4[(i >> 1) & 3] += p0 + p1;
                            const __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
                            packed[c * 16 + (i >> 1)] = *reinterpret_cast<const unsigned*>(&pk);
                        }
                    }
                }
            }
            const float rs = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
            l_run += rs;
            // value rows no key of the sequence has written (beyond its last key) may hold anything: cleared
            if (key0 + BKV > kv_total) {
                if (!mbar_wait(v_full + b, (j >> 1) & 1)) { if (lane == 0) atomicCAS(a.status, 0, TC_ATTN_V); ok = false; break; }
                if (r < BKV && key0 + r >= kv_total) {
#pragma unroll
                    for (int h = 0; h < SUB; ++h)
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            *reinterpret_cast<uint4*>(Vs + b * kVBytes + h * kPage + r * 128 + c * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");      // these writes become visible to the tensor core
            }
            tmem_st32_bits(taddr, packed);
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + t);
        }
        // the last product into O, then the row: O / l
        float o[HD];
        if (ok) {
            if (!mbar_wait(pv_done + (n_blocks - 1) % kSRing, ((n_blocks - 1) / kSRing) & 1)) { if (lane == 0) atomicCAS(a.status, 0, TC_ATTN_PV); ok = false; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        }
        if (ok) {
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
                float v[32];
                tmem_ld32(trow + kOCol + c * 32, v);
#pragma unroll
                for (int i = 0; i < 32; ++i) o[c * 32 + i] = v[i];
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        }
        if (ok && live) {
            const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
            __nv_bfloat16* dst = a.out + (size_t)(tok0 + q0 + r) * a.n_heads * HD + (size_t)head * HD;
#pragma unroll
            for (int d = 0; d < HD; d += 8) {
                unsigned pk[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const __nv_bfloat162 two = __floats2bfloat162_rn(o[d + 2 * e] * inv, o[d + 2 * e + 1] * inv);
                    pk[e] = *reinterpret_cast<const unsigned*>(&two);
                }
                *reinterpret_cast<uint4*>(dst + d) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            }
        }
    }
    // everybody meets; then the warp that took the tensor memory gives it back
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols));
    }
}

typedef CUresult (*TcAttnEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                        const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                        CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A bf16 matrix [rows, width] with row stride ld (elements) as the TMA sees it: boxes of box_rows x 64, 128-byte swizzle.
static bool attn_tc_map(const void* base, long long ld, long long rows, int width, int box_rows, CUtensorMap* out) {
    static TcAttnEncodeTiledFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess || !fn)
            return false;
        encode = (TcAttnEncodeTiledFn)fn;
    }
    static std::map<std::tuple<const void*, long long, long long, int, int>, CUtensorMap> maps;
    const auto key = std::make_tuple(base, ld, rows, width, box_rows);
    auto it = maps.find(key);
    if (it == maps.end()) {
        CUtensorMap m;
        const cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)rows};
        const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
        const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
        const cuuint32_t estr[2] = {1, 1};
        if (encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
        if (maps.size() > 4096) maps.clear();
        it = maps.emplace(key, m).first;
    }
    *out = it->second;
    return true;
}

template <int HD>
static int attn_prefill_tc_launch(const AttnPrefillTcArgs& a, const CUtensorMap& qmap, const CUtensorMap& pmap, dim3 grid, cudaStream_t stream) {
    constexpr int SUB = HD / 64;
    const size_t smem = (size_t)SUB * 128 * 128 + (size_t)(attn_tc::key_stages(HD) + attn_tc::kVStages) * SUB * 64 * 128 + 24 * 8 + 16 + 1024;
    static bool opted_in = false;
    if (!opted_in) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_prefill_tc_kernel<HD>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "attention prefill (tcgen05): %s", cudaGetErrorString(e));
        opted_in = true;
    }
    cudaError_t e = blm_launch_dependent(attn_prefill_tc_kernel<HD>, grid, dim3(attn_tc::kThreads), smem, stream, a, qmap, pmap);
    if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "attention prefill (tcgen05): %s", cudaGetErrorString(e));
    return BLM_OK;
}

// BLM_OK when the kernel took the step, -1 when the shape is not its own, else an error.
// q: the step's rows, token n's head h at q + n * q_stride + h * hd.
static int launch_attn_prefill_tc(const AttnPrefillTcArgs& a, const void* q, long long q_stride, const void* pool, int n_pages,
                                  int hd, int n_tokens, int n_seqs, int max_q_len, cudaStream_t stream) {
    const dim3 grid(a.n_heads, (max_q_len + attn_tc::BQ - 1) / attn_tc::BQ, n_seqs);
    if (grid.y > 65535 || grid.z > 65535 || (hd != 64 && hd != 128)) return -1;
    CUtensorMap qmap, pmap;
    if (!attn_tc_map(q, q_stride, n_tokens, a.n_heads * hd, attn_tc::BQ, &qmap) ||
        !attn_tc_map(pool, hd, (long long)n_pages * 2 * a.n_kv * 64, hd, 64, &pmap))
        return blm_fail(BLM_CUDA_ERROR, "attention prefill (tcgen05): cuTensorMapEncodeTiled failed");
    return hd == 64 ? attn_prefill_tc_launch<64>(a, qmap, pmap, grid, stream) : attn_prefill_tc_launch<128>(a, qmap, pmap, grid, stream);
}
