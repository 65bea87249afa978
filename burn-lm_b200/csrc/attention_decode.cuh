// Decode attention for bf16: one new token per sequence against its paged cache, grouped-query.  A block
// owns one (sequence, kv head, split of the sequence's pages).  Its producer warp reads the page numbers
// (32 at a time) and streams the pages into a ring in shared memory: TMA boxes of 64 keys x 64 lanes with
// the 128-byte swizzle (cp.async.bulk.tensor over the pool seen as a matrix), completion on mbarriers.
// The G query heads of the kv head are rows of a 16-row tensor-core tile, so scores and outputs are
// mma.sync.m16n8k16 products; the four warps of a consumer group take 16 keys of a page each, and one, two
// or four groups work on different pages at once (a warp alone on its scheduler waits out every latency
// of its chain).  The ring is as deep as the block's walk when few blocks run, two pages when many share
// an SM.  Warps and groups keep their own running (max, sum, output) and merge at the end; splits of a
// long sequence are merged by a second kernel.  Waits on mbarriers are bounded; one that runs out is
// recorded in the status word.
#pragma once
#include <cuda.h>

#include <map>
#include <tuple>

#include "common.cuh"

struct AttnDecodeArgs {
    const __nv_bfloat16* q;      // token n, head h at q + n * q_stride + h * HD
    long long q_stride;
    const __nv_bfloat16* pool;   // [pages][2][n_kv][64][HD]
    const int* block_table;
    int table_stride;
    const int* seq_table;        // optional: the block table's rows in the order of the step's sequences
    const int* cu_seqlens;
    const int* slot_of_seq;
    const int* start_pos;
    __nv_bfloat16* out;          // [N, n_heads * HD]
    float* part_acc;             // [N, n_heads, n_splits, HD]
    float* part_ml;              // [N, n_heads, n_splits, 2]: (max in natural-log units, sum)
    int n_heads, n_kv, window, n_splits;
    int group;                   // query heads per kv head, 1 to 8: rows 0 .. group-1 of the 16-row tile
    int pages_per_split;         // a sequence's keys are cut into blocks of about this many pages, n_splits blocks at most
    int n_stages;                // pages the ring of a block holds (a multiple of n_groups)
    int n_groups;                // groups of four consumer warps; group g takes pages g, g + n_groups, ... of the block's
    float scale_log2e;           // softmax scale times log2(e): scores live in base-2 units
    int* status;                 // 0, or 21 / 22 when a bounded wait ran out
    // 1: the kernel before this one let it start only after its own wait, so all but that kernel's work (the step's
    // positions and page tables, the cache pages of earlier tokens) is written and may be read before this kernel's
    // wait; only q and the page that holds the new token wait for it
    int ahead;
};

// How many of the n_splits blocks of a (sequence, kv head) work: one per `pages_per_split` pages the keys touch,
// n_splits at most.  With pages_per_split = 1 every sequence of n_splits pages or more takes them all; with the
// pages a block of the longest sequence the step may hold would walk, the sequences of a batch of unequal lengths
// take blocks in proportion to their lengths, all of about that many pages, instead of n_splits tiny ones each.
__host__ __device__ inline int attn_decode_active_splits(int key_lo, int kv_len, int n_splits, int pages_per_split) {
    const int n_pg = (kv_len - 1) / 64 - key_lo / 64 + 1;
    const int want = (n_pg + pages_per_split - 1) / pages_per_split;
    return want < 1 ? 1 : (want > n_splits ? n_splits : want);
}

namespace attn_decode {
constexpr unsigned kSpinLimit = 1u << 22;
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
__device__ __forceinline__ void bulk_copy(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
}  // namespace attn_decode

// How many pages the ring of a block holds.  With few blocks (one per SM or less) a block keeps all its
// pages in flight at once, up to what shared memory takes; with many blocks the rings are short, so that
// all blocks are resident at once (at batch 64, 512 blocks: two pages a ring and six blocks an SM measured
// best, ahead of three or four pages).
static inline int attn_decode_stages(int hd, int blocks, int pages_per_block) {
    const int page_kb = 2 * 64 * hd * 2 / 1024;                    // keys and values of a page of one kv head
    const int sms = blm_sm_count();
    const int room_kb = blocks <= sms ? 192 : (blocks <= 2 * sms ? 96 : 32);
    int s = room_kb / page_kb;
    if (s > pages_per_block) s = pages_per_block;
    return s < 2 ? 2 : s;
}
// Groups of consumer warps.  One warp per scheduler waits out every latency of its chain of dependent
// instructions; when a block is (almost) alone on its SM, several groups work on different pages at once.
// Head size 128 stops at two groups: with four (17 warps) a thread has 96 registers and the output tiles of a
// 128-lane head spill (measured, 8 sequences of 2,000 tokens: 35.7 us with four groups, 24.6 us with two).
static inline int attn_decode_groups(int blocks, int pages_per_block, int stages, int hd = 64) {
    const int sms = blm_sm_count();
    int ng = blocks <= sms ? (hd > 64 ? 2 : 4) : (blocks <= 2 * sms && hd <= 64 ? 2 : 1);
    while (ng > 1 && (ng > pages_per_block || ng > stages)) ng /= 2;
    return ng;
}

__device__ __forceinline__ void dec_ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void dec_ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void dec_mma(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The G query heads of a kv head are rows 0 .. G-1 of a 16-row tensor-core tile (the other rows are zero):
// S = Q K^T and O += P V run as mma.sync.m16n8k16, so a page costs a warp a few dozen instructions
// instead of hundreds.  A page arrives as TMA boxes of 64 keys x 64 lanes with the 128-byte swizzle, which
// ldmatrix reads without bank conflicts; the four consumer warps take 16 keys of every page each and keep
// their own running (max, sum, output), merged at the end.
template <int HD, int NG>
__global__ void __launch_bounds__((4 * NG + 1) * 32) attn_decode_kernel(const AttnDecodeArgs a, const __grid_constant__ CUtensorMap pool_map) {
    using namespace attn_decode;
    const int G = a.group;
    constexpr int WARPS = 4 * NG;      // consumer warps (NG groups of four); the warp after them is the producer
    const int S = a.n_stages;
    constexpr int SUB = HD / 64;       // 64-lane boxes per row
    constexpr int KS = HD / 16;        // k steps of Q K^T
    constexpr int DT = HD / 8;         // 8-wide output tiles
    constexpr unsigned BOX = 64 * 64 * 2;          // bytes of one box
    constexpr unsigned PB = SUB * BOX;             // bytes of the keys (or of the values) of one page of one kv head
    constexpr float LN2 = 0.6931471805599453f;
    extern __shared__ __align__(1024) unsigned char smem_dec_raw[];
    unsigned char* smem_dec = smem_dec_raw + ((1024u - (smem_u32(smem_dec_raw) & 1023u)) & 1023u);
    unsigned char* ring = smem_dec;                                                         // [S][k | v][SUB][64 x 128 bytes]
    float* sm_acc = reinterpret_cast<float*>(smem_dec + (size_t)S * 2 * PB);                // [WARPS][G][HD]
    float* sm_m = sm_acc + WARPS * G * HD;                                                  // [WARPS][G]
    float* sm_l = sm_m + WARPS * G;
    unsigned long long* full = reinterpret_cast<unsigned long long*>(sm_l + WARPS * G);
    unsigned long long* empty = full + S;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    pdl_launch_dependents();
    blm_trace(0x400);
    if (!a.ahead) pdl_wait();          // the queries and this step's keys are the work of the kernels before
    blm_trace(0x410);
    const int tok = seq;                         // one token per sequence: the packed row is the sequence
    const int pos = a.start_pos[seq];            // the new token's position; keys 0..pos are visible
    const int kv_len = pos + 1;
    const int key_lo = a.window > 0 ? max(0, kv_len - a.window) : 0;
    // Only some of the splits are active for a short sequence; the others leave at once and the combine kernel,
    // which computes the same number, does not look at them.
    const int active = attn_decode_active_splits(key_lo, kv_len, a.n_splits, a.pages_per_split);
    if (split >= active) return;
    const int pg_first = key_lo / 64, n_pg = (kv_len - 1) / 64 - pg_first + 1;
    const int per = (n_pg + active - 1) / active;
    const int pg_lo = pg_first + split * per;
    const int pg_hi = min(pg_first + n_pg, pg_lo + per);          // exclusive
    const int* pages = a.seq_table != nullptr ? a.seq_table + (size_t)seq * a.table_stride
                                              : a.block_table + (size_t)a.slot_of_seq[seq] * a.table_stride;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 4);          // the four warps of the group that reads the stage
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    if (warp == WARPS) {
        // ---------------- producer: streams the pages of this split ----------------
        // The warp reads the page numbers together, 32 at a time (one round trip instead of one per page);
        // lane 0 issues the copies.
        bool failed = false;
        int s = -1;                       // the stage of page i and the parity of its barriers' current phase
        unsigned phase = 0;
        for (int base = pg_lo, i = 0; base < pg_hi; base += 32) {
            const int mine = base + lane < pg_hi ? pages[base + lane] : 0;
            const int n = min(32, pg_hi - base);
            for (int j = 0; j < n; ++j, ++i) {
                const int page = __shfl_sync(0xffffffffu, mine, j);
                if (a.ahead && base + j == (kv_len - 1) / 64) pdl_wait();      // the page the new token was just written to
                if (++s == S) { s = 0; phase ^= 1; }
                if (lane != 0 || failed) continue;
                if (i >= S && !mbar_wait(empty + s, phase ^ 1)) {
                    atomicCAS(a.status, 0, 22);
                    failed = true;
                    continue;
                }
                // rows of the pool seen as a matrix [pages * 2 * n_kv * 64, HD]: keys, then values, of a page
                const int krow = ((page * 2) * a.n_kv + kvh) * 64, vrow = krow + a.n_kv * 64;
                mbar_expect_tx(full + s, 2 * PB);
                unsigned char* dst = ring + (size_t)s * 2 * PB;
#pragma unroll
                for (int h = 0; h < SUB; ++h) {
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
                                     smem_u32(dst + h * BOX)),
                                 "l"(&pool_map), "r"(h * 64), "r"(krow), "r"(smem_u32(full + s))
                                 : "memory");
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(
                                     smem_u32(dst + PB + h * BOX)),
                                 "l"(&pool_map), "r"(h * 64), "r"(vrow), "r"(smem_u32(full + s))
                                 : "memory");
                }
            }
        }
    } else {
        // ---------------- consumers: the warps of a group take 16 keys each of the group's pages ----------------
        // Q as the A operand: row g is head g of the group (rows G.. and 8.. are zero)
        if (a.ahead) pdl_wait();
        unsigned qf[KS][4];
        {
            const __nv_bfloat16* qrow = a.q + (size_t)tok * a.q_stride + (size_t)(kvh * G + (g < G ? g : 0)) * HD;
#pragma unroll
            for (int kk = 0; kk < KS; ++kk) {
                qf[kk][0] = g < G ? *reinterpret_cast<const unsigned*>(qrow + kk * 16 + 2 * t) : 0u;
                qf[kk][2] = g < G ? *reinterpret_cast<const unsigned*>(qrow + kk * 16 + 8 + 2 * t) : 0u;
                qf[kk][1] = 0u;
                qf[kk][3] = 0u;
            }
        }
        float o[DT][4];
#pragma unroll
        for (int d = 0; d < DT; ++d)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[d][e] = 0.f;
        float m_run = -INFINITY, l_run = 0.f;        // of row g (head g); every lane of a quad holds the same max
        auto swz = [](int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); };   // byte offset in a box

        // This warp's group takes every NG-th page; the ring's depth is a multiple of NG, so a stage always
        // serves the same group, which thus sees every phase of the stage's barriers.
        const int group = warp >> 2, quarter = warp & 3;
        int s = group - NG;
        unsigned phase = 0;
        for (int i = group, pg = pg_lo + group; pg < pg_hi; pg += NG, i += NG) {
            s += NG;
            if (s >= S) { s -= S; phase ^= 1; }
            if (!mbar_wait(full + s, phase)) {
                if (lane == 0) atomicCAS(a.status, 0, 21);
                break;
            }
            if (i == 0) blm_trace(0x430);
            const unsigned char* Kt = ring + (size_t)s * 2 * PB;
            const unsigned char* Vt = Kt + PB;
            // scores of this warp's 16 keys: two tiles of 8 keys
            float sc[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[nt][e] = 0.f;
#pragma unroll
                for (int kk = 0; kk < KS; kk += 2) {
                    const int chunk = 2 * kk + (lane >> 3);           // 16-byte chunk of the row: k steps kk and kk + 1
                    unsigned kb[4];
                    dec_ldmatrix_x4(kb, Kt + (chunk >> 3) * BOX + swz(quarter * 16 + nt * 8 + (lane & 7), chunk & 7));
                    dec_mma(sc[nt], qf[kk], kb[0], kb[1]);
                    dec_mma(sc[nt], qf[kk + 1], kb[2], kb[3]);
                }
            }
            // scale, mask, online softmax of row g
            float mx = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = pg * 64 + quarter * 16 + nt * 8 + 2 * t + e;
                    const float v = (key >= key_lo && key < kv_len) ? sc[nt][e] * a.scale_log2e : -INFINITY;
                    sc[nt][e] = v;
                    mx = fmaxf(mx, v);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run, mx);
            const float alpha = m_run == -INFINITY ? 0.f : exp2f(m_run - m_new);
            m_run = m_new;
            float p[2][2];
            float rs = 0.f;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    p[nt][e] = (sc[nt][e] == -INFINITY || m_new == -INFINITY) ? 0.f : exp2f(sc[nt][e] - m_new);
                    rs += p[nt][e];
                }
            l_run = l_run * alpha + rs;                 // this lane's share; summed over the quad at the end
            unsigned pf[4];
            {
                const __nv_bfloat162 p0 = __floats2bfloat162_rn(p[0][0], p[0][1]), p1 = __floats2bfloat162_rn(p[1][0], p[1][1]);
                pf[0] = *reinterpret_cast<const unsigned*>(&p0);     // row g, keys 2t, 2t + 1
                pf[2] = *reinterpret_cast<const unsigned*>(&p1);     // row g, keys 8 + 2t, ...
                pf[1] = 0u;
                pf[3] = 0u;
            }
#pragma unroll
            for (int d = 0; d < DT; ++d) {
                o[d][0] *= alpha;
                o[d][1] *= alpha;
            }
            // A masked key has weight zero, but 0 x NaN is NaN: rows of the value tile that hold no key of
            // this sequence (a page's unwritten tail, keys before the window) are cleared before they are read.
            if (pg * 64 + quarter * 16 + 15 >= kv_len || pg * 64 + quarter * 16 < key_lo) {
                const int row = quarter * 16 + (lane >> 1), key = pg * 64 + row;
                if (key >= kv_len || key < key_lo)
                    for (int c = lane & 1; c < HD / 8; c += 2)
                        *reinterpret_cast<uint4*>(const_cast<unsigned char*>(Vt) + (c >> 3) * BOX + swz(row, c & 7)) = make_uint4(0u, 0u, 0u, 0u);
                __syncwarp();
            }
            // O += P V over this warp's 16 keys
#pragma unroll
            for (int d = 0; d < DT; d += 2) {
                const int chunk = d + (lane >> 4);
                unsigned vb[4];
                dec_ldmatrix_x4_trans(vb, Vt + (chunk >> 3) * BOX + swz(quarter * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, chunk & 7));
                dec_mma(o[d], pf, vb[0], vb[1]);
                dec_mma(o[d + 1], pf, vb[2], vb[3]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + s);      // this warp has read its keys of the page
        }
        blm_trace(0x440);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
        if (g < G) {
#pragma unroll
            for (int d = 0; d < DT; ++d) {
                sm_acc[(warp * G + g) * HD + d * 8 + 2 * t] = o[d][0];
                sm_acc[(warp * G + g) * HD + d * 8 + 2 * t + 1] = o[d][1];
            }
            if (t == 0) { sm_m[warp * G + g] = m_run; sm_l[warp * G + g] = l_run; }
        }
    }
    __syncthreads();
    // merge the warps and write
    for (int idx = tid; idx < G * HD; idx += blockDim.x) {
        const int gg = idx / HD, d = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, sm_m[w * G + gg]);
        float L = 0.f, ov = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float scl = sm_m[w * G + gg] == -INFINITY ? 0.f : exp2f(sm_m[w * G + gg] - M);
            L += sm_l[w * G + gg] * scl;
            ov += sm_acc[(w * G + gg) * HD + d] * scl;
        }
        const int head = kvh * G + gg;
        if (active == 1) {
            a.out[(size_t)tok * a.n_heads * HD + (size_t)head * HD + d] = __float2bfloat16_rn(L > 0.f ? ov / L : 0.f);
        } else {
            const size_t pi = ((size_t)tok * a.n_heads + head) * a.n_splits + split;
            a.part_acc[pi * HD + d] = ov;
            if (d == 0) {
                a.part_ml[pi * 2] = M == -INFINITY ? -INFINITY : M * LN2;
                a.part_ml[pi * 2 + 1] = L;
            }
        }
    }
    blm_trace(0x450);
}

// Merges the partial results of the active splits: one warp per (token, head).
template <int HD>
__global__ void __launch_bounds__(128) attn_decode_combine_kernel(const AttnDecodeArgs a, int n_rows) {
    pdl_launch_dependents();
    pdl_wait();
    blm_trace(0x420);
    constexpr int DPL = HD / 32;       // dims per lane
    __shared__ float wts[4][64];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * 4 + warp;          // tok * n_heads + head
    if (row >= n_rows) return;
    const int tok = row / a.n_heads;                // one token per sequence: tok is the sequence
    const int kv_len = a.start_pos[tok] + 1;
    const int key_lo = a.window > 0 ? max(0, kv_len - a.window) : 0;
    const int active = attn_decode_active_splits(key_lo, kv_len, a.n_splits, a.pages_per_split);
    if (active == 1) return;                        // the split kernel wrote the output itself
    const float* ml = a.part_ml + (size_t)row * a.n_splits * 2;
    float m0 = lane < active ? ml[lane * 2] : -INFINITY, m1 = lane + 32 < active ? ml[(lane + 32) * 2] : -INFINITY;
    float l0 = lane < active ? ml[lane * 2 + 1] : 0.f, l1 = lane + 32 < active ? ml[(lane + 32) * 2 + 1] : 0.f;
    const float M = warp_max(fmaxf(m0, m1));
    const float w0 = m0 == -INFINITY ? 0.f : expf(m0 - M), w1 = m1 == -INFINITY ? 0.f : expf(m1 - M);
    const float L = warp_sum(l0 * w0 + l1 * w1);
    wts[warp][lane] = w0;
    wts[warp][lane + 32] = w1;
    __syncwarp();
    const float* acc = a.part_acc + (size_t)row * a.n_splits * HD;
    float o[DPL];
#pragma unroll
    for (int e = 0; e < DPL; ++e) o[e] = 0.f;
#pragma unroll 4
    for (int z = 0; z < active; ++z) {
        const float w = wts[warp][z];
#pragma unroll
        for (int e = 0; e < DPL; ++e) o[e] += acc[(size_t)z * HD + e * 32 + lane] * w;
    }
    const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
    for (int e = 0; e < DPL; ++e) a.out[(size_t)row * HD + e * 32 + lane] = __float2bfloat16_rn(o[e] * inv);
}

typedef CUresult (*DecEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                     const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The TMA's view of one cache line's pool [pages][2][n_kv][64][HD]: a matrix of pages * 2 * n_kv * 64 rows
// of HD lanes; boxes of 64 rows x 64 lanes with the 128-byte swizzle.
static bool attn_decode_pool_map(const void* pool, int n_pages, int n_kv, int hd, CUtensorMap* out) {
    static DecEncodeTiledFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess || !fn)
            return false;
        encode = (DecEncodeTiledFn)fn;
    }
    static std::map<std::tuple<const void*, int, int, int>, CUtensorMap> maps;
    const auto key = std::make_tuple(pool, n_pages, n_kv, hd);
    auto it = maps.find(key);
    if (it == maps.end()) {
        CUtensorMap m;
        const cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)n_pages * 2 * n_kv * 64};
        const cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
        const cuuint32_t box[2] = {64, 64};
        const cuuint32_t estr[2] = {1, 1};
        if (encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
        if (maps.size() > 4096) maps.clear();
        it = maps.emplace(key, m).first;
    }
    *out = it->second;
    return true;
}

template <int HD, int NG>
static bool attn_decode_launch_ng(AttnDecodeArgs a, dim3 grid, int n_pages, cudaStream_t stream) {
    const int G = a.group;
    auto bytes = [&](int stages) {
        return (size_t)stages * 2 * 64 * HD * 2 + (size_t)4 * a.n_groups * G * (HD + 2) * 4 + 2 * stages * 8 + 16 + 1024;
    };
    while (bytes(a.n_stages) > 220 * 1024 && a.n_stages > a.n_groups) a.n_stages -= a.n_groups;   // the warps' results need room too
    if (bytes(a.n_stages) > 220 * 1024) return false;
    const size_t smem = bytes(a.n_stages);
    CUtensorMap map;
    if (!attn_decode_pool_map(a.pool, n_pages, a.n_kv, HD, &map)) return false;
    static bool opted_in = false;
    if (!opted_in) {
        if (cudaFuncSetAttribute(attn_decode_kernel<HD, NG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess) return false;
        opted_in = true;
    }
    return blm_launch_dependent(attn_decode_kernel<HD, NG>, grid, dim3((4 * NG + 1) * 32), smem, stream, a, map) == cudaSuccess;
}

template <int HD>
static bool launch_attn_decode_g(const AttnDecodeArgs& a, dim3 grid, int n_pages, cudaStream_t stream) {
    if (a.group < 1 || a.group > 8) return false;
    switch (a.n_groups) {
        case 1: return attn_decode_launch_ng<HD, 1>(a, grid, n_pages, stream);
        case 2: return attn_decode_launch_ng<HD, 2>(a, grid, n_pages, stream);
        case 4: return attn_decode_launch_ng<HD, 4>(a, grid, n_pages, stream);
        default: return false;
    }
}

// true when the specialised kernels were launched; false: the shape is left to the general kernel
static bool launch_attn_decode(AttnDecodeArgs a, int hd, int group, int n_seqs, int n_pages, int max_kv_len, cudaStream_t stream) {
    const dim3 grid(a.n_splits, a.n_kv, n_seqs);
    a.group = group;
    // the longest walk of a block: the pages of the longest sequence (all the cache could hold, when the
    // caller does not say), shared out over the splits
    const int most_pages = max_kv_len > 0 ? (max_kv_len + 63) / 64 : 4 * a.n_splits;
    const int blocks = a.n_splits * a.n_kv * n_seqs, pages_per_block = (most_pages + a.n_splits - 1) / a.n_splits;
    // With more blocks than fill the SMs twice, a sequence takes blocks in proportion to its length (measured on the 3B
    // shape, 16 sequences of 64 to 4,200 tokens in 3 splits: a decode step 3.11 to 2.95 ms); with fewer, every sequence
    // takes all the splits, short blocks being what fills the SMs then (8 sequences of 2,100 tokens in a bound of 4,096:
    // 0.840 ms a step against 0.860).
    a.pages_per_split = (max_kv_len > 0 && blocks > 2 * blm_sm_count()) ? pages_per_block : 1;
    if (a.pages_per_split < 1) a.pages_per_split = 1;
    a.n_stages = attn_decode_stages(hd, blocks, pages_per_block);
    a.n_groups = attn_decode_groups(blocks, pages_per_block, a.n_stages, hd);
    a.n_stages -= a.n_stages % a.n_groups;
    const int n_rows = n_seqs * a.n_heads;
    if (hd == 64) {
        if (!launch_attn_decode_g<64>(a, grid, n_pages, stream)) return false;
        if (a.n_splits > 1) blm_launch_dependent(attn_decode_combine_kernel<64>, dim3((n_rows + 3) / 4), dim3(128), 0, stream, a, n_rows);
        return true;
    }
    if (hd == 128) {
        if (!launch_attn_decode_g<128>(a, grid, n_pages, stream)) return false;
        if (a.n_splits > 1) blm_launch_dependent(attn_decode_combine_kernel<128>, dim3((n_rows + 3) / 4), dim3(128), 0, stream, a, n_rows);
        return true;
    }
    return false;
}
