// Prompt attention for bf16 on the tensor cores: causal, grouped-query, over the paged cache.
//
// A block of 4 warps owns 64 consecutive query positions of one head of one sequence; a warp owns 16
// of them.  Keys and values come page by page (64 positions, which is also the tile) through a
// double buffer in shared memory filled by cp.async; S = Q K^T and O += P V run as
// mma.sync.m16n8k16 with fp32 accumulators, the softmax is the online one, in fp32 on the
// accumulator registers (scores in base-2 units), and P is rounded to bf16 only as an operand of the
// second product.  Shared tiles are swizzled by 16-byte chunks (chunk ^= row & 7) so that ldmatrix
// reads without bank conflicts.  Rows of a page beyond the sequence are zero-filled: the pool is
// never cleared.
#pragma once
#include "common.cuh"

struct AttnPrefillArgs {
    const __nv_bfloat16* q;      // token n, head h at q + n * q_stride + h * HD
    long long q_stride;
    const __nv_bfloat16* pool;   // [pages][2][n_kv][64][HD]
    const int* block_table;
    int table_stride;
    const int* cu_seqlens;
    const int* slot_of_seq;
    const int* start_pos;
    __nv_bfloat16* out;          // [N, n_heads * HD]
    int n_heads, n_kv, window;
    float scale_log2e;
};

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    const unsigned addr = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
}

template <int HD>
__global__ void __launch_bounds__(128) attn_prefill_kernel(const AttnPrefillArgs a) {
    constexpr int BM = 64, BN = 64;              // query positions per block, keys per tile (= page)
    constexpr int CH = HD / 8;                   // 16-byte chunks per row
    constexpr int KS = HD / 16;                  // k steps of S = Q K^T
    constexpr int DT = HD / 8;                   // 8-wide output tiles
    extern __shared__ __align__(128) unsigned char smem_pf[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_pf);            // [BM][HD], swizzled
    __nv_bfloat16* Ks = Qs + BM * HD;                                          // [2][BN][HD]
    __nv_bfloat16* Vs = Ks + 2 * BN * HD;                                      // [2][BN][HD]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int seq = blockIdx.z, head = blockIdx.y;
    const int tok0 = a.cu_seqlens[seq];
    const int q_len = a.cu_seqlens[seq + 1] - tok0;
    // later tiles have more keys to walk: start them first
    const int q0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * BM;
    if (q0 >= q_len) return;
    const int start = a.start_pos[seq];
    const int kv_len = start + q_len;
    const int kvh = head / (a.n_heads / a.n_kv);
    const int* pages = a.block_table + (size_t)a.slot_of_seq[seq] * a.table_stride;
    const size_t page_elems = (size_t)a.n_kv * BN * HD;

    auto swz = [](int row, int chunk) { return row * HD + ((chunk ^ (row & 7)) << 3); };   // element offset

    // Q tile -> shared (zero beyond the sequence's new tokens)
    for (int idx = tid; idx < BM * CH; idx += 128) {
        const int r = idx / CH, c = idx % CH;
        __nv_bfloat16* dst = Qs + swz(r, c);
        if (q0 + r < q_len) {
            const __nv_bfloat16* src = a.q + (size_t)(tok0 + q0 + r) * a.q_stride + (size_t)head * HD + c * 8;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
        } else {
            *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    auto load_tile = [&](int tile, int buf) {
        const int page = pages[tile];
        const __nv_bfloat16* kp = a.pool + (size_t)page * 2 * page_elems + (size_t)kvh * BN * HD;
        const __nv_bfloat16* vp = kp + page_elems;
        const int valid = min(BN, kv_len - tile * BN);
        for (int idx = tid; idx < BN * CH; idx += 128) {
            const int r = idx / CH, c = idx % CH;
            __nv_bfloat16* kd = Ks + buf * BN * HD + swz(r, c);
            __nv_bfloat16* vd = Vs + buf * BN * HD + swz(r, c);
            if (r < valid) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(kd)), "l"(kp + (size_t)r * HD + c * 8));
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(vd)), "l"(vp + (size_t)r * HD + c * 8));
            } else {
                *reinterpret_cast<uint4*>(kd) = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(vd) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };

    // keys this block walks: up to its last query's position, from the window's start
    const int p_first = start + q0, p_last = start + min(q0 + BM, q_len) - 1;
    const int tile_lo = a.window > 0 ? max(0, p_first - a.window + 1) / BN : 0;
    const int tile_hi = p_last / BN;     // inclusive

    load_tile(tile_lo, 0);
    asm volatile("cp.async.commit_group;\n" ::);

    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; ++d)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[d][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};    // rows g and g + 8 of the warp's 16
    unsigned qf[KS][4];
    const int row_lo = start + q0 + warp * 16 + g, row_hi = row_lo + 8;   // absolute positions of this thread's rows

    for (int tile = tile_lo; tile <= tile_hi; ++tile) {
        const int buf = (tile - tile_lo) & 1;
        if (tile < tile_hi) load_tile(tile + 1, buf ^ 1);
        asm volatile("cp.async.commit_group;\n" ::);
        asm volatile("cp.async.wait_group 1;\n" ::);      // this tile (and Q) have landed; the next may still fly
        __syncthreads();
        if (tile == tile_lo) {
#pragma unroll
            for (int kk = 0; kk < KS; ++kk)
                ldmatrix_x4(qf[kk], Qs + swz(warp * 16 + (lane & 15), 2 * kk + (lane >> 4)));
        }
        const __nv_bfloat16* Kb = Ks + buf * BN * HD;
        const __nv_bfloat16* Vb = Vs + buf * BN * HD;

        // S = Q K^T for 16 rows x 64 keys
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
            for (int kk = 0; kk < KS; kk += 2) {
                unsigned kb[4];     // b0, b1 of k step kk; b0, b1 of k step kk + 1
                ldmatrix_x4(kb, Kb + swz(nt * 8 + (lane & 7), 2 * kk + (lane >> 3)));
                mma_bf16(s[nt], qf[kk], kb[0], kb[1]);
                mma_bf16(s[nt], qf[kk + 1], kb[2], kb[3]);
            }
        }
        // scale, mask, online softmax
        const int key0 = tile * BN;
        const bool need_mask = key0 + BN - 1 > start + q0 + warp * 16 || (a.window > 0);
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[nt][e] * a.scale_log2e;
                if (need_mask) {
                    const int key = key0 + nt * 8 + 2 * t + (e & 1);
                    const int p = (e & 2) ? row_hi : row_lo;
                    if (key > p || (a.window > 0 && key <= p - a.window)) v = -INFINITY;
                }
                s[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        }
        float alpha[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            alpha[h] = m_run[h] == -INFINITY ? 0.f : exp2f(m_run[h] - m_new);
            m_run[h] = m_new;
        }
        float rs[2] = {0.f, 0.f};
        unsigned pf[4][4];      // P as the A operand of the second product: 4 k steps of 16 keys
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float m = m_run[e >> 1];
                p[e] = (s[nt][e] == -INFINITY || m == -INFINITY) ? 0.f : exp2f(s[nt][e] - m);
                rs[e >> 1] += p[e];
            }
            pf[nt >> 1][(nt & 1) * 2] = pack_bf16(p[0], p[1]);       // row g
            pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p[2], p[3]);   // row g + 8
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * alpha[h] + rs[h];   // this thread's share; summed over the quad at the end
#pragma unroll
        for (int d = 0; d < DT; ++d) {
            o[d][0] *= alpha[0]; o[d][1] *= alpha[0];
            o[d][2] *= alpha[1]; o[d][3] *= alpha[1];
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int d = 0; d < DT; d += 2) {
                unsigned vb[4];     // b0, b1 of output tile d; b0, b1 of output tile d + 1
                ldmatrix_x4_trans(vb, Vb + swz(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, d + (lane >> 4)));
                mma_bf16(o[d], pf[kk], vb[0], vb[1]);
                mma_bf16(o[d + 1], pf[kk], vb[2], vb[3]);
            }
        }
        __syncthreads();     // everybody is done with this buffer before the tile after next lands in it
    }

    // normalise and write
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    const float inv[2] = {l_run[0] > 0.f ? 1.0f / l_run[0] : 0.f, l_run[1] > 0.f ? 1.0f / l_run[1] : 0.f};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = q0 + warp * 16 + g + 8 * h;
        if (r >= q_len) continue;
        __nv_bfloat16* dst = a.out + (size_t)(tok0 + r) * a.n_heads * HD + (size_t)head * HD + 2 * t;
#pragma unroll
        for (int d = 0; d < DT; ++d)
            *reinterpret_cast<unsigned*>(dst + d * 8) = pack_bf16(o[d][2 * h] * inv[h], o[d][2 * h + 1] * inv[h]);
    }
}

// true when the kernel took the step
static bool launch_attn_prefill(const AttnPrefillArgs& a, int hd, int n_seqs, int max_q_len, cudaStream_t stream) {
    const dim3 grid((max_q_len + 63) / 64, a.n_heads, n_seqs);
    if (grid.y > 65535 || grid.z > 65535) return false;
    if (hd == 64) {
        attn_prefill_kernel<64><<<grid, 128, (64 + 4 * 64) * 64 * 2, stream>>>(a);
        return true;
    }
    if (hd == 128) {
        static bool opted_in = false;
        const int smem = (64 + 4 * 64) * 128 * 2;
        if (!opted_in) {
            if (cudaFuncSetAttribute(attn_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return false;
            opted_in = true;
        }
        attn_prefill_kernel<128><<<grid, 128, smem, stream>>>(a);
        return true;
    }
    return false;
}
