// Decode attention for bf16: one new token per sequence against its paged cache, grouped-query,
// keys split over blocks.  A block owns one (sequence, kv head, split); its 4 warps walk the keys of
// the split.  HD / 8 lanes share a key: each holds 8 lanes of the head (one 16-byte load of k, one of
// v), the partial dot products of the G query heads of the group are summed over those lanes with
// shuffles, and every lane keeps a running (max, sum, output slice) per head.  The running max is
// only raised when a score exceeds it, so a key costs one exponential per head.
#pragma once
#include "common.cuh"

struct AttnDecodeArgs {
    const __nv_bfloat16* q;      // token n, head h at q + n * q_stride + h * HD
    long long q_stride;
    const __nv_bfloat16* pool;   // [pages][2][n_kv][64][HD]
    const int* block_table;
    int table_stride;
    const int* cu_seqlens;
    const int* slot_of_seq;
    const int* start_pos;
    __nv_bfloat16* out;          // [N, n_heads * HD]
    float* part_acc;             // [N, n_heads, n_splits, HD]
    float* part_ml;              // [N, n_heads, n_splits, 2]: (max in natural-log units, sum)
    int n_heads, n_kv, window, n_splits;
    float scale_log2e;           // softmax scale times log2(e): scores live in base-2 units
};

// How many of the n_splits blocks of a (sequence, kv head) work: one for every 64 keys.
__host__ __device__ inline int attn_decode_active_splits(int span, int n_splits) {
    const int want = (span + 63) / 64;
    return want < 1 ? 1 : (want > n_splits ? n_splits : want);
}

template <int HD, int G>
__global__ void __launch_bounds__(128) attn_decode_kernel(const AttnDecodeArgs a) {
    constexpr int LPK = HD / 8;        // lanes per key
    constexpr int KPW = 32 / LPK;      // keys per warp per trip
    constexpr int WARPS = 4;
    constexpr float LN2 = 0.6931471805599453f;
    __shared__ float sm_acc[WARPS][G][HD];
    __shared__ float sm_m[WARPS][G], sm_l[WARPS][G];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sub = lane / LPK, li = lane % LPK;
    const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
    const int tok = a.cu_seqlens[seq];
    const int pos = a.start_pos[seq];            // the new token's position; keys 0..pos are visible
    const int kv_len = pos + 1;
    const int* pages = a.block_table + (size_t)a.slot_of_seq[seq] * a.table_stride;
    const size_t page_elems = (size_t)a.n_kv * 64 * HD;

    float qf[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const uint4 v = *reinterpret_cast<const uint4*>(a.q + (size_t)tok * a.q_stride + (size_t)(kvh * G + g) * HD + li * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            qf[g][2 * e] = f.x * a.scale_log2e;
            qf[g][2 * e + 1] = f.y * a.scale_log2e;
        }
    }
    float m[G], l[G], acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
    }

    // the keys of this split, in units of 16.  Only as many splits as the sequence has pages are
    // active (the grid is sized for the longest sequence the cache can hold); the others leave at once
    // and the combine kernel, which computes the same number, does not look at them.
    const int key_lo = a.window > 0 ? max(0, kv_len - a.window) : 0;
    const int span = kv_len - key_lo;
    const int active = attn_decode_active_splits(span, a.n_splits);
    if (split >= active) return;
    const int per = (((span + 15) / 16 + active - 1) / active) * 16;
    const int k_begin = key_lo + split * per;
    const int k_end = min(kv_len, k_begin + per);

    auto fetch = [&](int base, uint4& k4, uint4& v4) {
        const int key = base + sub;
        k4 = make_uint4(0u, 0u, 0u, 0u);
        v4 = k4;
        if (key < k_end) {
            const int page = pages[key >> 6];
            const __nv_bfloat16* kp = a.pool + (size_t)page * 2 * page_elems + ((size_t)kvh * 64 + (key & 63)) * HD + li * 8;
            k4 = *reinterpret_cast<const uint4*>(kp);
            v4 = *reinterpret_cast<const uint4*>(kp + page_elems);
        }
    };
    int base = k_begin + warp * KPW;
    uint4 kv4, vv4;
    fetch(base, kv4, vv4);
    while (base < k_end) {
        const int nbase = base + WARPS * KPW;
        uint4 kn4, vn4;
        fetch(nbase, kn4, vn4);        // the next trip's loads fly while this trip computes
        const bool live = base + sub < k_end;
        float kf[8], vf[8];
        {
            const __nv_bfloat162* kh = reinterpret_cast<const __nv_bfloat162*>(&kv4);
            const __nv_bfloat162* vh = reinterpret_cast<const __nv_bfloat162*>(&vv4);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 kk = __bfloat1622float2(kh[e]), vv = __bfloat1622float2(vh[e]);
                kf[2 * e] = kk.x; kf[2 * e + 1] = kk.y;
                vf[2 * e] = vv.x; vf[2 * e + 1] = vv.y;
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float s = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) s += qf[g][e] * kf[e];
#pragma unroll
            for (int o = LPK / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (live) {
                float p;
                if (s > m[g]) {            // a new maximum: rescale what was gathered so far
                    const float alpha = exp2f(m[g] - s);      // 0 the first time (m = -inf)
                    l[g] *= alpha;
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[g][e] *= alpha;
                    m[g] = s;
                    p = 1.f;
                } else {
                    p = exp2f(s - m[g]);
                }
                l[g] += p;
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[g][e] += p * vf[e];
            }
        }
        kv4 = kn4;
        vv4 = vn4;
        base = nbase;
    }

    // merge the key slots of a warp (lanes that differ above the LPK bits)
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float mo = __shfl_xor_sync(0xffffffffu, m[g], o);
            const float lo = __shfl_xor_sync(0xffffffffu, l[g], o);
            const float mn = fmaxf(m[g], mo);
            const float sa = m[g] == -INFINITY ? 0.f : exp2f(m[g] - mn);
            const float sb = mo == -INFINITY ? 0.f : exp2f(mo - mn);
            l[g] = l[g] * sa + lo * sb;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float ao = __shfl_xor_sync(0xffffffffu, acc[g][e], o);
                acc[g][e] = acc[g][e] * sa + ao * sb;
            }
            m[g] = mn;
        }
    }
    if (sub == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int e = 0; e < 8; ++e) sm_acc[warp][g][li * 8 + e] = acc[g][e];
            if (li == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
        }
    }
    __syncthreads();
    // merge the warps and write
    for (int idx = tid; idx < G * HD; idx += 128) {
        const int g = idx / HD, d = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, sm_m[w][g]);
        float L = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float sc = sm_m[w][g] == -INFINITY ? 0.f : exp2f(sm_m[w][g] - M);
            L += sm_l[w][g] * sc;
            o += sm_acc[w][g][d] * sc;
        }
        const int head = kvh * G + g;
        if (active == 1) {
            a.out[(size_t)tok * a.n_heads * HD + (size_t)head * HD + d] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
        } else {
            const size_t pi = ((size_t)tok * a.n_heads + head) * a.n_splits + split;
            a.part_acc[pi * HD + d] = o;
            if (d == 0) {
                a.part_ml[pi * 2] = M == -INFINITY ? -INFINITY : M * LN2;
                a.part_ml[pi * 2 + 1] = L;
            }
        }
    }
}

// Merges the partial results of the active splits: one warp per (token, head).
template <int HD>
__global__ void __launch_bounds__(128) attn_decode_combine_kernel(const AttnDecodeArgs a, int n_rows) {
    constexpr int DPL = HD / 32;       // dims per lane
    __shared__ float wts[4][64];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * 4 + warp;          // tok * n_heads + head
    if (row >= n_rows) return;
    const int tok = row / a.n_heads;                // one token per sequence: tok is the sequence
    const int kv_len = a.start_pos[tok] + 1;
    const int span = a.window > 0 ? min(kv_len, a.window) : kv_len;
    const int active = attn_decode_active_splits(span, a.n_splits);
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

template <int HD>
static bool launch_attn_decode_g(const AttnDecodeArgs& a, int group, dim3 grid, cudaStream_t stream) {
    switch (group) {
        case 1: attn_decode_kernel<HD, 1><<<grid, 128, 0, stream>>>(a); return true;
        case 2: attn_decode_kernel<HD, 2><<<grid, 128, 0, stream>>>(a); return true;
        case 4: attn_decode_kernel<HD, 4><<<grid, 128, 0, stream>>>(a); return true;
        case 8: attn_decode_kernel<HD, 8><<<grid, 128, 0, stream>>>(a); return true;
        default: return false;
    }
}

// true when the specialised kernels were launched; false: the shape is left to the general kernel
static bool launch_attn_decode(const AttnDecodeArgs& a, int hd, int group, int n_seqs, cudaStream_t stream) {
    const dim3 grid(a.n_splits, a.n_kv, n_seqs);
    const int n_rows = n_seqs * a.n_heads;
    if (hd == 64) {
        if (!launch_attn_decode_g<64>(a, group, grid, stream)) return false;
        if (a.n_splits > 1) attn_decode_combine_kernel<64><<<(n_rows + 3) / 4, 128, 0, stream>>>(a, n_rows);
        return true;
    }
    if (hd == 128) {
        if (!launch_attn_decode_g<128>(a, group, grid, stream)) return false;
        if (a.n_splits > 1) attn_decode_combine_kernel<128><<<(n_rows + 3) / 4, 128, 0, stream>>>(a, n_rows);
        return true;
    }
    return false;
}
