// Row-wise kernels of a decoder step: embedding gather, residual add + RMS norm, rotary position
// encoding fused with the cache append, gated activation, dtype conversion.
// All statistics, angles and sums are fp32 (angles fp64); values are rounded once when stored.
#include "common.cuh"

BLM_API const char* blm_elementwise_last_error() { return g_blm_error; }

// ---------------------------------------------------------------------------------------------
// embedding: out[n, :] = table[tokens[n], :]  (fp32 residual stream from a bf16 or fp32 table)
// With `xg` the kernel also leaves the input of the norm that reads the stream first, as the products that write
// the stream do: xg[n, :] = bf16(out[n, :] * gamma) and ssq[n] = the row's sum of squares (one part: a row of up to
// `ssq_row` tokens), so that the first product of a decode step need not normalise the stream in every block.
// ---------------------------------------------------------------------------------------------
template <typename TT>
__global__ void embed_kernel(const int* __restrict__ tokens, const TT* __restrict__ table,
                             float* __restrict__ out, int width, int vocab, const void* __restrict__ gamma, int gamma_f32,
                             __nv_bfloat16* __restrict__ xg, float* __restrict__ ssq) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    blm_trace(0x220);
    const int n = blockIdx.x;
    int tok = tokens[n];
    if ((unsigned)tok >= (unsigned)vocab) tok = 0;  // ids are validated on the host; never read wild
    const TT* row = table + (size_t)tok * width;
    float* o = out + (size_t)n * width;
    if (xg == nullptr) {
        for (int d = threadIdx.x; d < width; d += blockDim.x) o[d] = to_f32(row[d]);
        return;
    }
    float ss = 0.f;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        const float v = to_f32(row[d]);
        const float g = gamma_f32 ? reinterpret_cast<const float*>(gamma)[d] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(gamma)[d]);
        o[d] = v;
        xg[(size_t)n * width + d] = __float2bfloat16_rn(v * g);
        ss += v * v;
    }
    const float total = block_sum(ss, red);
    if (threadIdx.x == 0) ssq[n] = total;
}

BLM_API int blm_embed(const int* tokens, const void* table, int table_dtype, float* out,
                      int n_tokens, int width, int vocab, const void* gamma, int gamma_f32, void* xg, float* ssq, int ssq_row,
                      cudaStream_t stream) {
    if (n_tokens == 0) return BLM_OK;
    BLM_REQUIRE(n_tokens > 0 && width > 0 && vocab > 0, "embed: bad sizes");
    BLM_REQUIRE(xg == nullptr || (gamma != nullptr && ssq != nullptr && n_tokens <= ssq_row), "embed: a norm is handed over with gamma and room for %d sums", n_tokens);
    const int threads = width >= 1024 ? 256 : 128;
    __nv_bfloat16* x = (__nv_bfloat16*)xg;
    if (table_dtype == BLM_F32)
        blm_launch_dependent(embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const float*)table, out, width, vocab, gamma, gamma_f32, x, ssq);
    else if (table_dtype == BLM_BF16)
        blm_launch_dependent(embed_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const __nv_bfloat16*)table, out, width, vocab, gamma, gamma_f32, x, ssq);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "embed: table dtype %d", table_dtype);
    return blm_check_launch("embed");
}

// ---------------------------------------------------------------------------------------------
// residual add + RMS norm.
//   rows == nullptr: for every row n: resid[n] += delta[n] (fp32, stored), out[n] = norm(resid[n])
//   rows != nullptr: out[i] = norm(resid[rows[i]] + delta[rows[i]]), resid is left as it is
// delta may be null (nothing to add).  gamma is fp32 or bf16 whatever the activations are.
// ---------------------------------------------------------------------------------------------
template <typename TA, typename TG>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TA* __restrict__ delta,
                                   const TG* __restrict__ gamma, TA* __restrict__ out,
                                   const int* __restrict__ rows, int width, float eps) {
    extern __shared__ float row_buf[];  // [width] + 33 for the reduction
    float* red = row_buf + width;
    const int src = rows ? rows[blockIdx.x] : blockIdx.x;
    float* r = resid + (size_t)src * width;
    const TA* dl = delta ? delta + (size_t)src * width : nullptr;
    float ss = 0.f;
    for (int d = threadIdx.x; d < width; d += blockDim.x) {
        float h = r[d];
        if (dl) h += to_f32(dl[d]);
        row_buf[d] = h;
        ss += h * h;
        if (!rows && dl) r[d] = h;
    }
    const float total = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
    TA* o = out + (size_t)blockIdx.x * width;
    for (int d = threadIdx.x; d < width; d += blockDim.x)
        o[d] = from_f32<TA>(row_buf[d] * inv * to_f32(gamma[d]));
}

// bf16 activations, width a multiple of 8: 16-byte accesses, the row kept in registers when it fits
template <typename TG>
__global__ void add_rmsnorm_bf16_vec_kernel(float* __restrict__ resid, const __nv_bfloat16* __restrict__ delta,
                                            const TG* __restrict__ gamma, __nv_bfloat16* __restrict__ out,
                                            const int* __restrict__ rows, int width, float eps) {
    __shared__ float red[33];
    constexpr int MAXV = 4;                 // 8-lane groups per thread: width <= blockDim * 8 * MAXV
    const int src = rows ? rows[blockIdx.x] : blockIdx.x;
    float* r = resid + (size_t)src * width;
    const __nv_bfloat16* dl = delta ? delta + (size_t)src * width : nullptr;
    float h[MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
        const int d = (v * blockDim.x + threadIdx.x) * 8;
        if (d < width) {
            const float4 a = *reinterpret_cast<const float4*>(r + d), b = *reinterpret_cast<const float4*>(r + d + 4);
            h[v][0] = a.x; h[v][1] = a.y; h[v][2] = a.z; h[v][3] = a.w; h[v][4] = b.x; h[v][5] = b.y; h[v][6] = b.z; h[v][7] = b.w;
            if (dl) {
                const uint4 dv = *reinterpret_cast<const uint4*>(dl + d);
                const __nv_bfloat162* dp = reinterpret_cast<const __nv_bfloat162*>(&dv);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(dp[e]);
                    h[v][2 * e] += f.x;
                    h[v][2 * e + 1] += f.y;
                }
                if (!rows) {
                    *reinterpret_cast<float4*>(r + d) = make_float4(h[v][0], h[v][1], h[v][2], h[v][3]);
                    *reinterpret_cast<float4*>(r + d + 4) = make_float4(h[v][4], h[v][5], h[v][6], h[v][7]);
                }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += h[v][e] * h[v][e];
        }
    }
    const float total = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
    __nv_bfloat16* o = out + (size_t)blockIdx.x * width;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
        const int d = (v * blockDim.x + threadIdx.x) * 8;
        if (d < width) {
            uint4 ov;
            __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
            for (int e = 0; e < 4; ++e)
                op[e] = __floats2bfloat162_rn(h[v][2 * e] * inv * to_f32(gamma[d + 2 * e]), h[v][2 * e + 1] * inv * to_f32(gamma[d + 2 * e + 1]));
            *reinterpret_cast<uint4*>(o + d) = ov;
        }
    }
}

template <typename TA, typename TG>
static int launch_add_rmsnorm(float* resid, const void* delta, const void* gamma, void* out,
                              const int* rows, int n_rows, int width, float eps, cudaStream_t stream) {
    if (sizeof(TA) == 2 && width % 8 == 0 && width <= 256 * 8 * 4 && ((size_t)resid & 15) == 0 && ((size_t)out & 15) == 0 &&
        (delta == nullptr || ((size_t)delta & 15) == 0)) {
        const int threads = width >= 2048 ? 256 : 128;
        if (width <= threads * 8 * 4) {
            add_rmsnorm_bf16_vec_kernel<TG><<<n_rows, threads, 0, stream>>>(resid, (const __nv_bfloat16*)delta, (const TG*)gamma,
                                                                              (__nv_bfloat16*)out, rows, width, eps);
            return blm_check_launch("add_rmsnorm");
        }
    }
    const size_t smem = (size_t)(width + 33) * sizeof(float);
    BLM_REQUIRE(smem <= 200 * 1024, "rms norm: width %d is beyond the 51,000 this kernel holds in shared memory", width);
    auto k = add_rmsnorm_kernel<TA, TG>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "rms norm: %s", cudaGetErrorString(e));
    }
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    k<<<n_rows, threads, smem, stream>>>(resid, (const TA*)delta, (const TG*)gamma, (TA*)out, rows, width, eps);
    return blm_check_launch("add_rmsnorm");
}

BLM_API int blm_add_rmsnorm(float* resid, const void* delta, const void* gamma, int gamma_dtype,
                            void* out, int act_dtype, const int* rows, int n_rows, int width,
                            float eps, cudaStream_t stream) {
    if (n_rows == 0) return BLM_OK;
    BLM_REQUIRE(n_rows > 0 && width > 0, "rms norm: bad sizes");
    if (act_dtype == BLM_F32 && gamma_dtype == BLM_F32)
        return launch_add_rmsnorm<float, float>(resid, delta, gamma, out, rows, n_rows, width, eps, stream);
    if (act_dtype == BLM_F32 && gamma_dtype == BLM_BF16)
        return launch_add_rmsnorm<float, __nv_bfloat16>(resid, delta, gamma, out, rows, n_rows, width, eps, stream);
    if (act_dtype == BLM_BF16 && gamma_dtype == BLM_F32)
        return launch_add_rmsnorm<__nv_bfloat16, float>(resid, delta, gamma, out, rows, n_rows, width, eps, stream);
    if (act_dtype == BLM_BF16 && gamma_dtype == BLM_BF16)
        return launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(resid, delta, gamma, out, rows, n_rows, width, eps, stream);
    return blm_fail(BLM_BAD_ARGUMENT, "rms norm: dtypes %d/%d", act_dtype, gamma_dtype);
}

// ---------------------------------------------------------------------------------------------
// rotary position encoding of q and k, fused with the append of k and v to the paged cache.
//   qkv [N, (H + 2 KV) * hd]: q heads, then k heads, then v heads of every token.
//   q is rotated in place; rotated k and plain v go to the page that holds the token's position.
//   cache pool of one layer: [pages][2 (k, v)][KV][page_size][hd].
//   The angle pos * inv_freq[i] and its sine and cosine are computed in fp64 and applied in fp32,
//   so no position is too far for the table and long contexts lose nothing to the angle.
//   pairing 0: lanes (i, i + rot/2); pairing 1: lanes (2i, 2i + 1); pairing 2: pair i sits at lanes
//   (16 (i / 8) + i % 8, that + 8), the order in which a 16-row tile of a matrix product holds the pairs
//   of a head whose rows were dealt out that way.  rot == 0: no rotation.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_append_kernel(T* __restrict__ qkv, const int* __restrict__ token_seq,
                                   const int* __restrict__ token_pos, const int* __restrict__ slot_of_seq,
                                   const int* __restrict__ block_table, int table_stride,
                                   const double* __restrict__ inv_freq, int rot, int pairing,
                                   T* __restrict__ pool, int n_heads, int n_kv, int hd, int page_size,
                                   int write_cache, const float2* __restrict__ table, int table_len) {
    // one item per thread: a rotated pair of q or k, a lane of k beyond the rotated ones, or two lanes of v
    const int n = blockIdx.y;
    const int item = blockIdx.x * blockDim.x + threadIdx.x;
    const int half = rot >> 1;
    const int n_pairs = (n_heads + n_kv) * half;
    const int n_tail = write_cache ? n_kv * (hd - rot) : 0;
    const int n_v = write_cache ? n_kv * (hd >> 1) : 0;
    if (item >= n_pairs + n_tail + n_v) return;
    const int pos = token_pos[n];
    T* row = qkv + (size_t)n * (size_t)(n_heads + 2 * n_kv) * hd;
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (write_cache) {
        const int seq = token_seq[n];
        if (seq < 0) return;         // a row of no sequence (padding): nothing of it reaches the cache
        const int slot = slot_of_seq[seq];
        const int page = block_table[(size_t)slot * table_stride + pos / page_size];
        const size_t page_elems = (size_t)n_kv * page_size * hd;
        kdst = pool + (size_t)page * 2 * page_elems + (size_t)(pos % page_size) * hd;
        vdst = kdst + page_elems;
    }
    const size_t head_stride_cache = (size_t)page_size * hd;
    if (item < n_pairs) {
        const int h = item / half, i = item % half;
        float c, s;
        if (pos < table_len) {       // the same numbers, computed once by rope_table_kernel
            const float2 v = table[(size_t)pos * half + i];
            c = v.x;
            s = v.y;
        } else {
            double sd, cd;
            sincos((double)pos * inv_freq[i], &sd, &cd);
            c = (float)cd;
            s = (float)sd;
        }
        const int la = pairing == 1 ? 2 * i : (pairing == 2 ? 16 * (i >> 3) + (i & 7) : i);
        const int lb = pairing == 1 ? la + 1 : (pairing == 2 ? la + 8 : i + half);
        T* hp = row + (size_t)h * hd;
        const float a = to_f32(hp[la]), b = to_f32(hp[lb]);
        const T ra = from_f32<T>(a * c - b * s), rb = from_f32<T>(a * s + b * c);
        T* dst = (h < n_heads || !kdst) ? hp : kdst + (size_t)(h - n_heads) * head_stride_cache;
        dst[la] = ra;
        dst[lb] = rb;
    } else if (item < n_pairs + n_tail) {
        const int tail = hd - rot, j = item - n_pairs;
        const int h = j / tail, l = rot + j % tail;
        kdst[(size_t)h * head_stride_cache + l] = row[(size_t)(n_heads + h) * hd + l];
    } else {
        const int j = item - n_pairs - n_tail;
        const int h = j / (hd >> 1), l = 2 * (j % (hd >> 1));
        const T* vsrc = row + (size_t)(n_heads + n_kv + h) * hd + l;
        T* vd = vdst + (size_t)h * head_stride_cache + l;
        vd[0] = vsrc[0];
        vd[1] = vsrc[1];
    }
}

// bf16, the whole head rotated, pairs (i, i + hd/2) or tiled (`tiled`: pairing 2 above), hd a multiple of 16,
// positions inside the table: eight pairs per thread with 16-byte accesses
__global__ void rope_append_bf16_vec_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ token_seq,
                                            const int* __restrict__ token_pos, const int* __restrict__ slot_of_seq,
                                            const int* __restrict__ block_table, int table_stride,
                                            __nv_bfloat16* __restrict__ pool, int n_heads, int n_kv, int hd, int page_size,
                                            int write_cache, const float2* __restrict__ table, int tiled) {
    pdl_launch_dependents();
    pdl_wait();
    blm_trace(0x210);
    const int n = blockIdx.y;
    const int item = blockIdx.x * blockDim.x + threadIdx.x;
    const int half = hd >> 1, cpp = half >> 3;                  // chunks of 8 pairs per head
    const int n_rot = (n_heads + n_kv) * cpp;
    const int n_v = write_cache ? n_kv * (hd >> 3) : 0;
    if (item >= n_rot + n_v) return;
    const int pos = token_pos[n];
    __nv_bfloat16* row = qkv + (size_t)n * (size_t)(n_heads + 2 * n_kv) * hd;
    __nv_bfloat16* kdst = nullptr;
    __nv_bfloat16* vdst = nullptr;
    if (write_cache) {
        const int seq = token_seq[n];
        if (seq < 0) return;         // a row of no sequence (padding): nothing of it reaches the cache
        const int slot = slot_of_seq[seq];
        const int page = block_table[(size_t)slot * table_stride + pos / page_size];
        const size_t page_elems = (size_t)n_kv * page_size * hd;
        kdst = pool + (size_t)page * 2 * page_elems + (size_t)(pos % page_size) * hd;
        vdst = kdst + page_elems;
    }
    const size_t head_stride_cache = (size_t)page_size * hd;
    if (item < n_rot) {
        const int h = item / cpp, i = (item % cpp) * 8;
        __nv_bfloat16* hp = row + (size_t)h * hd;
        const int la = tiled ? 2 * i : i, lb = tiled ? 2 * i + 8 : i + half;      // where the eight pairs' two halves lie
        const uint4 av = *reinterpret_cast<const uint4*>(hp + la), bv = *reinterpret_cast<const uint4*>(hp + lb);
        const float4* cs = reinterpret_cast<const float4*>(table + (size_t)pos * half + i);
        const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&av);
        const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&bv);
        uint4 ra, rb;
        __nv_bfloat162* rap = reinterpret_cast<__nv_bfloat162*>(&ra);
        __nv_bfloat162* rbp = reinterpret_cast<__nv_bfloat162*>(&rb);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float4 t = cs[e];                  // (cos, sin) of pairs 2e and 2e + 1
            const float2 a2 = __bfloat1622float2(ap[e]), b2 = __bfloat1622float2(bp[e]);
            rap[e] = __floats2bfloat162_rn(a2.x * t.x - b2.x * t.y, a2.y * t.z - b2.y * t.w);
            rbp[e] = __floats2bfloat162_rn(a2.x * t.y + b2.x * t.x, a2.y * t.w + b2.y * t.z);
        }
        __nv_bfloat16* dst = (h < n_heads || !kdst) ? hp : kdst + (size_t)(h - n_heads) * head_stride_cache;
        *reinterpret_cast<uint4*>(dst + la) = ra;
        *reinterpret_cast<uint4*>(dst + lb) = rb;
    } else {
        const int j = item - n_rot;
        const int h = j / (hd >> 3), l = (j % (hd >> 3)) * 8;
        *reinterpret_cast<uint4*>(vdst + (size_t)h * head_stride_cache + l) =
            *reinterpret_cast<const uint4*>(row + (size_t)(n_heads + n_kv + h) * hd + l);
    }
}

BLM_API int blm_rope_append(void* qkv, int dtype, const int* token_seq, const int* token_pos,
                            const int* slot_of_seq, const int* block_table, int table_stride,
                            const double* inv_freq, int rot, int pairing, void* pool, int n_tokens,
                            int n_heads, int n_kv, int hd, int page_size, int write_cache,
                            const float2* table, int table_len, int table_covers_step, cudaStream_t stream) {
    if (n_tokens == 0) return BLM_OK;
    BLM_REQUIRE(rot >= 0 && rot <= hd && rot % 2 == 0, "rotary: %d rotated lanes of a head of %d", rot, hd);
    BLM_REQUIRE(rot == 0 || inv_freq != nullptr, "rotary: no frequencies");
    BLM_REQUIRE(pairing >= 0 && pairing <= 2, "rotary: pairing %d", pairing);
    BLM_REQUIRE(pairing != 2 || rot % 16 == 0, "rotary: tiled pairs need a multiple of 16 rotated lanes, got %d", rot);
    BLM_REQUIRE(hd % 2 == 0, "rotary: odd head size %d", hd);
    const int threads = 128;
    const int items = (n_heads + n_kv) * (rot / 2) + (write_cache ? n_kv * (hd - rot) + n_kv * (hd / 2) : 0);
    if (items == 0) return BLM_OK;
    const dim3 grid((items + threads - 1) / threads, n_tokens);
    BLM_REQUIRE(grid.y <= 65535, "rotary: %d tokens in one step (at most 65535)", n_tokens);
    const size_t smem = 0;
    if (dtype == BLM_BF16 && rot == hd && pairing != 1 && hd % 16 == 0 && table != nullptr && table_len > 0 &&
        ((size_t)qkv & 15) == 0 && (!write_cache || ((size_t)pool & 15) == 0) && ((size_t)table & 15) == 0) {
        // every position of the step must lie inside the table for this path; the host makes the table
        // as long as the cache's longest sequence, and a step never goes beyond that
        const int vitems = (n_heads + n_kv) * (hd / 16) + (write_cache ? n_kv * (hd / 8) : 0);
        const dim3 vgrid((vitems + threads - 1) / threads, n_tokens);
        if (table_covers_step) {
            blm_launch_dependent(rope_append_bf16_vec_kernel, vgrid, dim3(threads), 0, stream, (__nv_bfloat16*)qkv, token_seq, token_pos,
                                 slot_of_seq, block_table, table_stride, (__nv_bfloat16*)pool, n_heads, n_kv, hd, page_size,
                                 write_cache, table, pairing == 2 ? 1 : 0);
            return blm_check_launch("rope_append");
        }
    }
    if (dtype == BLM_F32)
        rope_append_kernel<float><<<grid, threads, smem, stream>>>((float*)qkv, token_seq, token_pos, slot_of_seq, block_table, table_stride, inv_freq, rot, pairing, (float*)pool, n_heads, n_kv, hd, page_size, write_cache, table, table_len);
    else if (dtype == BLM_BF16)
        rope_append_kernel<__nv_bfloat16><<<grid, threads, smem, stream>>>((__nv_bfloat16*)qkv, token_seq, token_pos, slot_of_seq, block_table, table_stride, inv_freq, rot, pairing, (__nv_bfloat16*)pool, n_heads, n_kv, hd, page_size, write_cache, table, table_len);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "rotary: dtype %d", dtype);
    return blm_check_launch("rope_append");
}

// (cos, sin) of pos * inv_freq[i] for pos < n_pos, in fp64, rounded to fp32: what rope_append_kernel
// computes on the fly, once for all steps
__global__ void rope_table_kernel(const double* __restrict__ inv_freq, float2* __restrict__ table, int n_pos, int half) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_pos * half) return;
    const int pos = (int)(idx / half), i = (int)(idx % half);
    double s, c;
    sincos((double)pos * inv_freq[i], &s, &c);
    table[idx] = make_float2((float)c, (float)s);
}

BLM_API int blm_rope_table(const double* inv_freq, float* table, int n_pos, int half, cudaStream_t stream) {
    if (n_pos == 0 || half == 0) return BLM_OK;
    const size_t total = (size_t)n_pos * half;
    rope_table_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(inv_freq, (float2*)table, n_pos, half);
    return blm_check_launch("rope_table");
}

// ---------------------------------------------------------------------------------------------
// gated activation: out[n, i] = silu(gate_i) * up_i, computed in fp32.  The fused product gu[n, 2 I]
// holds gate then up (tile == 0), or tiles of `tile` gates followed by the `tile` ups of the same outputs.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inner, size_t total, int tile) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t n = idx / inner;
        const int i = (int)(idx % inner);
        const size_t gi = tile ? (size_t)(i / tile) * 2 * tile + i % tile : (size_t)i;
        const size_t ui = tile ? gi + tile : (size_t)inner + i;
        const float g = to_f32(gu[n * 2 * inner + gi]);
        const float u = to_f32(gu[n * 2 * inner + ui]);
        out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

// bf16, eight outputs per thread: 16-byte loads of the gates and of the ups, one 16-byte store
__global__ void swiglu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int inner,
                                     size_t total8, int tile) {
    const int per_row = inner >> 3;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t n = idx / per_row;
        const int i = (int)(idx % per_row) * 8;
        const size_t gi = tile ? (size_t)(i / tile) * 2 * tile + i % tile : (size_t)i;
        const size_t ui = tile ? gi + tile : (size_t)inner + i;
        const uint4 gv = *reinterpret_cast<const uint4*>(gu + n * 2 * inner + gi);
        const uint4 uv = *reinterpret_cast<const uint4*>(gu + n * 2 * inner + ui);
        const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&uv);
        uint4 ov;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 g = __bfloat1622float2(gp[e]), u = __bfloat1622float2(up[e]);
            op[e] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
        }
        *reinterpret_cast<uint4*>(out + n * inner + i) = ov;
    }
}

BLM_API int blm_swiglu(const void* gu, void* out, int dtype, int n_rows, int inner, int tile, cudaStream_t stream) {
    if (n_rows == 0) return BLM_OK;
    BLM_REQUIRE(tile >= 0 && (tile == 0 || inner % tile == 0), "swiglu: tiles of %d do not divide %d", tile, inner);
    const size_t total = (size_t)n_rows * inner;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < blm_sm_count() * 16 ? (total + threads - 1) / threads : blm_sm_count() * 16);
    if (dtype == BLM_BF16 && inner % 8 == 0 && (tile == 0 || tile % 8 == 0) && ((size_t)gu & 15) == 0 && ((size_t)out & 15) == 0) {
        const size_t total8 = total / 8;
        const int b8 = (int)((total8 + threads - 1) / threads < blm_sm_count() * 16 ? (total8 + threads - 1) / threads : blm_sm_count() * 16);
        swiglu_bf16x8_kernel<<<b8, threads, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inner, total8, tile);
        return blm_check_launch("swiglu");
    }
    if (dtype == BLM_F32)
        swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, inner, total, tile);
    else if (dtype == BLM_BF16)
        swiglu_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, inner, total, tile);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "swiglu: dtype %d", dtype);
    return blm_check_launch("swiglu");
}

// ---------------------------------------------------------------------------------------------
// dtype conversion (for a layer whose weights are stored in fp32 inside a bf16 model)
// ---------------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void convert_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t total) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x)
        out[idx] = from_f32<TO>(to_f32(in[idx]));
}

BLM_API int blm_convert(const void* in, int in_dtype, void* out, int out_dtype, size_t total, cudaStream_t stream) {
    if (total == 0) return BLM_OK;
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < blm_sm_count() * 16 ? (total + threads - 1) / threads : blm_sm_count() * 16);
    if (in_dtype == BLM_F32 && out_dtype == BLM_BF16)
        convert_kernel<float, __nv_bfloat16><<<blocks, threads, 0, stream>>>((const float*)in, (__nv_bfloat16*)out, total);
    else if (in_dtype == BLM_BF16 && out_dtype == BLM_F32)
        convert_kernel<__nv_bfloat16, float><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)in, (float*)out, total);
    else
        return blm_fail(BLM_BAD_ARGUMENT, "convert: %d -> %d", in_dtype, out_dtype);
    return blm_check_launch("convert");
}

// ---------------------------------------------------------------------------------------------
// between two decode steps that run without the host: the sampled token becomes the next input,
// every position moves on by one, and the token is appended to the history of the run
// ---------------------------------------------------------------------------------------------
__global__ void decode_advance_kernel(int* __restrict__ tokens, int* __restrict__ pos, const int* __restrict__ sampled,
                                      int* __restrict__ history, int* __restrict__ step_no, long long* __restrict__ counters,
                                      int batch, int history_steps) {
    pdl_launch_dependents();
    pdl_wait();
    blm_trace(0x230);
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    const int s = *step_no;
    if (b < batch) {
        const int t = sampled[b];
        tokens[b] = t;
        pos[b] += 1;
        if (counters) counters[b] += 1;
        if (history && s < history_steps) history[(size_t)s * batch + b] = t;
    }
}
// a launch of its own, so that every block of the kernel above has read the old value
__global__ void bump_kernel(int* step_no) {
    pdl_launch_dependents();
    pdl_wait();
    *step_no += 1;
}

// Once per step and group of cache lines, for every layer of the group: the page each new token goes to, and the
// block table's rows put in the order of the step's sequences.  The kernels that append to the cache and that walk
// a sequence's pages then read one array each instead of following token -> sequence -> slot -> table.
__global__ void step_tables_kernel(const int* __restrict__ token_seq, const int* __restrict__ token_pos, const int* __restrict__ slot_of_seq,
                                   const int* __restrict__ block_table, int table_stride, int page_size, int n_tokens, int n_seqs,
                                   int* __restrict__ token_page, int* __restrict__ seq_table) {
    pdl_launch_dependents();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n_tokens) {
        const int seq = token_seq[idx];
        token_page[idx] = seq >= 0 ? block_table[(size_t)slot_of_seq[seq] * table_stride + token_pos[idx] / page_size] : -1;   // -1: a row of no sequence
    }
    const int cell = idx - n_tokens;
    if (cell >= 0 && cell < n_seqs * table_stride)
        seq_table[cell] = block_table[(size_t)slot_of_seq[cell / table_stride] * table_stride + cell % table_stride];
}

BLM_API int blm_step_tables(const int* token_seq, const int* token_pos, const int* slot_of_seq, const int* block_table, int table_stride,
                            int page_size, int n_tokens, int n_seqs, int* token_page, int* seq_table, cudaStream_t stream) {
    const long long total = (long long)n_tokens + (long long)n_seqs * table_stride;
    if (total == 0) return BLM_OK;
    BLM_REQUIRE(page_size > 0 && table_stride > 0, "step_tables: page size %d, table stride %d", page_size, table_stride);
    blm_launch_dependent(step_tables_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, token_seq, token_pos, slot_of_seq,
                         block_table, table_stride, page_size, n_tokens, n_seqs, token_page, seq_table);
    return blm_check_launch("step_tables");
}

BLM_API int blm_decode_advance(int* tokens, int* pos, const int* sampled, int* history, int* step_no,
                               long long* counters, int batch, int history_steps, cudaStream_t stream) {
    if (batch == 0) return BLM_OK;
    BLM_REQUIRE(step_no != nullptr, "decode_advance: no step counter");
    blm_launch_dependent(decode_advance_kernel, dim3((batch + 127) / 128), dim3(128), 0, stream, tokens, pos, sampled, history, step_no,
                         counters, batch, history_steps);
    blm_launch_dependent(bump_kernel, dim3(1), dim3(1), 0, stream, step_no);
    return blm_check_launch("decode_advance");
}
