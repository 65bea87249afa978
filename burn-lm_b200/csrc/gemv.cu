// Skinny matrix products for decode steps: y[N, M] = x[N, K] . W[M, K]^T with N <= 64 tokens, bf16
// weights streamed once from HBM at full width, fp32 accumulation on the tensor cores.
//
// The weight matrix is the "A" operand of mma.sync.m16n8k16 (16 weight rows per warp), the tokens
// are the "B" operand (8 tokens per instruction), so one pass over W serves every token.  A thread
// loads 16 contiguous bytes of a weight row straight from global memory; the k index inside an
// instruction is permuted the same way for both operands, which a dot product does not notice, so
// no shuffle or shared-memory transpose of the weights is needed.  The tokens sit in shared memory.
//
// Fused around the product, to save launches and activation traffic:
//   prologue  x = rmsnorm(resid[rows]) * gamma computed by every block from the fp32 residual stream
//   epilogue  store (bf16 or fp32) | silu(gate) * up (rows i and I + i of a fused [gate; up] weight)
//             | resid += y (the residual add of the stream, exactly one writer per element)
// A block is WR row tiles x WK slices of K (8 warps); the K slices are summed through shared memory
// in a fixed order, so results are deterministic and do not depend on the other tokens of the batch.
#include <mma.h>

#include "common.cuh"

BLM_API const char* blm_gemv_last_error() { return g_blm_error; }

constexpr int kGemvThreads = 256;
constexpr int kUnroll = 4;  // 32-wide k units per loop trip: 8 x 16-byte loads in flight per thread

enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_RESID_ADD = 2 };

struct GemvArgs {
    const __nv_bfloat16* w;
    long long ldw;
    int M;              // outputs (for EPI_SWIGLU: the inner size I; W has 2 I rows, up at row I + i)
    int K;
    long long up_off;   // row offset of the "up" half for EPI_SWIGLU
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
    int wr, wk;              // warps: row tiles x k slices (wr * wk == 8)
    int kc;                  // k chunk staged in shared memory at a time (multiple of 32)
};

__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <int NBT>
__global__ void __launch_bounds__(kGemvThreads) gemv_kernel(const GemvArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int wr = warp / a.wk, wk = warp % a.wk;
    const int nrows = NBT * 8;
    const int xstride = a.kc + 8;                                  // bf16 elements; 16 bytes of padding
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem);    // [nrows][xstride]
    float* red = reinterpret_cast<float*>(smem + (size_t)nrows * xstride * 2);   // [wk][wr*16][nrows]
    float* inv_rms = red + (size_t)a.wk * a.wr * 16 * nrows;       // [nrows]

    // the two weight rows of this thread
    long long row_lo, row_hi;
    bool ok_lo, ok_hi;
    if (a.epi == EPI_SWIGLU) {
        const int i = (blockIdx.x * a.wr + wr) * 8 + g;
        ok_lo = ok_hi = i < a.M;
        row_lo = i;
        row_hi = a.up_off + i;
    } else {
        const int r = (blockIdx.x * a.wr + wr) * 16 + g;
        ok_lo = r < a.M;
        ok_hi = r + 8 < a.M;
        row_lo = r;
        row_hi = r + 8;
    }
    const __nv_bfloat16* wlo = a.w + row_lo * a.ldw + 8 * t;
    const __nv_bfloat16* whi = a.w + row_hi * a.ldw + 8 * t;

    float c[NBT][4];
#pragma unroll
    for (int j = 0; j < NBT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) c[j][e] = 0.f;

    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    auto load_w = [&](int unit, int unit_end, uint4& lo, uint4& hi) {
        const int k = unit * 32 + 8 * t;
        const bool in = unit < unit_end && k < a.K;
        lo = (in && ok_lo) ? ld_stream(wlo + (size_t)unit * 32) : zero4;
        hi = (in && ok_hi) ? ld_stream(whi + (size_t)unit * 32) : zero4;
    };

    for (int kc0 = 0; kc0 < a.K; kc0 += a.kc) {
        const int kc_len = min(a.kc, a.K - kc0);
        // this warp's units of the chunk
        const int units = (kc_len + 31) / 32;
        const int per = (units + a.wk - 1) / a.wk;
        const int u_begin = kc0 / 32 + wk * per;
        const int u_end = kc0 / 32 + min(units, (wk + 1) * per);
        // weights do not depend on the tokens: start streaming them before the tokens are staged
        uint4 lo[kUnroll], hi[kUnroll];
#pragma unroll
        for (int i = 0; i < kUnroll; ++i) load_w(u_begin + i, u_end, lo[i], hi[i]);

        if (kc0 == 0 && a.resid != nullptr) {
            // row statistics of the norm prologue: one pass over the stream rows (they sit in L2)
            for (int r = warp; r < nrows; r += kGemvThreads / 32) {
                float ss = 0.f;
                if (r < a.N) {
                    const float* src = a.resid + (size_t)(a.rows ? a.rows[r] : r) * a.K;
                    for (int k = lane * 4; k < a.K; k += 128) {
                        const float4 v = *reinterpret_cast<const float4*>(src + k);
                        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                    }
                }
                ss = warp_sum(ss);
                if (lane == 0) inv_rms[r] = 1.0f / sqrtf(ss / (float)a.K + a.eps);
            }
        }

        __syncthreads();   // the chunk before this one is consumed; inv_rms is visible
        const int staged = units * 32;   // whole units: what lies beyond K is zero, never left as it was
        for (int idx = tid; idx < nrows * (staged / 4); idx += kGemvThreads) {
            const int r = idx / (staged / 4), k = (idx % (staged / 4)) * 4;
            __nv_bfloat162 p0, p1;
            if (r < a.N && k < kc_len) {
                if (a.resid != nullptr) {
                    const float* src = a.resid + (size_t)(a.rows ? a.rows[r] : r) * a.K + kc0 + k;
                    const float4 v = *reinterpret_cast<const float4*>(src);
                    const float s = inv_rms[r];
                    float g0, g1, g2, g3;
                    if (a.gamma_f32) {
                        const float4 gv = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.gamma) + kc0 + k);
                        g0 = gv.x; g1 = gv.y; g2 = gv.z; g3 = gv.w;
                    } else {
                        const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(reinterpret_cast<const __nv_bfloat16*>(a.gamma) + kc0 + k);
                        const float2 ga = __bfloat1622float2(gp[0]), gb = __bfloat1622float2(gp[1]);
                        g0 = ga.x; g1 = ga.y; g2 = gb.x; g3 = gb.y;
                    }
                    p0 = __floats2bfloat162_rn(v.x * s * g0, v.y * s * g1);
                    p1 = __floats2bfloat162_rn(v.z * s * g2, v.w * s * g3);
                } else {
                    const __nv_bfloat162* src = reinterpret_cast<const __nv_bfloat162*>(a.x + (size_t)r * a.ldx + kc0 + k);
                    p0 = src[0];
                    p1 = src[1];
                }
            } else {
                p0 = p1 = __floats2bfloat162_rn(0.f, 0.f);
            }
            __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(xs + (size_t)r * xstride + k);
            dst[0] = p0;
            dst[1] = p1;
        }
        __syncthreads();

        for (int u = u_begin; u < u_end; u += kUnroll) {
            uint4 nlo[kUnroll], nhi[kUnroll];
#pragma unroll
            for (int i = 0; i < kUnroll; ++i) load_w(u + kUnroll + i, u_end, nlo[i], nhi[i]);
#pragma unroll
            for (int i = 0; i < kUnroll; ++i) {
                if (u + i < u_end) {
                    const int k = (u + i) * 32 - kc0 + 8 * t;
#pragma unroll
                    for (int j = 0; j < NBT; ++j) {
                        const uint4 xv = *reinterpret_cast<const uint4*>(xs + (size_t)(j * 8 + g) * xstride + k);
                        mma16816(c[j], lo[i].x, hi[i].x, lo[i].y, hi[i].y, xv.x, xv.y);
                        mma16816(c[j], lo[i].z, hi[i].z, lo[i].w, hi[i].w, xv.z, xv.w);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < kUnroll; ++i) { lo[i] = nlo[i]; hi[i] = nhi[i]; }
        }
    }

    // sum the k slices in a fixed order, then the epilogue
    const int tile_rows = a.wr * 16;
#pragma unroll
    for (int j = 0; j < NBT; ++j) {
        float* dst = red + ((size_t)wk * tile_rows + wr * 16) * nrows;
        dst[(size_t)g * nrows + j * 8 + 2 * t] = c[j][0];
        dst[(size_t)g * nrows + j * 8 + 2 * t + 1] = c[j][1];
        dst[(size_t)(g + 8) * nrows + j * 8 + 2 * t] = c[j][2];
        dst[(size_t)(g + 8) * nrows + j * 8 + 2 * t + 1] = c[j][3];
    }
    __syncthreads();
    auto total = [&](int r, int b) {
        float s = 0.f;
        for (int z = 0; z < a.wk; ++z) s += red[((size_t)z * tile_rows + r) * nrows + b];
        return s;
    };
    if (a.epi == EPI_SWIGLU) {
        const int outs = a.wr * 8;
        for (int idx = tid; idx < outs * a.N; idx += kGemvThreads) {
            const int b = idx / outs, o = idx % outs;
            const int i = blockIdx.x * outs + o;
            if (i < a.M) {
                const int r = (o / 8) * 16 + (o % 8);
                const float gate = total(r, b), up = total(r + 8, b);
                const float v = gate / (1.0f + expf(-gate)) * up;
                reinterpret_cast<__nv_bfloat16*>(a.y)[(size_t)b * a.ldy + i] = __float2bfloat16_rn(v);
            }
        }
    } else {
        for (int idx = tid; idx < tile_rows * a.N; idx += kGemvThreads) {
            const int b = idx / tile_rows, r = idx % tile_rows;
            const int m = blockIdx.x * tile_rows + r;
            if (m < a.M) {
                const float v = total(r, b);
                if (a.epi == EPI_RESID_ADD) a.acc[(size_t)b * a.M + m] += v;
                else if (a.y_f32) reinterpret_cast<float*>(a.y)[(size_t)b * a.ldy + m] = v;
                else reinterpret_cast<__nv_bfloat16*>(a.y)[(size_t)b * a.ldy + m] = __float2bfloat16_rn(v);
            }
        }
    }
}

// Shared memory the kernel needs for a shape, and the k chunk it picks; 0 when the shape does not fit.
static size_t gemv_plan(int N, int K, int wr, int wk, int* kc_out, int* nbt_out) {
    int nbt = 1;
    while (nbt * 8 < N) nbt *= 2;
    if (nbt > 8) return 0;
    const int nrows = nbt * 8;
    const size_t fixed = (size_t)wk * wr * 16 * nrows * 4 + (size_t)nrows * 4;
    const size_t budget = 100 * 1024;     // two blocks per SM
    int kc = (K + 31) / 32 * 32;
    while ((size_t)nrows * (kc + 8) * 2 + fixed > budget && kc > 256) kc = ((kc / 2) + 31) / 32 * 32;
    if ((size_t)nrows * (kc + 8) * 2 + fixed > 200 * 1024) return 0;
    *kc_out = kc;
    *nbt_out = nbt;
    return (size_t)nrows * (kc + 8) * 2 + fixed;
}

// 1 when blm_gemv takes the shape, else 0 (the caller then uses the library product).
BLM_API int blm_gemv_supported(int N, int M, int K) {
    int kc, nbt;
    return N >= 1 && N <= 64 && K % 8 == 0 && K >= 32 && M >= 1 && gemv_plan(N, K, 1, 8, &kc, &nbt) > 0;
}

BLM_API int blm_gemv(const void* w, long long ldw, int M, int K, long long up_off, const void* x, long long ldx,
                     const float* resid, const void* gamma, int gamma_f32, float eps, const int* rows, int N,
                     void* y, long long ldy, int y_f32, float* acc, int epi, cudaStream_t stream) {
    if (N == 0 || M == 0) return BLM_OK;
    BLM_REQUIRE(N >= 1 && N <= 64, "gemv: %d tokens (1..64)", N);
    BLM_REQUIRE(K % 8 == 0 && K >= 32, "gemv: K = %d must be a multiple of 8, at least 32", K);
    BLM_REQUIRE((x != nullptr) != (resid != nullptr), "gemv: give either x or the stream to normalise");
    BLM_REQUIRE(x == nullptr || ldx % 8 == 0, "gemv: x rows must be 16-byte aligned");
    BLM_REQUIRE(ldw % 8 == 0, "gemv: weight rows must be 16-byte aligned");
    BLM_REQUIRE(epi == EPI_STORE || epi == EPI_SWIGLU || epi == EPI_RESID_ADD, "gemv: epilogue %d", epi);
    BLM_REQUIRE(epi != EPI_RESID_ADD || acc != nullptr, "gemv: no stream to add into");
    BLM_REQUIRE(epi == EPI_RESID_ADD || y != nullptr, "gemv: no output");
    BLM_REQUIRE(resid == nullptr || K % 4 == 0, "gemv: norm prologue needs K %% 4 == 0");
    GemvArgs a;
    a.w = (const __nv_bfloat16*)w; a.ldw = ldw; a.M = M; a.K = K; a.up_off = up_off;
    a.x = (const __nv_bfloat16*)x; a.ldx = ldx; a.resid = resid; a.gamma = gamma; a.gamma_f32 = gamma_f32; a.eps = eps;
    a.rows = rows; a.N = N; a.y = y; a.ldy = ldy; a.y_f32 = y_f32; a.acc = acc; a.epi = epi;
    // blocks: enough of them to fill 148 SMs a few times over; small M takes more k slices per block
    const int out_per_tile = epi == EPI_SWIGLU ? 8 : 16;
    const int tiles = (M + out_per_tile - 1) / out_per_tile;
    int wr = 1;
    while (wr < 8 && tiles / (wr * 2) >= 2 * 148) wr *= 2;
    a.wr = wr; a.wk = 8 / wr;
    int nbt;
    const size_t smem = gemv_plan(N, K, a.wr, a.wk, &a.kc, &nbt);
    BLM_REQUIRE(smem > 0, "gemv: the shape N=%d K=%d does not fit shared memory", N, K);
    const int grid = (tiles + wr - 1) / wr;
    auto launch = [&](auto kernel) -> int {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "gemv: %s", cudaGetErrorString(e));
        }
        kernel<<<grid, kGemvThreads, smem, stream>>>(a);
        return blm_check_launch("gemv");
    };
    switch (nbt) {
        case 1: return launch(gemv_kernel<1>);
        case 2: return launch(gemv_kernel<2>);
        case 4: return launch(gemv_kernel<4>);
        default: return launch(gemv_kernel<8>);
    }
}
