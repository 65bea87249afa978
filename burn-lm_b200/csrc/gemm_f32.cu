// y[N, M] = x[N, K] . W[M, K]^T in true fp32: FFMA on CUDA cores, no tensor-core mode of any kind.
// This is the matrix product of the 32-bit path; it is slow on purpose of being exact: the sum over
// K runs in one fixed order that depends on neither N nor M, so a token's result is the same
// whatever else is in the batch.
#include "common.cuh"

BLM_API const char* blm_gemm_last_error() { return g_blm_error; }

constexpr int BM = 64, BN = 64, BK = 16;

__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                       float* __restrict__ y, int N, int M, int K,
                                                       long long ldx, long long ldw, long long ldy) {
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int n0 = blockIdx.y * BM, m0 = blockIdx.x * BN;
    const int tn = (tid / 16) * 4, tm = (tid % 16) * 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 x 16 elements of each operand, 4 per thread; consecutive threads walk K (coalesced)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            const int r = idx / BK, c = idx % BK;
            const int k = k0 + c;
            xs[c][r] = (n0 + r < N && k < K) ? x[(size_t)(n0 + r) * ldx + k] : 0.f;
            ws[c][r] = (m0 + r < M && k < K) ? w[(size_t)(m0 + r) * ldw + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(&xs[k][tn]);
            const float4 b = *reinterpret_cast<const float4*>(&ws[k][tm]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (n0 + tn + i < N && m0 + tm + j < M) y[(size_t)(n0 + tn + i) * ldy + m0 + tm + j] = acc[i][j];
}

BLM_API int blm_gemm_f32(const float* x, const float* w, float* y, int N, int M, int K,
                         long long ldx, long long ldw, long long ldy, cudaStream_t stream) {
    if (N == 0 || M == 0) return BLM_OK;
    BLM_REQUIRE(N > 0 && M > 0 && K > 0, "gemm_f32: bad sizes %d %d %d", N, M, K);
    const dim3 grid((M + BN - 1) / BN, (N + BM - 1) / BM);
    BLM_REQUIRE(grid.y <= 65535, "gemm_f32: too many rows (%d)", N);
    gemm_f32_kernel<<<grid, 256, 0, stream>>>(x, w, y, N, M, K, ldx, ldw, ldy);
    return blm_check_launch("gemm_f32");
}
