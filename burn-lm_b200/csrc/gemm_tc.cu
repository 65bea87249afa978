// Matrix product for prompts on the 5th-generation tensor cores: y[M, N] = x[M, K] . W[N, K]^T, bf16
// operands, fp32 accumulation in tensor memory, with the gated activation or the addition into the fp32
// residual stream fused into the epilogue.
//
// Persistent blocks, one per SM, walk 128 x 256 tiles of y.  Warp 0 (one thread) is the producer: TMA
// tile loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of 128 x 64 of x and 256 x 64 of W per stage
// into a ring of four stages, completion on mbarriers.  Warp 1 allocates all 512 columns of tensor
// memory (two accumulators) and (one thread) issues tcgen05.mma.cta_group::1.kind::f16 (M 128, N 256,
// K 16) four times per stage from shared-memory descriptors; tcgen05.commit frees the stage when the
// tensor core has read it.  Warps 2..5 are the epilogue: when a tile's last commit lands they read its
// accumulator with tcgen05.ld (a warp reads the 32 lanes of its quarter, 16 columns at a time) and
// store bf16, while the tensor core already fills the other accumulator with the next tile; for a fused
// [gate; up] weight laid out in tiles of 8 gate rows followed by their 8 up rows, 16 columns are
// exactly 8 gates and their 8 ups, so silu(gate) * up is formed in registers and the [M, 2 I]
// intermediate never exists; with the stream epilogue the product is added into an fp32 [M, N] matrix in place
// (one writer per element), so a prompt step's output and down products need no bf16 round trip.  Edges: the TMA fills what lies outside x or W with zeros, the epilogue
// stores only what lies inside y.
//
// Every mbarrier wait is bounded; a wait that runs out records a code in the caller's status word and
// the block goes on to its end, where the tensor memory is given back.
#include <cuda.h>

#include <map>
#include <tuple>

#include "common.cuh"

BLM_API const char* blm_gemm_tc_last_error() { return g_blm_error; }

namespace {

constexpr int BM = 128, BN = 256, BK = 64;      // block tile; BK bf16 = 128 bytes = one swizzle row
constexpr int kStages = 4;
constexpr int kThreads = 192;                   // producer warp, mma warp, 4 epilogue warps
constexpr int kTmemCols = 512;                  // two fp32 accumulators of 256 columns: one per output column
constexpr unsigned kABytes = BM * BK * 2, kBBytes = BN * BK * 2;
constexpr unsigned kSpinLimit = 1u << 22;

enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_RESID_ADD = 2 };
enum { TC_OK = 0, TC_TIMEOUT_FULL = 11, TC_TIMEOUT_EMPTY = 12, TC_TIMEOUT_ACCUM = 13, TC_TIMEOUT_DRAIN = 14 };

struct TcArgs {
    __nv_bfloat16* y;
    long long ldy;
    float* acc;         // EPI_RESID_ADD: fp32 [M, N] (row stride ldy), the product is added into it
    int M, N, K;        // N: rows of W
    int epi;
    int* status;
};

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
    {   // a phase that is over already answers at once (the blocking form takes some hundred cycles even then)
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
// shared-memory operand descriptor: K-major tile of rows of 128 bytes, 128-byte swizzle; 8-row groups
// 1024 bytes apart
__device__ __forceinline__ unsigned long long umma_desc(const void* tile) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_u32(tile) >> 4) & 0x3fff);      // start address
    d |= (unsigned long long)1 << 16;                               // leading byte offset (unused with a swizzle)
    d |= (unsigned long long)(1024 >> 4) << 32;                     // stride byte offset
    d |= (unsigned long long)1 << 46;                               // descriptor version of this architecture
    d |= (unsigned long long)2 << 61;                               // 128-byte swizzle
    return d;
}
// instruction descriptor of kind::f16: fp32 accumulator, bf16 x bf16, both K-major, M 128, N 256
constexpr unsigned kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);

__device__ __forceinline__ void umma(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc, unsigned accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(kIdesc), "r"(accumulate)
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

// Stores 16 accumulator columns of one row: plain (16 outputs), gated (8 gates and their 8 ups -> 8 outputs), or
// added into the fp32 stream.  The end is a parameter of the kernel: each variant carries only its own code.
template <int EPI>
__device__ __forceinline__ void store_columns(const TcArgs& a, const float (&v)[16], int row, int n0, int j) {
    if (row >= a.M) return;
    if (EPI == EPI_RESID_ADD) {
        const int c0 = n0 + j * 16;
        if (c0 >= a.N) return;
        float* dst = a.acc + (size_t)row * a.ldy + c0;
        if (c0 + 16 <= a.N && ((a.ldy & 3) == 0)) {
            // all loads first
            const float4 o0 = reinterpret_cast<const float4*>(dst)[0], o1 = reinterpret_cast<const float4*>(dst)[1];
            const float4 o2 = reinterpret_cast<const float4*>(dst)[2], o3 = reinterpret_cast<const float4*>(dst)[3];
            reinterpret_cast<float4*>(dst)[0] = make_float4(o0.x + v[0], o0.y + v[1], o0.z + v[2], o0.w + v[3]);
            reinterpret_cast<float4*>(dst)[1] = make_float4(o1.x + v[4], o1.y + v[5], o1.z + v[6], o1.w + v[7]);
            reinterpret_cast<float4*>(dst)[2] = make_float4(o2.x + v[8], o2.y + v[9], o2.z + v[10], o2.w + v[11]);
            reinterpret_cast<float4*>(dst)[3] = make_float4(o3.x + v[12], o3.y + v[13], o3.z + v[14], o3.w + v[15]);
        } else {
            for (int e = 0; e < 16 && c0 + e < a.N; ++e) dst[e] += v[e];
        }
        return;
    }
    if (EPI == EPI_SWIGLU) {
        const int inner = a.N >> 1, o0 = (n0 >> 1) + j * 8;
        if (o0 >= inner) return;
        unsigned packed[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float g0 = v[2 * e], g1 = v[2 * e + 1], u0 = v[8 + 2 * e], u1 = v[8 + 2 * e + 1];
            const __nv_bfloat162 p = __floats2bfloat162_rn(g0 / (1.0f + expf(-g0)) * u0, g1 / (1.0f + expf(-g1)) * u1);
            packed[e] = *reinterpret_cast<const unsigned*>(&p);
        }
        __nv_bfloat16* dst = a.y + (size_t)row * a.ldy + o0;
        if (o0 + 8 <= inner && ((a.ldy & 7) == 0)) {
            *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        } else {
            const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(packed);
            for (int e = 0; e < 8 && o0 + e < inner; ++e) dst[e] = src[e];
        }
    } else {
        const int c0 = n0 + j * 16;
        if (c0 >= a.N) return;
        unsigned packed[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const __nv_bfloat162 p = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
            packed[e] = *reinterpret_cast<const unsigned*>(&p);
        }
        __nv_bfloat16* dst = a.y + (size_t)row * a.ldy + c0;
        if (c0 + 16 <= a.N && ((a.ldy & 7) == 0)) {
            reinterpret_cast<uint4*>(dst)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            reinterpret_cast<uint4*>(dst)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        } else {
            const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(packed);
            for (int e = 0; e < 16 && c0 + e < a.N; ++e) dst[e] = src[e];
        }
    }
}

template <int EPI>
__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(const TcArgs a, const __grid_constant__ CUtensorMap xmap,
                                                              const __grid_constant__ CUtensorMap wmap) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* As = smem;                                  // [kStages][BM][128 bytes]
    unsigned char* Bs = smem + kStages * kABytes;              // [kStages][BN][128 bytes]
    unsigned long long* full = reinterpret_cast<unsigned long long*>(Bs + kStages * kBBytes);
    unsigned long long* empty = full + kStages;
    unsigned long long* acc_full = empty + kStages;            // [2] the tensor core has finished an accumulator
    unsigned long long* acc_empty = acc_full + 2;              // [2] the epilogue has read it
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (a.M + BM - 1) / BM, n_tiles = (a.N + BN - 1) / BN;
    const int tiles = m_tiles * n_tiles;
    const int k_iters = (a.K + BK - 1) / BK;
    // tile t: rows (t % m_tiles), columns (t / m_tiles): the blocks that run together share W tiles in L2

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full + b, 1);
            mbar_init(acc_empty + b, 4);       // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        // tensor memory for the accumulators: the whole warp asks, the address lands in shared memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const unsigned tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- producer ----------------
            unsigned it = 0;        // stages issued so far, over all tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
                for (int k = 0; k < k_iters; ++k, ++it) {
                    const int s = it % kStages;
                    if (it >= (unsigned)kStages && !mbar_wait(empty + s, ((it / kStages) - 1) & 1)) {
                        atomicCAS(a.status, TC_OK, TC_TIMEOUT_EMPTY);
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(full + s, kABytes + kBBytes);
                    tma_load_2d(As + s * kABytes, &xmap, k * BK, m0, full + s);
                    tma_load_2d(Bs + s * kBBytes, &wmap, k * BK, n0, full + s);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- tensor core ----------------
            unsigned it = 0;
            int n_tile = 0;
            bool ok = true;
            // operand descriptors: the address field counts 16 bytes, so a stage further is an addition
            const unsigned long long a_desc = umma_desc(As), b_desc = umma_desc(Bs);
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++n_tile) {
                const int b = n_tile & 1;
                if (n_tile >= 2 && !mbar_wait(acc_empty + b, ((n_tile >> 1) - 1) & 1)) {      // the epilogue has read this accumulator
                    atomicCAS(a.status, TC_OK, TC_TIMEOUT_DRAIN);
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned tmem_d = tmem_base + (unsigned)(b * BN);
                for (int k = 0; k < k_iters; ++k, ++it) {
                    const int s = it % kStages;
                    if (!mbar_wait(full + s, (it / kStages) & 1)) {
                        atomicCAS(a.status, TC_OK, TC_TIMEOUT_FULL);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const unsigned long long ad = a_desc + (unsigned)(s * (kABytes >> 4)), bd = b_desc + (unsigned)(s * (kBBytes >> 4));
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk)      // 16 bf16 = 32 bytes further along the swizzled row: +2 in the address field
                        umma(tmem_d, ad + 2 * kk, bd + 2 * kk, (k > 0 || kk > 0) ? 1u : 0u);
                    umma_commit(empty + s);                   // the stage is free when these products have read it
                }
                umma_commit(acc_full + b);                    // the accumulator is complete when everything issued is done
            }
        }
    } else {
        // ---------------- epilogue: warp w reads lanes 32 (w % 4) .. of the accumulators ----------------
        const int quarter = warp & 3;
        int n_tile = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++n_tile) {
            const int b = n_tile & 1;
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
            if (!mbar_wait(acc_full + b, (n_tile >> 1) & 1)) {
                if (lane == 0) atomicCAS(a.status, TC_OK, TC_TIMEOUT_ACCUM);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(b * BN);
            const int row = m0 + quarter * 32 + lane;
#pragma unroll 1
            for (int j = 0; j < BN / 16; ++j) {
                float v[16];
                tmem_ld16(taddr + j * 16, v);
                store_columns<EPI>(a, v, row, n0, j);
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + b);        // this warp has read its quarter
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The TMA's view of a K-major bf16 matrix [rows, K] (row stride ld): boxes of box_rows x 64, 128-byte swizzle.
int make_map(const void* base, long long ld, int rows, int K, int box_rows, bool cache, CUtensorMap* out) {
    static EncodeTiledFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
            return blm_fail(BLM_CUDA_ERROR, "gemm_tc: the driver has no cuTensorMapEncodeTiled");
        encode = (EncodeTiledFn)fn;
    }
    static std::map<std::tuple<const void*, long long, int, int, int>, CUtensorMap> maps;
    const auto key = std::make_tuple(base, ld, rows, K, box_rows);
    if (cache) {
        auto it = maps.find(key);
        if (it != maps.end()) {
            *out = it->second;
            return BLM_OK;
        }
    }
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return blm_fail(BLM_CUDA_ERROR, "gemm_tc: cuTensorMapEncodeTiled failed (%d)", (int)r);
    if (cache) {
        if (maps.size() > 4096) maps.clear();
        maps.emplace(key, *out);
    }
    return BLM_OK;
}

}  // namespace

// 1 when blm_gemm_tc takes the shape
BLM_API int blm_gemm_tc_supported(int M, int N, int K) { return M >= 1 && N >= 16 && K >= 64 && K % 8 == 0; }

// y[M, N] = x[M, K] . w[N, K]^T (epi 0), or y[M, N / 2] = silu(gate) * up for a weight in tiles of 8 gate rows
// followed by their 8 up rows (epi 1), or y[M, N] += x . w^T with y fp32 (epi 2: the residual stream).  x, w
// bfloat16, y bfloat16 but for epi 2; ldx, ldw, ldy in elements.
BLM_API int blm_gemm_tc(const void* x, long long ldx, const void* w, long long ldw, void* y, long long ldy, int M, int N, int K,
                        int epi, int* status, cudaStream_t stream) {
    if (M == 0 || N == 0) return BLM_OK;
    BLM_REQUIRE(blm_gemm_tc_supported(M, N, K), "gemm_tc: shape %d x %d x %d (K a multiple of 8, at least 64)", M, N, K);
    BLM_REQUIRE(ldx % 8 == 0 && ldw % 8 == 0 && ((size_t)x & 15) == 0 && ((size_t)w & 15) == 0,
                "gemm_tc: operand rows must be 16-byte aligned");
    BLM_REQUIRE(epi == EPI_STORE || epi == EPI_RESID_ADD || (epi == EPI_SWIGLU && N % 16 == 0), "gemm_tc: epilogue %d with %d weight rows", epi, N);
    BLM_REQUIRE(epi != EPI_RESID_ADD || ((size_t)y & 15) == 0, "gemm_tc: the stream must be 16-byte aligned");
    BLM_REQUIRE(status != nullptr, "gemm_tc: no status word");
    CUtensorMap xmap, wmap;
    int rc = make_map(x, ldx, M, K, BM, false, &xmap);
    if (rc != BLM_OK) return rc;
    rc = make_map(w, ldw, N, K, BN, true, &wmap);
    if (rc != BLM_OK) return rc;
    TcArgs a;
    a.y = (__nv_bfloat16*)y; a.acc = (float*)y; a.ldy = ldy; a.M = M; a.N = N; a.K = K; a.epi = epi; a.status = status;
    const size_t smem = (size_t)kStages * (kABytes + kBBytes) + (2 * kStages + 4) * 8 + 16 + 1024;
    static bool opted_in = false;
    if (!opted_in) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<EPI_STORE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_kernel<EPI_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_kernel<EPI_RESID_ADD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return blm_fail(BLM_CUDA_ERROR, "gemm_tc: %s", cudaGetErrorString(e));
        opted_in = true;
    }
    const long long tiles = (long long)((N + BN - 1) / BN) * ((M + BM - 1) / BM);
    const int grid = (int)(tiles < blm_sm_count() ? tiles : blm_sm_count());        // persistent: one block per SM
    if (epi == EPI_SWIGLU) gemm_tc_kernel<EPI_SWIGLU><<<grid, kThreads, smem, stream>>>(a, xmap, wmap);
    else if (epi == EPI_RESID_ADD) gemm_tc_kernel<EPI_RESID_ADD><<<grid, kThreads, smem, stream>>>(a, xmap, wmap);
    else gemm_tc_kernel<EPI_STORE><<<grid, kThreads, smem, stream>>>(a, xmap, wmap);
    return blm_check_launch("gemm_tc");
}
