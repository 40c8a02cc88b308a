// Block-scaled fp8 GEMM on the 5th-generation tensor cores:
//     C[M,N] = sum over 128-deep K blocks b of  sa[m,b] * sw[n,b] * (A8[m, b] . W8[n, b])
// A8 / W8 are fp8 e4m3; sa holds one fp32 scale per (row, 128 columns) of the activation (1 x 128
// quantisation, produced by pie_quant_act_fp8), sw one per (row, 128 columns) of the weight
// (128 x 128 checkpoint blocks expanded to rows when the weight is loaded).
//
// One CTA per 128 x BN output tile, persistent over tiles:
//   warp 0      TMA producer: per K block one 128 x 128-byte tile of A8 and one bn x 128-byte tile
//               of W8 (128-byte swizzle) into a ring of slots
//   warp 1      four tcgen05.mma.kind::f8f6f4 (K = 32 each) per K block into one of two TMEM
//               buffers, starting from zero each block; tcgen05.commit frees the ring slot and
//               publishes the block's partial product
//   warps 2-5   read the partial product from TMEM, scale it by sa * sw and add it to fp32
//               accumulators in registers (one output row per thread); after the last block the
//               usual epilogue (store / +residual / SwiGLU) writes bf16
// The per-block rescale in registers is what block scaling costs; the MMAs of block b+1 overlap it
// through the second TMEM buffer. Every wait is bounded (status word, drain, TMEM freed).
//
// Replaces the reference's dequantise-to-bf16 kernel followed by a library GEMM for block-scaled
// fp8 weights (driver/cuda/src/ops/gemm.cpp:1166-1211, driver/cuda/src/kernels/dequant_fp8.cu:41).
#include <cuda_fp8.h>

#include "gemm_common.cuh"

namespace pie {
using namespace sm100;

constexpr int F8_BK = 128;   // fp8 elements (= bytes) per K block: one swizzle span

template <int BN>
struct Fp8Cfg {
    static constexpr uint32_t A_BYTES = GEMM_BM * F8_BK;
    static constexpr uint32_t B_BYTES = BN * F8_BK;
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = BN == 128 ? 5 : 7;
    static constexpr uint32_t TMEM_COLS = 2 * BN;
    static constexpr uint32_t SCALE_BYTES = 4 * 2 * BN * 4;   // per epilogue warp: weight scales of the block being folded, double-buffered
    static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + SCALE_BYTES + 16384;
};

// Instruction descriptor, kind::f8f6f4: e4m3 x e4m3 -> fp32, both operands K-major.
//   [4,6) D format (1 = f32)  [7,10) A format (0 = e4m3)  [10,13) B format (0 = e4m3)
//   [17,23) N >> 3  [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc_e4m3(int m, int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
template <int BN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                const float* __restrict__ sa, const float* __restrict__ sw, bf16* __restrict__ C,
                const bf16* __restrict__ R, int M, int N, int K, int ldc, int ldr, int* status, int bn,
                const __grid_constant__ TpArgs tp) {
    using Cfg = Fp8Cfg<BN>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_addr(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    uint8_t* tiles_ptr = smem_raw + (tiles - raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles_ptr + STAGES * Cfg::STAGE_BYTES);
    const uint32_t bar0 = tiles + STAGES * Cfg::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2 * STAGES + 4);
    float* sw_s = reinterpret_cast<float*>(tiles_ptr + STAGES * Cfg::STAGE_BYTES + 256);          // [4 warps][2][BN]
    uint8_t* stage_base = tiles_ptr + STAGES * Cfg::STAGE_BYTES + 256 + Cfg::SCALE_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
    const int tiles_n = (N + bn - 1) / bn;
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (K + F8_BK - 1) / F8_BK;
    const uint32_t stage_tx = Cfg::A_BYTES + (uint32_t)bn * F8_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 4);
        }
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        tmem_alloc(smem_addr(const_cast<uint32_t*>(tmem_slot)), Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&tma_a);
            tma_prefetch_desc(&tma_b);
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int m_blk = tile % tiles_m, n_blk = tile / tiles_m;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, status, PIE_ERR_WAIT_TMA)) { ok = false; break; }
                    mbar_arrive_expect_tx(full_bar(s), stage_tx);
                    const uint32_t dst = tiles + s * Cfg::STAGE_BYTES;
                    tma_load_2d(dst, &tma_a, full_bar(s), kb * F8_BK, m_blk * GEMM_BM);
                    tma_load_2d(dst + Cfg::A_BYTES, &tma_b, full_bar(s), kb * F8_BK, n_blk * bn);
                }
            }
            const uint32_t first = it > (uint32_t)STAGES ? it - STAGES : 0u;
            for (uint32_t j = first; j < it; ++j)
                mbar_wait(full_bar(j % STAGES), (j / STAGES) & 1u, status, PIE_ERR_WAIT_TMA, 200000000ll);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc_e4m3(GEMM_BM, bn);
            uint32_t it = 0;      // counts K blocks = TMEM buffer uses
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t buf = it & 1u, bph = (it >> 1) & 1u;
                    if (!mbar_wait(tempty_bar(buf), bph ^ 1u, status, PIE_ERR_WAIT_EPILOGUE)) { ok = false; break; }
                    if (!mbar_wait(full_bar(s), (it / STAGES) & 1u, status, PIE_ERR_WAIT_TMA)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = tiles + s * Cfg::STAGE_BYTES;
                    const uint64_t adesc = make_smem_desc_sw128(a_addr);
                    const uint64_t bdesc = make_smem_desc_sw128(a_addr + Cfg::A_BYTES);
                    const uint32_t d_tmem = tmem_base + buf * BN;
#pragma unroll
                    for (int k = 0; k < F8_BK / 32; ++k)
                        umma_f8(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, k != 0);
                    umma_commit(empty_bar(s));
                    umma_commit(tfull_bar(buf));
                }
            }
        }
    } else {
        // accumulate + epilogue: 128 threads, thread = one output row of the tile
        const int q = warp & 3;
        float* sw_w = sw_s + (warp - 2) * 2 * BN;      // this warp's copy: no barrier across warps is needed
        uint32_t it = 0;
        bool ok = true;
        const int kbs = (K + 127) / 128;       // columns of the scale tables
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            const int m_blk = tile % tiles_m, n_blk = tile / tiles_m;
            const int row = m_blk * GEMM_BM + q * 32 + lane;
            const int n0 = n_blk * bn;
            float acc[BN];
#pragma unroll
            for (int c = 0; c < BN; ++c) acc[c] = 0.f;
            // scales of the next K block are fetched one block ahead (global latency hidden behind
            // the wait for the MMAs and the fold of the current block); lane l keeps the weight
            // scales of columns l, l+32, ... in registers and hands them to its warp through smem
            constexpr int SPL = BN / 32;
            float sw_n[SPL], sa_n;
            auto fetch = [&](int kb) {
#pragma unroll
                for (int u = 0; u < SPL; ++u) {
                    const int c = u * 32 + lane;
                    sw_n[u] = (c < bn && n0 + c < N) ? __ldg(sw + (size_t)(n0 + c) * kbs + kb) : 0.f;
                }
                sa_n = row < M ? __ldg(sa + (size_t)row * kbs + kb) : 0.f;
            };
            fetch(0);
            for (int kb = 0; kb < num_kb; ++kb, ++it) {
                const uint32_t buf = it & 1u, bph = (it >> 1) & 1u;
                float* sws = sw_w + buf * BN;
#pragma unroll
                for (int u = 0; u < SPL; ++u) sws[u * 32 + lane] = sw_n[u];
                const float sa_r = sa_n;
                if (kb + 1 < num_kb) fetch(kb + 1);
                __syncwarp();
                const bool got = mbar_wait(tfull_bar(buf), bph, status, PIE_ERR_WAIT_MMA);
                if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
                tc_fence_after();
                const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
#pragma unroll
                for (int c = 0; c < BN / 32; ++c) {
                    if (c * 32 < bn) {
                        uint32_t v[32];
                        tmem_ld_32x32(t_row + c * 32, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            acc[c * 32 + j] = fmaf(__uint_as_float(v[j]), sa_r * sws[c * 32 + j], acc[c * 32 + j]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty_bar(buf));
            }
            if (!ok) break;
            uint8_t* stage = stage_base + (warp - 2) * 4096;
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) {
                if (c * 64 < bn) {
                    uint32_t v0[32], v1[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        v0[j] = __float_as_uint(acc[c * 64 + j]);
                        v1[j] = __float_as_uint(acc[c * 64 + 32 + j]);
                    }
                    epilogue_store_64<EPI>(v0, v1, stage, m_blk * GEMM_BM + q * 32, n0 + c * 64, M, N, C, ldc, R, ldr,
                                           tp, min(N, n0 + bn));
                }
            }
            if (EPI == EPI_RS) {
                // this warp's rows of the tile are in the owners' receive buffers: count the arrival
                __threadfence_system();
                __syncwarp();
                if (lane == 0) rs_publish_arrival(tp, num_tiles * 4);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// 1 x 128 activation quantisation: one warp per (row, 128-column block).
__global__ void quant_act_fp8_kernel(const bf16* __restrict__ x, int ldx, uint8_t* __restrict__ x8, float* __restrict__ sx,
                                     int M, int K) {
    const int kbs = (K + 127) / 128;
    const long gw = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (gw >= (long)M * kbs) return;
    const int row = (int)(gw / kbs), kb = (int)(gw - (long)row * kbs);
    const int c = kb * 128 + lane * 4;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (c < K) {
        const uint2 raw = *reinterpret_cast<const uint2*>(x + (size_t)row * ldx + c);
        const bf162* p = reinterpret_cast<const bf162*>(&raw);
        const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = warp_max(amax);
    const float scale = fmaxf(amax, 1e-12f) / 448.f;
    const float inv = 1.f / scale;
    if (c < K) {
        const __nv_fp8x4_storage_t q4 = __nv_cvt_float2_to_fp8x2(make_float2(v[0] * inv, v[1] * inv), __NV_SATFINITE, __NV_E4M3) |
                                        ((uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(v[2] * inv, v[3] * inv), __NV_SATFINITE, __NV_E4M3) << 16);
        *reinterpret_cast<uint32_t*>(x8 + (size_t)row * K + c) = q4;
    }
    if (lane == 0) sx[(size_t)row * kbs + kb] = scale;
}

}  // namespace pie

using namespace pie;

extern "C" int pie_make_tma_2d_bf16(CUtensorMap* map, const void* ptr, long rows, long cols, long ld, int box_rows);

typedef CUresult (*EncodeTiledFn8)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 2-D uint8 row-major [rows, cols]; box = box_rows x 128 bytes with the 128-byte swizzle.
static int make_tma_2d_u8(CUtensorMap* map, const void* ptr, long rows, long cols, long ld, int box_rows) {
    static EncodeTiledFn8 enc = nullptr;
    if (!enc) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return -1;
        enc = reinterpret_cast<EncodeTiledFn8>(p);
    }
    if (((uintptr_t)ptr & 15) || ld % 16) return -2;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld};
    cuuint32_t box[2] = {(cuuint32_t)F8_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return (int)enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
}

// x [M, K] bf16 -> x8 [M, K] e4m3 (dense, leading dimension K) and sx [M, ceil(K/128)].
PIE_API int pie_quant_act_fp8(const void* x, int ldx, void* x8, float* sx, int M, int K, cudaStream_t st) {
    if (M <= 0) return 0;
    if (K % 16 || ldx % 4) return (int)cudaErrorInvalidValue;
    const long warps = (long)M * ((K + 127) / 128);
    const int blocks = (int)((warps * 32 + 255) / 256);
    quant_act_fp8_kernel<<<blocks, 256, 0, st>>>((const bf16*)x, ldx, (uint8_t*)x8, sx, M, K);
    return (int)cudaGetLastError();
}

// C[M,N] (or [M,N/2] with SwiGLU) from fp8 operands and their scales (see the header comment).
static int gemm_fp8_launch(const void* A8, const float* sa, const void* W8, const float* sw, void* C,
                           const void* R, int M, int N, int K, int ldc, int ldr, int epilogue, int* status,
                           int num_sms, cudaStream_t st, const TpArgs& tp);

PIE_API int pie_gemm_fp8_blockscaled(const void* A8, const float* sa, const void* W8, const float* sw, void* C,
                                     const void* R, int M, int N, int K, int ldc, int ldr, int epilogue, int* status,
                                     int num_sms, cudaStream_t st) {
    if (epilogue == EPI_RS) return (int)cudaErrorInvalidValue;
    return gemm_fp8_launch(A8, sa, W8, sw, C, R, M, N, K, ldc, ldr, epilogue, status, num_sms, st, TpArgs{});
}

// Tensor-parallel form: with EPI_RS every output row goes to its owner rank's receive buffer
// (`tp_blob` = the communicator's TpArgs, rows_per_rank rows per owner), as in pie_gemm_bf16_tp.
PIE_API int pie_gemm_fp8_blockscaled_tp(const void* A8, const float* sa, const void* W8, const float* sw, void* C,
                                        int M, int N, int K, int ldc, int epilogue, const void* tp_blob,
                                        int rows_per_rank, int* status, int num_sms, cudaStream_t st) {
    TpArgs tp = *reinterpret_cast<const TpArgs*>(tp_blob);
    tp.rows_per_rank = rows_per_rank;
    tp.gated = 0;
    if (epilogue == EPI_RS && (rows_per_rank % 32 || rows_per_rank <= 0)) return (int)cudaErrorInvalidValue;
    return gemm_fp8_launch(A8, sa, W8, sw, C, nullptr, M, N, K, ldc, 0, epilogue, status, num_sms, st, tp);
}

static int gemm_fp8_launch(const void* A8, const float* sa, const void* W8, const float* sw, void* C,
                           const void* R, int M, int N, int K, int ldc, int ldr, int epilogue, int* status,
                           int num_sms, cudaStream_t st, const TpArgs& tp) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 16 || N % 16 || (epilogue != EPI_RS && ldc % 8) || (epilogue == EPI_RESIDUAL && ldr % 8))
        return (int)cudaErrorInvalidValue;
    if (epilogue == EPI_SWIGLU && N % 32) return (int)cudaErrorInvalidValue;
    const int tm = (M + GEMM_BM - 1) / GEMM_BM;
    // tile width: the widest of {128, 112, ..., 16} whose tile count fills its waves best
    int bn = 128;
    double best = 1e30;
    for (int cand = 128; cand >= 16; cand -= 16) {
        const long tiles = (long)tm * ((N + cand - 1) / cand);
        const long waves = (tiles + num_sms - 1) / num_sms;
        const double cost = (double)waves * (cand + 24);
        if (cost < best) { best = cost; bn = cand; }
    }
    const int bt = bn <= 64 ? 64 : 128;
    CUtensorMap ta, tb;
    if (make_tma_2d_u8(&ta, A8, M, K, K, GEMM_BM) != 0) return (int)cudaErrorInvalidValue;
    if (make_tma_2d_u8(&tb, W8, N, K, K, bn) != 0) return (int)cudaErrorInvalidValue;
    const long tiles = (long)tm * ((N + bn - 1) / bn);
    const int grid = (int)(tiles < num_sms ? tiles : num_sms);
#define GO(BN_, EPI_)                                                                                         \
    {                                                                                                         \
        auto kern = gemm_fp8_kernel<BN_, EPI_>;                                                               \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,               \
                                             (int)Fp8Cfg<BN_>::SMEM_BYTES);                                   \
        if (e != cudaSuccess) return (int)e;                                                                  \
        kern<<<grid, GEMM_THREADS, Fp8Cfg<BN_>::SMEM_BYTES, st>>>(ta, tb, sa, sw, (bf16*)C, (const bf16*)R, M, N, K, \
                                                                  ldc, ldr, status, bn, tp);                  \
        return (int)cudaGetLastError();                                                                       \
    }
#define GOE(BN_)                                                  \
    switch (epilogue) {                                           \
        case EPI_STORE: GO(BN_, EPI_STORE)                        \
        case EPI_RESIDUAL: GO(BN_, EPI_RESIDUAL)                  \
        case EPI_SWIGLU: GO(BN_, EPI_SWIGLU)                      \
        case EPI_RS: GO(BN_, EPI_RS)                              \
        default: return (int)cudaErrorInvalidValue;               \
    }
    if (bt == 128) { GOE(128) } else { GOE(64) }
#undef GOE
#undef GO
    return (int)cudaErrorInvalidValue;
}
