// bf16 GEMM on the 5th-generation tensor cores:  C[M,N] = A[M,K] * W[N,K]^T.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer: 128x64 A tiles and BNx64 W tiles (128-byte swizzle)
//               into a STAGES-deep shared-memory ring, completion on mbarriers
//   warp 1      allocates TMEM and issues tcgen05.mma (128 x BN x 16) from one
//               thread; tcgen05.commit frees ring slots and publishes accumulators
//   warps 2-5   epilogue: tcgen05.ld of the fp32 accumulator (two accumulator
//               stages in TMEM, so the next tile's MMAs overlap this store),
//               optional fused residual add or SwiGLU, bf16 store
// Every mbarrier wait is bounded; on a time-out the kernel records a status
// word, drains its copies, frees TMEM and returns.
//
// Replaces the reference's cuBLASLt/cuBLAS dispatch
// (driver/cuda/src/ops/gemm.cpp:326-415, 607-640) and its separate
// residual-add / SwiGLU passes (driver/cuda/src/kernels/swiglu.cu:180-260).
#include <algorithm>

#include "gemm_common.cuh"

namespace pie {
using namespace sm100;

constexpr int GEMM_KSUB = 1;                       // 64-column sub-tiles per ring slot (2 measured no faster)
constexpr int GEMM_KSTEP = GEMM_BK * GEMM_KSUB;    // K covered by one ring slot

// OCC = CTAs per SM the instantiation is sized for. Two per SM (half the ring each) lets one
// CTA's prologue, fix-up and epilogue overlap the other's streaming; it pays for skinny problems
// where those fixed parts are a large share of a CTA's life.
template <int BN, int OCC = 1>
struct GemmCfg {
    // one ring slot holds KSUB consecutive 64-column sub-tiles of each operand (one swizzle span
    // each), so a barrier round trip and a commit cover KSUB * 4 MMAs
    static constexpr int KSUB = GEMM_KSUB;
    static constexpr uint32_t A_SUB = GEMM_BM * GEMM_BK * 2;
    static constexpr uint32_t B_SUB = BN * GEMM_BK * 2;
    static constexpr uint32_t A_BYTES = KSUB * A_SUB;
    static constexpr uint32_t B_BYTES = KSUB * B_SUB;
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (BN == 256 ? 4 : (BN == 128 ? 6 : 8)) / OCC / KSUB;
    static constexpr uint32_t TMEM_COLS = 2 * BN;
    static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ + 16384 /*epilogue staging*/;
};

// BN is the widest tile the instantiation has room for (ring slots, TMEM columns); the launch
// picks the actual width bn <= BN, a multiple of 16, so that the tile count fills the machine's
// waves; the W tensor map's box has bn rows.
// GROUPED: mixture-of-experts form. A holds token rows sorted by expert in 128-row tiles,
// tile_expert[m_tile] names the expert whose weights ([E*N, K] under tma_b) the tile multiplies,
// or -1 for an unused tile, which every role skips. Whole-tile scheduling only.
template <int BN, int EPI, bool GROUPED = false, int OCC = 1>
__global__ void __launch_bounds__(GEMM_THREADS, OCC)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 bf16* __restrict__ C, const bf16* __restrict__ R, int M, int N, int K, int ldc,
                 int ldr, int* status, const __grid_constant__ TpArgs tp, const StreamKArgs sk,
                 const int* __restrict__ tile_expert, int bn) {
    using Cfg = GemmCfg<BN, OCC>;
    constexpr int STAGES = Cfg::STAGES;
    constexpr bool SWAPPED = EPI >= EPI_STORE_T;   // tma_a walks the weights, tma_b the activation
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

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
    const int tiles_n = (N + bn - 1) / bn;
    const int num_tiles = tiles_m * tiles_n;
    const uint32_t stage_tx = Cfg::A_BYTES + (uint32_t)bn * (GEMM_KSTEP * 2);
    const int num_kb = (K + GEMM_KSTEP - 1) / GEMM_KSTEP;

    if (threadIdx.x == 0) {
        trace_stamp(sk.trace, 0);
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
    if (threadIdx.x == 0) trace_stamp(sk.trace, 1);
    pdl_trigger();

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tma_a);
            tma_prefetch_desc(&tma_b);
            uint32_t it = 0;
            bool ok = true;
            // The weight tiles depend on nothing: they stream into the ring at once. The activation
            // tiles wait for the producing kernel (grid dependency) and, under tensor parallelism,
            // for every rank's push of the gathered activation; their loads are parked meanwhile.
            bool dep_ready = false;
            int pending = 0;
            int q_kb[STAGES], q_row[STAGES], q_stage[STAGES];
            uint32_t seen = 0;    // owners whose push this producer has observed
            auto resolve = [&]() {
                pdl_wait();
                for (int j = 0; j < pending && ok; ++j) {
                    if (tp.gated) ok = ag_gate_wait_rows(tp, status, q_row[j], SWAPPED ? bn : GEMM_BM, seen);
                    if (!ok) break;
#pragma unroll
                    for (int u = 0; u < Cfg::KSUB; ++u) {
                        if (SWAPPED)
                            tma_load_2d(tiles + q_stage[j] * Cfg::STAGE_BYTES + Cfg::A_BYTES + u * Cfg::B_SUB, &tma_b,
                                        full_bar(q_stage[j]), q_kb[j] * GEMM_KSTEP + u * GEMM_BK, q_row[j]);
                        else
                            tma_load_2d(tiles + q_stage[j] * Cfg::STAGE_BYTES + u * Cfg::A_SUB, &tma_a, full_bar(q_stage[j]),
                                        q_kb[j] * GEMM_KSTEP + u * GEMM_BK, q_row[j]);
                    }
                }
                pending = 0;
                dep_ready = true;
            };
            SegmentWalk walk(sk.enabled != 0, num_tiles, num_kb, blockIdx.x, gridDim.x);
            Segment seg;
            while (ok && walk.next(seg)) {
                const int m_blk = seg.tile % tiles_m, n_blk = seg.tile / tiles_m;
                int b_row = n_blk * bn;
                if (GROUPED) {
                    if (!dep_ready) resolve();       // the tile table itself comes from the previous kernel
                    const int e = tile_expert[m_blk];
                    if (e < 0) continue;
                    b_row += e * N;
                }
                // Every tile walks K in ascending order: an output element then sees the same
                // summation order whatever tile shape the plan picked (rotating the start per tile
                // was measured and did not help).
                for (int kb = seg.kb0; kb < seg.kb1 && ok; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!dep_ready && it >= (uint32_t)STAGES) resolve();
                    if (!ok) break;
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, status, PIE_ERR_WAIT_TMA)) { ok = false; break; }
                    const uint32_t a_dst = tiles + s * Cfg::STAGE_BYTES;
                    if (PIE_DIAG(sk.dbg & 6)) {   // diagnostics: 2 = no activation loads, 4 = no weight loads, 6 = neither
                        const uint32_t tx = ((sk.dbg & 2) ? 0u : Cfg::A_BYTES) + ((sk.dbg & 4) ? 0u : (uint32_t)bn * (GEMM_KSTEP * 2));
                        mbar_arrive_expect_tx(full_bar(s), tx);
                        for (int u = 0; u < Cfg::KSUB; ++u) {
                            if (!(sk.dbg & 4))
                                tma_load_2d(a_dst + Cfg::A_BYTES + u * Cfg::B_SUB, &tma_b, full_bar(s), kb * GEMM_KSTEP + u * GEMM_BK, b_row);
                            if (!(sk.dbg & 2))
                                tma_load_2d(a_dst + u * Cfg::A_SUB, &tma_a, full_bar(s), kb * GEMM_KSTEP + u * GEMM_BK, m_blk * GEMM_BM);
                        }
                        continue;
                    }
                    if (dep_ready && tp.gated &&
                        !ag_gate_wait_rows(tp, status, SWAPPED ? b_row : m_blk * GEMM_BM, SWAPPED ? bn : GEMM_BM, seen)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(full_bar(s), stage_tx);
                    // the operand that holds the weights goes first; the activation operand (tma_a, or
                    // tma_b of a swapped launch) waits for its producer
                    if (!SWAPPED || dep_ready) {
#pragma unroll
                        for (int u = 0; u < Cfg::KSUB; ++u)
                            tma_load_2d(a_dst + Cfg::A_BYTES + u * Cfg::B_SUB, &tma_b, full_bar(s), kb * GEMM_KSTEP + u * GEMM_BK, b_row);
                    }
                    if (SWAPPED || dep_ready) {
#pragma unroll
                        for (int u = 0; u < Cfg::KSUB; ++u)
                            tma_load_2d(a_dst + u * Cfg::A_SUB, &tma_a, full_bar(s), kb * GEMM_KSTEP + u * GEMM_BK, m_blk * GEMM_BM);
                    }
                    if (!dep_ready) {
                        q_kb[pending] = kb; q_row[pending] = SWAPPED ? b_row : m_blk * GEMM_BM; q_stage[pending] = s;
                        ++pending;
                    }
                }
            }
            if (!dep_ready) resolve();
            // no copy of this CTA may still be in flight when it exits
            const uint32_t first = it > (uint32_t)STAGES ? it - STAGES : 0u;
            for (uint32_t j = first; j < it; ++j)
                mbar_wait(full_bar(j % STAGES), (j / STAGES) & 1u, status, PIE_ERR_WAIT_TMA,
                          200000000ll);
        }
    } else if (warp == 1) {
        // -------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = make_idesc_bf16(GEMM_BM, bn);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            SegmentWalk walk(sk.enabled != 0, num_tiles, num_kb, blockIdx.x, gridDim.x);
            Segment seg;
            if (GROUPED) pdl_wait();
            for (; ok && walk.next(seg); ++tcount) {
                if (GROUPED && tile_expert[seg.tile % tiles_m] < 0) { --tcount; continue; }
                const uint32_t acc = tcount & 1u, aph = (tcount >> 1) & 1u;
                if (!mbar_wait(tempty_bar(acc), aph ^ 1u, status, PIE_ERR_WAIT_EPILOGUE)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = seg.kb0; kb < seg.kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait(full_bar(s), ph, status, PIE_ERR_WAIT_TMA)) { ok = false; break; }
                    if (it == 0) trace_stamp(sk.trace, 2);
                    tc_fence_after();
                    const uint32_t a_addr = tiles + s * Cfg::STAGE_BYTES;
                    if (!PIE_DIAG(sk.dbg & 1)) {
#pragma unroll
                        for (int u = 0; u < Cfg::KSUB; ++u) {
                            const uint64_t adesc = make_smem_desc_sw128(a_addr + u * Cfg::A_SUB);
                            const uint64_t bdesc = make_smem_desc_sw128(a_addr + Cfg::A_BYTES + u * Cfg::B_SUB);
#pragma unroll
                            for (int k = 0; k < GEMM_BK / 16; ++k)
                                umma_bf16(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, ((kb - seg.kb0) | u | k) != 0);
                        }
                    }
                    umma_commit(empty_bar(s));
                }
                if (ok) umma_commit(tfull_bar(acc));
            }
            trace_stamp(sk.trace, 3);
        }
    } else {
        // ----------------------------------------------------------- epilogue
        const int q = warp & 3;  // TMEM lanes [32q, 32q+32) belong to this warp
        uint32_t tcount = 0;
        pdl_wait();   // outputs, residual and the stream-K workspace may still be in use by the previous kernel
        SegmentWalk walk(sk.enabled != 0, num_tiles, num_kb, blockIdx.x, gridDim.x);
        Segment seg;
        const long long total_units = (long long)num_tiles * num_kb;
        for (; walk.next(seg); ++tcount) {
            const int m_blk = seg.tile % tiles_m, n_blk = seg.tile / tiles_m;
            if (GROUPED && tile_expert[m_blk] < 0) { --tcount; continue; }
            const uint32_t acc = tcount & 1u, aph = (tcount >> 1) & 1u;
            const bool got = mbar_wait(tfull_bar(acc), aph, status, PIE_ERR_WAIT_MMA);
            if (!__all_sync(0xffffffffu, got)) break;
            if (warp == 2 && lane == 0) trace_stamp(sk.trace, tcount == 0 ? 4 : 5);
            tc_fence_after();
            const int row = m_blk * GEMM_BM + q * 32 + lane;
            const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
            const bool partial = seg.kb0 != 0 || seg.kb1 != num_kb;
            // a 32-row quarter that lies wholly past M has nothing to park, reduce or store
            const bool rows_valid = m_blk * GEMM_BM + q * 32 < M;
            bool finalise = rows_valid;
            int c_first = 0, c_last = -1;
            if (partial && rows_valid) {
                // park this warp's 32 rows of the partial tile, then count the arrival
                // workspace layout per (slot, warp): [chunk of 32 columns][float4 j][lane], so that every
                // store/load instruction of a warp moves 512 contiguous bytes
                uint4* mine = reinterpret_cast<uint4*>(sk.ws) + (size_t)(blockIdx.x + seg.tile) * (GEMM_BM * BN / 4) +
                              (size_t)q * (32 * BN / 4) + lane;
#pragma unroll 1
                for (int c = 0; c < (bn + 31) / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(t_row + c * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        mine[(c * 8 + j) * 32] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
                __threadfence();
                __syncwarp();
                c_first = streamk_cta_of((long long)seg.tile * num_kb, total_units, gridDim.x);
                c_last = streamk_cta_of((long long)(seg.tile + 1) * num_kb - 1, total_units, gridDim.x);
                int last = 0;
                if (lane == 0) {
                    int* ctr = sk.cnt + seg.tile * 4 + q;
                    last = (atomicAdd(ctr, 1) + 1 == c_last - c_first + 1) ? 1 : 0;
                    if (last) *ctr = 0;
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                finalise = last != 0;
                if (finalise) __threadfence();
            }
            if (finalise) {
                uint8_t* stage = tiles_ptr + STAGES * Cfg::STAGE_BYTES + 256 + (warp - 2) * 4096;
#pragma unroll 1
                for (int c = 0; c < (bn + 63) / 64; ++c) {
                    uint32_t v0[32], v1[32];
                    tmem_ld_32x32(t_row + c * 64, v0);
                    tmem_ld_32x32(t_row + c * 64 + 32, v1);
                    tmem_ld_wait();
                    if (partial) {
                        // Sum every contributor's parked partial (this CTA's own included) in CTA
                        // order: the result does not depend on which CTA happened to arrive last.
#pragma unroll
                        for (int j = 0; j < 32; ++j) v0[j] = v1[j] = 0u;
                        for (int cc = c_first; cc <= c_last; ++cc) {
                            const float4* other = reinterpret_cast<const float4*>(sk.ws) +
                                                  (size_t)(cc + seg.tile) * (GEMM_BM * BN / 4) +
                                                  (size_t)q * (32 * BN / 4) + (size_t)c * 16 * 32 + lane;
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const float4 a4 = __ldcg(other + j * 32), b4 = __ldcg(other + (8 + j) * 32);
                                v0[4 * j] = __float_as_uint(__uint_as_float(v0[4 * j]) + a4.x);
                                v0[4 * j + 1] = __float_as_uint(__uint_as_float(v0[4 * j + 1]) + a4.y);
                                v0[4 * j + 2] = __float_as_uint(__uint_as_float(v0[4 * j + 2]) + a4.z);
                                v0[4 * j + 3] = __float_as_uint(__uint_as_float(v0[4 * j + 3]) + a4.w);
                                v1[4 * j] = __float_as_uint(__uint_as_float(v1[4 * j]) + b4.x);
                                v1[4 * j + 1] = __float_as_uint(__uint_as_float(v1[4 * j + 1]) + b4.y);
                                v1[4 * j + 2] = __float_as_uint(__uint_as_float(v1[4 * j + 2]) + b4.z);
                                v1[4 * j + 3] = __float_as_uint(__uint_as_float(v1[4 * j + 3]) + b4.w);
                            }
                        }
                    }
                    if constexpr (EPI >= EPI_STORE_T)
                        epilogue_store_64_t<EPI>(v0, v1, stage, m_blk * GEMM_BM + q * 32, n_blk * bn + c * 64, M,
                                                 min(N, (n_blk + 1) * bn), C, ldc, R, ldr);
                    else
                        epilogue_store_64<EPI>(v0, v1, stage, m_blk * GEMM_BM + q * 32, n_blk * bn + c * 64, M, N, C,
                                               ldc, R, ldr, tp, min(N, (n_blk + 1) * bn));
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
            // one arrival per (tile, quarter): the finaliser's for a valid quarter, the owner of the
            // tile's last k-block for a quarter past M
            if (EPI == EPI_RS && (rows_valid ? finalise : seg.kb1 == num_kb)) {
                // publish: this warp's rows of the tile are in the owners' buffers
                __threadfence_system();
                __syncwarp();
                if (lane == 0) {
                    const int total = num_tiles * 4;
                    if (atomicAdd(tp.rs_done, 1) + 1 == total) {
                        *tp.rs_done = 0;
                        const int e = *reinterpret_cast<volatile int*>(tp.rs_epoch) + 1;
                        *reinterpret_cast<volatile int*>(tp.rs_epoch) = e;
                        __threadfence_system();
                        for (int p = 0; p < tp.world; ++p)
                            *reinterpret_cast<volatile int*>(tp.peer_rs_flags[p] + tp.rank) = e;
                    }
                }
            }
        }
    }
    if (warp == 2 && lane == 0) trace_stamp(sk.trace, 6);
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) trace_stamp(sk.trace, 7);
    if (warp == 1) {
        __syncwarp();  // lane 0 ran the MMA loop alone: reconverge before the aligned dealloc
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

}  // namespace pie

using namespace pie;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D bf16 row-major [rows, cols] with leading dimension ld (elements); box is
// box_rows x 64 columns with the 128-byte swizzle.
extern "C" int pie_make_tma_2d_bf16(CUtensorMap* map, const void* ptr, long rows, long cols, long ld,
                                    int box_rows) {
    EncodeTiledFn enc = get_encode_fn();
    if (!enc) return -1;
    if (((uintptr_t)ptr & 15) || (ld * 2) % 16) return -2;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)GEMM_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                     box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return (int)r;
}

// Per-device stream-K workspace, registered once by the caller (pie_gemm_set_workspace).
struct GemmWorkspace {
    float* ws = nullptr;
    long ws_floats = 0;
    int* cnt = nullptr;
    int cnt_ints = 0;
};
static GemmWorkspace g_gemm_ws[64];

// ws: fp32 scratch for partial tiles; cnt: zero-initialised arrival counters (the kernel leaves
// them zero). Without a registered workspace every GEMM runs with whole-tile scheduling.
PIE_API int pie_gemm_set_workspace(int device, float* ws, long ws_floats, int* cnt, int cnt_ints) {
    if (device < 0 || device >= 64) return (int)cudaErrorInvalidValue;
    g_gemm_ws[device] = GemmWorkspace{ws, ws_floats, cnt, cnt_ints};
    return 0;
}

// Diagnostics, only in a build with -DPIE_GEMM_DIAG (otherwise both setters answer
// cudaErrorNotSupported and the kernels carry no diagnostic code).
// trace: the single-CTA kernel writes 8 globaltimer stamps per CTA (start, set-up done, first tile
// landed, last MMA issued, first/last accumulator ready, epilogue done, all roles done) into
// trace[grid][8]. debug bits (results are then meaningless): 1 skips the MMAs, 2 the activation
// loads, 4 the weight loads.
static unsigned long long* g_gemm_trace = nullptr;
static int g_gemm_dbg = 0;
#ifdef PIE_GEMM_DIAG
PIE_API int pie_gemm_set_debug(int bits) { g_gemm_dbg = bits; return 0; }
PIE_API int pie_gemm_set_trace(unsigned long long* trace) { g_gemm_trace = trace; return 0; }
#else
PIE_API int pie_gemm_set_debug(int) { return (int)cudaErrorNotSupported; }
PIE_API int pie_gemm_set_trace(unsigned long long*) { return (int)cudaErrorNotSupported; }
#endif

int g_pie_pdl = 0;
// 1: launch the library's kernels with programmatic stream serialisation, so that a kernel's
// prologue and weight prefetch overlap the tail of its predecessor.
PIE_API int pie_set_pdl(int enabled) { g_pie_pdl = enabled; return 0; }

// 0: single-CTA tiles only; 1: CTA pairs (cta_group::2) where the shape allows (default)
static int g_gemm_pairs = 1;
PIE_API int pie_gemm_set_pairs(int enabled) { g_gemm_pairs = enabled; return 0; }

// Batches of up to this many rows run with swapped operands (0: never): the weight rows take the
// 128-row side of the MMA and the batch the narrow side, so each CTA streams a [128 x K-slice]
// block of the weights against the whole (small) activation instead of re-reading the activation
// once per narrow weight tile.
static int g_gemm_swap_max_m = 128;
PIE_API int pie_gemm_set_swap(int max_m) { g_gemm_swap_max_m = max_m; return 0; }

int pie_gemm2_dispatch(const void* A, const void* W, void* C, const void* R, int M, int N, int K, int lda,
                       int ldw, int ldc, int ldr, int epilogue, int* status, int num_sms, cudaStream_t st,
                       const TpArgs* tp_in, float* ws, long ws_floats, int* cnt, int cnt_ints, int* handled);

struct GemmPlan {
    int bn;        // tile width of the launch (multiple of 16)
    int grid, streamk;
    int bn_t() const { return bn <= 64 ? 64 : (bn <= 128 ? 128 : 256); }   // instantiation that holds it
};

// Tile width and scheduling from a small analytical model (times in ns).
//   A tile of width bn costs per 64-deep k-block the slower of its MMAs (128 x bn x 64) and of
//   filling its ring slot (the activation rows + bn weight rows of 128 B); whole-tile scheduling
//   runs ceil(tiles / SMs) waves of such tiles, so the width is chosen to make the tile count
//   fill its waves. The weights also have to come out of HBM once. Stream-K (even split of all
//   k-blocks, partial tiles fixed up through the workspace) competes when no width fills the waves.
//   force_bn > 0 fixes the width; allow_sk = false keeps whole-tile scheduling.
// Tuning aid: a plan (tile width, grid, stream-K) that replaces the planner's choice for every
// following single-CTA launch until cleared with bn = 0. The caller owns its validity.
static GemmPlan g_plan_override{0, 0, 0};
PIE_API int pie_gemm_set_plan_override(int bn, int grid, int streamk) {
    if (bn < 0 || bn > 256 || bn % 16) return (int)cudaErrorInvalidValue;
    g_plan_override = GemmPlan{bn, grid, streamk};
    return 0;
}

static GemmPlan plan_gemm(int M, int N, int K, int num_sms, int force_bn, const GemmWorkspace& w,
                          bool allow_sk = true) {
    if (g_plan_override.bn > 0) {
        GemmPlan p = g_plan_override;
        const long tiles = (long)((M + GEMM_BM - 1) / GEMM_BM) * ((N + p.bn - 1) / p.bn);
        if (!p.streamk) p.grid = (int)std::min<long>(tiles, p.grid > 0 ? p.grid : num_sms);
        else if (!w.ws || (long)(p.grid + tiles) * GEMM_BM * (p.bn <= 64 ? 64 : (p.bn <= 128 ? 128 : 256)) > w.ws_floats ||
                 tiles * 4 > w.cnt_ints) p.streamk = 0, p.grid = (int)std::min<long>(tiles, num_sms);
        return p;
    }
    const int tm = (M + GEMM_BM - 1) / GEMM_BM;
    const int num_kb = (K + GEMM_KSTEP - 1) / GEMM_KSTEP;
    // The plan depends on M only through the number of 128-row tiles: every batch size within a
    // tile count takes the same tile width and K split, hence the same summation order, so a
    // request's numbers do not change with the company it is batched with.
    const double a_rows = 128.0;
    const double mma_ns = 1.08, fill_ns = 0.62;                  // per tile column / per 128-byte operand row
    const double hbm_ns = (double)N * K * 2.0 / 6.0e3;           // all weights once at ~6 TB/s
    const double launch_ns = 3000.0, wave_ns = 700.0, fixup_ns = 4500.0;
    GemmPlan best{64, 1, 0};
    double best_cost = 1e30;
    for (int bn = 256; bn >= 16; bn -= 16) {
        if (force_bn > 0 && bn != force_bn) continue;
        if (force_bn <= 0 && bn > 16 && bn - 16 >= N) continue;  // wider than the matrix: pure waste
        const int bt = bn <= 64 ? 64 : (bn <= 128 ? 128 : 256);
        const long tiles = (long)tm * ((N + bn - 1) / bn);
        const double kb_ns = GEMM_KSUB * std::max(mma_ns * bn, fill_ns * (a_rows + bn));
        const double tile_ns = num_kb * kb_ns + wave_ns;
        const long waves = (tiles + num_sms - 1) / num_sms;
        const double active = (double)std::min<long>(tiles, num_sms);
        // an SM keeps (stages x bn x 128 B) of weights in flight; ~1.6 us to turn them around
        const int stages = (bt == 256 ? 4 : (bt == 128 ? 6 : 8)) / GEMM_KSUB;
        const double per_sm_gbs = std::min(90.0, stages * bn * 128.0 * GEMM_KSUB / 1600.0);
        const double hbm_eff = std::max(hbm_ns, (double)N * K * 2.0 / (active * per_sm_gbs));
        const double dp = std::max(waves * tile_ns, hbm_eff) + launch_ns;
        if (dp < best_cost) {
            best_cost = dp;
            best = GemmPlan{bn, (int)std::min<long>(tiles, num_sms), 0};
        }
        // stream-K at the three native widths only, and only over a K long enough to be worth
        // splitting (short-K problems keep one summation order whatever the batch size)
        if (!allow_sk || !w.ws || (bn != bt) || K < 2048) continue;
        const long units = tiles * num_kb;
        const long grid = std::min<long>(units * GEMM_KSUB / 16, num_sms);   // at least 1024 of K per CTA
        if (grid < 1 || tiles > 2L * num_sms || tiles % grid == 0) continue;
        if ((grid + tiles) * (long)GEMM_BM * bt > w.ws_floats || tiles * 4 > w.cnt_ints) continue;
        const double sk_hbm = std::max(hbm_ns, (double)N * K * 2.0 / (grid * per_sm_gbs));
        const double sk = std::max((double)units / grid * kb_ns, sk_hbm) + fixup_ns + launch_ns;
        if (sk < best_cost) {
            best_cost = sk;
            best = GemmPlan{bn, (int)grid, 1};
        }
    }
    return best;
}

// The plan the single-CTA kernel would use (introspection, tests): out = {bn, grid, streamk}.
PIE_API int pie_gemm_plan(int M, int N, int K, int num_sms, int with_workspace, int* out) {
    GemmWorkspace w{};
    if (with_workspace) {
        w.ws = reinterpret_cast<float*>(16);
        w.ws_floats = 3L * num_sms * 128 * 256;
        w.cnt_ints = 2 * num_sms * 4;
    }
    const GemmPlan p = plan_gemm(M, N, K, num_sms, 0, w);
    out[0] = p.bn; out[1] = p.grid; out[2] = p.streamk;
    return 0;
}

template <int BN, int EPI>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, void* C, const void* R, int M,
                       int N, int K, int ldc, int ldr, int* status, const GemmPlan& plan,
                       const GemmWorkspace& w, cudaStream_t st, const TpArgs& tp = TpArgs{}) {
    using Cfg = GemmCfg<BN>;
    auto kern = gemm_bf16_kernel<BN, EPI>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    StreamKArgs sk{w.ws, w.cnt, plan.streamk, g_gemm_dbg, g_gemm_trace};
    e = launch_pdl(kern, dim3(plan.grid), dim3(GEMM_THREADS), Cfg::SMEM_BYTES, st, ta, tb, (bf16*)C, (const bf16*)R,
                   M, N, K, ldc, ldr, status, tp, sk, (const int*)nullptr, plan.bn);
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

static int current_workspace(GemmWorkspace* out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    *out = (dev >= 0 && dev < 64) ? g_gemm_ws[dev] : GemmWorkspace{};
    return 0;
}

// C[M,N] (or [M,N/2] for the SwiGLU epilogue) = A[M,K] * W[N,K]^T.
// `status` is a device int that stays 0 unless a bounded wait ran out.
PIE_API int pie_gemm_bf16(const void* A, const void* W, void* C, const void* R, int M, int N, int K,
                          int lda, int ldw, int ldc, int ldr, int epilogue, int force_bn,
                          int* status, int num_sms, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || N % 8 || ldc % 8 || (epilogue == EPI_RESIDUAL && ldr % 8))
        return (int)cudaErrorInvalidValue;
    if (epilogue == EPI_SWIGLU && N % 32) return (int)cudaErrorInvalidValue;
    GemmWorkspace w;
    if (int rc = current_workspace(&w)) return rc;
    if (g_gemm_pairs && force_bn == 0) {
        int handled = 0;
        const int rc = pie_gemm2_dispatch(A, W, C, R, M, N, K, lda, ldw, ldc, ldr, epilogue, status, num_sms, st,
                                          nullptr, w.ws, w.ws_floats, w.cnt, w.cnt_ints, &handled);
        if (handled || rc) return rc;
    }
    if (force_bn == 0 && M <= (g_gemm_swap_max_m >= 1000 ? 128 : g_gemm_swap_max_m) && M <= 128 && N >= 128 && K >= 512) {
        // C^T = W * A^T: rows of the launch are output features, its one column tile the batch
        const int bt = M <= 64 ? 64 : 128;
        const GemmPlan plan = plan_gemm(N, bt, K, num_sms, bt, w, true);
        // Measured (Llama-3.1-8B shapes, 8 to 128 rows): the swapped launch wins where its 128-row
        // feature tiles cannot fill the machine by themselves and K is long enough that each CTA of
        // the K split keeps 20 or more k-blocks (qkv 31 -> 27 us, down 59 -> 47 us at 64 rows); with
        // shorter splits the fix-up of the partial tiles costs more than the narrow direct tiles. Up to 128 rows the
        // decode step still gains (96 requests 8.41 -> 7.96 ms, 128 requests 9.20 -> 8.99 ms).
        const long s_tiles = (N + GEMM_BM - 1) / GEMM_BM, s_kb = (K + GEMM_KSTEP - 1) / GEMM_KSTEP;
        const bool take = g_gemm_swap_max_m >= 1000 ||
                          (plan.streamk && s_tiles <= num_sms && s_tiles * s_kb >= 20L * plan.grid);
        CUtensorMap ta, tb;
        if (!take) goto direct;
        if (pie_make_tma_2d_bf16(&ta, W, N, K, ldw, GEMM_BM) != 0) return (int)cudaErrorInvalidValue;
        if (pie_make_tma_2d_bf16(&tb, A, M, K, lda, bt) != 0) return (int)cudaErrorInvalidValue;
#define GO_T(BN_)                                                                                   \
    switch (epilogue) {                                                                           \
        case EPI_STORE: return launch_gemm<BN_, EPI_STORE_T>(ta, tb, C, R, N, M, K, ldc, ldr, status, plan, w, st); \
        case EPI_RESIDUAL: return launch_gemm<BN_, EPI_RESIDUAL_T>(ta, tb, C, R, N, M, K, ldc, ldr, status, plan, w, st); \
        case EPI_SWIGLU: return launch_gemm<BN_, EPI_SWIGLU_T>(ta, tb, C, R, N, M, K, ldc, ldr, status, plan, w, st); \
        default: return (int)cudaErrorInvalidValue;                                               \
    }
        if (bt == 64) { GO_T(64) } else { GO_T(128) }
#undef GO_T
    }
direct:
    bool allow_sk = true;
    if (force_bn < 0) { allow_sk = false; force_bn = -force_bn == 1 ? 0 : -force_bn; }  // negative: whole-tile only
    if (force_bn > 256 || force_bn % 16) return (int)cudaErrorInvalidValue;
    const GemmPlan plan = plan_gemm(M, N, K, num_sms, force_bn, w, allow_sk);
    const int bn = plan.bn_t();
    CUtensorMap ta, tb;
    if (pie_make_tma_2d_bf16(&ta, A, M, K, lda, GEMM_BM) != 0) return (int)cudaErrorInvalidValue;
    if (pie_make_tma_2d_bf16(&tb, W, N, K, ldw, plan.bn) != 0) return (int)cudaErrorInvalidValue;
#define GO(BN_)                                                                                   \
    switch (epilogue) {                                                                           \
        case EPI_STORE: return launch_gemm<BN_, EPI_STORE>(ta, tb, C, R, M, N, K, ldc, ldr, status, plan, w, st); \
        case EPI_RESIDUAL: return launch_gemm<BN_, EPI_RESIDUAL>(ta, tb, C, R, M, N, K, ldc, ldr, status, plan, w, st); \
        case EPI_SWIGLU: return launch_gemm<BN_, EPI_SWIGLU>(ta, tb, C, R, M, N, K, ldc, ldr, status, plan, w, st); \
        default: return (int)cudaErrorInvalidValue;                                               \
    }
    if (bn == 256) { GO(256) }
    else if (bn == 128) { GO(128) }
    else if (bn == 64) { GO(64) }
#undef GO
    return (int)cudaErrorInvalidValue;
}

// Tensor-parallel GEMM: `tp_blob` points at a host copy of TpArgs (see pie_tp_args_size).
//   epilogue EPI_RS  : y = A * W^T is not stored locally; each row goes to its owner's receive buffer
//   gated (tp.gated) : A is the all-gathered activation; loads wait for every rank's push flag
PIE_API int pie_tp_args_size() { return (int)sizeof(TpArgs); }

PIE_API int pie_tp_fill_args(void* blob, const int* ag_flags, const int* ag_epoch, void* const* peer_recv,
                             int* const* peer_rs_flags, int* rs_done, int* rs_epoch, int world, int rank,
                             int rows_per_rank, int gated) {
    if (world > TP_MAX_RANKS || world < 1) return (int)cudaErrorInvalidValue;
    TpArgs a{};
    a.ag_flags = ag_flags; a.ag_epoch = ag_epoch; a.rs_done = rs_done; a.rs_epoch = rs_epoch;
    for (int i = 0; i < world; ++i) {
        a.peer_recv[i] = (bf16*)peer_recv[i];
        a.peer_rs_flags[i] = peer_rs_flags[i];
    }
    a.world = world; a.rank = rank; a.rows_per_rank = rows_per_rank; a.gated = gated;
    *reinterpret_cast<TpArgs*>(blob) = a;
    return 0;
}

PIE_API int pie_gemm_bf16_tp(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw,
                             int ldc, int epilogue, const void* tp_blob, int rows_per_rank, int gated,
                             int force_bn, int* status, int num_sms, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 || N % 8) return (int)cudaErrorInvalidValue;
    if (epilogue == EPI_SWIGLU && N % 32) return (int)cudaErrorInvalidValue;
    TpArgs tp = *reinterpret_cast<const TpArgs*>(tp_blob);
    tp.rows_per_rank = rows_per_rank;
    tp.gated = gated;
    if (epilogue == EPI_RS && (rows_per_rank % 32 || rows_per_rank <= 0)) return (int)cudaErrorInvalidValue;
    GemmWorkspace w;
    if (int rc = current_workspace(&w)) return rc;
    if (g_gemm_pairs && force_bn == 0) {
        int handled = 0;
        const int rc = pie_gemm2_dispatch(A, W, C, nullptr, M, N, K, lda, ldw, ldc, 0, epilogue, status, num_sms,
                                          st, &tp, w.ws, w.ws_floats, w.cnt, w.cnt_ints, &handled);
        if (handled || rc) return rc;
    }
    if (force_bn < 0 || force_bn > 256 || force_bn % 16) return (int)cudaErrorInvalidValue;
    const GemmPlan plan = plan_gemm(M, N, K, num_sms, force_bn, w);
    const int bn = plan.bn_t();
    CUtensorMap ta, tb;
    if (pie_make_tma_2d_bf16(&ta, A, M, K, lda, GEMM_BM) != 0) return (int)cudaErrorInvalidValue;
    if (pie_make_tma_2d_bf16(&tb, W, N, K, ldw, plan.bn) != 0) return (int)cudaErrorInvalidValue;
#define GO(BN_)                                                                                    \
    switch (epilogue) {                                                                            \
        case EPI_STORE: return launch_gemm<BN_, EPI_STORE>(ta, tb, C, nullptr, M, N, K, ldc, 0, status, plan, w, st, tp);   \
        case EPI_SWIGLU: return launch_gemm<BN_, EPI_SWIGLU>(ta, tb, C, nullptr, M, N, K, ldc, 0, status, plan, w, st, tp); \
        case EPI_RS: return launch_gemm<BN_, EPI_RS>(ta, tb, C, nullptr, M, N, K, ldc, 0, status, plan, w, st, tp);         \
        default: return (int)cudaErrorInvalidValue;                                                \
    }
    if (bn == 256) { GO(256) }
    else if (bn == 128) { GO(128) }
    else if (bn == 64) { GO(64) }
#undef GO
    return (int)cudaErrorInvalidValue;
}

// Grouped (mixture-of-experts) GEMM: A [max_mtiles*128, K] holds token rows sorted by expert in
// 128-row tiles; W is [E, N, K] contiguous; tile_expert [max_mtiles] (device) gives each tile's
// expert or -1. C [max_mtiles*128, N] (or N/2 with the SwiGLU epilogue). Graph-safe: the launch
// shape depends only on max_mtiles.
PIE_API int pie_grouped_gemm_bf16(const void* A, const void* W, void* C, const int* tile_expert, int max_mtiles,
                                  int num_experts, int N, int K, int lda, int ldc, int epilogue, int* status,
                                  int num_sms, cudaStream_t st) {
    if (max_mtiles <= 0 || N <= 0 || num_experts <= 0) return 0;
    if (K <= 0 || K % 8 || N % 8 || ldc % 8) return (int)cudaErrorInvalidValue;
    if (epilogue == EPI_SWIGLU && N % 32) return (int)cudaErrorInvalidValue;
    const int M = max_mtiles * GEMM_BM;
    const int bn = N >= 128 ? 128 : 64;
    CUtensorMap ta, tb;
    if (pie_make_tma_2d_bf16(&ta, A, M, K, lda, GEMM_BM) != 0) return (int)cudaErrorInvalidValue;
    if (pie_make_tma_2d_bf16(&tb, W, (long)num_experts * N, K, K, bn) != 0) return (int)cudaErrorInvalidValue;
    const long tiles = (long)max_mtiles * ((N + bn - 1) / bn);
    const int grid = (int)(tiles < num_sms ? tiles : num_sms);
    StreamKArgs sk{nullptr, nullptr, 0, 0, nullptr};
    TpArgs tp{};
#define GO(BN_, EPI_)                                                                                     \
    {                                                                                                     \
        auto kern = gemm_bf16_kernel<BN_, EPI_, true>;                                                    \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                                             (int)GemmCfg<BN_>::SMEM_BYTES);                              \
        if (e != cudaSuccess) return (int)e;                                                              \
        e = launch_pdl(kern, dim3(grid), dim3(GEMM_THREADS), GemmCfg<BN_>::SMEM_BYTES, st, ta, tb, (bf16*)C, \
                       (const bf16*)nullptr, M, N, K, ldc, 0, status, tp, sk, tile_expert, bn);               \
        return (int)(e != cudaSuccess ? e : cudaGetLastError());                                          \
    }
    if (epilogue == EPI_STORE) {
        if (bn == 128) GO(128, EPI_STORE) else GO(64, EPI_STORE)
    } else if (epilogue == EPI_SWIGLU) {
        if (bn == 128) GO(128, EPI_SWIGLU) else GO(64, EPI_SWIGLU)
    }
#undef GO
    return (int)cudaErrorInvalidValue;
}
