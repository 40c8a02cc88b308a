// bf16 GEMM on CTA pairs (tcgen05 cta_group::2):  C[M,N] = A[M,K] * W[N,K]^T, 256 x BN per pair.
//
// Two CTAs of a 2-CTA cluster share one output tile. Each CTA TMA-loads its own 128 rows of A
// and its own half of the W tile (BN/2 rows) into its shared memory (plain per-CTA loads, no
// multicast); the leader CTA issues tcgen05.mma.cta_group::2, which reads both CTAs' shared
// memory and accumulates 128 rows in each CTA's TMEM. Compared with the single-CTA kernel this
// halves the shared-memory fill per flop (the measured limit of that kernel) and leaves room
// for a deeper TMA ring.
//
// Roles per CTA: warp 0 TMA producer; warp 1 MMA issuer (leader) or full-barrier relay
// (follower: forwards "my stage landed" to the leader); warps 2-5 epilogue of the CTA's own
// 128 rows. tcgen05.commit signals the ring-slot and accumulator barriers of both CTAs.
// Same epilogues, stream-K schedule and tensor-parallel hooks as gemm_tcgen05.cu; every wait
// on an mbarrier is bounded. The two cluster-wide barriers (start, end) are reached by every
// thread on every path.
#include "gemm_common.cuh"

namespace pie {
using namespace sm100;

template <int BN>
struct Gemm2Cfg {
    static constexpr uint32_t A_BYTES = GEMM_BM * GEMM_BK * 2;       // this CTA's 128 rows
    static constexpr uint32_t B_BYTES = (BN / 2) * GEMM_BK * 2;      // this CTA's half of the W tile
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = BN == 256 ? 6 : 8;
    static constexpr uint32_t TMEM_COLS = 2 * BN;
    static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 512 /*barriers*/ + 16384 /*epilogue staging*/;
};

template <int BN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                  bf16* __restrict__ C, const bf16* __restrict__ R, int M, int N, int K, int ldc, int ldr,
                  int* status, const __grid_constant__ TpArgs tp, const StreamKArgs sk) {
    using Cfg = Gemm2Cfg<BN>;
    constexpr int STAGES = Cfg::STAGES;
    constexpr int PAIR_M = 2 * GEMM_BM;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_addr(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    uint8_t* tiles_ptr = smem_raw + (tiles - raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles_ptr + STAGES * Cfg::STAGE_BYTES);
    const uint32_t bar0 = tiles + STAGES * Cfg::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
    auto peer_bar = [&](int s) { return bar0 + 8u * (2 * STAGES + s); };   // leader: follower's stage landed
    auto tfull_bar = [&](int a) { return bar0 + 8u * (3 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar0 + 8u * (3 * STAGES + 2 + a); };  // leader's is the one in use
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 3 * STAGES + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t crank = cluster_ctarank();
    const bool leader = crank == 0;
    const bool relay = PIE_DIAG(sk.dbg & 4) != 0;
    const int pid = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int tiles_m = (M + PAIR_M - 1) / PAIR_M;
    const int tiles_n = (N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (K + GEMM_BK - 1) / GEMM_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
            mbar_init(peer_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 8);   // 4 epilogue warps of each CTA
        }
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        tmem_alloc_2cta(smem_addr(const_cast<uint32_t*>(tmem_slot)), Cfg::TMEM_COLS);
        tmem_relinquish_2cta();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // both CTAs' barriers exist before anyone signals across
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer (each CTA)
        if (lane == 0) {
            tma_prefetch_desc(&tma_a);
            tma_prefetch_desc(&tma_b);
            uint32_t it = 0;
            bool ok = true;
            uint32_t seen = 0;
            const uint32_t leader_full0 = map_to_cta(full_bar(0), 0);
            SegmentWalk walk(sk.enabled != 0, num_tiles, num_kb, pid, npairs);
            Segment seg;
            while (ok && walk.next(seg)) {
                const int m_blk = seg.tile % tiles_m, n_blk = seg.tile / tiles_m;
                if (tp.gated && !ag_gate_wait_rows(tp, status, m_blk * PAIR_M + (int)crank * GEMM_BM, GEMM_BM, seen)) {
                    ok = false;
                    break;
                }
                for (int kb = seg.kb0; kb < seg.kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait_cluster(empty_bar(s), ph ^ 1u, status, PIE_ERR_WAIT_TMA)) { ok = false; break; }
                    const uint32_t a_dst = tiles + s * Cfg::STAGE_BYTES;
                    const int a_row = m_blk * PAIR_M + (int)crank * GEMM_BM;
                    const int b_row = n_blk * BN + (int)crank * (BN / 2);
                    if (relay) {
                        if (PIE_DIAG(sk.dbg & 2)) { mbar_arrive(full_bar(s)); continue; }
                        mbar_arrive_expect_tx(full_bar(s), Cfg::STAGE_BYTES);
                        tma_load_2d(a_dst, &tma_a, full_bar(s), kb * GEMM_BK, a_row);
                        tma_load_2d(a_dst + Cfg::A_BYTES, &tma_b, full_bar(s), kb * GEMM_BK, b_row);
                    } else {
                        // both CTAs' loads complete on the leader's barrier, armed for the pair's bytes
                        if (PIE_DIAG(sk.dbg & 2)) { if (leader) mbar_arrive(full_bar(s)); continue; }
                        if (leader) mbar_arrive_expect_tx(full_bar(s), 2 * Cfg::STAGE_BYTES);
                        const uint32_t lbar = leader_full0 + 8u * s;
                        tma_load_2d_pair(a_dst, &tma_a, lbar, kb * GEMM_BK, a_row);
                        tma_load_2d_pair(a_dst + Cfg::A_BYTES, &tma_b, lbar, kb * GEMM_BK, b_row);
                    }
                }
            }
            // no copy into this CTA may be in flight when it exits: with direct signalling the
            // leader's barriers cover the pair and both CTAs meet at the cluster barrier below
            if (relay || leader) {
                const uint32_t first = it > (uint32_t)STAGES ? it - STAGES : 0u;
                for (uint32_t j = first; j < it; ++j)
                    mbar_wait_cluster(full_bar(j % STAGES), (j / STAGES) & 1u, status, PIE_ERR_WAIT_TMA, 200000000ll);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && !leader && relay) {
            // ---------------------------------------------------- follower: relay "stage landed"
            uint32_t it = 0;
            bool ok = true;
            SegmentWalk walk(sk.enabled != 0, num_tiles, num_kb, pid, npairs);
            Segment seg;
            while (ok && walk.next(seg)) {
                for (int kb = seg.kb0; kb < seg.kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(full_bar(s), (it / STAGES) & 1u, status, PIE_ERR_WAIT_TMA)) { ok = false; break; }
                    mbar_arrive_cluster(map_to_cta(peer_bar(s), 0));
                }
            }
        } else if (lane == 0 && leader) {
            // ---------------------------------------------------- leader: MMA issuer of the pair
            constexpr uint32_t idesc = make_idesc_bf16(PAIR_M, BN);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            SegmentWalk walk(sk.enabled != 0, num_tiles, num_kb, pid, npairs);
            Segment seg;
            for (; ok && walk.next(seg); ++tcount) {
                const uint32_t acc = tcount & 1u, aph = (tcount >> 1) & 1u;
                if (!mbar_wait_cluster(tempty_bar(acc), aph ^ 1u, status, PIE_ERR_WAIT_EPILOGUE)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = seg.kb0; kb < seg.kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait_cluster(full_bar(s), ph, status, PIE_ERR_WAIT_TMA) ||
                        (relay && !mbar_wait_cluster(peer_bar(s), ph, status, PIE_ERR_WAIT_TMA))) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = tiles + s * Cfg::STAGE_BYTES;
                    const uint64_t adesc = make_smem_desc_sw128(a_addr);
                    const uint64_t bdesc = make_smem_desc_sw128(a_addr + Cfg::A_BYTES);
                    if (!PIE_DIAG(sk.dbg & 1)) {
#pragma unroll
                        for (int k = 0; k < GEMM_BK / 16; ++k)
                            umma_bf16_2cta(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, ((kb - seg.kb0) | k) != 0);
                    }
                    umma_commit_2cta(empty_bar(s), 3);   // slot s is free in both CTAs
                }
                if (ok) umma_commit_2cta(tfull_bar(acc), 3);
            }
        }
    } else {
        // ----------------------------------------------------------- epilogue (own 128 rows)
        const int q = warp & 3;
        uint32_t tcount = 0;
        SegmentWalk walk(sk.enabled != 0, num_tiles, num_kb, pid, npairs);
        Segment seg;
        const long long total_units = (long long)num_tiles * num_kb;
        const uint32_t leader_tempty0 = map_to_cta(tempty_bar(0), 0);
        const uint32_t leader_tempty1 = map_to_cta(tempty_bar(1), 0);
        for (; walk.next(seg); ++tcount) {
            const int m_blk = seg.tile % tiles_m, n_blk = seg.tile / tiles_m;
            const uint32_t acc = tcount & 1u, aph = (tcount >> 1) & 1u;
            const bool got = mbar_wait_cluster(tfull_bar(acc), aph, status, PIE_ERR_WAIT_MMA);
            if (!__all_sync(0xffffffffu, got)) break;
            tc_fence_after();
            const int row_in_pair = (int)crank * GEMM_BM + q * 32 + lane;
            const int row = m_blk * PAIR_M + row_in_pair;
            const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
            const bool partial = seg.kb0 != 0 || seg.kb1 != num_kb;
            bool finalise = true;
            int c_first = 0, c_last = -1;
            if (partial) {
                // workspace layout per (slot, warp): [chunk of 32 columns][float4 j][lane], so that every
                // store/load instruction of a warp moves 512 contiguous bytes
                uint4* mine = reinterpret_cast<uint4*>(sk.ws) + (size_t)(pid + seg.tile) * (PAIR_M * BN / 4) +
                              (size_t)((int)crank * 4 + q) * (32 * BN / 4) + lane;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(t_row + c * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        mine[(c * 8 + j) * 32] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
                __threadfence();
                __syncwarp();
                c_first = streamk_cta_of((long long)seg.tile * num_kb, total_units, npairs);
                c_last = streamk_cta_of((long long)(seg.tile + 1) * num_kb - 1, total_units, npairs);
                int last = 0;
                if (lane == 0) {
                    int* ctr = sk.cnt + seg.tile * 8 + (int)crank * 4 + q;
                    last = (atomicAdd(ctr, 1) + 1 == c_last - c_first + 1) ? 1 : 0;
                    if (last) *ctr = 0;
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                finalise = last != 0;
                if (finalise) __threadfence();
            }
            if (finalise) {
                uint8_t* stage = tiles_ptr + STAGES * Cfg::STAGE_BYTES + 512 + (warp - 2) * 4096;
#pragma unroll 1
                for (int c = 0; c < BN / 64; ++c) {
                    uint32_t v0[32], v1[32];
                    tmem_ld_32x32(t_row + c * 64, v0);
                    tmem_ld_32x32(t_row + c * 64 + 32, v1);
                    tmem_ld_wait();
                    if (partial) {
                        // every contributor's parked partial (this pair's own included) in pair
                        // order, so the sum does not depend on which pair arrived last
#pragma unroll
                        for (int j = 0; j < 32; ++j) v0[j] = v1[j] = 0u;
                        for (int cc = c_first; cc <= c_last; ++cc) {
                            const float4* other = reinterpret_cast<const float4*>(sk.ws) +
                                                  (size_t)(cc + seg.tile) * (PAIR_M * BN / 4) +
                                                  (size_t)((int)crank * 4 + q) * (32 * BN / 4) + (size_t)c * 16 * 32 + lane;
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
                    epilogue_store_64<EPI>(v0, v1, stage, m_blk * PAIR_M + (int)crank * GEMM_BM + q * 32,
                                           n_blk * BN + c * 64, M, N, C, ldc, R, ldr, tp, N);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (leader) mbar_arrive(tempty_bar(acc));
                else mbar_arrive_cluster(acc ? leader_tempty1 : leader_tempty0);
            }
            if (EPI == EPI_RS && finalise) {
                __threadfence_system();
                __syncwarp();
                if (lane == 0) rs_publish_arrival(tp, num_tiles * 8);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // the peer may still read this CTA's shared memory / signal its barriers
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_2cta(tmem_base, Cfg::TMEM_COLS);
    }
}

}  // namespace pie

using namespace pie;

extern "C" int pie_make_tma_2d_bf16(CUtensorMap* map, const void* ptr, long rows, long cols, long ld, int box_rows);

static int g_pair_dbg = 0;
#ifdef PIE_GEMM_DIAG
extern "C" __attribute__((visibility("default"))) int pie_gemm_set_pair_debug(int bits) { g_pair_dbg = bits; return 0; }
#else
extern "C" __attribute__((visibility("default"))) int pie_gemm_set_pair_debug(int) { return (int)cudaErrorNotSupported; }
#endif

// Problems below these MAC counts go to the single-CTA kernel (second value: when K < 8192).
static double g_pair_min_macs = 1.0e10, g_pair_min_macs_short_k = 2.0e10;
// Tuning aid: pair tile width (64 / 128 / 256) and stream-K (-1 auto, 0 off, 1 on) instead of the dispatcher's choice.
static int g_pair_force_bn = 0, g_pair_force_sk = -1;
extern "C" __attribute__((visibility("default"))) int pie_gemm_set_pair_plan(int bn, int streamk) {
    if (bn != 0 && bn != 64 && bn != 128 && bn != 256) return (int)cudaErrorInvalidValue;
    g_pair_force_bn = bn;
    g_pair_force_sk = streamk;
    return 0;
}
extern "C" __attribute__((visibility("default"))) int pie_gemm_set_pair_thresholds(double min_macs, double min_macs_short_k) {
    g_pair_min_macs = min_macs;
    g_pair_min_macs_short_k = min_macs_short_k;
    return 0;
}

template <int BN, int EPI>
static int launch_gemm2(const CUtensorMap& ta, const CUtensorMap& tb, void* C, const void* R, int M, int N,
                        int K, int ldc, int ldr, int* status, int pairs, int streamk, float* ws, int* cnt,
                        cudaStream_t st, const TpArgs& tp) {
    using Cfg = Gemm2Cfg<BN>;
    auto kern = gemm2_bf16_kernel<BN, EPI>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    StreamKArgs sk{ws, cnt, streamk, g_pair_dbg};
    kern<<<2 * pairs, GEMM_THREADS, Cfg::SMEM_BYTES, st>>>(ta, tb, (bf16*)C, (const bf16*)R, M, N, K, ldc, ldr,
                                                           status, tp, sk);
    return (int)cudaGetLastError();
}

// CTA-pair GEMM entry used by the public GEMM functions. Sets *handled = 0 (and launches nothing)
// when the shape is better served by the single-CTA kernel.
int pie_gemm2_dispatch(const void* A, const void* W, void* C, const void* R, int M, int N, int K, int lda,
                       int ldw, int ldc, int ldr, int epilogue, int* status, int num_sms, cudaStream_t st,
                       const TpArgs* tp_in, float* ws, long ws_floats, int* cnt, int cnt_ints, int* handled) {
    *handled = 0;
    // small problems are launch/fix-up bound: the single-CTA kernel's narrower tiles fill the machine
    // better. Measured cross-over on B200 (M = 256 / 512 decode shapes): pairs win from 2e10 MACs,
    // and from 1e10 when K is long (the 14336-deep down projection).
    const double macs = (double)M * N * K;
    if (M <= GEMM_BM || N < 128 || num_sms < 2 || macs < g_pair_min_macs || (macs < g_pair_min_macs_short_k && K < 8192)) return 0;
    const int bn = g_pair_force_bn ? g_pair_force_bn : (N >= 256 ? 256 : 128);
    const int pairs_max = num_sms / 2;
    const int num_kb = (K + GEMM_BK - 1) / GEMM_BK;
    const long tiles = (long)((M + 2 * GEMM_BM - 1) / (2 * GEMM_BM)) * ((N + bn - 1) / bn);
    int pairs = (int)(tiles < pairs_max ? tiles : pairs_max);
    int streamk = 0;
    {
        const long waves = (tiles + pairs_max - 1) / pairs_max;
        const long units = tiles * num_kb;
        const long gp = units / 16 < pairs_max ? units / 16 : pairs_max;   // >= 16 k-blocks per pair
        if (ws && gp >= 1 && tiles % gp != 0 && tiles <= 2L * pairs_max &&
            (gp + tiles) * 2L * GEMM_BM * bn <= ws_floats && tiles * 8 <= cnt_ints) {
            const double dp = (double)waves, skc = (double)tiles / gp + 0.12;
            if ((skc < 0.92 * dp && g_pair_force_sk != 0) || g_pair_force_sk == 1) { streamk = 1; pairs = (int)gp; }
        }
    }
    CUtensorMap ta, tb;
    if (pie_make_tma_2d_bf16(&ta, A, M, K, lda, GEMM_BM) != 0) return (int)cudaErrorInvalidValue;
    if (pie_make_tma_2d_bf16(&tb, W, N, K, ldw, bn / 2) != 0) return (int)cudaErrorInvalidValue;
    const TpArgs tp = tp_in ? *tp_in : TpArgs{};
    *handled = 1;
#define GO(BN_)                                                                                                     \
    switch (epilogue) {                                                                                             \
        case EPI_STORE: return launch_gemm2<BN_, EPI_STORE>(ta, tb, C, R, M, N, K, ldc, ldr, status, pairs, streamk, ws, cnt, st, tp);       \
        case EPI_RESIDUAL: return launch_gemm2<BN_, EPI_RESIDUAL>(ta, tb, C, R, M, N, K, ldc, ldr, status, pairs, streamk, ws, cnt, st, tp); \
        case EPI_SWIGLU: return launch_gemm2<BN_, EPI_SWIGLU>(ta, tb, C, R, M, N, K, ldc, ldr, status, pairs, streamk, ws, cnt, st, tp);     \
        case EPI_RS: return launch_gemm2<BN_, EPI_RS>(ta, tb, C, R, M, N, K, ldc, ldr, status, pairs, streamk, ws, cnt, st, tp);             \
        default: *handled = 0; return (int)cudaErrorInvalidValue;                                                   \
    }
    if (bn == 256) { GO(256) } else if (bn == 128) { GO(128) } else { GO(64) }
#undef GO
    return (int)cudaErrorInvalidValue;
}
