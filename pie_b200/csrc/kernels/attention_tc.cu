// Paged prefill attention on the 5th-generation tensor cores (head_dim 64 or 128, 16-token pages).
//
// One CTA per (tile of 128 or 256 packed query rows, KV head); a row is (query token, head within
// the GQA group), so a CTA covers 128 / G or 256 / G tokens of one request as one or two MMA tiles of
// 128 rows that share the K and V tiles. KV is walked in blocks of 64 keys:
//   warp 0      TMA producer: the Q tiles once (3-D boxes over [tokens, heads, d]); per block the K
//               and the V rows of its four pages (2-D boxes of 16 rows x 64 columns, 128-byte
//               swizzle) into a ring of K tiles and a ring of V tiles (K is needed two blocks
//               before V); pages past the end come from the cache's pad page
//   1 warp per tile: tcgen05.mma issuer: S = Q K^T (128 x 64, K-major operands) into one of two TMEM
//               buffers, issued two blocks ahead; O += P V (128 x 128; P from shared memory, V as
//               an MN-major operand straight from its [key, d] tile) into the tile's TMEM
//               accumulator as soon as the softmax warps hand over P, then the next S into the
//               buffer just freed
//   4 warps per tile: softmax, one row per thread: S from TMEM, mask (causal / window / custom bits;
//               skipped for blocks fully inside the causal region), exponentials against a
//               reference maximum, P as bf16 into a swizzled shared-memory tile for the PV MMA.
//               The reference maximum follows the true one lazily: only when a block maximum
//               outgrows it by 2^8 does the warp rescale its rows of O in TMEM (tcgen05.ld / st),
//               so most blocks cost one exp per score and no pass over O.
// The two tiles' softmax and MMA phases interleave on the SM: while one tile's rows are in the
// exponentials the tensor cores work on the other's.
// Every wait is bounded; on a time-out the kernel records a status word and leaves.
//
// Replaces the FlashInfer FA2 paged prefill kernel the reference calls
// (driver/cuda/src/ops/attention_flashinfer.cu:848, plans :612,:1075) and this library's own
// mma.sync version for the shapes it covers.
#include "tcgen05.cuh"

namespace pie {
using namespace sm100;

constexpr int AT_ROWS = 128;     // packed query rows per MMA tile
constexpr int AT_BK = 64;        // keys per block
constexpr int AT_D = 128;          // widest head: fixes the TMEM budget (S[2] x 64 + O x D columns per tile)
constexpr int AT_STAGES = 3;      // K ring and V ring, each of this many 16 KB tiles
constexpr uint32_t AT_Q_HALF = AT_ROWS * 64 * 2;               // 16 KB: [128 rows x 64 d]; a Q tile is D / 64 of them
constexpr uint32_t AT_KV_HALF = AT_BK * 64 * 2;                // 8 KB: [64 keys x 64 d]; a K or V tile is D / 64 of them
constexpr uint32_t AT_P_BYTES = AT_ROWS * AT_BK * 2;           // 16 KB
constexpr int AT_TILE_BARS = 8;                                // s_full[2] p_full[2] p_empty[2] pv_done o_final
constexpr float AT_RESCALE_LOG2 = 8.f;                         // the reference maximum may lag the true one by 2^8

template <int NT, int D = AT_D>
struct AtCfg {
    static constexpr int THREADS = 32 * (1 + NT) + 128 * NT;   // producer, one MMA warp per tile, softmax warps
    static constexpr int HALVES = D / 64;
    static constexpr uint32_t Q_BYTES = HALVES * AT_Q_HALF;
    static constexpr uint32_t KV_TILE = HALVES * AT_KV_HALF;
    static constexpr uint32_t SMEM = NT * Q_BYTES + 2 * AT_STAGES * KV_TILE + NT * 2 * AT_P_BYTES + 1024 + 512;
    static constexpr uint32_t TMEM_COLS = 256 * NT;             // per tile: S[2] x 64 columns, O x 128
};

// K-major SW128 descriptor is make_smem_desc_sw128 (tcgen05.cuh). MN-major SW128: the contiguous
// dimension is N (64 elements = one 128-byte row), 8 K-rows form a 1024-byte group (stride field),
// the next 64-element span of N starts `lbo` bytes further (leading field).
__device__ __forceinline__ uint64_t make_smem_desc_sw128_mn(uint32_t saddr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// kind::f16 instruction descriptor with an MN-major B operand (bit 16)
__host__ __device__ constexpr uint32_t make_idesc_bf16_bmn(int m, int n) {
    return make_idesc_bf16(m, n) | (1u << 16);
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];\n" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float fast_tanh(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// CAP: soft-capped scores (Gemma-2). A raw score s becomes cap_post * tanh(s * cap_pre) with cap_pre = sm_scale / cap
// and cap_post = cap / sm_scale, so that the unchanged scale by sm_scale * log2(e) gives cap * tanh(s * sm_scale / cap).
// G = query heads per KV head; NT = MMA tiles of 128 rows per CTA (they share the K/V stages);
// D = head dimension (64 or 128).
template <int G, int NT, int D, bool CAP = false>
__global__ void __launch_bounds__(AtCfg<NT, D>::THREADS, 1)
paged_prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_kv,
                             const int* __restrict__ page_indices, const int* __restrict__ kv_page_indptr,
                             const int* __restrict__ qo_indptr, const int* __restrict__ kv_lens,
                             const int* __restrict__ tile_req, const int* __restrict__ tile_qstart,
                             const uint32_t* __restrict__ mask_bits, const long* __restrict__ mask_word_indptr,
                             bf16* __restrict__ out, float* __restrict__ lse_out, const float* __restrict__ sinks_log2,
                             int hq, int hkv, int pad_page, float scale_log2, int window_left, int* status,
                             float cap_pre, float cap_post) {
    constexpr int TQ = AT_ROWS / G;          // query tokens per MMA tile
    constexpr int HALVES = D / 64;
    constexpr uint32_t AT_Q_BYTES = AtCfg<NT, D>::Q_BYTES, AT_KV_TILE = AtCfg<NT, D>::KV_TILE;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_addr(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t q_s = base;
    const uint32_t k_s = q_s + NT * AT_Q_BYTES;                  // K ring
    const uint32_t v_s = k_s + AT_STAGES * AT_KV_TILE;            // V ring
    const uint32_t p_s = v_s + AT_STAGES * AT_KV_TILE;
    const uint32_t bar0 = p_s + NT * 2 * AT_P_BYTES;
    auto q_full = [&]() { return bar0; };
    auto k_full = [&](int s) { return bar0 + 8u * (1 + s); };
    auto k_empty = [&](int s) { return bar0 + 8u * (1 + AT_STAGES + s); };       // one arrival per MMA warp
    auto v_full = [&](int s) { return bar0 + 8u * (1 + 2 * AT_STAGES + s); };
    auto v_empty = [&](int s) { return bar0 + 8u * (1 + 3 * AT_STAGES + s); };   // one arrival per MMA warp
    auto tbar = [&](int t, int i) { return bar0 + 8u * (1 + 4 * AT_STAGES + t * AT_TILE_BARS + i); };
    auto s_full = [&](int t, int b) { return tbar(t, b); };
    auto p_full = [&](int t, int b) { return tbar(t, 2 + b); };
    auto p_empty = [&](int t, int b) { return tbar(t, 4 + b); };
    auto pv_done = [&](int t) { return tbar(t, 6); };     // one phase per PV MMA of the tile
    auto o_final = [&](int t) { return tbar(t, 7); };     // the tile's last PV MMA has completed
    volatile uint32_t* tmem_slot =
        reinterpret_cast<volatile uint32_t*>(base_ptr + (bar0 - base) + 8u * (1 + 4 * AT_STAGES + NT * AT_TILE_BARS));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, h = blockIdx.y;
    const int req = tile_req[tile], qstart = tile_qstart[tile];
    const int q_base = qo_indptr[req];
    const int qo_len = qo_indptr[req + 1] - q_base;
    const int kv_len = kv_lens[req];
    const int* pages = page_indices + kv_page_indptr[req];
    const bool custom = mask_bits != nullptr;
    // keys visible to MMA tile t: up to the causal limit of its last query token
    auto tile_kv_hi = [&](int t) {
        const int first = qstart + t * TQ;
        if (first >= qo_len) return 0;
        const int last_q = min(first + TQ, qo_len) - 1;
        return custom ? kv_len : max(0, min(kv_len, kv_len - qo_len + last_q + 1));
    };
    int nkb_t[NT], nkb = 0, kv_hi = 0;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const int hi = tile_kv_hi(t);
        nkb_t[t] = (hi + AT_BK - 1) / AT_BK;
        nkb = max(nkb, nkb_t[t]);
        kv_hi = max(kv_hi, hi);
    }
    const int npages = (kv_hi + 15) >> 4;

    if (threadIdx.x == 0) {
        mbar_init(q_full(), 1);
        for (int s = 0; s < AT_STAGES; ++s) {
            mbar_init(k_full(s), 1);
            mbar_init(k_empty(s), NT);
            mbar_init(v_full(s), 1);
            mbar_init(v_empty(s), NT);
        }
        for (int t = 0; t < NT; ++t) {
            for (int b = 0; b < 2; ++b) {
                mbar_init(s_full(t, b), 1);
                mbar_init(p_full(t, b), 4);
                mbar_init(p_empty(t, b), 1);
            }
            mbar_init(pv_done(t), 1);
            mbar_init(o_final(t), 1);
        }
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        tmem_alloc(smem_addr(const_cast<uint32_t*>(tmem_slot)), AtCfg<NT, D>::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0 && nkb > 0) {
            tma_prefetch_desc(&tma_q);
            tma_prefetch_desc(&tma_kv);
            mbar_arrive_expect_tx(q_full(), NT * AT_Q_BYTES);
#pragma unroll
            for (int t = 0; t < NT; ++t) {
#pragma unroll
                for (int half = 0; half < HALVES; ++half)
                    tma_load_3d(q_s + t * AT_Q_BYTES + half * AT_Q_HALF, &tma_q, q_full(), half * 64, h * G,
                                q_base + qstart + t * TQ);
            }
            bool ok = true;
            for (int j = 0; j < nkb && ok; ++j) {
                const int s = j % AT_STAGES;
                const uint32_t par = ((j / AT_STAGES) & 1u) ^ 1u;
                int pg_id[4];
#pragma unroll
                for (int pg = 0; pg < 4; ++pg) {
                    const int pi = j * 4 + pg;
                    pg_id[pg] = pi < npages ? pages[pi] : pad_page;
                }
                if (!mbar_wait(k_empty(s), par, status, PIE_ERR_WAIT_TMA)) { ok = false; break; }
                mbar_arrive_expect_tx(k_full(s), AT_KV_TILE);
#pragma unroll
                for (int pg = 0; pg < 4; ++pg) {
                    const int krow = ((pg_id[pg] * 2) * hkv + h) * 16;
#pragma unroll
                    for (int half = 0; half < HALVES; ++half)
                        tma_load_2d(k_s + s * AT_KV_TILE + half * AT_KV_HALF + pg * 2048, &tma_kv, k_full(s), half * 64, krow);
                }
                if (!mbar_wait(v_empty(s), par, status, PIE_ERR_WAIT_TMA)) { ok = false; break; }
                mbar_arrive_expect_tx(v_full(s), AT_KV_TILE);
#pragma unroll
                for (int pg = 0; pg < 4; ++pg) {
                    const int vrow = ((pg_id[pg] * 2 + 1) * hkv + h) * 16;
#pragma unroll
                    for (int half = 0; half < HALVES; ++half)
                        tma_load_2d(v_s + s * AT_KV_TILE + half * AT_KV_HALF + pg * 2048, &tma_kv, v_full(s), half * 64, vrow);
                }
            }
            // no copy may be in flight when the CTA exits
            const int first = nkb > AT_STAGES ? nkb - AT_STAGES : 0;
            for (int j = first; j < nkb; ++j) {
                mbar_wait(k_full(j % AT_STAGES), (j / AT_STAGES) & 1u, status, PIE_ERR_WAIT_TMA, 200000000ll);
                mbar_wait(v_full(j % AT_STAGES), (j / AT_STAGES) & 1u, status, PIE_ERR_WAIT_TMA, 200000000ll);
            }
        }
    } else if (warp <= NT) {
        // ------------------------------------------------ MMA warp of tile t: S two blocks ahead of PV
        const int t = warp - 1;
        if (lane == 0 && nkb > 0) {
            constexpr uint32_t idesc_s = make_idesc_bf16(AT_ROWS, AT_BK);
            constexpr uint32_t idesc_o = make_idesc_bf16_bmn(AT_ROWS, D);
            const int my = NT == 1 ? nkb : (t == 0 ? nkb_t[0] : nkb_t[NT - 1]);
            const uint32_t tm_s = tmem_base + t * 256, tm_o = tm_s + 128;
            const uint64_t q_desc0 = make_smem_desc_sw128(q_s + t * AT_Q_BYTES);
            bool ok = mbar_wait(q_full(), 0, status, PIE_ERR_WAIT_TMA);
            // S_t(j) = Q_t K_j^T into S buffer j & 1. Every MMA warp waits for and releases every K and V
            // tile, also those its (shorter) tile does not use, so that the rings advance in step.
            auto issue_s = [&](int j) {
                const int s = j % AT_STAGES;
                if (!mbar_wait(k_full(s), (j / AT_STAGES) & 1u, status, PIE_ERR_WAIT_TMA)) { ok = false; return; }
                if (j < my) {
                    tc_fence_after();
                    const uint64_t k_desc0 = make_smem_desc_sw128(k_s + s * AT_KV_TILE);
                    // descriptors count in 16-byte units: the next 64-wide half of d is AT_Q_HALF / AT_KV_HALF further
#pragma unroll
                    for (int half = 0; half < HALVES; ++half)
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma_bf16(tm_s + (j & 1) * AT_BK, q_desc0 + half * (AT_Q_HALF >> 4) + 2u * k,
                                      k_desc0 + half * (AT_KV_HALF >> 4) + 2u * k, idesc_s, (half | k) != 0);
                    umma_commit(s_full(t, j & 1));
                }
                umma_commit(k_empty(s));
            };
            if (ok) issue_s(0);
            if (ok && nkb > 1) issue_s(1);
            for (int j = 0; j < nkb && ok; ++j) {
                const int s = j % AT_STAGES;
                const uint32_t b = j & 1u, ph = (j >> 1) & 1u;
                if (!mbar_wait(v_full(s), (j / AT_STAGES) & 1u, status, PIE_ERR_WAIT_TMA)) { ok = false; break; }
                if (j < my) {
                    // softmax has read S_t(j) and written P_t(j)
                    if (!mbar_wait(p_full(t, b), ph, status, PIE_ERR_WAIT_EPILOGUE)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t p_desc = make_smem_desc_sw128(p_s + (t * 2 + b) * AT_P_BYTES);
#pragma unroll
                    for (int k = 0; k < AT_BK / 16; ++k)      // 16 keys: 32 bytes along a P row, two 8-row groups of V
                        umma_bf16(tm_o, p_desc + 2u * k, make_smem_desc_sw128_mn(v_s + s * AT_KV_TILE + k * 2048, AT_KV_HALF),
                                  idesc_o, (j | k) != 0);
                    umma_commit(pv_done(t));
                    umma_commit(p_empty(t, b));
                    if (j == my - 1) umma_commit(o_final(t));
                }
                umma_commit(v_empty(s));
                if (j + 2 < nkb) issue_s(j + 2);      // overwrites the S buffer that block j has just left
            }
        }
    } else {
        // ---------------------------------------------- softmax warps: thread = row of MMA tile t
        const int t = (warp - 1 - NT) >> 2;
        const int q4 = warp & 3;                        // the TMEM lane quarter this warp may access
        const int row = q4 * 32 + lane;
        const int qtok = qstart + t * TQ + row / G;
        const bool valid = qtok < qo_len;
        const int lim = valid ? (custom ? kv_len : kv_len - qo_len + qtok + 1) : 0;
        const int lo = (window_left >= 0 && valid) ? max(0, kv_len - qo_len + qtok - window_left) : 0;
        const int mask_words = (kv_len + 31) >> 5;
        const uint32_t* row_mask = (custom && valid) ? mask_bits + mask_word_indptr[req] + (size_t)qtok * mask_words : nullptr;
        const uint32_t tm_t = tmem_base + t * 256 + ((uint32_t)(q4 * 32) << 16);
        const uint32_t tm_o = tm_t + 128;
        const float thr_raw = AT_RESCALE_LOG2 / scale_log2;
        const int my_nkb = NT == 1 ? nkb : (t == 0 ? nkb_t[0] : nkb_t[NT - 1]);
        float m_ref = -INFINITY, l = 0.f;    // exponents are taken against m_ref (raw score units)
        bool ok = true;
        for (int j = 0; j < my_nkb && ok; ++j) {
            const uint32_t b = j & 1u, ph = (j >> 1) & 1u;
            const bool got = mbar_wait(s_full(t, b), ph, status, PIE_ERR_WAIT_MMA);
            if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
            tc_fence_after();
            float sv[AT_BK];
#pragma unroll
            for (int c = 0; c < AT_BK / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(tm_t + b * AT_BK + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    sv[c * 32 + i] = CAP ? cap_post * fast_tanh(__uint_as_float(v[i]) * cap_pre) : __uint_as_float(v[i]);
            }
            const int kb0 = j * AT_BK;
            const bool inner = !custom && kb0 + AT_BK <= lim && kb0 >= lo;
            if (!__all_sync(0xffffffffu, inner)) {
                // 64-bit allow mask of this row for the block
                const int n = lim - kb0, nl = lo - kb0;
                unsigned long long allow = n >= 64 ? ~0ull : (n <= 0 ? 0ull : ((1ull << n) - 1ull));
                if (nl > 0) allow &= nl >= 64 ? 0ull : ~((1ull << nl) - 1ull);
                if (row_mask && allow) {
                    const unsigned long long w0 = row_mask[kb0 >> 5];
                    const unsigned long long w1 = (kb0 + 32 < kv_len) ? row_mask[(kb0 >> 5) + 1] : 0u;
                    allow &= w0 | (w1 << 32);
                }
#pragma unroll
                for (int i = 0; i < AT_BK; ++i)
                    if (!((allow >> i) & 1ull)) sv[i] = -INFINITY;
            }
            float bm0 = sv[0], bm1 = sv[1], bm2 = sv[2], bm3 = sv[3];
#pragma unroll
            for (int i = 4; i < AT_BK; i += 4) {
                bm0 = fmaxf(bm0, sv[i]);
                bm1 = fmaxf(bm1, sv[i + 1]);
                bm2 = fmaxf(bm2, sv[i + 2]);
                bm3 = fmaxf(bm3, sv[i + 3]);
            }
            const float bm = fmaxf(fmaxf(bm0, bm1), fmaxf(bm2, bm3));
            // the reference maximum moves only when a row's block maximum outgrows it by 2^8: the
            // accumulator in TMEM is then rescaled by the warp (tcgen05.ld/st are warp-wide)
            const bool grow = bm > m_ref + thr_raw;
            if (__any_sync(0xffffffffu, grow)) {
                const float m_new = fmaxf(m_ref, bm);
                const float alpha = (m_new == -INFINITY) ? 1.f : fast_exp2((m_ref - m_new) * scale_log2);
                m_ref = m_new;
                l *= alpha;
                if (j > 0) {
                    const bool done = mbar_wait(pv_done(t), (j - 1) & 1u, status, PIE_ERR_WAIT_MMA);
                    if (!__all_sync(0xffffffffu, done)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t v[32];
                        tmem_ld_32x32(tm_o + c * 32, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        tmem_st_32x32(tm_o + c * 32, v);
                    }
                    tmem_st_wait();
                }
            }
            const float neg = (m_ref == -INFINITY) ? 0.f : -m_ref * scale_log2;
            const bool freed = mbar_wait(p_empty(t, b), ph ^ 1u, status, PIE_ERR_WAIT_MMA);
            if (!__all_sync(0xffffffffu, freed)) { ok = false; break; }
            // P row (64 bf16 = 128 bytes) into the swizzled tile: 16-byte chunk c of row r at r*128 + ((c ^ (r & 7)) << 4)
            uint8_t* prow = base_ptr + (p_s - base) + (t * 2 + b) * AT_P_BYTES + row * 128;
            float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                float pv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) pv[i] = fast_exp2(__fmaf_rn(sv[c * 8 + i], scale_log2, neg));
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    ps0 += pv[i];
                    ps1 += pv[i + 1];
                }
                *reinterpret_cast<bf16x8*>(prow + ((c ^ (row & 7)) << 4)) = pack8(pv);
            }
            l += ps0 + ps1;
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(t, b));
        }
        if (ok && my_nkb > 0) {
            // pv_done cannot serve here: a parity wait tells apart only neighbouring phases, and by now
            // that barrier may be one phase short of the last or already past it
            const bool done = mbar_wait(o_final(t), 0, status, PIE_ERR_WAIT_MMA);
            ok = __all_sync(0xffffffffu, done);
        }
        if (ok && my_nkb > 0) {
            tc_fence_after();
            const int head = h * G + row % G;
            // attention sink: a per-head logit in the softmax denominator without a value row
            if (sinks_log2 && l > 0.f) l += exp2f(sinks_log2[head] - m_ref * scale_log2);
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* dst = out + ((size_t)(q_base + (valid ? qtok : 0)) * hq + head) * D;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(tm_o + c * 32, v);
                tmem_ld_wait();
                if (valid) {
#pragma unroll
                    for (int i8 = 0; i8 < 4; ++i8) {
                        float tv[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) tv[i] = __uint_as_float(v[i8 * 8 + i]) * inv;
                        *reinterpret_cast<bf16x8*>(dst + c * 32 + i8 * 8) = pack8(tv);
                    }
                }
            }
            if (valid && lse_out)
                lse_out[(size_t)(q_base + qtok) * hq + head] =
                    l > 0.f ? (m_ref * scale_log2 + log2f(l)) * 0.6931471805599453f : -INFINITY;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, AtCfg<NT, D>::TMEM_COLS);
    }
}

}  // namespace pie

using namespace pie;

typedef CUresult (*EncodeTiledFnA)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFnA at_encoder() {
    static EncodeTiledFnA enc = nullptr;
    if (!enc) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        enc = reinterpret_cast<EncodeTiledFnA>(p);
    }
    return enc;
}

// 1 when the tensor-core kernel covers the shape (head_dim 64 or 128, 16-token pages, group size dividing 128).
PIE_API int pie_prefill_attn_tc_supported(int hq, int hkv, int head_dim, int page_size) {
    if (hkv <= 0 || hq % hkv) return 0;
    const int g = hq / hkv;
    return (head_dim == 128 || head_dim == 64) && page_size == 16 && (g == 1 || g == 2 || g == 4 || g == 8 || g == 16) ? 1 : 0;
}

// Same contract as pie_paged_prefill_attn, with tiles of tile_rows / group query tokens (tile_rows = 128 or
// 256: one or two MMA tiles per CTA) and `total_pages` = pages of kv_layer including the pad page (last).
// softcap > 0 (tile_rows 256 only): softmax over softcap * tanh(q.k * sm_scale / softcap).
PIE_API int pie_paged_prefill_attn_tc_softcap(const void* q, const void* kv_layer, const int* page_indices,
                                              const int* kv_page_indptr, const int* qo_indptr, const int* kv_lens,
                                              const int* tile_req, const int* tile_qstart, int num_tiles,
                                              const uint32_t* mask_bits, const long* mask_word_indptr, void* out,
                                              float* lse_out, int n_tokens, int hq, int hkv, int head_dim, int total_pages,
                                              float sm_scale, int window_left, int tile_rows, const float* sinks_log2,
                                              int* status, float softcap, cudaStream_t st) {
    if (num_tiles <= 0) return 0;
    const int D_ = head_dim;
    if (!pie_prefill_attn_tc_supported(hq, hkv, head_dim, 16) || (tile_rows != 128 && tile_rows != 256) || !status)
        return (int)cudaErrorInvalidValue;
    if (softcap > 0.f && tile_rows != 256) return (int)cudaErrorInvalidValue;
    EncodeTiledFnA enc = at_encoder();
    if (!enc) return (int)cudaErrorNotSupported;
    const int G = hq / hkv;
    CUtensorMap tq, tkv;
    {
        cuuint64_t dims[3] = {(cuuint64_t)D_, (cuuint64_t)hq, (cuuint64_t)n_tokens};
        cuuint64_t strides[2] = {(cuuint64_t)D_ * 2, (cuuint64_t)hq * D_ * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(AT_ROWS / G)};
        cuuint32_t estr[3] = {1, 1, 1};
        if (enc(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return (int)cudaErrorInvalidValue;
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)D_, (cuuint64_t)total_pages * 2 * hkv * 16};
        cuuint64_t strides[1] = {(cuuint64_t)D_ * 2};
        cuuint32_t box[2] = {64, 16};
        cuuint32_t estr[2] = {1, 1};
        if (enc(&tkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(kv_layer), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return (int)cudaErrorInvalidValue;
    }
    const float scale_log2 = sm_scale * 1.4426950408889634f;
    dim3 grid(num_tiles, hkv);
    const float cap_pre = softcap > 0.f ? sm_scale / softcap : 0.f, cap_post = softcap > 0.f ? softcap / sm_scale : 0.f;
#define GO4(G_, NT_, D__, CAP_)                                                                                       \
    {                                                                                                                 \
        auto kern = paged_prefill_attn_tc_kernel<G_, NT_, D__, CAP_>;                                                 \
        using Cfg = AtCfg<NT_, D__>;                                                                                  \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM);      \
        if (e != cudaSuccess) return (int)e;                                                                          \
        kern<<<grid, Cfg::THREADS, Cfg::SMEM, st>>>(                                                                  \
            tq, tkv, page_indices, kv_page_indptr, qo_indptr, kv_lens, tile_req, tile_qstart, mask_bits,              \
            mask_word_indptr, (bf16*)out, lse_out, sinks_log2, hq, hkv, total_pages - 1, scale_log2, window_left,     \
            status, cap_pre, cap_post);                                                                               \
        return (int)cudaGetLastError();                                                                               \
    }
#define GO2(G_, NT_)           \
    if (D_ == 128) GO4(G_, NT_, 128, false) else GO4(G_, NT_, 64, false)
#define GO(G_)                 \
    if (softcap > 0.f) { if (D_ == 128) GO4(G_, 2, 128, true) else GO4(G_, 2, 64, true) } \
    else if (tile_rows == 128) GO2(G_, 1) else GO2(G_, 2)
    switch (G) {
        case 1: GO(1)
        case 2: GO(2)
        case 4: GO(4)
        case 8: GO(8)
        case 16: GO(16)
    }
#undef GO
#undef GO2
#undef GO4
    return (int)cudaErrorInvalidValue;
}

PIE_API int pie_paged_prefill_attn_tc(const void* q, const void* kv_layer, const int* page_indices,
                                      const int* kv_page_indptr, const int* qo_indptr, const int* kv_lens,
                                      const int* tile_req, const int* tile_qstart, int num_tiles,
                                      const uint32_t* mask_bits, const long* mask_word_indptr, void* out,
                                      float* lse_out, int n_tokens, int hq, int hkv, int head_dim, int total_pages,
                                      float sm_scale,
                                      int window_left, int tile_rows, const float* sinks_log2, int* status,
                                      cudaStream_t st) {
    return pie_paged_prefill_attn_tc_softcap(q, kv_layer, page_indices, kv_page_indptr, qo_indptr, kv_lens, tile_req,
                                             tile_qstart, num_tiles, mask_bits, mask_word_indptr, out, lse_out, n_tokens,
                                             hq, hkv, head_dim, total_pages, sm_scale, window_left, tile_rows, sinks_log2,
                                             status, 0.f, st);
}

