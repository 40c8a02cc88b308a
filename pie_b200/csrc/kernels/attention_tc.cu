// Paged prefill attention on the 5th-generation tensor cores (head_dim 128, 16-token pages).
//
// One CTA per (tile of 128 packed query rows, KV head); a row is (query token, head within the
// GQA group), so a tile covers 128 / G tokens of one request. KV is walked in blocks of 64 keys:
//   warp 0      TMA producer: the Q tile once (3-D box over [tokens, heads, d]); per block the K
//               and V rows of its four pages (2-D boxes of 16 rows x 64 columns, 128-byte
//               swizzle) into a ring of stages; pages past the end come from the cache's pad page
//   warp 1      tcgen05.mma issuer: S = Q K^T (128 x 64, K-major operands) into one of two TMEM
//               buffers, then O_blk = P V (128 x 128; P from shared memory, V as an MN-major
//               operand straight from its [key, d] tile) into one of two more
//   warps 2-5   softmax, one row per thread: S from TMEM, mask (causal / window / custom bits),
//               running max and sum, P as bf16 into a swizzled shared-memory tile for the next
//               MMA, and the running output in registers: O = (O + O_blk) * alpha per block
// The score and output MMAs of neighbouring blocks overlap the softmax through the double
// buffers. Every wait is bounded; on a time-out the kernel records a status word and leaves.
//
// Replaces the FlashInfer FA2 paged prefill kernel the reference calls
// (driver/cuda/src/ops/attention_flashinfer.cu:848, plans :612,:1075) and this library's own
// mma.sync version for the shapes it covers.
#include "tcgen05.cuh"

namespace pie {
using namespace sm100;

constexpr int AT_ROWS = 128;     // packed query rows per tile
constexpr int AT_BK = 64;        // keys per block
constexpr int AT_D = 128;
constexpr int AT_STAGES = 3;
constexpr int AT_THREADS = 192;
constexpr uint32_t AT_Q_BYTES = AT_ROWS * AT_D * 2;            // two 16 KB halves
constexpr uint32_t AT_KV_TILE = AT_BK * AT_D * 2;              // 16 KB: two 8 KB halves [64 keys x 64 d]
constexpr uint32_t AT_STAGE_BYTES = 2 * AT_KV_TILE;            // K then V
constexpr uint32_t AT_P_BYTES = AT_ROWS * AT_BK * 2;           // 16 KB
constexpr uint32_t AT_SMEM = AT_Q_BYTES + AT_STAGES * AT_STAGE_BYTES + 2 * AT_P_BYTES + 1024 + 512;
constexpr uint32_t AT_TMEM_COLS = 512;                          // S[2] x 64 + O_blk[2] x 128 = 384 -> 512

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

template <int G>
__global__ void __launch_bounds__(AT_THREADS, 1)
paged_prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_kv,
                             const int* __restrict__ page_indices, const int* __restrict__ kv_page_indptr,
                             const int* __restrict__ qo_indptr, const int* __restrict__ kv_lens,
                             const int* __restrict__ tile_req, const int* __restrict__ tile_qstart,
                             const uint32_t* __restrict__ mask_bits, const long* __restrict__ mask_word_indptr,
                             bf16* __restrict__ out, float* __restrict__ lse_out, int hq, int hkv, int pad_page,
                             float scale_log2, int window_left, int* status) {
    constexpr int TQ = AT_ROWS / G;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_addr(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t q_s = base;
    const uint32_t kv_s = q_s + AT_Q_BYTES;
    const uint32_t p_s = kv_s + AT_STAGES * AT_STAGE_BYTES;
    const uint32_t bar0 = p_s + 2 * AT_P_BYTES;
    // barriers: q_full, kv_full[ST], kv_empty[ST], s_full[2], s_empty[2], p_full[2], p_empty[2], o_full[2], o_empty[2]
    auto q_full = [&]() { return bar0; };
    auto kv_full = [&](int s) { return bar0 + 8u * (1 + s); };
    auto kv_empty = [&](int s) { return bar0 + 8u * (1 + AT_STAGES + s); };
    auto s_full = [&](int b) { return bar0 + 8u * (1 + 2 * AT_STAGES + b); };
    auto s_empty = [&](int b) { return bar0 + 8u * (3 + 2 * AT_STAGES + b); };
    auto p_full = [&](int b) { return bar0 + 8u * (5 + 2 * AT_STAGES + b); };
    auto p_empty = [&](int b) { return bar0 + 8u * (7 + 2 * AT_STAGES + b); };
    auto o_full = [&](int b) { return bar0 + 8u * (9 + 2 * AT_STAGES + b); };
    auto o_empty = [&](int b) { return bar0 + 8u * (11 + 2 * AT_STAGES + b); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + (bar0 - base) + 8u * (13 + 2 * AT_STAGES));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, h = blockIdx.y;
    const int req = tile_req[tile], qstart = tile_qstart[tile];
    const int q_base = qo_indptr[req];
    const int qo_len = qo_indptr[req + 1] - q_base;
    const int kv_len = kv_lens[req];
    const int* pages = page_indices + kv_page_indptr[req];
    const bool custom = mask_bits != nullptr;
    const int last_q = min(qstart + TQ, qo_len) - 1;
    const int kv_hi = custom ? kv_len : max(0, min(kv_len, kv_len - qo_len + last_q + 1));
    const int nkb = (kv_hi + AT_BK - 1) / AT_BK;
    const int npages = (kv_hi + 15) >> 4;

    if (threadIdx.x == 0) {
        mbar_init(q_full(), 1);
        for (int s = 0; s < AT_STAGES; ++s) {
            mbar_init(kv_full(s), 1);
            mbar_init(kv_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(s_full(b), 1);
            mbar_init(s_empty(b), 4);
            mbar_init(p_full(b), 4);
            mbar_init(p_empty(b), 1);
            mbar_init(o_full(b), 1);
            mbar_init(o_empty(b), 4);
        }
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        tmem_alloc(smem_addr(const_cast<uint32_t*>(tmem_slot)), AT_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tm_s = tmem_base;                // S buffers: columns [0, 64) and [64, 128)
    const uint32_t tm_o = tmem_base + 128;          // O_blk buffers: columns [128, 256) and [256, 384)

    if (warp == 0) {
        if (lane == 0 && nkb > 0) {
            tma_prefetch_desc(&tma_q);
            tma_prefetch_desc(&tma_kv);
            mbar_arrive_expect_tx(q_full(), AT_Q_BYTES);
            tma_load_3d(q_s, &tma_q, q_full(), 0, h * G, q_base + qstart);
            tma_load_3d(q_s + AT_Q_BYTES / 2, &tma_q, q_full(), 64, h * G, q_base + qstart);
            bool ok = true;
            for (int j = 0; j < nkb && ok; ++j) {
                const int s = j % AT_STAGES;
                if (!mbar_wait(kv_empty(s), ((j / AT_STAGES) & 1u) ^ 1u, status, PIE_ERR_WAIT_TMA)) { ok = false; break; }
                mbar_arrive_expect_tx(kv_full(s), AT_STAGE_BYTES);
                const uint32_t kdst = kv_s + s * AT_STAGE_BYTES;
                for (int pg = 0; pg < 4; ++pg) {
                    const int pi = j * 4 + pg;
                    const int page = pi < npages ? pages[pi] : pad_page;
                    const int krow = ((page * 2) * hkv + h) * 16;
                    const int vrow = ((page * 2 + 1) * hkv + h) * 16;
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        tma_load_2d(kdst + half * (AT_KV_TILE / 2) + pg * 2048, &tma_kv, kv_full(s), half * 64, krow);
                        tma_load_2d(kdst + AT_KV_TILE + half * (AT_KV_TILE / 2) + pg * 2048, &tma_kv, kv_full(s), half * 64, vrow);
                    }
                }
            }
            // no copy may be in flight when the CTA exits
            const int first = nkb > AT_STAGES ? nkb - AT_STAGES : 0;
            for (int j = first; j < nkb; ++j)
                mbar_wait(kv_full(j % AT_STAGES), (j / AT_STAGES) & 1u, status, PIE_ERR_WAIT_TMA, 200000000ll);
        }
    } else if (warp == 1) {
        if (lane == 0 && nkb > 0) {
            constexpr uint32_t idesc_s = make_idesc_bf16(AT_ROWS, AT_BK);
            constexpr uint32_t idesc_o = make_idesc_bf16_bmn(AT_ROWS, AT_D);
            bool ok = mbar_wait(q_full(), 0, status, PIE_ERR_WAIT_TMA);
            auto issue_pv = [&](int j) {
                const int s = j % AT_STAGES;
                const uint32_t b = j & 1u, ph = (j >> 1) & 1u;
                if (!mbar_wait(p_full(b), ph, status, PIE_ERR_WAIT_EPILOGUE)) { ok = false; return; }
                if (!mbar_wait(o_empty(b), ph ^ 1u, status, PIE_ERR_WAIT_EPILOGUE)) { ok = false; return; }
                tc_fence_after();
                const uint32_t v_addr = kv_s + s * AT_STAGE_BYTES + AT_KV_TILE;
                const uint32_t p_addr = p_s + b * AT_P_BYTES;
#pragma unroll
                for (int k = 0; k < AT_BK / 16; ++k) {
                    const uint64_t adesc = make_smem_desc_sw128(p_addr) + 2u * k;                       // 16 keys = 32 bytes along a P row
                    const uint64_t bdesc = make_smem_desc_sw128_mn(v_addr + k * 2048, AT_KV_TILE / 2);  // 16 keys = two 8-row groups
                    umma_bf16(tm_o + b * AT_D, adesc, bdesc, idesc_o, k != 0);
                }
                umma_commit(o_full(b));
                umma_commit(kv_empty(s));
                umma_commit(p_empty(b));
            };
            for (int j = 0; j < nkb && ok; ++j) {
                const int s = j % AT_STAGES;
                const uint32_t b = j & 1u, ph = (j >> 1) & 1u;
                if (!mbar_wait(kv_full(s), (j / AT_STAGES) & 1u, status, PIE_ERR_WAIT_TMA)) { ok = false; break; }
                if (!mbar_wait(s_empty(b), ph ^ 1u, status, PIE_ERR_WAIT_EPILOGUE)) { ok = false; break; }
                tc_fence_after();
                const uint32_t k_addr = kv_s + s * AT_STAGE_BYTES;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint64_t adesc = make_smem_desc_sw128(q_s + half * (AT_Q_BYTES / 2));
                    const uint64_t bdesc = make_smem_desc_sw128(k_addr + half * (AT_KV_TILE / 2));
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        umma_bf16(tm_s + b * AT_BK, adesc + 2u * k, bdesc + 2u * k, idesc_s, (half | k) != 0);
                }
                umma_commit(s_full(b));
                if (j >= 1) issue_pv(j - 1);
            }
            if (ok) issue_pv(nkb - 1);
        }
    } else {
        // ------------------------------------------------------------ softmax + output (thread = row)
        const int q4 = warp & 3;
        const int row = q4 * 32 + lane;
        const int qtok = qstart + row / G;
        const bool valid = qtok < qo_len;
        const int lim = valid ? (custom ? kv_len : kv_len - qo_len + qtok + 1) : 0;
        const int lo = (window_left >= 0 && valid) ? max(0, kv_len - qo_len + qtok - window_left) : 0;
        const int mask_words = (kv_len + 31) >> 5;
        const uint32_t* row_mask = (custom && valid) ? mask_bits + mask_word_indptr[req] + (size_t)qtok * mask_words : nullptr;
        const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
        float o[AT_D];
#pragma unroll
        for (int c = 0; c < AT_D; ++c) o[c] = 0.f;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        auto fold_o = [&](int j, float alpha) {
            // o = (o + O_blk_j) * alpha
            const uint32_t b = j & 1u, ph = (j >> 1) & 1u;
            const bool got = mbar_wait(o_full(b), ph, status, PIE_ERR_WAIT_MMA);
            if (!__all_sync(0xffffffffu, got)) { ok = false; return; }
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < AT_D / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(tm_o + lane_base + b * AT_D + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[c * 32 + i] = (o[c * 32 + i] + __uint_as_float(v[i])) * alpha;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_empty(b));
        };
        for (int j = 0; j < nkb && ok; ++j) {
            const uint32_t b = j & 1u, ph = (j >> 1) & 1u;
            const bool got = mbar_wait(s_full(b), ph, status, PIE_ERR_WAIT_MMA);
            if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
            tc_fence_after();
            float sv[AT_BK];
#pragma unroll
            for (int c = 0; c < AT_BK / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32(tm_s + lane_base + b * AT_BK + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) sv[c * 32 + i] = __uint_as_float(v[i]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_empty(b));
            // mask and running max
            const int kb0 = j * AT_BK;
            uint32_t mw0 = 0xffffffffu, mw1 = 0xffffffffu;
            if (row_mask) {
                mw0 = row_mask[kb0 >> 5];
                mw1 = (kb0 + 32 < kv_len) ? row_mask[(kb0 >> 5) + 1] : 0u;
            }
            float bm = -INFINITY;
#pragma unroll
            for (int i = 0; i < AT_BK; ++i) {
                const int key = kb0 + i;
                const bool allow = key < lim && key >= lo && (((i < 32 ? mw0 : mw1) >> (i & 31)) & 1u);
                sv[i] = allow ? sv[i] * scale_log2 : -INFINITY;
                bm = fmaxf(bm, sv[i]);
            }
            const float m_new = fmaxf(m, bm);
            const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m - m_new);   // m = -inf, m_new finite -> 0
            float psum = 0.f;
            // P row (64 bf16 = 128 bytes) into the swizzled tile: 16-byte chunk c of row r at r*128 + ((c ^ (r & 7)) << 4)
            if (!mbar_wait(p_empty(b), ph ^ 1u, status, PIE_ERR_WAIT_MMA)) ok = false;
            if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
            uint8_t* prow = base_ptr + (p_s - base) + b * AT_P_BYTES + row * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                float pv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float sx = sv[c * 8 + i];
                    pv[i] = (sx == -INFINITY) ? 0.f : exp2f(sx - m_new);
                }
                // the sum uses the bf16-rounded values the MMA will see
                bf16x8 pk = pack8(pv);
                float pr[8];
                unpack8(pk, pr);
#pragma unroll
                for (int i = 0; i < 8; ++i) psum += pr[i];
                *reinterpret_cast<bf16x8*>(prow + ((c ^ (row & 7)) << 4)) = pk;
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(b));
            l = l * alpha + psum;
            m = m_new;
            if (j >= 1) fold_o(j - 1, alpha);
        }
        if (ok && nkb > 0) fold_o(nkb - 1, 1.f);
        if (valid && ok) {
            const int head = h * G + row % G;
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* dst = out + ((size_t)(q_base + qtok) * hq + head) * AT_D;
#pragma unroll
            for (int c = 0; c < AT_D / 8; ++c) {
                float t[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) t[i] = o[c * 8 + i] * inv;
                *reinterpret_cast<bf16x8*>(dst + c * 8) = pack8(t);
            }
            if (lse_out)
                lse_out[(size_t)(q_base + qtok) * hq + head] = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, AT_TMEM_COLS);
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

// 1 when the tensor-core kernel covers the shape (head_dim 128, 16-token pages, group size dividing 128).
PIE_API int pie_prefill_attn_tc_supported(int hq, int hkv, int head_dim, int page_size) {
    if (hkv <= 0 || hq % hkv) return 0;
    const int g = hq / hkv;
    return head_dim == 128 && page_size == 16 && (g == 1 || g == 2 || g == 4 || g == 8 || g == 16) ? 1 : 0;
}

// Same contract as pie_paged_prefill_attn, with tiles of 128 / group query tokens
// (pie_prefill_tc_tile_tokens) and `total_pages` = pages of kv_layer including the pad page (last).
PIE_API int pie_prefill_tc_tile_tokens(int group) { return AT_ROWS / group; }

PIE_API int pie_paged_prefill_attn_tc(const void* q, const void* kv_layer, const int* page_indices,
                                      const int* kv_page_indptr, const int* qo_indptr, const int* kv_lens,
                                      const int* tile_req, const int* tile_qstart, int num_tiles,
                                      const uint32_t* mask_bits, const long* mask_word_indptr, void* out,
                                      float* lse_out, int n_tokens, int hq, int hkv, int total_pages, float sm_scale,
                                      int window_left, int* status, cudaStream_t st) {
    if (num_tiles <= 0) return 0;
    if (!pie_prefill_attn_tc_supported(hq, hkv, AT_D, 16)) return (int)cudaErrorInvalidValue;
    EncodeTiledFnA enc = at_encoder();
    if (!enc) return (int)cudaErrorNotSupported;
    const int G = hq / hkv;
    CUtensorMap tq, tkv;
    {
        cuuint64_t dims[3] = {(cuuint64_t)AT_D, (cuuint64_t)hq, (cuuint64_t)n_tokens};
        cuuint64_t strides[2] = {(cuuint64_t)AT_D * 2, (cuuint64_t)hq * AT_D * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(AT_ROWS / G)};
        cuuint32_t estr[3] = {1, 1, 1};
        if (enc(&tq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return (int)cudaErrorInvalidValue;
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)AT_D, (cuuint64_t)total_pages * 2 * hkv * 16};
        cuuint64_t strides[1] = {(cuuint64_t)AT_D * 2};
        cuuint32_t box[2] = {64, 16};
        cuuint32_t estr[2] = {1, 1};
        if (enc(&tkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(kv_layer), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return (int)cudaErrorInvalidValue;
    }
    const float scale_log2 = sm_scale * 1.4426950408889634f;
    dim3 grid(num_tiles, hkv);
#define GO(G_)                                                                                                  \
    {                                                                                                           \
        auto kern = paged_prefill_attn_tc_kernel<G_>;                                                           \
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)AT_SMEM);  \
        if (e != cudaSuccess) return (int)e;                                                                    \
        kern<<<grid, AT_THREADS, AT_SMEM, st>>>(tq, tkv, page_indices, kv_page_indptr, qo_indptr, kv_lens, tile_req, \
                                                tile_qstart, mask_bits, mask_word_indptr, (bf16*)out, lse_out, hq, hkv, \
                                                total_pages - 1, scale_log2, window_left, status);             \
        return (int)cudaGetLastError();                                                                         \
    }
    switch (G) {
        case 1: GO(1)
        case 2: GO(2)
        case 4: GO(4)
        case 8: GO(8)
        case 16: GO(16)
    }
#undef GO
    return (int)cudaErrorInvalidValue;
}
