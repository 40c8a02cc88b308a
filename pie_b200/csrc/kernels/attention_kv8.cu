// Paged decode attention over fp8 (e4m3) KV pages with one fp32 scale per (token, KV head).
//
// KV layer layout: data [pages][2][Hkv][page_size][D] bytes (K then V per page) and scales
// [pages][2][Hkv][page_size] fp32; a stored row is x / scale rounded to e4m3 with
// scale = max|x| / 448, written by qk_norm_rope_kvwrite (elementwise.cu). Decode is bound by the
// KV bytes it streams, so halving them is the point: per 16-token block a warp copies 2 KB of K
// and 2 KB of V (instead of 4 KB each) plus 128 B of scales with cp.async, expands the bytes to
// f16 in shared memory (one cvt per pair; e4m3 is exact in f16), and runs the same m16n8k16
// tensor-core tiles as the bf16 kernel with f16 operands. The scales never touch the tiles:
// S[:, t] is multiplied by the K scale of token t after QK^T, and P[:, t] by the V scale of token
// t before PV. Work items, split-KV partial results and the merge pass are those of the bf16
// kernel (attention.cu); shared-prefix items are not supported here.
//
// Reference behaviour: the reference stores fp8 / int8 KV with per-token-head side scales
// (driver/cuda/src/kv_cache.hpp:1-202, kernels/kv_paged.cu:188-325) and dequantises the active
// pages to a bf16 scratch before FlashInfer runs (kernels/kv_paged.cu:418-496); here the decode
// kernel reads the fp8 pages directly.
#include <cuda_fp8.h>

#include "common.cuh"

extern "C" int pie_decode_merge(const float* o_part, const float* lse_part, const int* req_item_indptr, void* out,
                                int num_reqs, int hq, int hkv, int head_dim, const float* sinks_log2, int max_items,
                                cudaStream_t st);
extern "C" int* pie_status_word_current();

namespace pie {
namespace kv8 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// two e4m3 bytes -> f16x2 (exact)
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint16_t v) {
    const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)v, __NV_E4M3);
    return (uint32_t)h.x | ((uint32_t)h.y << 16);
}
// Byte offset of 16-byte chunk `chunk` of row `row` in a [rows][D] 16-bit tile, chunks XOR-swizzled by row.
template <int D>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return (uint32_t)(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}

constexpr int WARPS = 4;
constexpr int STAGES = 3;

// shared memory: Q tile (f16) | per warp: fp8 ring [STAGES][K 16xD, V 16xD bytes] + scales [STAGES][2][16] | per warp one
// f16 K tile and one f16 V tile. The merge space of an item reuses the per-warp regions.
template <int D>
struct Layout {
    static constexpr int Q_BYTES = 16 * D * 2;
    static constexpr int RAW_TILE = 16 * D;                       // one fp8 K or V block
    static constexpr int RING = STAGES * (2 * RAW_TILE + 128);    // + 16 K scales + 16 V scales
    static constexpr int F16_TILE = 16 * D * 2;
    static constexpr int WARP_BYTES = RING + 2 * F16_TILE;
    static constexpr int TOTAL = Q_BYTES + WARPS * WARP_BYTES;
};

template <int D, int G>
__global__ void __launch_bounds__(WARPS * 32)
paged_decode_attn_kv8_kernel(const bf16* __restrict__ q, const uint8_t* __restrict__ kv_layer,
                             const float* __restrict__ kv_scale, const int* __restrict__ page_indices,
                             const int* __restrict__ kv_page_indptr, const int* __restrict__ item_req,
                             const int* __restrict__ item_start, const int* __restrict__ item_end,
                             const int* __restrict__ req_item_indptr, const int* __restrict__ num_items_ptr,
                             bf16* __restrict__ out, float* __restrict__ o_part, float* __restrict__ lse_part, int hq,
                             int hkv, int page_size, float scale_log2, int window_left,
                             const float* __restrict__ sinks_log2, int max_items, int num_reqs,
                             int* __restrict__ status) {
    static_assert(G <= 16, "at most 16 query heads per KV head");
    using L = Layout<D>;
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr int CH = D / 8;          // 16-byte chunks per f16 row
    constexpr int CH8 = D / 16;        // 16-byte chunks per fp8 row
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t q_smem = smem_u32(smem);
    uint8_t* wbase = smem + L::Q_BYTES + warp * L::WARP_BYTES;
    const uint32_t k16 = smem_u32(wbase + L::RING), v16 = k16 + L::F16_TILE;
    pdl_trigger();
    pdl_wait();
    int n_items = *num_items_ptr;
    if (n_items > max_items || n_items < 0) {
        if (threadIdx.x == 0 && blockIdx.x == 0 && status) atomicCAS(status, 0, PIE_ERR_BOUNDS);
        n_items = n_items < 0 ? 0 : max_items;
    }
    const long total = (long)n_items * hkv;

    for (long w = blockIdx.x; w < total; w += gridDim.x) {
        const int it = (int)(w / hkv), h = (int)(w - (long)it * hkv);
        const int req = item_req[it];
        if (req < 0 || req >= num_reqs) {
            if (threadIdx.x == 0 && status) atomicCAS(status, 0, PIE_ERR_BOUNDS);
            continue;
        }
        const int kv_start = item_start[it], kv_end = item_end[it];
        const int kv_lo = window_left >= 0 ? max(0, item_end[req_item_indptr[req + 1] - 1] - 1 - window_left) : 0;
        __syncthreads();  // previous item's merge reads are done
        // Q tile in f16: rows < G are the heads of this KV head, the rest zeros
        for (int c = threadIdx.x; c < 16 * CH; c += blockDim.x) {
            const int row = c / CH, col = c - row * CH;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < G) {
                const uint4 raw = *reinterpret_cast<const uint4*>(q + ((size_t)req * hq + h * G + row) * D + col * 8);
                const bf162* b = reinterpret_cast<const bf162*>(&raw);
                uint32_t* o = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(b[e]);
                    o[e] = pack_f16(f.x, f.y);
                }
            }
            *reinterpret_cast<uint4*>(smem + swz<D>(row, col)) = v;
        }
        __syncthreads();
        uint32_t qf[D / 16][4];
        {
            const int mi = lane >> 3, r = lane & 7;
            const int row = r + (mi & 1) * 8;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)
                ldsm_x4(q_smem + swz<D>(row, ks * 2 + (mi >> 1)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
        }
        float o_acc[D / 8][4];
#pragma unroll
        for (int i = 0; i < D / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

        const int nb_total = (kv_end - kv_start + 15) >> 4;
        const int my_count = nb_total > warp ? (nb_total - warp + WARPS - 1) / WARPS : 0;
        const int* pages = page_indices + kv_page_indptr[req];

        auto issue = [&](int j) {
            const int tok0 = kv_start + (warp + WARPS * j) * 16;
            const int page = pages[tok0 / page_size];
            const int off = tok0 % page_size;
            const size_t kblk = (((size_t)page * 2) * hkv + h) * page_size + off;       // in tokens
            const size_t vblk = (((size_t)page * 2 + 1) * hkv + h) * page_size + off;
            uint8_t* st = wbase + (j % STAGES) * (2 * L::RAW_TILE + 128);
            const uint32_t kdst = smem_u32(st), vdst = kdst + L::RAW_TILE, sdst = vdst + L::RAW_TILE;
#pragma unroll
            for (int i = 0; i < (16 * CH8 + 31) / 32; ++i) {
                const int c = lane + 32 * i;
                if (c < 16 * CH8) {
                    cp_async16(kdst + c * 16, kv_layer + kblk * D + (size_t)c * 16);
                    cp_async16(vdst + c * 16, kv_layer + vblk * D + (size_t)c * 16);
                }
            }
            if (lane < 4) cp_async16(sdst + lane * 16, kv_scale + kblk + lane * 4);
            else if (lane < 8) cp_async16(sdst + 64 + (lane - 4) * 16, kv_scale + vblk + (lane - 4) * 4);
        };
#pragma unroll
        for (int s = 0; s < STAGES - 1; ++s) {
            if (s < my_count) issue(s);
            cp_async_commit();
        }
        for (int i = 0; i < my_count; ++i) {
            if (i + STAGES - 1 < my_count) issue(i + STAGES - 1);
            cp_async_commit();
            cp_async_wait<STAGES - 1>();
            __syncwarp();
            const uint8_t* st = wbase + (i % STAGES) * (2 * L::RAW_TILE + 128);
            // expand the block: every 16-byte chunk of fp8 becomes two 16-byte chunks of f16 in the swizzled tiles
#pragma unroll
            for (int u = 0; u < (16 * CH8 + 31) / 32; ++u) {
                const int c = lane + 32 * u;
                if (c < 16 * CH8) {
                    const int row = c / CH8, c8 = c - row * CH8;
#pragma unroll
                    for (int kv = 0; kv < 2; ++kv) {
                        const uint4 raw = *reinterpret_cast<const uint4*>(st + kv * L::RAW_TILE + c * 16);
                        const uint16_t* p2 = reinterpret_cast<const uint16_t*>(&raw);
                        uint4 lo, hi;
                        lo.x = e4m3x2_to_f16x2(p2[0]); lo.y = e4m3x2_to_f16x2(p2[1]);
                        lo.z = e4m3x2_to_f16x2(p2[2]); lo.w = e4m3x2_to_f16x2(p2[3]);
                        hi.x = e4m3x2_to_f16x2(p2[4]); hi.y = e4m3x2_to_f16x2(p2[5]);
                        hi.z = e4m3x2_to_f16x2(p2[6]); hi.w = e4m3x2_to_f16x2(p2[7]);
                        uint8_t* dst = wbase + L::RING + kv * L::F16_TILE;
                        *reinterpret_cast<uint4*>(dst + swz<D>(row, 2 * c8)) = lo;
                        *reinterpret_cast<uint4*>(dst + swz<D>(row, 2 * c8 + 1)) = hi;
                    }
                }
            }
            const float* ksc = reinterpret_cast<const float*>(st + 2 * L::RAW_TILE);
            const float* vsc = ksc + 16;
            __syncwarp();
            const int tok0 = kv_start + (warp + WARPS * i) * 16;
            const int nvalid = kv_end - tok0;
            uint32_t allow = nvalid >= 16 ? 0xffffu : ((1u << nvalid) - 1u);
            if (kv_lo > tok0) allow &= kv_lo - tok0 >= 16 ? 0u : ~((1u << (kv_lo - tok0)) - 1u);
            // ---- S = Q K^T (raw e4m3 values), column scale, online softmax, O += (P * v-scale) V
            const int mi = lane >> 3, r = lane & 7, t = lane & 3;
            float s[2][2][4];
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int b = 0; b < 2; ++b) s[a][b][0] = s[a][b][1] = s[a][b][2] = s[a][b][3] = 0.f;
            {
                const int token = r + (mi >> 1) * 8;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    uint32_t b00, b01, b10, b11;
                    ldsm_x4(k16 + swz<D>(token, ks * 2 + (mi & 1)), b00, b01, b10, b11);
                    mma_f16(s[0][ks & 1], qf[ks], b00, b01);
                    mma_f16(s[1][ks & 1], qf[ks], b10, b11);
                }
            }
            float p[2][4], vs[2][2];
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int tok = j * 8 + 2 * t + (e & 1);
                    float v = (s[j][0][e] + s[j][1][e]) * (scale_log2 * ksc[tok]);
                    v = ((allow >> tok) & 1u) ? v : -INFINITY;
                    p[j][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                vs[j][0] = (nvalid > j * 8 + 2 * t) ? vsc[j * 8 + 2 * t] : 0.f;
                vs[j][1] = (nvalid > j * 8 + 2 * t + 1) ? vsc[j * 8 + 2 * t + 1] : 0.f;
            }
            float alpha[2], mref[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
                mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
                const float mnew = fmaxf(m_run[hh], mx[hh]);
                mref[hh] = (mnew == -INFINITY) ? 0.f : mnew;
                alpha[hh] = exp2f(m_run[hh] - mref[hh]);
                m_run[hh] = mnew;
            }
            float rs[2] = {0.f, 0.f};
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    p[j][e] = exp2f(p[j][e] - mref[e >> 1]);
                    rs[e >> 1] += p[j][e];
                }
            l_run[0] = l_run[0] * alpha[0] + rs[0];
            l_run[1] = l_run[1] * alpha[1] + rs[1];
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                o_acc[n][0] *= alpha[0];
                o_acc[n][1] *= alpha[0];
                o_acc[n][2] *= alpha[1];
                o_acc[n][3] *= alpha[1];
            }
            uint32_t pa[4];
            pa[0] = pack_f16(p[0][0] * vs[0][0], p[0][1] * vs[0][1]);
            pa[1] = pack_f16(p[0][2] * vs[0][0], p[0][3] * vs[0][1]);
            pa[2] = pack_f16(p[1][0] * vs[1][0], p[1][1] * vs[1][1]);
            pa[3] = pack_f16(p[1][2] * vs[1][0], p[1][3] * vs[1][1]);
            {
                const int token = r + (mi & 1) * 8;
#pragma unroll
                for (int np = 0; np < D / 16; ++np) {
                    uint32_t v0, v1, v2, v3;
                    ldsm_x4_t(v16 + swz<D>(token, np * 2 + (mi >> 1)), v0, v1, v2, v3);
                    mma_f16(o_acc[2 * np], pa, v0, v1);
                    mma_f16(o_acc[2 * np + 1], pa, v2, v3);
                }
            }
            __syncwarp();
        }
        cp_async_wait<0>();
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
            l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
        }
        __syncthreads();  // every warp is done with its buffers: reuse as merge space
        float* sm_m = reinterpret_cast<float*>(smem + L::Q_BYTES);   // [W][16]
        float* sm_l = sm_m + WARPS * 16;                              // [W][16]
        float* sm_o = sm_l + WARPS * 16;                              // [W][G][D]
        {
            const int g = lane >> 2, t = lane & 3;
            if (t == 0) {
                sm_m[warp * 16 + g] = m_run[0];
                sm_l[warp * 16 + g] = l_run[0];
                sm_m[warp * 16 + g + 8] = m_run[1];
                sm_l[warp * 16 + g + 8] = l_run[1];
            }
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                if (g < G) {
                    sm_o[(warp * G + g) * D + n * 8 + 2 * t] = o_acc[n][0];
                    sm_o[(warp * G + g) * D + n * 8 + 2 * t + 1] = o_acc[n][1];
                }
                if (G > 8 && g + 8 < G) {
                    sm_o[(warp * G + g + 8) * D + n * 8 + 2 * t] = o_acc[n][2];
                    sm_o[(warp * G + g + 8) * D + n * 8 + 2 * t + 1] = o_acc[n][3];
                }
            }
        }
        __syncthreads();
        const bool single = (req_item_indptr[req + 1] - req_item_indptr[req]) == 1;
        for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
            const int row = idx / D, dim = idx - row * D;
            float M = -INFINITY;
#pragma unroll
            for (int ww = 0; ww < WARPS; ++ww) M = fmaxf(M, sm_m[ww * 16 + row]);
            float Ls = 0.f, O = 0.f;
            if (M != -INFINITY) {
#pragma unroll
                for (int ww = 0; ww < WARPS; ++ww) {
                    const float sc = exp2f(sm_m[ww * 16 + row] - M);
                    Ls += sm_l[ww * 16 + row] * sc;
                    O += sm_o[(ww * G + row) * D + dim] * sc;
                }
            }
            float val = Ls > 0.f ? O / Ls : 0.f;
            if (single) {
                if (sinks_log2 && Ls > 0.f) val = O / (Ls + exp2f(sinks_log2[h * G + row] - M));
                out[((size_t)req * hq + h * G + row) * D + dim] = __float2bfloat16(val);
            } else {
                o_part[(((size_t)it * hkv + h) * G + row) * D + dim] = val;
                if (dim == 0) lse_part[((size_t)it * hkv + h) * G + row] = Ls > 0.f ? M + log2f(Ls) : -INFINITY;
            }
        }
    }
}

// Expand fp8 pages to bf16: dst page j (of a compact scratch [n][2][Hkv][page][D] bf16) = source page src_pages[j].
template <int D>
__global__ void dequant_kv_pages_kernel(const uint8_t* __restrict__ kv8, const float* __restrict__ scale,
                                        const int* __restrict__ src_pages, bf16* __restrict__ dst, int rows_per_page) {
    const int j = blockIdx.x;
    const size_t src = (size_t)src_pages[j] * rows_per_page, dbase = (size_t)j * rows_per_page;
    for (int rix = threadIdx.x / (D / 8); rix < rows_per_page; rix += blockDim.x / (D / 8)) {
        const int c = threadIdx.x % (D / 8);                       // 8 elements per thread
        const float sc = scale[src + rix];
        const uint2 raw = *reinterpret_cast<const uint2*>(kv8 + (src + rix) * D + c * 8);
        const uint16_t* p2 = reinterpret_cast<const uint16_t*>(&raw);
        float f[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t h2 = e4m3x2_to_f16x2(p2[e]);
            const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&h2));
            f[2 * e] = v.x * sc;
            f[2 * e + 1] = v.y * sc;
        }
        *reinterpret_cast<bf16x8*>(dst + (dbase + rix) * D + c * 8) = pack8(f);
    }
}

}  // namespace kv8
}  // namespace pie

using namespace pie;

// Decode attention over fp8 KV pages (see the header of this file). Arguments as pie_paged_decode_attn_window
// plus the per-(token, head) scales of the layer.
PIE_API int pie_paged_decode_attn_kv8(const void* q, const void* kv_layer, const float* kv_scale,
                                      const int* page_indices, const int* kv_page_indptr, const int* item_req,
                                      const int* item_start, const int* item_end, const int* req_item_indptr,
                                      const int* num_items_ptr, void* out, float* scratch, int max_items,
                                      int num_reqs, int hq, int hkv, int head_dim, int page_size, float sm_scale,
                                      int num_ctas, int window_left, const float* sinks_log2, cudaStream_t st) {
    if (num_reqs <= 0) return 0;
    if (hkv <= 0 || hq % hkv || page_size % 16) return (int)cudaErrorInvalidValue;
    const int group = hq / hkv;
    float* o_part = scratch;
    float* lse_part = scratch + (size_t)max_items * hq * head_dim;
    const float scale_log2 = sm_scale * 1.4426950408889634f;
    int* status = pie_status_word_current();
#define GO(D_, G_)                                                                                            \
    {                                                                                                         \
        auto kern = kv8::paged_decode_attn_kv8_kernel<D_, G_>;                                                \
        constexpr int SM = kv8::Layout<D_>::TOTAL;                                                            \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM);                          \
        launch_pdl(kern, dim3(num_ctas), dim3(kv8::WARPS * 32), SM, st, (const bf16*)q, (const uint8_t*)kv_layer, \
                   kv_scale, page_indices, kv_page_indptr, item_req, item_start, item_end, req_item_indptr,  \
                   num_items_ptr, (bf16*)out, o_part, lse_part, hq, hkv, page_size, scale_log2, window_left,  \
                   sinks_log2, max_items, num_reqs, status);                                                  \
    }
#define GO_D(D_)                                                     \
    switch (group) {                                                 \
        case 1: GO(D_, 1) break;                                     \
        case 2: GO(D_, 2) break;                                     \
        case 4: GO(D_, 4) break;                                     \
        case 8: GO(D_, 8) break;                                     \
        case 16: GO(D_, 16) break;                                   \
        default: return (int)cudaErrorInvalidValue;                  \
    }
    if (head_dim == 128) { GO_D(128) }
    else if (head_dim == 64) { GO_D(64) }
    else return (int)cudaErrorInvalidValue;
#undef GO_D
#undef GO
    int err = (int)cudaGetLastError();
    if (err) return err;
    return pie_decode_merge(o_part, lse_part, req_item_indptr, out, num_reqs, hq, hkv, head_dim, sinks_log2,
                            max_items, st);
}

// dst[j] (bf16 page of a compact scratch) = dequantised source page src_pages[j], for n pages of one layer.
PIE_API int pie_dequant_kv_pages(const void* kv8_layer, const float* scale_layer, const int* src_pages, void* dst,
                                 int n, int hkv, int page_size, int head_dim, cudaStream_t st) {
    if (n <= 0) return 0;
    const int rows = 2 * hkv * page_size;
    if (head_dim == 128)
        kv8::dequant_kv_pages_kernel<128><<<n, 256, 0, st>>>((const uint8_t*)kv8_layer, scale_layer, src_pages, (bf16*)dst, rows);
    else if (head_dim == 64)
        kv8::dequant_kv_pages_kernel<64><<<n, 256, 0, st>>>((const uint8_t*)kv8_layer, scale_layer, src_pages, (bf16*)dst, rows);
    else
        return (int)cudaErrorInvalidValue;
    return (int)cudaGetLastError();
}
