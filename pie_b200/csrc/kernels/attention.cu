// Paged attention over inferlet-owned page tables.
//
//  * paged_decode_attn: one query token per request, GQA heads of one KV head
//    packed as the rows of a 16-row tensor-core tile, split-KV over a host-built
//    list of (request, kv range) work items walked by a persistent grid (graph
//    safe: the item count is read from device memory), partial results merged
//    by a second kernel when a request has more than one item.
//  * paged_prefill_attn: ragged query lengths, causal or custom bit-mask,
//    optional sliding window, 64-row tiles of (query token, head-in-group).
//
// KV layer layout: [pages][2][Hkv][page_size][D] bf16 (K then V per page), so a
// (page, head) K or V block is one contiguous page_size*D*2-byte run.
// page_size must be a multiple of 16.
//
// Reference behaviour: driver/cuda/src/ops/attention_flashinfer.cu:301-312,714
// (decode, split-KV plan), :612,848,1075 (prefill, custom mask, window).
#include "common.cuh"

namespace pie {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                          uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    bf162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a [rows][D] bf16 tile
// whose chunks are XOR-swizzled with the row index (bank-conflict-free ldmatrix).
template <int D>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return (uint32_t)(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}

template <int D>
struct AttnState {
    float o[D / 8][4];
    float m[2];
    float l[2];
    __device__ __forceinline__ void init() {
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.f;
    }
};

// One warp: S = Q(16 x D) K(16 tokens)^T, online softmax, O += P V.
// allow0/allow1: bit c set when token c of the block is visible to row g /
// row g+8 of the warp's tile (g = lane/4).
// CAP (Gemma-2's soft-capped scores): the scores pass through cap * tanh(s * sm_scale / cap) before the softmax;
// scale_log2 then carries sm_scale / cap and cap_log2 = cap * log2(e).
__device__ __forceinline__ float tanh_approx(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D, bool CAP = false>
__device__ __forceinline__ void attn_block16(const uint32_t (&qf)[D / 16][4], uint32_t k_smem,
                                             uint32_t v_smem, float scale_log2, uint32_t allow0,
                                             uint32_t allow1, AttnState<D>& st, float cap_log2 = 0.f) {
    const int lane = threadIdx.x & 31;
    const int mi = lane >> 3, r = lane & 7;
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
            ldsm_x4(k_smem + swz<D>(token, ks * 2 + (mi & 1)), b00, b01, b10, b11);
            mma_bf16(s[0][ks & 1], qf[ks], b00, b01);
            mma_bf16(s[1][ks & 1], qf[ks], b10, b11);
        }
    }
    const int t = lane & 3;
    float p[2][4];
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int tok = j * 8 + 2 * t + (e & 1);
            const uint32_t allow = (e >> 1) ? allow1 : allow0;
            float v = (s[j][0][e] + s[j][1][e]) * scale_log2;
            if (CAP) v = cap_log2 * tanh_approx(v);
            v = ((allow >> tok) & 1u) ? v : -INFINITY;
            p[j][e] = v;
            mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
    float alpha[2], mref[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float mnew = fmaxf(st.m[h], mx[h]);
        mref[h] = (mnew == -INFINITY) ? 0.f : mnew;
        alpha[h] = exp2f(st.m[h] - mref[h]);
        st.m[h] = mnew;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            p[j][e] = exp2f(p[j][e] - mref[e >> 1]);
            rs[e >> 1] += p[j][e];
        }
    st.l[0] = st.l[0] * alpha[0] + rs[0];
    st.l[1] = st.l[1] * alpha[1] + rs[1];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        st.o[n][0] *= alpha[0];
        st.o[n][1] *= alpha[0];
        st.o[n][2] *= alpha[1];
        st.o[n][3] *= alpha[1];
    }
    uint32_t pa[4];
    pa[0] = pack_bf16(p[0][0], p[0][1]);
    pa[1] = pack_bf16(p[0][2], p[0][3]);
    pa[2] = pack_bf16(p[1][0], p[1][1]);
    pa[3] = pack_bf16(p[1][2], p[1][3]);
    {
        const int token = r + (mi & 1) * 8;
#pragma unroll
        for (int np = 0; np < D / 16; ++np) {
            uint32_t v0, v1, v2, v3;
            ldsm_x4_t(v_smem + swz<D>(token, np * 2 + (mi >> 1)), v0, v1, v2, v3);
            mma_bf16(st.o[2 * np], pa, v0, v1);
            mma_bf16(st.o[2 * np + 1], pa, v2, v3);
        }
    }
}

// Load the warp's 16 x D query tile fragments from a swizzled smem tile.
template <int D>
__device__ __forceinline__ void load_q_frags(uint32_t q_smem, int row0, uint32_t (&qf)[D / 16][4]) {
    const int lane = threadIdx.x & 31;
    const int mi = lane >> 3, r = lane & 7;
    const int row = row0 + r + (mi & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks)
        ldsm_x4(q_smem + swz<D>(row, ks * 2 + (mi >> 1)), qf[ks][0], qf[ks][1], qf[ks][2],
                qf[ks][3]);
}

// ------------------------------------------------------------------ decode
constexpr int DEC_WARPS = 4;
constexpr int DEC_STAGES = 3;

template <int D>
constexpr int decode_smem_bytes() {
    return 16 * D * 2 + DEC_WARPS * DEC_STAGES * 2 * 16 * D * 2;
}

// CASCADE: shared-prefix items. A work item may then cover a KV range that up to 16 / G requests
// (the "members" of a tile: forks of one context, whose leading pages are the same physical pages)
// have in common: the Q tile holds the heads of all members (row = member * G + head), the keys and
// values of the range are read ONCE, and every member gets its own partial result. Partial results go
// to slots: a request's slots are [req_item_indptr[r], req_item_indptr[r + 1]) and a shared item with
// chunk index c fills slot req_item_indptr[member] + c of every member; an unshared item names its
// slot directly. The merge pass combines a request's slots as before.
//   item_slot  [items]  : chunk index (shared item) or slot (unshared item)
//   item_tile  [items]  : row of tile_members for a shared item, -1 otherwise
//   tile_members [tiles][16] : request of each member, -1 for unused rows
// Without CASCADE the three arrays are unused and slot == item index.
template <int D, int G, bool CASCADE, bool CAP = false>
__global__ void __launch_bounds__(DEC_WARPS * 32)
paged_decode_attn_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kv_layer,
                         const int* __restrict__ page_indices,
                         const int* __restrict__ kv_page_indptr, const int* __restrict__ item_req,
                         const int* __restrict__ item_start, const int* __restrict__ item_end,
                         const int* __restrict__ req_item_indptr,
                         const int* __restrict__ num_items_ptr, bf16* __restrict__ out,
                         float* __restrict__ o_part, float* __restrict__ lse_part, int hq, int hkv,
                         int page_size, float scale_log2, int window_left,
                         const float* __restrict__ sinks_log2, int max_items, int num_reqs,
                         int* __restrict__ status, const int* __restrict__ item_slot,
                         const int* __restrict__ item_tile, const int* __restrict__ tile_members,
                         float cap_log2) {
    static_assert(G <= 16, "at most 16 query heads per KV head");
    constexpr int ROWS = CASCADE ? (16 / G) * G : G;      // rows of the Q tile in use
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr int CH = D / 8;              // 16-byte chunks per row
    constexpr int TILE_BYTES = 16 * D * 2; // one 16-token K or V tile
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t q_smem = smem_u32(smem);
    const uint32_t warp_smem = q_smem + TILE_BYTES + warp * DEC_STAGES * 2 * TILE_BYTES;
    pdl_trigger();
    pdl_wait();
    // The work count lives in device memory (graph replays refresh it): never trust it past the
    // size of the scratch the launcher was given. Work beyond that is dropped and reported.
    int n_items = *num_items_ptr;
    if (n_items > max_items || n_items < 0) {
        if (threadIdx.x == 0 && blockIdx.x == 0 && status) atomicCAS(status, 0, PIE_ERR_BOUNDS);
        n_items = n_items < 0 ? 0 : max_items;
    }
    const long total = (long)n_items * hkv;

    for (long w = blockIdx.x; w < total; w += gridDim.x) {
        const int it = (int)(w / hkv), h = (int)(w - (long)it * hkv);
        const int req = item_req[it];
        if (req < 0 || req >= num_reqs) {      // block-uniform: a corrupt item is skipped, not followed
            if (threadIdx.x == 0 && status) atomicCAS(status, 0, PIE_ERR_BOUNDS);
            continue;
        }
        const int kv_start = item_start[it], kv_end = item_end[it];
        const int tile = CASCADE ? item_tile[it] : -1;
        const int* members = (CASCADE && tile >= 0) ? tile_members + (size_t)tile * 16 : nullptr;
        // sliding window: the query sits at position kv_len - 1 (kv_len = end of the request's last
        // item) and sees keys >= kv_len - 1 - window_left; items start on a 16-token boundary below that
        // (plans with shared items carry no window)
        const int kv_lo = (!CASCADE && window_left >= 0)
                              ? max(0, item_end[req_item_indptr[req + 1] - 1] - 1 - window_left) : 0;
        __syncthreads();  // previous item's merge reads are done
        // Q tile: rows < G are the heads of this KV head (of member row / G in a shared item), the rest zeros
        for (int c = threadIdx.x; c < 16 * CH; c += blockDim.x) {
            const int row = c / CH, col = c - row * CH;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < ROWS) {
                int rq = req;
                if (CASCADE) {
                    const int mem = row / G;
                    rq = members ? members[mem] : (mem == 0 ? req : -1);
                    if (rq >= num_reqs) rq = -1;
                }
                if (rq >= 0)
                    v = *reinterpret_cast<const uint4*>(q + ((size_t)rq * hq + h * G + (row % G)) * D + col * 8);
            }
            *reinterpret_cast<uint4*>(smem + swz<D>(row, col)) = v;
        }
        __syncthreads();
        uint32_t qf[D / 16][4];
        load_q_frags<D>(q_smem, 0, qf);

        AttnState<D> st;
        st.init();
        const int nb_total = (kv_end - kv_start + 15) >> 4;
        const int my_count = nb_total > warp ? (nb_total - warp + DEC_WARPS - 1) / DEC_WARPS : 0;
        const int* pages = page_indices + kv_page_indptr[req];

        auto issue = [&](int j) {
            const int tok0 = kv_start + (warp + DEC_WARPS * j) * 16;
            const int page = pages[tok0 / page_size];
            const int off = tok0 % page_size;
            const bf16* ksrc = kv_layer + ((((size_t)page * 2) * hkv + h) * page_size + off) * D;
            const bf16* vsrc = kv_layer + ((((size_t)page * 2 + 1) * hkv + h) * page_size + off) * D;
            const uint32_t kdst = warp_smem + (j % DEC_STAGES) * 2 * TILE_BYTES;
            const uint32_t vdst = kdst + TILE_BYTES;
#pragma unroll
            for (int i = 0; i < (16 * CH) / 32; ++i) {
                const int c = lane + 32 * i;
                const int row = c / CH, col = c - row * CH;
                cp_async16(kdst + swz<D>(row, col), ksrc + (size_t)c * 8);
                cp_async16(vdst + swz<D>(row, col), vsrc + (size_t)c * 8);
            }
        };
#pragma unroll
        for (int s = 0; s < DEC_STAGES - 1; ++s) {
            if (s < my_count) issue(s);
            cp_async_commit();
        }
        for (int i = 0; i < my_count; ++i) {
            if (i + DEC_STAGES - 1 < my_count) issue(i + DEC_STAGES - 1);
            cp_async_commit();
            cp_async_wait<DEC_STAGES - 1>();
            __syncwarp();
            const int tok0 = kv_start + (warp + DEC_WARPS * i) * 16;
            const int nvalid = kv_end - tok0;
            uint32_t allow = nvalid >= 16 ? 0xffffu : ((1u << nvalid) - 1u);
            if (kv_lo > tok0) allow &= kv_lo - tok0 >= 16 ? 0u : ~((1u << (kv_lo - tok0)) - 1u);
            const uint32_t kt = warp_smem + (i % DEC_STAGES) * 2 * TILE_BYTES;
            attn_block16<D, CAP>(qf, kt, kt + TILE_BYTES, scale_log2, allow, allow, st, cap_log2);
            __syncwarp();
        }
        cp_async_wait<0>();
        // row sums across the 4 lanes that share a row
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            st.l[hh] += __shfl_xor_sync(0xffffffffu, st.l[hh], 1);
            st.l[hh] += __shfl_xor_sync(0xffffffffu, st.l[hh], 2);
        }
        __syncthreads();  // every warp is done with its K/V stages: reuse as merge space
        float* sm_m = reinterpret_cast<float*>(smem + TILE_BYTES);  // [W][16]
        float* sm_l = sm_m + DEC_WARPS * 16;                         // [W][16]
        float* sm_o = sm_l + DEC_WARPS * 16;                         // [W][ROWS][D]
        {
            const int g = lane >> 2, t = lane & 3;
            if (t == 0) {
                sm_m[warp * 16 + g] = st.m[0];
                sm_l[warp * 16 + g] = st.l[0];
                sm_m[warp * 16 + g + 8] = st.m[1];
                sm_l[warp * 16 + g + 8] = st.l[1];
            }
#pragma unroll
            for (int n = 0; n < D / 8; ++n) {
                if (g < ROWS) {
                    sm_o[(warp * ROWS + g) * D + n * 8 + 2 * t] = st.o[n][0];
                    sm_o[(warp * ROWS + g) * D + n * 8 + 2 * t + 1] = st.o[n][1];
                }
                if (ROWS > 8 && g + 8 < ROWS) {
                    sm_o[(warp * ROWS + g + 8) * D + n * 8 + 2 * t] = st.o[n][2];
                    sm_o[(warp * ROWS + g + 8) * D + n * 8 + 2 * t + 1] = st.o[n][3];
                }
            }
        }
        __syncthreads();
        const bool single = !(CASCADE && members) && (req_item_indptr[req + 1] - req_item_indptr[req]) == 1;
        const int my_slot = CASCADE ? item_slot[it] : it;
        for (int idx = threadIdx.x; idx < ROWS * D; idx += blockDim.x) {
            const int row = idx / D, dim = idx - row * D;
            int rq = req, slot = my_slot, hrow = row;
            if (CASCADE) {
                const int mem = row / G;
                hrow = row - mem * G;
                if (members) {
                    rq = members[mem];
                    if (rq < 0 || rq >= num_reqs) continue;
                    slot = req_item_indptr[rq] + my_slot;
                } else if (mem != 0) {
                    continue;
                }
                if (slot < 0 || slot >= max_items) {          // a plan that outgrew the scratch: drop, report
                    if (status) atomicCAS(status, 0, PIE_ERR_BOUNDS);
                    continue;
                }
            }
            float M = -INFINITY;
#pragma unroll
            for (int ww = 0; ww < DEC_WARPS; ++ww) M = fmaxf(M, sm_m[ww * 16 + row]);
            float L = 0.f, O = 0.f;
            if (M != -INFINITY) {
#pragma unroll
                for (int ww = 0; ww < DEC_WARPS; ++ww) {
                    const float sc = exp2f(sm_m[ww * 16 + row] - M);
                    L += sm_l[ww * 16 + row] * sc;
                    O += sm_o[(ww * ROWS + row) * D + dim] * sc;
                }
            }
            float val = L > 0.f ? O / L : 0.f;
            if (single) {
                // attention sink: a per-head logit that takes probability mass but has no value row
                if (sinks_log2 && L > 0.f) val = O / (L + exp2f(sinks_log2[h * G + hrow] - M));
                out[((size_t)rq * hq + h * G + hrow) * D + dim] = __float2bfloat16(val);
            } else {
                o_part[(((size_t)slot * hkv + h) * G + hrow) * D + dim] = val;
                if (dim == 0)
                    lse_part[((size_t)slot * hkv + h) * G + hrow] = L > 0.f ? M + log2f(L) : -INFINITY;
            }
        }
    }
}

// Merge the partial results of requests that were split into several items.
template <int D>
__global__ void paged_decode_merge_kernel(const float* __restrict__ o_part,
                                          const float* __restrict__ lse_part,
                                          const int* __restrict__ req_item_indptr,
                                          bf16* __restrict__ out, int hq, int hkv, int group,
                                          const float* __restrict__ sinks_log2, int max_items) {
    const int req = blockIdx.x, qh = blockIdx.y;
    pdl_trigger();
    pdl_wait();
    const int a = req_item_indptr[req], b = min(req_item_indptr[req + 1], max_items);
    if (b - a <= 1) return;
    const int kvh = qh / group, row = qh - kvh * group;
    float M = -INFINITY;
    for (int i = a; i < b; ++i) M = fmaxf(M, lse_part[((size_t)i * hkv + kvh) * group + row]);
    for (int dim = threadIdx.x; dim < D; dim += blockDim.x) {
        float L = 0.f, O = 0.f;
        if (M != -INFINITY) {
            for (int i = a; i < b; ++i) {
                const size_t base = ((size_t)i * hkv + kvh) * group + row;
                const float sc = exp2f(lse_part[base] - M);
                L += sc;
                O += o_part[base * D + dim] * sc;
            }
            if (sinks_log2) L += exp2f(sinks_log2[qh] - M);
        }
        out[((size_t)req * hq + qh) * D + dim] = __float2bfloat16(L > 0.f ? O / L : 0.f);
    }
}

// ----------------------------------------------------------------- prefill
constexpr int PF_WARPS = 4;
constexpr int PF_ROWS = 64;  // packed (token, head-in-group) rows per tile
constexpr int PF_KV = 64;    // KV tokens per pipeline stage

template <int D>
constexpr int prefill_smem_bytes() {
    return PF_ROWS * D * 2 + 2 * 2 * PF_KV * D * 2;
}

template <int D, int G, bool CAP = false>
__global__ void __launch_bounds__(PF_WARPS * 32)
paged_prefill_attn_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kv_layer,
                          const int* __restrict__ page_indices,
                          const int* __restrict__ kv_page_indptr,
                          const int* __restrict__ qo_indptr, const int* __restrict__ kv_lens,
                          const int* __restrict__ tile_req, const int* __restrict__ tile_qstart,
                          const uint32_t* __restrict__ mask_bits,
                          const long* __restrict__ mask_word_indptr, bf16* __restrict__ out,
                          float* __restrict__ lse_out, const float* __restrict__ sinks_log2, int hq, int hkv, int page_size,
                          float scale_log2, int window_left, float cap_log2) {
    extern __shared__ __align__(1024) uint8_t smem[];
    constexpr int CH = D / 8;
    constexpr int TQ = PF_ROWS / G;  // query tokens per tile
    constexpr int Q_BYTES = PF_ROWS * D * 2;
    constexpr int KV_TILE = PF_KV * D * 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, h = blockIdx.y;
    const int req = tile_req[tile], qstart = tile_qstart[tile];
    const int q_base = qo_indptr[req];
    const int qo_len = qo_indptr[req + 1] - q_base;
    const int kv_len = kv_lens[req];
    const int* pages = page_indices + kv_page_indptr[req];
    const bool custom = mask_bits != nullptr;
    const int mask_words = (kv_len + 31) >> 5;
    const uint32_t* req_mask = custom ? mask_bits + mask_word_indptr[req] : nullptr;

    const uint32_t q_smem = smem_u32(smem);
    const uint32_t kv_smem = q_smem + Q_BYTES;
    for (int c = threadIdx.x; c < PF_ROWS * CH; c += blockDim.x) {
        const int row = c / CH, col = c - row * CH;
        const int qt = qstart + row / G;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (qt < qo_len)
            v = *reinterpret_cast<const uint4*>(
                q + ((size_t)(q_base + qt) * hq + h * G + row % G) * D + col * 8);
        *reinterpret_cast<uint4*>(smem + swz<D>(row, col)) = v;
    }
    __syncthreads();
    uint32_t qf[D / 16][4];
    load_q_frags<D>(q_smem, warp * 16, qf);

    // per-thread rows g and g+8 of the warp tile
    const int g = lane >> 2;
    int qtok[2], lim[2], lo[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int row = warp * 16 + g + hh * 8;
        qtok[hh] = qstart + row / G;
        const bool valid = qtok[hh] < qo_len;
        // causal: query token i of qo_len sees kv positions < kv_len - qo_len + i + 1
        lim[hh] = valid ? (custom ? kv_len : kv_len - qo_len + qtok[hh] + 1) : 0;
        lo[hh] = (window_left >= 0 && valid) ? max(0, kv_len - qo_len + qtok[hh] - window_left) : 0;
    }
    const int last_q = min(qstart + TQ, qo_len) - 1;
    const int kv_hi = custom ? kv_len : max(0, min(kv_len, kv_len - qo_len + last_q + 1));
    // the warp's last row has the largest causal limit of the warp
    const int warp_last_q = min(qstart + (warp * 16 + 15) / G, qo_len - 1);
    const int warp_hi = custom ? kv_len : kv_len - qo_len + warp_last_q + 1;
    const int nkb = (kv_hi + PF_KV - 1) / PF_KV;

    auto load_stage = [&](int kb) {
        const uint32_t kdst = kv_smem + (kb & 1) * 2 * KV_TILE;
        const uint32_t vdst = kdst + KV_TILE;
#pragma unroll
        for (int i = 0; i < (PF_KV * CH) / (PF_WARPS * 32); ++i) {
            const int c = threadIdx.x + PF_WARPS * 32 * i;
            const int row = c / CH, col = c - row * CH;
            const int tok = kb * PF_KV + row;
            if (tok < kv_hi) {
                const int page = pages[tok / page_size];
                const int off = tok % page_size;
                const bf16* ksrc =
                    kv_layer + ((((size_t)page * 2) * hkv + h) * page_size + off) * D + col * 8;
                const bf16* vsrc =
                    kv_layer + ((((size_t)page * 2 + 1) * hkv + h) * page_size + off) * D + col * 8;
                cp_async16(kdst + swz<D>(row, col), ksrc);
                cp_async16(vdst + swz<D>(row, col), vsrc);
            } else {
                // rows past the end are multiplied by p == 0: they must be finite
                *reinterpret_cast<uint4*>(smem + (vdst - q_smem) + swz<D>(row, col)) =
                    make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(smem + (kdst - q_smem) + swz<D>(row, col)) =
                    make_uint4(0, 0, 0, 0);
            }
        }
    };

    AttnState<D> st;
    st.init();
    if (nkb > 0) load_stage(0);
    cp_async_commit();
    for (int kb = 0; kb < nkb; ++kb) {
        if (kb + 1 < nkb) load_stage(kb + 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t kt = kv_smem + (kb & 1) * 2 * KV_TILE;
#pragma unroll
        for (int sb = 0; sb < PF_KV / 16; ++sb) {
            const int tb = kb * PF_KV + sb * 16;
            if (tb >= warp_hi || tb >= kv_hi) break;
            uint32_t allow[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int n = lim[hh] - tb;
                uint32_t a = n >= 16 ? 0xffffu : (n <= 0 ? 0u : ((1u << n) - 1u));
                const int nl = lo[hh] - tb;
                if (nl > 0) a &= nl >= 16 ? 0u : ~((1u << nl) - 1u);
                if (custom && a) {
                    const uint32_t wv = req_mask[(size_t)qtok[hh] * mask_words + (tb >> 5)];
                    a &= (wv >> (tb & 31)) & 0xffffu;
                }
                allow[hh] = a;
            }
            attn_block16<D, CAP>(qf, kt + sb * 16 * D * 2, kt + KV_TILE + sb * 16 * D * 2, scale_log2,
                                 allow[0], allow[1], st, cap_log2);
        }
        __syncthreads();
    }
    cp_async_wait<0>();
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        st.l[hh] += __shfl_xor_sync(0xffffffffu, st.l[hh], 1);
        st.l[hh] += __shfl_xor_sync(0xffffffffu, st.l[hh], 2);
    }
    const int t = lane & 3;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        if (qtok[hh] >= qo_len) continue;
        const int row = warp * 16 + g + hh * 8;
        const int head = h * G + row % G;
        if (sinks_log2 && st.l[hh] > 0.f) st.l[hh] += exp2f(sinks_log2[head] - st.m[hh]);
        const float inv = st.l[hh] > 0.f ? 1.f / st.l[hh] : 0.f;
        bf16* dst = out + ((size_t)(q_base + qtok[hh]) * hq + head) * D;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            bf162 v = __floats2bfloat162_rn(st.o[n][2 * hh] * inv, st.o[n][2 * hh + 1] * inv);
            *reinterpret_cast<bf162*>(dst + n * 8 + 2 * t) = v;
        }
        if (lse_out && t == 0)
            lse_out[(size_t)(q_base + qtok[hh]) * hq + head] =
                st.l[hh] > 0.f ? (st.m[hh] + log2f(st.l[hh])) * 0.6931471805599453f : -INFINITY;
    }
}

}  // namespace pie

using namespace pie;

#define DISPATCH_DG(D_, G_, ...)                                      \
    do {                                                               \
        bool ok_ = true;                                               \
        if (D_ == 128) {                                               \
            constexpr int D = 128;                                     \
            switch (G_) {                                              \
                case 1: { constexpr int G = 1; __VA_ARGS__; } break;          \
                case 2: { constexpr int G = 2; __VA_ARGS__; } break;          \
                case 4: { constexpr int G = 4; __VA_ARGS__; } break;          \
                case 8: { constexpr int G = 8; __VA_ARGS__; } break;          \
                case 16: { constexpr int G = 16; __VA_ARGS__; } break;        \
                default: ok_ = false;                                  \
            }                                                          \
        } else if (D_ == 256) {                                        \
            constexpr int D = 256;                                     \
            switch (G_) {                                              \
                case 1: { constexpr int G = 1; __VA_ARGS__; } break;          \
                case 2: { constexpr int G = 2; __VA_ARGS__; } break;          \
                case 4: { constexpr int G = 4; __VA_ARGS__; } break;          \
                case 8: { constexpr int G = 8; __VA_ARGS__; } break;          \
                default: ok_ = false;                                  \
            }                                                          \
        } else if (D_ == 64) {                                         \
            constexpr int D = 64;                                      \
            switch (G_) {                                              \
                case 1: { constexpr int G = 1; __VA_ARGS__; } break;          \
                case 2: { constexpr int G = 2; __VA_ARGS__; } break;          \
                case 4: { constexpr int G = 4; __VA_ARGS__; } break;          \
                case 8: { constexpr int G = 8; __VA_ARGS__; } break;          \
                case 16: { constexpr int G = 16; __VA_ARGS__; } break;        \
                default: ok_ = false;                                  \
            }                                                          \
        } else {                                                       \
            ok_ = false;                                               \
        }                                                              \
        if (!ok_) return (int)cudaErrorInvalidValue;                   \
    } while (0)

// Status word of the current device for the bounds reports of the decode kernel (see
// pie_set_status_word); null when the embedder registered none: the kernel then only clamps.
namespace {
constexpr int kStatusDevices = 64;
int* g_status_word[kStatusDevices] = {};
int* status_word() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kStatusDevices) return nullptr;
    return g_status_word[dev];
}
}  // namespace

// Register a device int32 (on the current device) that kernels without a status argument set to a
// PieKernelStatus code when they drop work; pass null to unregister.
PIE_API int pie_set_status_word(int* word) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kStatusDevices) return (int)cudaErrorInvalidValue;
    g_status_word[dev] = word;
    return 0;
}

// The status word registered for the current device (null if none): for kernels of other files.
PIE_API int* pie_status_word_current() { return status_word(); }

// Merge pass of split-KV decode on its own (used by the fp8-KV decode kernel of attention_kv8.cu).
PIE_API int pie_decode_merge(const float* o_part, const float* lse_part, const int* req_item_indptr, void* out,
                             int num_reqs, int hq, int hkv, int head_dim, const float* sinks_log2, int max_items,
                             cudaStream_t st) {
    if (num_reqs <= 0) return 0;
    dim3 grid(num_reqs, hq);
    const int group = hq / hkv;
    if (head_dim == 128)
        launch_pdl(paged_decode_merge_kernel<128>, grid, dim3(128), 0, st, o_part, lse_part, req_item_indptr,
                   (bf16*)out, hq, hkv, group, sinks_log2, max_items);
    else if (head_dim == 256)
        launch_pdl(paged_decode_merge_kernel<256>, grid, dim3(256), 0, st, o_part, lse_part, req_item_indptr,
                   (bf16*)out, hq, hkv, group, sinks_log2, max_items);
    else if (head_dim == 64)
        launch_pdl(paged_decode_merge_kernel<64>, grid, dim3(64), 0, st, o_part, lse_part, req_item_indptr,
                   (bf16*)out, hq, hkv, group, sinks_log2, max_items);
    else
        return (int)cudaErrorInvalidValue;
    return (int)cudaGetLastError();
}

// Scratch sizes (in floats) a caller must provide for `max_items` work items.
PIE_API long pie_decode_attn_scratch_floats(int max_items, int hq, int head_dim) {
    return (long)max_items * hq * head_dim + (long)max_items * hq;
}

static int launch_decode(const void* q, const void* kv_layer, const int* page_indices,
                         const int* kv_page_indptr, const int* item_req, const int* item_start,
                         const int* item_end, const int* req_item_indptr, const int* num_items_ptr,
                         void* out, float* scratch, int max_items, int num_reqs, int hq, int hkv,
                         int head_dim, int page_size, float sm_scale, int num_ctas, int run_merge,
                         int window_left, const float* sinks_log2, const int* item_slot,
                         const int* item_tile, const int* tile_members, cudaStream_t st, float softcap = 0.f) {
    if (num_reqs <= 0) return 0;
    if (hkv <= 0 || hq % hkv || page_size % 16) return (int)cudaErrorInvalidValue;
    const bool cascade = item_tile != nullptr;
    if (cascade && (!item_slot || !tile_members || window_left >= 0 || softcap > 0.f)) return (int)cudaErrorInvalidValue;
    const int group = hq / hkv;
    float* o_part = scratch;
    float* lse_part = scratch + (size_t)max_items * hq * head_dim;
    const float scale_log2 = softcap > 0.f ? sm_scale / softcap : sm_scale * 1.4426950408889634f;
    const float cap_log2 = softcap * 1.4426950408889634f;
    DISPATCH_DG(head_dim, group, {
        constexpr int SM = decode_smem_bytes<D>();
        if (softcap > 0.f) {
            auto kern = paged_decode_attn_kernel<D, G, false, true>;
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM);
            launch_pdl(kern, dim3(num_ctas), dim3(DEC_WARPS * 32), SM, st,
                (const bf16*)q, (const bf16*)kv_layer, page_indices, kv_page_indptr, item_req,
                item_start, item_end, req_item_indptr, num_items_ptr, (bf16*)out, o_part, lse_part, hq,
                hkv, page_size, scale_log2, window_left, sinks_log2, max_items, num_reqs, status_word(),
                (const int*)nullptr, (const int*)nullptr, (const int*)nullptr, cap_log2);
        } else if (cascade) {
            auto kern = paged_decode_attn_kernel<D, G, true>;
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM);
            launch_pdl(kern, dim3(num_ctas), dim3(DEC_WARPS * 32), SM, st,
                (const bf16*)q, (const bf16*)kv_layer, page_indices, kv_page_indptr, item_req,
                item_start, item_end, req_item_indptr, num_items_ptr, (bf16*)out, o_part, lse_part, hq,
                hkv, page_size, scale_log2, window_left, sinks_log2, max_items, num_reqs, status_word(),
                item_slot, item_tile, tile_members, 0.f);
        } else {
            auto kern = paged_decode_attn_kernel<D, G, false>;
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM);
            launch_pdl(kern, dim3(num_ctas), dim3(DEC_WARPS * 32), SM, st,
                (const bf16*)q, (const bf16*)kv_layer, page_indices, kv_page_indptr, item_req,
                item_start, item_end, req_item_indptr, num_items_ptr, (bf16*)out, o_part, lse_part, hq,
                hkv, page_size, scale_log2, window_left, sinks_log2, max_items, num_reqs, status_word(),
                (const int*)nullptr, (const int*)nullptr, (const int*)nullptr, 0.f);
        }
    });
    int err = (int)cudaGetLastError();
    if (err || !run_merge) return err;
    dim3 grid(num_reqs, hq);
    if (head_dim == 128)
        launch_pdl(paged_decode_merge_kernel<128>, grid, dim3(128), 0, st, (const float*)o_part,
                   (const float*)lse_part, req_item_indptr, (bf16*)out, hq, hkv, group, sinks_log2, max_items);
    else if (head_dim == 256)
        launch_pdl(paged_decode_merge_kernel<256>, grid, dim3(256), 0, st, (const float*)o_part,
                   (const float*)lse_part, req_item_indptr, (bf16*)out, hq, hkv, group, sinks_log2, max_items);
    else
        launch_pdl(paged_decode_merge_kernel<64>, grid, dim3(64), 0, st, (const float*)o_part,
                   (const float*)lse_part, req_item_indptr, (bf16*)out, hq, hkv, group, sinks_log2, max_items);
    return (int)cudaGetLastError();
}

// window_left >= 0: each request's single query token sees only the last window_left + 1 keys; the
// caller's items then start at the 16-token boundary at or below the first visible key (items that
// start lower are masked). sinks_log2 (optional, [hq], logit * log2(e)): per-head attention sinks.
PIE_API int pie_paged_decode_attn_window(const void* q, const void* kv_layer, const int* page_indices,
                                         const int* kv_page_indptr, const int* item_req,
                                         const int* item_start, const int* item_end,
                                         const int* req_item_indptr, const int* num_items_ptr,
                                         void* out, float* scratch, int max_items, int num_reqs, int hq,
                                         int hkv, int head_dim, int page_size, float sm_scale,
                                         int num_ctas, int run_merge, int window_left,
                                         const float* sinks_log2, cudaStream_t st) {
    return launch_decode(q, kv_layer, page_indices, kv_page_indptr, item_req, item_start, item_end, req_item_indptr,
                         num_items_ptr, out, scratch, max_items, num_reqs, hq, hkv, head_dim, page_size, sm_scale,
                         num_ctas, run_merge, window_left, sinks_log2, nullptr, nullptr, nullptr, st);
}

// The same with soft-capped scores (softcap > 0): softmax over softcap * tanh(q.k * sm_scale / softcap).
PIE_API int pie_paged_decode_attn_softcap(const void* q, const void* kv_layer, const int* page_indices,
                                          const int* kv_page_indptr, const int* item_req,
                                          const int* item_start, const int* item_end,
                                          const int* req_item_indptr, const int* num_items_ptr,
                                          void* out, float* scratch, int max_items, int num_reqs, int hq,
                                          int hkv, int head_dim, int page_size, float sm_scale,
                                          int num_ctas, int run_merge, int window_left,
                                          const float* sinks_log2, float softcap, cudaStream_t st) {
    return launch_decode(q, kv_layer, page_indices, kv_page_indptr, item_req, item_start, item_end, req_item_indptr,
                         num_items_ptr, out, scratch, max_items, num_reqs, hq, hkv, head_dim, page_size, sm_scale,
                         num_ctas, run_merge, window_left, sinks_log2, nullptr, nullptr, nullptr, st, softcap);
}

// Decode attention over a plan with shared-prefix items (see the kernel): requests that were forked
// from one context read their common pages once. item_req of a shared item names the member whose
// page table addresses the range. req_item_indptr counts partial-result slots, all below max_items.
PIE_API int pie_paged_decode_attn_cascade(const void* q, const void* kv_layer, const int* page_indices,
                                          const int* kv_page_indptr, const int* item_req,
                                          const int* item_start, const int* item_end,
                                          const int* req_item_indptr, const int* num_items_ptr,
                                          void* out, float* scratch, int max_items, int num_reqs, int hq,
                                          int hkv, int head_dim, int page_size, float sm_scale,
                                          int num_ctas, const float* sinks_log2, const int* item_slot,
                                          const int* item_tile, const int* tile_members, cudaStream_t st) {
    if (!item_tile) return (int)cudaErrorInvalidValue;
    return launch_decode(q, kv_layer, page_indices, kv_page_indptr, item_req, item_start, item_end, req_item_indptr,
                         num_items_ptr, out, scratch, max_items, num_reqs, hq, hkv, head_dim, page_size, sm_scale,
                         num_ctas, 1, -1, sinks_log2, item_slot, item_tile, tile_members, st);
}

PIE_API int pie_paged_decode_attn(const void* q, const void* kv_layer, const int* page_indices,
                                  const int* kv_page_indptr, const int* item_req,
                                  const int* item_start, const int* item_end,
                                  const int* req_item_indptr, const int* num_items_ptr,
                                  void* out, float* scratch, int max_items, int num_reqs, int hq,
                                  int hkv, int head_dim, int page_size, float sm_scale,
                                  int num_ctas, int run_merge, cudaStream_t st) {
    return pie_paged_decode_attn_window(q, kv_layer, page_indices, kv_page_indptr, item_req, item_start, item_end,
                                        req_item_indptr, num_items_ptr, out, scratch, max_items, num_reqs, hq, hkv,
                                        head_dim, page_size, sm_scale, num_ctas, run_merge, -1, nullptr, st);
}

// softcap > 0: softmax over softcap * tanh(q.k * sm_scale / softcap) (Gemma-2).
PIE_API int pie_paged_prefill_attn_softcap(const void* q, const void* kv_layer, const int* page_indices,
                                           const int* kv_page_indptr, const int* qo_indptr,
                                           const int* kv_lens, const int* tile_req, const int* tile_qstart,
                                           int num_tiles, const uint32_t* mask_bits,
                                           const long* mask_word_indptr, void* out, float* lse_out, int hq,
                                           int hkv, int head_dim, int page_size, float sm_scale,
                                           int window_left, const float* sinks_log2, float softcap,
                                           cudaStream_t st) {
    if (num_tiles <= 0) return 0;
    if (hkv <= 0 || hq % hkv || page_size % 16) return (int)cudaErrorInvalidValue;
    const int group = hq / hkv;
    const float scale_log2 = softcap > 0.f ? sm_scale / softcap : sm_scale * 1.4426950408889634f;
    const float cap_log2 = softcap * 1.4426950408889634f;
    dim3 grid(num_tiles, hkv);
    DISPATCH_DG(head_dim, group, {
        constexpr int SM = prefill_smem_bytes<D>();
        if (softcap > 0.f) {
            auto kern = paged_prefill_attn_kernel<D, G, true>;
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM);
            kern<<<grid, PF_WARPS * 32, SM, st>>>(
                (const bf16*)q, (const bf16*)kv_layer, page_indices, kv_page_indptr, qo_indptr, kv_lens,
                tile_req, tile_qstart, mask_bits, mask_word_indptr, (bf16*)out, lse_out, sinks_log2, hq, hkv,
                page_size, scale_log2, window_left, cap_log2);
        } else {
            auto kern = paged_prefill_attn_kernel<D, G, false>;
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM);
            kern<<<grid, PF_WARPS * 32, SM, st>>>(
                (const bf16*)q, (const bf16*)kv_layer, page_indices, kv_page_indptr, qo_indptr, kv_lens,
                tile_req, tile_qstart, mask_bits, mask_word_indptr, (bf16*)out, lse_out, sinks_log2, hq, hkv,
                page_size, scale_log2, window_left, 0.f);
        }
    });
    return (int)cudaGetLastError();
}

PIE_API int pie_paged_prefill_attn(const void* q, const void* kv_layer, const int* page_indices,
                                   const int* kv_page_indptr, const int* qo_indptr,
                                   const int* kv_lens, const int* tile_req, const int* tile_qstart,
                                   int num_tiles, const uint32_t* mask_bits,
                                   const long* mask_word_indptr, void* out, float* lse_out, int hq,
                                   int hkv, int head_dim, int page_size, float sm_scale,
                                   int window_left, const float* sinks_log2, cudaStream_t st) {
    return pie_paged_prefill_attn_softcap(q, kv_layer, page_indices, kv_page_indptr, qo_indptr, kv_lens, tile_req,
                                          tile_qstart, num_tiles, mask_bits, mask_word_indptr, out, lse_out, hq, hkv,
                                          head_dim, page_size, sm_scale, window_left, sinks_log2, 0.f, st);
}

// Query tokens covered by one prefill tile for a given GQA group size.
PIE_API int pie_prefill_tile_tokens(int group) { return PF_ROWS / group; }

// ------------------------------------------------- allocation-free variant
// See pie_noalloc.h: split-KV decode attention whose scratch lives in this
// library instead of being passed in, for callers that cannot allocate.
#include <stdio.h>
#include <mutex>
#include "pie_noalloc.h"

// Split-KV partial outputs and log-sum-exps of the allocation-free entry point.
// Host code must not use this name as an address: it is a host-side stand-in;
// the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float pie_noalloc_scratch[PIE_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mutex;

// Device address of the scratch array on the current device (looked up once per device).
int noalloc_scratch_for_current_device(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return PIE_NOALLOC_ERR_SETUP;
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[dev]) {
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, pie_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!p) return PIE_NOALLOC_ERR_SETUP;
        g_noalloc_ptr[dev] = p;
    }
    *out = g_noalloc_ptr[dev];
    return 0;
}
}  // namespace

PIE_API int pie_paged_decode_attn_noalloc(const void* q, const void* kv_layer,
                                          const int* page_indices, const int* kv_page_indptr,
                                          const int* item_req, const int* item_start,
                                          const int* item_end, const int* req_item_indptr,
                                          const int* num_items_ptr, void* out, int max_items,
                                          int num_reqs, int hq, int hkv, int head_dim,
                                          int page_size, float sm_scale, int num_ctas,
                                          cudaStream_t stream) {
    if (max_items < 0 || hq <= 0 || head_dim <= 0) return (int)cudaErrorInvalidValue;
    const long need = pie_decode_attn_scratch_floats(max_items, hq, head_dim);
    if (need > (long)PIE_NOALLOC_SCRATCH_FLOATS) {
        fprintf(stderr,
                "pie_paged_decode_attn_noalloc: max_items=%d, hq=%d, head_dim=%d need %ld floats of "
                "scratch; the built-in array holds %u. Use fewer work items or pie_paged_decode_attn "
                "with your own buffer.\n",
                max_items, hq, head_dim, need, (unsigned)PIE_NOALLOC_SCRATCH_FLOATS);
        return PIE_NOALLOC_ERR_TOO_LARGE;
    }
    float* scratch = nullptr;
    const int rc = noalloc_scratch_for_current_device(&scratch);
    if (rc != 0) return rc;
    return pie_paged_decode_attn(q, kv_layer, page_indices, kv_page_indptr, item_req, item_start,
                                 item_end, req_item_indptr, num_items_ptr, out, scratch, max_items,
                                 num_reqs, hq, hkv, head_dim, page_size, sm_scale, num_ctas, 1, stream);
}
