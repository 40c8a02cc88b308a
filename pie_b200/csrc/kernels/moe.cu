// Mixture-of-experts plumbing around the grouped tcgen05 GEMM (gemm_tcgen05.cu, GROUPED form):
//   pie_moe_route    softmax over E router logits, top-k, optional renormalisation; every route
//                    (token, j) takes a position inside its expert's segment with one atomic
//   pie_moe_align    per-expert segments padded to 128-row tiles: seg_start[e], tile_expert[tile]
//   pie_moe_permute  token rows -> expert-sorted rows
//   pie_moe_combine  out[t] = residual[t] + sum_j w[t,j] * y[slot(t,j)]; the _rs form stores this
//                    rank's partial rows into the row owners' receive buffers (peer stores)
// Expert parallelism in the row-sharded tensor-parallel design: the all-gather push of the
// normalised activations already delivers every token to every rank (the dispatch), each rank
// routes all tokens but gives slots only to its own experts, and the combine is a reduce-scatter
// by peer stores that the owner's reduce+norm kernel sums.
// Everything is sized by static upper bounds and reads its counts on the device, so the whole
// block can sit inside a CUDA graph.
//
// Replaces driver/cuda/src/kernels/topk_softmax.cu:19 (router) and the pointer-array / aligned
// dispatch family of driver/cuda/src/kernels/moe_dispatch.cu:12-760 with its cuBLAS batched GEMMs
// (driver/cuda/src/model/qwen3_5_moe_forward.cpp:1315-1558).
#include "gemm_common.cuh"

namespace pie {

constexpr int MOE_MAX_E = 512;
constexpr int MOE_TILE = 128;

// One warp per token. logits [N, E] (bf16 or fp32), E <= 512.
// ids receives the expert index relative to e_lo, or -1 for an expert outside [e_lo, e_lo+e_cnt)
// (expert parallelism: those routes belong to another rank and take no slot here).
template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ logits, int ld, int n, int E, int k, int renorm,
                                 int e_lo, int e_cnt, int* __restrict__ ids, float* __restrict__ w,
                                 int* __restrict__ pos, int* __restrict__ counts) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= n) return;
    const T* row = logits + (size_t)warp * ld;
    float v[MOE_MAX_E / 32];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < MOE_MAX_E / 32; ++i) {
        const int e = i * 32 + lane;
        v[i] = e < E ? (float)row[e] : -INFINITY;
        mx = fmaxf(mx, v[i]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < MOE_MAX_E / 32; ++i) {
        v[i] = (i * 32 + lane) < E ? __expf(v[i] - mx) : -1.f;   // -1 = excluded
        if (v[i] > 0.f) sum += v[i];
    }
    sum = warp_sum(sum);
    float picked_sum = 0.f;
    float my_w = 0.f;
    int my_id = 0;
    for (int j = 0; j < k; ++j) {
        float best = -2.f;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < MOE_MAX_E / 32; ++i) {
            const int e = i * 32 + lane;
            if (v[i] > best) { best = v[i]; bi = e; }     // lowest index wins ties within a lane
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if ((bi & 31) == lane) v[bi >> 5] = -1.f;
        picked_sum += best;
        if (lane == j) { my_w = best; my_id = bi; }
    }
    if (lane < k) {
        const float denom = renorm ? picked_sum : sum;
        const int local = my_id - e_lo;
        const bool mine = local >= 0 && local < e_cnt;
        ids[(size_t)warp * k + lane] = mine ? local : -1;
        w[(size_t)warp * k + lane] = my_w / denom;
        pos[(size_t)warp * k + lane] = mine ? atomicAdd(counts + local, 1) : -1;
    }
}

// Single block. counts [E] -> seg_start [E] (row of the expert's first slot), tile_expert
// [max_mtiles]; counts are copied to counts_out (may be null) and zeroed for the next call.
__global__ void moe_align_kernel(int* __restrict__ counts, int E, int max_mtiles, int* __restrict__ seg_start,
                                 int* __restrict__ tile_expert, int* __restrict__ counts_out) {
    __shared__ int tiles_of[MOE_MAX_E];
    __shared__ int start_of[MOE_MAX_E + 1];
    const int tid = threadIdx.x;
    for (int e = tid; e < E; e += blockDim.x) {
        const int c = counts[e];
        tiles_of[e] = (c + MOE_TILE - 1) / MOE_TILE;
        if (counts_out) counts_out[e] = c;
        counts[e] = 0;
    }
    __syncthreads();
    if (tid == 0) {
        int acc = 0;
        for (int e = 0; e < E; ++e) {
            start_of[e] = acc;
            acc += tiles_of[e];
        }
        start_of[E] = acc;
    }
    __syncthreads();
    for (int e = tid; e < E; e += blockDim.x) {
        seg_start[e] = start_of[e] * MOE_TILE;
        for (int t = start_of[e]; t < start_of[e + 1] && t < max_mtiles; ++t) tile_expert[t] = e;
    }
    for (int t = start_of[E] + tid; t < max_mtiles; t += blockDim.x) tile_expert[t] = -1;
}

// One block per route: xs[slot] = x[token]; routes of experts that are not local (ids < 0) take
// no slot.
__global__ void moe_permute_kernel(const bf16* __restrict__ x, int ldx, const int* __restrict__ ids,
                                   const int* __restrict__ pos, const int* __restrict__ seg_start, int H, int k,
                                   bf16* __restrict__ xs, int* __restrict__ slot_of) {
    const int route = blockIdx.x;
    const int e = ids[route];
    if (e < 0) {
        if (threadIdx.x == 0) slot_of[route] = -1;
        return;
    }
    const int slot = seg_start[e] + pos[route];
    if (threadIdx.x == 0) slot_of[route] = slot;
    const bf16x8* src = reinterpret_cast<const bf16x8*>(x + (size_t)(route / k) * ldx);
    bf16x8* dst = reinterpret_cast<bf16x8*>(xs + (size_t)slot * H);
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) dst[c] = src[c];
}

// One block per token. RS: the (partial) row goes to the receive buffer of the rank that owns
// token t (reduce-scatter by peer stores, same protocol as the GEMM's EPI_RS epilogue); the last
// block to finish raises this rank's flag on every owner.
template <bool RS>
__global__ void moe_combine_kernel(const bf16* __restrict__ y, const int* __restrict__ slot_of,
                                   const float* __restrict__ w, const bf16* __restrict__ residual, int ldr, int H,
                                   int k, bf16* __restrict__ out, int ldo, const __grid_constant__ TpArgs tp) {
    const int t = blockIdx.x;
    bf16* dst_row;
    if (RS) {
        const int owner = t / tp.rows_per_rank;
        dst_row = tp.peer_recv[owner] + ((size_t)tp.rank * tp.rows_per_rank + (t - owner * tp.rows_per_rank)) * (size_t)H;
    } else {
        dst_row = out + (size_t)t * ldo;
    }
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
        float acc[8];
        if (residual) unpack8(*reinterpret_cast<const bf16x8*>(residual + (size_t)t * ldr + c * 8), acc);
        else
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = 0.f;
        for (int j = 0; j < k; ++j) {
            const int slot = slot_of[(size_t)t * k + j];
            if (slot < 0) continue;
            const float wj = w[(size_t)t * k + j];
            float v[8];
            unpack8(*reinterpret_cast<const bf16x8*>(y + (size_t)slot * H + c * 8), v);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] += wj * v[i];
        }
        *reinterpret_cast<bf16x8*>(dst_row + c * 8) = pack8(acc);
    }
    if (RS) {
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) rs_publish_arrival(tp, (int)gridDim.x);
    }
}

}  // namespace pie

using namespace pie;

// logits_fp32: 0 = bf16 logits, 1 = fp32. counts must be zero on entry (pie_moe_align leaves it so).
PIE_API int pie_moe_route(const void* logits, int logits_fp32, int ld, int n, int E, int k, int renorm, int e_lo,
                          int e_cnt, int* ids, float* w, int* pos, int* counts, cudaStream_t st) {
    if (n <= 0) return 0;
    if (E > MOE_MAX_E || k > 32 || k > E || k <= 0) return (int)cudaErrorInvalidValue;
    const int threads = 128, blocks = (n * 32 + threads - 1) / threads;
    if (logits_fp32)
        moe_route_kernel<float><<<blocks, threads, 0, st>>>((const float*)logits, ld, n, E, k, renorm, e_lo, e_cnt, ids, w, pos, counts);
    else
        moe_route_kernel<bf16><<<blocks, threads, 0, st>>>((const bf16*)logits, ld, n, E, k, renorm, e_lo, e_cnt, ids, w, pos, counts);
    return (int)cudaGetLastError();
}

PIE_API int pie_moe_align(int* counts, int E, int max_mtiles, int* seg_start, int* tile_expert, int* counts_out,
                          cudaStream_t st) {
    if (E > MOE_MAX_E || E <= 0) return (int)cudaErrorInvalidValue;
    moe_align_kernel<<<1, 256, 0, st>>>(counts, E, max_mtiles, seg_start, tile_expert, counts_out);
    return (int)cudaGetLastError();
}

PIE_API int pie_moe_permute(const void* x, int ldx, const int* ids, const int* pos, const int* seg_start, int n,
                            int H, int k, void* xs, int* slot_of, cudaStream_t st) {
    if (n <= 0) return 0;
    if (H % 8 || ldx % 8) return (int)cudaErrorInvalidValue;
    moe_permute_kernel<<<n * k, 128, 0, st>>>((const bf16*)x, ldx, ids, pos, seg_start, H, k, (bf16*)xs, slot_of);
    return (int)cudaGetLastError();
}

PIE_API int pie_moe_combine(const void* y, const int* slot_of, const float* w, const void* residual, int ldr, int n,
                            int H, int k, void* out, int ldo, cudaStream_t st) {
    if (n <= 0) return 0;
    if (H % 8 || ldo % 8 || (residual && ldr % 8)) return (int)cudaErrorInvalidValue;
    moe_combine_kernel<false><<<n, 128, 0, st>>>((const bf16*)y, slot_of, w, (const bf16*)residual, ldr, H, k,
                                                 (bf16*)out, ldo, TpArgs{});
    return (int)cudaGetLastError();
}

// Tensor/expert-parallel combine: this rank's partial sum of every token row (its local experts, or
// its slice of every expert) is stored into the row owner's receive buffer; `tp_blob` is the TpArgs
// blob of the communicator. The owner then runs pie_tp_reduce_norm_push as after a row-parallel GEMM.
PIE_API int pie_moe_combine_rs(const void* y, const int* slot_of, const float* w, int n, int H, int k,
                               const void* tp_blob, int rows_per_rank, cudaStream_t st) {
    if (n <= 0) return 0;
    if (H % 8 || rows_per_rank <= 0) return (int)cudaErrorInvalidValue;
    TpArgs tp = *reinterpret_cast<const TpArgs*>(tp_blob);
    tp.rows_per_rank = rows_per_rank;
    moe_combine_kernel<true><<<n, 128, 0, st>>>((const bf16*)y, slot_of, w, nullptr, 0, H, k, nullptr, H, tp);
    return (int)cudaGetLastError();
}

// ----------------------------------------------------------------------- GPT-OSS expert epilogues
// The expert-sorted rows of a grouped GEMM carry their expert in the tile table (128 rows per tile).
// gate/up columns are interleaved: act[r, j] = (clamp(up) + 1) * g * sigmoid(1.702 g), g = min(gate, limit),
// after adding the expert's bias. Rows of unused tiles (expert < 0) are left alone.
// Counterpart of gpt_oss_glu in the reference (driver/cuda/src/kernels/swiglu.cu).
namespace pie {
__global__ void moe_bias_glu_kernel(const bf16* __restrict__ gu, const bf16* __restrict__ bias,
                                    const int* __restrict__ tile_expert, bf16* __restrict__ act, int inter,
                                    float limit) {
    const int row = blockIdx.x;
    const int e = tile_expert[row >> 7];
    if (e < 0) return;
    const bf16* src = gu + (size_t)row * 2 * inter;
    const bf16* b = bias + (size_t)e * 2 * inter;
    bf16* dst = act + (size_t)row * inter;
    for (int c = threadIdx.x * 4; c < inter; c += blockDim.x * 4) {      // 4 outputs = 8 interleaved inputs
        float x[8], bb[8], y[4];
        unpack8(*reinterpret_cast<const bf16x8*>(src + 2 * c), x);
        unpack8(*reinterpret_cast<const bf16x8*>(b + 2 * c), bb);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float g = fminf(x[2 * i] + bb[2 * i], limit);
            const float u = fminf(fmaxf(x[2 * i + 1] + bb[2 * i + 1], -limit), limit);
            y[i] = (u + 1.f) * g / (1.f + __expf(-1.702f * g));
        }
        bf162 lo = __floats2bfloat162_rn(y[0], y[1]), hi = __floats2bfloat162_rn(y[2], y[3]);
        *reinterpret_cast<uint2*>(dst + c) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
}

__global__ void moe_row_bias_kernel(bf16* __restrict__ y, const bf16* __restrict__ bias,
                                    const int* __restrict__ tile_expert, int H) {
    const int row = blockIdx.x;
    const int e = tile_expert[row >> 7];
    if (e < 0) return;
    bf16* dst = y + (size_t)row * H;
    const bf16* b = bias + (size_t)e * H;
    for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
        float x[8], bb[8];
        unpack8(*reinterpret_cast<const bf16x8*>(dst + c), x);
        unpack8(*reinterpret_cast<const bf16x8*>(b + c), bb);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] += bb[i];
        *reinterpret_cast<bf16x8*>(dst + c) = pack8(x);
    }
}
}  // namespace pie

// act[rows, inter] from gu[rows, 2 * inter] + bias[E, 2 * inter]; rows = mtiles * 128.
PIE_API int pie_moe_bias_glu(const void* gu, const void* bias, const int* tile_expert, void* act, int mtiles, int inter,
                             float limit, cudaStream_t st) {
    if (mtiles <= 0) return 0;
    if (inter % 4) return (int)cudaErrorInvalidValue;
    pie::moe_bias_glu_kernel<<<mtiles * 128, 128, 0, st>>>((const bf16*)gu, (const bf16*)bias, tile_expert, (bf16*)act,
                                                           inter, limit);
    return (int)cudaGetLastError();
}

// y[rows, H] += bias[expert of row, H]
PIE_API int pie_moe_row_bias(void* y, const void* bias, const int* tile_expert, int mtiles, int H, cudaStream_t st) {
    if (mtiles <= 0) return 0;
    if (H % 8) return (int)cudaErrorInvalidValue;
    pie::moe_row_bias_kernel<<<mtiles * 128, 128, 0, st>>>((bf16*)y, (const bf16*)bias, tile_expert, H);
    return (int)cudaGetLastError();
}
