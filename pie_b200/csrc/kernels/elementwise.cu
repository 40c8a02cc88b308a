// Bandwidth-bound helper kernels of the model forward: embedding gather,
// RMSNorm (+residual add), SwiGLU, per-head q/k RMSNorm + RoPE + paged KV
// write, row gather, KV page copy and BRLE -> bitmask expansion.
//
// Counterparts in the reference (behaviour only, the code is new):
//   driver/cuda/src/kernels/embed.cu:11,28      row gather (+vocab shard)
//   driver/cuda/src/kernels/rmsnorm.cu:15-190   RMSNorm / residual variants
//   driver/cuda/src/kernels/swiglu.cu:180-260   silu(g)*u on packed [N,2I]
//   driver/cuda/src/kernels/split_packed.cu:62  qk-norm + rope + KV write
//   driver/cuda/src/kernels/kv_paged.cu:28-80   tail-append KV slot write
//   driver/cuda/src/kernels/gather_rows.cu:11   compact rows
//   driver/cuda/src/swap_pool.cpp               page copies
//   driver/cuda/src/brle.cpp                    BRLE decode (host in the reference)
#include <cuda_fp8.h>

#include "common.cuh"

namespace pie {

// ---------------------------------------------------------------- embedding
// out[t,:] = table[tok[t]-vocab_start,:] if the id is in this rank's shard
// else zeros (the shards are summed by the following reduce).
__global__ void embed_gather_kernel(const int* __restrict__ tokens, const bf16* __restrict__ table,
                                    bf16* __restrict__ out, int hidden, int vocab_start,
                                    int vocab_count) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = tokens[t] - vocab_start;
    const int nvec = hidden >> 3;
    bf16x8* dst = reinterpret_cast<bf16x8*>(out + (size_t)t * hidden);
    if (id < 0 || id >= vocab_count) {
        bf16x8 z;
#pragma unroll
        for (int i = 0; i < 4; ++i) z.v[i] = __floats2bfloat162_rn(0.f, 0.f);
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = z;
        return;
    }
    const bf16x8* src = reinterpret_cast<const bf16x8*>(table + (size_t)id * hidden);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = src[i];
}

// ------------------------------------------------------------------ rmsnorm
// If `delta` is non-null: residual[t,:] += delta[t,:] first (stored back in
// bf16), and the norm is taken of the updated residual. out may alias delta.
// VEC_PER_THREAD 8-element vectors are cached in registers between passes.
template <int MAXV>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const bf16* x, const bf16* delta, bf16* residual_out,
               const bf16* __restrict__ w, bf16* out, int hidden, float eps, float w_offset) {
    __shared__ float red[32];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int nvec = hidden >> 3;
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)t * hidden);
    const bf16x8* dr = delta ? reinterpret_cast<const bf16x8*>(delta + (size_t)t * hidden) : nullptr;
    bf16x8* rr = residual_out ? reinterpret_cast<bf16x8*>(residual_out + (size_t)t * hidden) : nullptr;
    float cache[MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i < nvec) {
            unpack8(xr[i], cache[j]);
            if (dr) {
                float d[8];
                unpack8(dr[i], d);
#pragma unroll
                for (int k = 0; k < 8; ++k) cache[j][k] += d[k];
                bf16x8 p = pack8(cache[j]);
                // the normalised value is computed from the rounded residual so
                // that a later reader of the bf16 residual sees the same numbers
                unpack8(p, cache[j]);
                if (rr) rr[i] = p;
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) ss += cache[j][k] * cache[j][k];
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)hidden + eps);
    const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
    bf16x8* orow = reinterpret_cast<bf16x8*>(out + (size_t)t * hidden);
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i < nvec) {
            float wv[8], o[8];
            unpack8(wr[i], wv);
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = cache[j][k] * inv * (wv[k] + w_offset);
            orow[i] = pack8(o);
        }
    }
}

// ------------------------------------------------------------------- swiglu
__global__ void swiglu_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int inter,
                              long total_vec) {
    const int vec_per_row = inter >> 3;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total_vec;
         i += (long)gridDim.x * blockDim.x) {
        const long row = i / vec_per_row;
        const int c = (int)(i - row * vec_per_row);
        const bf16x8* g = reinterpret_cast<const bf16x8*>(gu + row * 2 * (long)inter) + c;
        const bf16x8* u = reinterpret_cast<const bf16x8*>(gu + row * 2 * (long)inter + inter) + c;
        float gf[8], uf[8], o[8];
        unpack8(*g, gf);
        unpack8(*u, uf);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = gf[k] / (1.f + __expf(-gf[k])) * uf[k];
        reinterpret_cast<bf16x8*>(out + row * (long)inter)[c] = pack8(o);
    }
}

// GLU over INTERLEAVED columns (gate_0, up_0, gate_1, up_1, ...), the layout of the fused gate / up weights:
// out[r, j] = act(gu[r, 2j]) * gu[r, 2j + 1]. ACT 0: SiLU, 1: tanh-approximated GELU (Gemma's GeGLU).
template <int ACT>
__global__ void glu_interleaved_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, long total_vec) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total_vec; i += (long)gridDim.x * blockDim.x) {
        const bf16x8* src = reinterpret_cast<const bf16x8*>(gu) + 2 * i;
        float a[8], b[8], o[8];
        unpack8(src[0], a);
        unpack8(src[1], b);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float g = k < 4 ? a[2 * k] : b[2 * k - 8], u = k < 4 ? a[2 * k + 1] : b[2 * k - 7];
            if (ACT == 0) {
                o[k] = g / (1.f + __expf(-g)) * u;
            } else {
                const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
                o[k] = 0.5f * g * (1.f + t) * u;
            }
        }
        reinterpret_cast<bf16x8*>(out)[i] = pack8(o);
    }
}

// -------------------------------------------- q/k norm + rope + paged KV write
// One warp per (token, head) of the packed qkv row [Hq*d | Hkv*d | Hkv*d].
// q heads: optional RMSNorm over the head (weight qn[d]) then rotate-half RoPE,
// written to q_out[t, h, :]. k heads: same with kn, written to the K half of
// the token's KV slot. v heads: copied to the V half.
// KV layer layout: [pages][2][Hkv][page_size][d]; slot = page*page_size + off.
// A negative slot skips the KV write (padding tokens of a graph bucket).
// KV8: the K and V rows are stored as e4m3 bytes with one fp32 scale per (token, KV head) row,
// scale = max|x| / 448 (kv_layer then addresses bytes, kv_scale [pages][2][Hkv][page_size] floats).
template <int D, bool KV8>
__global__ void __launch_bounds__(256)
qk_norm_rope_kvwrite_kernel(const bf16* __restrict__ qkv, const int* __restrict__ positions,
                            const int* __restrict__ slots, const float* __restrict__ inv_freq,
                            const bf16* __restrict__ qn, const bf16* __restrict__ kn,
                            bf16* __restrict__ q_out, bf16* __restrict__ kv_layer, int n_tokens,
                            int hq, int hkv, int page_size, float eps, int qkv_stride,
                            float* __restrict__ kv_scale, const bf16* __restrict__ bias) {
    constexpr int EP = D / 64;  // elements per lane per half
    pdl_trigger();
    pdl_wait();
    const int heads = hq + 2 * hkv;
    const long gw = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (gw >= (long)n_tokens * heads) return;
    const int t = (int)(gw / heads);
    const int h = (int)(gw - (long)t * heads);
    const bf16* src = qkv + (size_t)t * qkv_stride + (size_t)h * D;
    float lo[EP], hi[EP];
#pragma unroll
    for (int e = 0; e < EP; ++e) {
        lo[e] = __bfloat162float(src[lane * EP + e]);
        hi[e] = __bfloat162float(src[D / 2 + lane * EP + e]);
    }
    if (bias) {     // projection bias (Qwen2): added here instead of by a pass of its own over the packed rows, rounded as that pass would
        const bf16* bp = bias + (size_t)h * D;
#pragma unroll
        for (int e = 0; e < EP; ++e) {
            lo[e] = __bfloat162float(__float2bfloat16(lo[e] + __bfloat162float(bp[lane * EP + e])));
            hi[e] = __bfloat162float(__float2bfloat16(hi[e] + __bfloat162float(bp[D / 2 + lane * EP + e])));
        }
    }
    const bool is_q = h < hq;
    const bool is_k = !is_q && h < hq + hkv;
    if (is_q || is_k) {
        const bf16* nw = is_q ? qn : kn;
        if (nw) {
            float ss = 0.f;
#pragma unroll
            for (int e = 0; e < EP; ++e) ss += lo[e] * lo[e] + hi[e] * hi[e];
            ss = warp_sum(ss);
            const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
            for (int e = 0; e < EP; ++e) {
                // round to bf16 after the norm as a separate norm kernel would
                lo[e] = __bfloat162float(__float2bfloat16(
                    lo[e] * inv * __bfloat162float(nw[lane * EP + e])));
                hi[e] = __bfloat162float(__float2bfloat16(
                    hi[e] * inv * __bfloat162float(nw[D / 2 + lane * EP + e])));
            }
        }
        const float pos = (float)positions[t];
#pragma unroll
        for (int e = 0; e < EP; ++e) {
            float s, c;
            sincosf(pos * inv_freq[lane * EP + e], &s, &c);
            const float a = lo[e], b = hi[e];
            lo[e] = a * c - b * s;
            hi[e] = b * c + a * s;
        }
    }
    bf16* dst;
    if (is_q) {
        dst = q_out + ((size_t)t * hq + h) * D;
    } else {
        const int slot = slots[t];
        if (slot < 0) return;
        const int page = slot / page_size, off = slot - page * page_size;
        const int kvh = is_k ? (h - hq) : (h - hq - hkv);
        const size_t row = (((size_t)page * 2 + (is_k ? 0 : 1)) * hkv + kvh) * page_size + off;
        if (KV8) {
            float amax = 0.f;
#pragma unroll
            for (int e = 0; e < EP; ++e) amax = fmaxf(amax, fmaxf(fabsf(lo[e]), fabsf(hi[e])));
            amax = warp_max(amax);
            const float scale = fmaxf(amax, 1e-12f) * (1.0f / 448.0f);
            const float inv = 1.0f / scale;
            uint8_t* d8 = reinterpret_cast<uint8_t*>(kv_layer) + row * D;
#pragma unroll
            for (int e = 0; e < EP; ++e) {
                d8[lane * EP + e] = (uint8_t)__nv_cvt_float_to_fp8(lo[e] * inv, __NV_SATFINITE, __NV_E4M3);
                d8[D / 2 + lane * EP + e] = (uint8_t)__nv_cvt_float_to_fp8(hi[e] * inv, __NV_SATFINITE, __NV_E4M3);
            }
            if (lane == 0) kv_scale[row] = scale;
            return;
        }
        dst = kv_layer + row * D;
    }
#pragma unroll
    for (int e = 0; e < EP; ++e) {
        dst[lane * EP + e] = __float2bfloat16(lo[e]);
        dst[D / 2 + lane * EP + e] = __float2bfloat16(hi[e]);
    }
}

// --------------------------------------------------------------- row gather
__global__ void gather_rows_kernel(const bf16* __restrict__ in, const int* __restrict__ idx,
                                   bf16* __restrict__ out, int hidden) {
    const int r = blockIdx.x;
    const bf16x8* src = reinterpret_cast<const bf16x8*>(in + (size_t)idx[r] * hidden);
    bf16x8* dst = reinterpret_cast<bf16x8*>(out + (size_t)r * hidden);
    for (int i = threadIdx.x; i < (hidden >> 3); i += blockDim.x) dst[i] = src[i];
}

// ---------------------------------------------------------------- page copy
// kv is [layers][pages][page_bytes]; copies src[i] -> dst[i] in every layer.
__global__ void copy_pages_kernel(uint4* __restrict__ kv, const int* __restrict__ src,
                                  const int* __restrict__ dst, long page_vec, long layer_vec) {
    const int pair = blockIdx.x, layer = blockIdx.y;
    const uint4* s = kv + layer * layer_vec + (long)src[pair] * page_vec;
    uint4* d = kv + layer * layer_vec + (long)dst[pair] * page_vec;
    for (long i = threadIdx.x; i < page_vec; i += blockDim.x) d[i] = s[i];
}

// --------------------------------------------------------------- brle expand
// Row r has runs run_ends[indptr[r] .. indptr[r+1]) given as cumulative end
// offsets; run 0 is a run of zeros, run 1 of ones, alternating. Bits past the
// last run are `tail_value`. Output: bitmask[r, words] with bit i of the row at
// word i/32, bit i%32.
__global__ void brle_expand_kernel(const uint32_t* __restrict__ run_ends,
                                   const int* __restrict__ indptr, uint32_t* __restrict__ out,
                                   int words, int nbits, int tail_value) {
    const int r = blockIdx.y;
    const uint32_t* ends = run_ends + indptr[r];
    const int nr = indptr[r + 1] - indptr[r];
    for (int w = blockIdx.x * blockDim.x + threadIdx.x; w < words; w += gridDim.x * blockDim.x) {
        const uint32_t base = (uint32_t)w * 32u;
        // first run whose end is > base
        int lo = 0, hi = nr;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (ends[mid] > base) hi = mid; else lo = mid + 1;
        }
        uint32_t word = 0;
        uint32_t bit = base;
        int run = lo;
        const uint32_t limit = min(base + 32u, (uint32_t)nbits);
        while (bit < limit) {
            uint32_t end;
            int val;
            if (run < nr) { end = min(ends[run], limit); val = run & 1; }
            else { end = limit; val = tail_value; }
            if (val && end > bit) {
                const uint32_t n = end - bit;
                const uint32_t m = (n >= 32u) ? 0xffffffffu : ((1u << n) - 1u);
                word |= m << (bit - base);
            }
            bit = max(end, bit);
            ++run;
            if (run > nr + 1) break;
        }
        out[(size_t)r * words + w] = word;
    }
}

// The same for rows of different lengths in one launch: row r has row_nbits[r] bits and its words start at
// out + row_word_offset[r] (rows of one request back to back: the layout the prefill kernels read custom masks in).
__global__ void brle_expand_ragged_kernel(const uint32_t* __restrict__ run_ends, const int* __restrict__ indptr,
                                          uint32_t* __restrict__ out, const long* __restrict__ row_word_offset,
                                          const int* __restrict__ row_nbits, int tail_value) {
    const int r = blockIdx.y;
    const uint32_t* ends = run_ends + indptr[r];
    const int nr = indptr[r + 1] - indptr[r];
    const int nbits = row_nbits[r];
    const int words = (nbits + 31) >> 5;
    uint32_t* dst = out + row_word_offset[r];
    for (int w = blockIdx.x * blockDim.x + threadIdx.x; w < words; w += gridDim.x * blockDim.x) {
        const uint32_t base = (uint32_t)w * 32u;
        int lo = 0, hi = nr;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (ends[mid] > base) hi = mid; else lo = mid + 1;
        }
        uint32_t word = 0, bit = base;
        int run = lo;
        const uint32_t limit = min(base + 32u, (uint32_t)nbits);
        while (bit < limit) {
            uint32_t end;
            int val;
            if (run < nr) { end = min(ends[run], limit); val = run & 1; }
            else { end = limit; val = tail_value; }
            if (val && end > bit) {
                const uint32_t n = end - bit;
                word |= ((n >= 32u) ? 0xffffffffu : ((1u << n) - 1u)) << (bit - base);
            }
            bit = max(end, bit);
            if (++run > nr + 1) break;
        }
        dst[w] = word;
    }
}

}  // namespace pie

using namespace pie;

PIE_API int pie_embed_gather(const int* tokens, const void* table, void* out, int n_tokens,
                             int hidden, int vocab_start, int vocab_count, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (hidden % 8) return (int)cudaErrorInvalidValue;
    launch_pdl(embed_gather_kernel, dim3(n_tokens), dim3(128), 0, st, tokens, (const bf16*)table, (bf16*)out, hidden,
                                                  vocab_start, vocab_count);
    return (int)cudaGetLastError();
}

PIE_API int pie_rmsnorm(const void* x, const void* delta, void* residual_out, const void* w,
                        void* out, int rows, int hidden, float eps, float w_offset,
                        cudaStream_t st) {
    if (rows <= 0) return 0;
    if (hidden % 8 || hidden > 256 * 8 * 8) return (int)cudaErrorInvalidValue;
    const int nvec = hidden / 8;
    const int per = (nvec + 255) / 256;
#define LAUNCH(MV)                                                                              \
    launch_pdl(rmsnorm_kernel<MV>, dim3(rows), dim3(256), 0, st, (const bf16*)x, (const bf16*)delta, \
               (bf16*)residual_out, (const bf16*)w, (bf16*)out, hidden, eps, w_offset)
    if (per <= 1) LAUNCH(1);
    else if (per <= 2) LAUNCH(2);
    else if (per <= 4) LAUNCH(4);
    else LAUNCH(8);
#undef LAUNCH
    return (int)cudaGetLastError();
}

// fp8 (e4m3) weights with one fp32 scale per (row, 128 columns): out = bf16(w8 * scale).
// 16 weights per thread. Replaces driver/cuda/src/kernels/dequant_fp8.cu:41 (per-group expand).
__global__ void dequant_fp8_rowblock_kernel(const uint8_t* __restrict__ w8, const float* __restrict__ scale,
                                            bf16* __restrict__ out, int K, long total_vec) {
    const int vec_per_row = K >> 4;
    const int kblocks = (K + 127) >> 7;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total_vec; i += (long)gridDim.x * blockDim.x) {
        const long row = i / vec_per_row;
        const int c = (int)(i - row * vec_per_row) << 4;
        const float sc = scale[row * kblocks + (c >> 7)];
        const uint4 raw = *reinterpret_cast<const uint4*>(w8 + row * (long)K + c);
        const __nv_fp8x2_storage_t* p2 = reinterpret_cast<const __nv_fp8x2_storage_t*>(&raw);
        float f[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2(p2[j], __NV_E4M3);
            const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&h2));
            f[2 * j] = v.x * sc;
            f[2 * j + 1] = v.y * sc;
        }
        bf16x8* dst = reinterpret_cast<bf16x8*>(out + row * (long)K + c);
        dst[0] = pack8(f);
        dst[1] = pack8(f + 8);
    }
}

PIE_API int pie_dequant_fp8_rowblock(const void* w8, const float* scale, void* out, long rows, int K,
                                     cudaStream_t st) {
    if (rows <= 0) return 0;
    if (K % 16) return (int)cudaErrorInvalidValue;
    const long total = rows * (K / 16);
    const int blocks = (int)min((total + 255) / 256, (long)148 * 32);
    dequant_fp8_rowblock_kernel<<<blocks, 256, 0, st>>>((const uint8_t*)w8, scale, (bf16*)out, K, total);
    return (int)cudaGetLastError();
}

PIE_API int pie_swiglu(const void* gate_up, void* out, long rows, int inter, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (inter % 8) return (int)cudaErrorInvalidValue;
    const long total = rows * (inter / 8);
    const int blocks = (int)min((total + 255) / 256, (long)148 * 16);
    swiglu_kernel<<<blocks, 256, 0, st>>>((const bf16*)gate_up, (bf16*)out, inter, total);
    return (int)cudaGetLastError();
}

PIE_API int pie_glu_interleaved(const void* gate_up, void* out, long rows, int inter, int act, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (inter % 8 || act < 0 || act > 1) return (int)cudaErrorInvalidValue;
    const long total = rows * (inter / 8);
    const int blocks = (int)min((total + 255) / 256, (long)148 * 16);
    if (act == 0)
        glu_interleaved_kernel<0><<<blocks, 256, 0, st>>>((const bf16*)gate_up, (bf16*)out, total);
    else
        glu_interleaved_kernel<1><<<blocks, 256, 0, st>>>((const bf16*)gate_up, (bf16*)out, total);
    return (int)cudaGetLastError();
}

PIE_API int pie_qk_bias_norm_rope_kvwrite(const void* qkv, const void* qkv_bias, const int* positions, const int* slots,
                                          const float* inv_freq, const void* q_norm_w, const void* k_norm_w,
                                          void* q_out, void* kv_layer, float* kv_scale, int n_tokens, int hq,
                                          int hkv, int head_dim, int page_size, float eps, int qkv_stride,
                                          cudaStream_t st);

PIE_API int pie_qk_norm_rope_kvwrite(const void* qkv, const int* positions, const int* slots,
                                     const float* inv_freq, const void* q_norm_w,
                                     const void* k_norm_w, void* q_out, void* kv_layer,
                                     int n_tokens, int hq, int hkv, int head_dim, int page_size,
                                     float eps, int qkv_stride, cudaStream_t st) {
    return pie_qk_bias_norm_rope_kvwrite(qkv, nullptr, positions, slots, inv_freq, q_norm_w, k_norm_w, q_out, kv_layer,
                                         nullptr, n_tokens, hq, hkv, head_dim, page_size, eps, qkv_stride, st);
}

// The same with fp8 KV pages: kv_layer holds e4m3 bytes, kv_scale one fp32 per (token, KV head) row.
PIE_API int pie_qk_norm_rope_kvwrite_kv8(const void* qkv, const int* positions, const int* slots,
                                         const float* inv_freq, const void* q_norm_w, const void* k_norm_w,
                                         void* q_out, void* kv_layer, float* kv_scale, int n_tokens, int hq,
                                         int hkv, int head_dim, int page_size, float eps, int qkv_stride,
                                         cudaStream_t st) {
    if (!kv_scale) return (int)cudaErrorInvalidValue;
    return pie_qk_bias_norm_rope_kvwrite(qkv, nullptr, positions, slots, inv_freq, q_norm_w, k_norm_w, q_out, kv_layer,
                                         kv_scale, n_tokens, hq, hkv, head_dim, page_size, eps, qkv_stride, st);
}

// The general form: optional projection bias [(hq + 2 hkv) * head_dim] added to the packed rows first; kv_scale non-null
// selects fp8 KV pages (head_dim 64 / 128).
PIE_API int pie_qk_bias_norm_rope_kvwrite(const void* qkv, const void* qkv_bias, const int* positions, const int* slots,
                                          const float* inv_freq, const void* q_norm_w, const void* k_norm_w,
                                          void* q_out, void* kv_layer, float* kv_scale, int n_tokens, int hq,
                                          int hkv, int head_dim, int page_size, float eps, int qkv_stride,
                                          cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    const long warps = (long)n_tokens * (hq + 2 * hkv);
    const int blocks = (int)((warps + 7) / 8);
#define LAUNCH(D, KV8)                                                                           \
    launch_pdl(qk_norm_rope_kvwrite_kernel<D, KV8>, dim3(blocks), dim3(256), 0, st,             \
        (const bf16*)qkv, positions, slots, inv_freq, (const bf16*)q_norm_w,                    \
        (const bf16*)k_norm_w, (bf16*)q_out, (bf16*)kv_layer, n_tokens, hq, hkv, page_size, eps, \
        qkv_stride, kv_scale, (const bf16*)qkv_bias)
    if (kv_scale) {
        if (head_dim == 64) LAUNCH(64, true);
        else if (head_dim == 128) LAUNCH(128, true);
        else return (int)cudaErrorInvalidValue;
    } else {
        if (head_dim == 64) LAUNCH(64, false);
        else if (head_dim == 128) LAUNCH(128, false);
        else if (head_dim == 256) LAUNCH(256, false);
        else return (int)cudaErrorInvalidValue;
    }
#undef LAUNCH
    return (int)cudaGetLastError();
}

PIE_API int pie_gather_rows(const void* in, const int* idx, void* out, int rows, int hidden,
                            cudaStream_t st) {
    if (rows <= 0) return 0;
    if (hidden % 8) return (int)cudaErrorInvalidValue;
    gather_rows_kernel<<<rows, 128, 0, st>>>((const bf16*)in, idx, (bf16*)out, hidden);
    return (int)cudaGetLastError();
}

PIE_API int pie_copy_pages(void* kv, const int* src, const int* dst, int n_pairs, int layers,
                           long page_bytes, long layer_bytes, cudaStream_t st) {
    if (n_pairs <= 0) return 0;
    if (page_bytes % 16 || layer_bytes % 16) return (int)cudaErrorInvalidValue;
    dim3 grid(n_pairs, layers);
    copy_pages_kernel<<<grid, 256, 0, st>>>((uint4*)kv, src, dst, page_bytes / 16,
                                            layer_bytes / 16);
    return (int)cudaGetLastError();
}

PIE_API int pie_brle_expand(const uint32_t* run_ends, const int* indptr, uint32_t* out, int rows,
                            int nbits, int tail_value, cudaStream_t st) {
    if (rows <= 0) return 0;
    const int words = (nbits + 31) / 32;
    dim3 grid(min((words + 127) / 128, 1024), rows);
    brle_expand_kernel<<<grid, 128, 0, st>>>(run_ends, indptr, out, words, nbits, tail_value);
    return (int)cudaGetLastError();
}

PIE_API int pie_brle_expand_ragged(const uint32_t* run_ends, const int* indptr, uint32_t* out, const long* row_word_offset,
                                   const int* row_nbits, int rows, int max_words, int tail_value, cudaStream_t st) {
    if (rows <= 0 || max_words <= 0) return 0;
    dim3 grid(min((max_words + 127) / 128, 64), rows);
    brle_expand_ragged_kernel<<<grid, 128, 0, st>>>(run_ends, indptr, out, row_word_offset, row_nbits, tail_value);
    return (int)cudaGetLastError();
}

// ------------------------------------------------------------- token feed
// Decode pipelining: the input token of row i is the token sampled for row
// src_row[i] by the previous step (still on the device), unless src_row[i] < 0,
// in which case the host-provided token already in `tokens` stays.
namespace pie {
__global__ void feed_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ src_row,
                                   const int* __restrict__ prev_sampled, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const int s = src_row[i];
        if (s >= 0) tokens[i] = prev_sampled[s];
    }
}
}  // namespace pie

namespace pie {
// Debug check of an index table before the kernels that trust it run: an entry outside [lo, hi) is
// recorded (first one wins) and nothing is dereferenced.
__global__ void validate_indices_kernel(const int* __restrict__ v, int n, int lo, int hi, int table_code,
                                        int* __restrict__ status) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int x = v[i];
    if (x < lo || x >= hi) {
        if (atomicCAS(&status[0], 0, PIE_ERR_BOUNDS) == 0) status[1] = (table_code << 24) | min(i, 0xFFFFFF);
    }
}
}  // namespace pie

PIE_API int pie_validate_indices(const int* v, int n, int lo, int hi, int table_code, int* status, cudaStream_t st) {
    if (n <= 0) return 0;
    pie::validate_indices_kernel<<<(n + 255) / 256, 256, 0, st>>>(v, n, lo, hi, table_code, status);
    return (int)cudaGetLastError();
}

PIE_API int pie_feed_tokens(int* tokens, const int* src_row, const int* prev_sampled, int n,
                            cudaStream_t st) {
    if (n <= 0) return 0;
    pie::feed_tokens_kernel<<<(n + 255) / 256, 256, 0, st>>>(tokens, src_row, prev_sampled, n);
    return (int)cudaGetLastError();
}
