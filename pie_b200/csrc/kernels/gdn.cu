// Recurrent mixers of the hybrid models. Mamba-2 (state-space) is at the end of the file; first the
// Gated DeltaNet (linear attention) mixer: the short causal convolution over the
// q | k | v channels with its per-slot tail state, and the gated delta-rule recurrence with the gated
// RMSNorm on its output. One launch serves a ragged batch (prefill chunks and decode rows alike): the
// state of every request lives in its slot of the recurrent-state cache and is carried from fire to fire.
//
//   conv:       y[t, c] = silu( sum_j w[c, j] * x[t - (K-1) + j, c] ), inputs before the first token of
//               this fire come from the slot's last K-1 inputs (zeros after a reset)
//   recurrence: per value head, S in R^{dk x dv} (fp32):
//               S <- S * exp(g);  delta = (v - k^T S) * beta;  S <- S + k (x) delta;  o = q^T S
//               with q, k L2-normalised (q also scaled by dk^-1/2), beta = sigmoid(b),
//               g = -exp(A_log) * softplus(a + dt_bias)
//   output:     out = RMSNorm(o) * w_norm * silu(z)
//
// The recurrence kernel is the plain token-serial form: one CTA per (request, value head), one thread per
// state column, the column's dk values in registers. It is exact for any chunking of a sequence.
//
// Counterpart in the reference (behaviour only): driver/cuda/src/kernels/gated_delta_net.cu
// (l2norm, g / beta, recurrent_step*), driver/cuda/src/recurrent_state_cache.cpp (slot layout, slot copy).
#include "common.cuh"

namespace pie {

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// x: [N, F] fused projection (first C columns are the convolved channels); state: [S, C, K-1] fp32.
template <int K>
__global__ void gdn_conv_kernel(const bf16* __restrict__ x, int x_stride, const bf16* __restrict__ w,
                                const bf16* __restrict__ bias, const float* __restrict__ state,
                                const int* __restrict__ qo_indptr,
                                const int* __restrict__ tok_req, const int* __restrict__ slots,
                                const int* __restrict__ reset, float* __restrict__ y, int n, int c) {
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    const int t = blockIdx.y;
    if (ch >= c || t >= n) return;
    const int r = tok_req[t];
    if (slots[r] < 0) return;          // a padding request of a decode graph's bucket: no state, no output
    const int first = qo_indptr[r];
    const int i = t - first;
    const bool fresh = reset[r] != 0;
    const float* st = state + ((size_t)slots[r] * c + ch) * (K - 1);
    float acc = bias ? __bfloat162float(bias[ch]) : 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) {
        const int idx = i - (K - 1) + j;
        float v;
        if (idx >= 0) v = __bfloat162float(x[(size_t)(first + idx) * x_stride + ch]);
        else v = fresh ? 0.f : st[(K - 1) + idx];
        acc += __bfloat162float(w[ch * K + j]) * v;
    }
    y[(size_t)t * c + ch] = silu_f(acc);
}

// New tail of every request's slot: its last K-1 inputs (older ones come from the previous tail).
template <int K>
__global__ void gdn_conv_state_kernel(const bf16* __restrict__ x, int x_stride, float* __restrict__ state,
                                      const int* __restrict__ qo_indptr, const int* __restrict__ slots,
                                      const int* __restrict__ reset, int c) {
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (ch >= c) return;
    const int first = qo_indptr[r], len = qo_indptr[r + 1] - first;
    if (len <= 0 || slots[r] < 0) return;
    float* st = state + ((size_t)slots[r] * c + ch) * (K - 1);
    const bool fresh = reset[r] != 0;
    float nv[K - 1];
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
        const int idx = len - (K - 1) + j;                 // position within this fire's rows
        if (idx >= 0) nv[j] = __bfloat162float(x[(size_t)(first + idx) * x_stride + ch]);
        else nv[j] = fresh ? 0.f : st[(K - 1) + idx];
    }
#pragma unroll
    for (int j = 0; j < K - 1; ++j) st[j] = nv[j];
}

// grid (requests, value heads), block = SPLIT * dv threads (<= 256). A state column S[:, j] is held in
// registers by SPLIT adjacent lanes, DK / SPLIT rows each; their partial dot products meet through
// shuffles. SPLIT = 2 for dk = 128 (64 rows per lane). Measured: a four-way split with 512-thread blocks
// (no spills, 16 warps per SM) is slower - 542 against 471 us for 256 decode rows - because the three
// block-wide reductions per token grow with the block.
template <int DK, int SPLIT>
__global__ void __launch_bounds__(256)
gdn_recurrent_kernel(const float* __restrict__ conv, const bf16* __restrict__ x, int x_stride,
                     const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                     const bf16* __restrict__ norm_w, float* __restrict__ rec_state,
                     const int* __restrict__ qo_indptr, const int* __restrict__ slots,
                     const int* __restrict__ reset, bf16* __restrict__ out, int hk, int hv, int dv, float eps) {
    constexpr int ROWS = DK / SPLIT;
    __shared__ float sq[DK], sk[DK], red[32], sc[2];
    const int r = blockIdx.x, h = blockIdx.y;
    const int j = threadIdx.x / SPLIT, part = threadIdx.x % SPLIT;
    const int first = qo_indptr[r], len = qo_indptr[r + 1] - first;
    if (len <= 0 || slots[r] < 0) return;
    const int kh = h / (hv / hk);
    const int c = 2 * hk * DK + hv * dv;
    float* sp = rec_state + (((size_t)slots[r] * hv + h) * DK + (size_t)part * ROWS) * dv + j;
    float S[ROWS];
    if (reset[r]) {
#pragma unroll
        for (int i = 0; i < ROWS; ++i) S[i] = 0.f;
    } else {
#pragma unroll
        for (int i = 0; i < ROWS; ++i) S[i] = sp[(size_t)i * dv];
    }
    const float decay_rate = -__expf(a_log[h]);
    const float bias = dt_bias[h];
    const float wn = __bfloat162float(norm_w[j]);
    const float* mq = sq + part * ROWS;
    const float* mk = sk + part * ROWS;
    for (int t = 0; t < len; ++t) {
        const size_t row = (size_t)(first + t);
        const float* cr = conv + row * c;
        // q, k of this value head's key head: L2 norms over dk
        float q2 = 0.f, k2 = 0.f;
        for (int i = threadIdx.x; i < DK; i += blockDim.x) {
            const float qv = cr[kh * DK + i], kv = cr[hk * DK + kh * DK + i];
            sq[i] = qv;
            sk[i] = kv;
            q2 += qv * qv;
            k2 += kv * kv;
        }
        q2 = block_sum(q2, red);
        k2 = block_sum(k2, red);
        if (threadIdx.x == 0) {
            const bf16* xr = x + row * x_stride + c + hv * dv;
            sc[0] = 1.f / (1.f + __expf(-__bfloat162float(xr[h])));                        // beta
            sc[1] = __expf(decay_rate * softplus_f(__bfloat162float(xr[hv + h]) + bias));   // exp(g)
        }
        __syncthreads();
        const float qs = rsqrtf(q2 + 1e-6f) * rsqrtf((float)DK), ks = rsqrtf(k2 + 1e-6f);
        const float beta = sc[0], decay = sc[1];
        const float v = cr[2 * hk * DK + h * dv + j];
        float kv = 0.f;
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            S[i] *= decay;
            kv += mk[i] * S[i];
        }
        if (SPLIT >= 2) kv += __shfl_xor_sync(0xffffffffu, kv, 1);
        if (SPLIT == 4) kv += __shfl_xor_sync(0xffffffffu, kv, 2);
        const float delta = (v - kv * ks) * beta * ks;          // k is used normalised on both sides
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            S[i] += mk[i] * delta;
            o += mq[i] * S[i];
        }
        if (SPLIT >= 2) o += __shfl_xor_sync(0xffffffffu, o, 1);
        if (SPLIT == 4) o += __shfl_xor_sync(0xffffffffu, o, 2);
        o *= qs;
        const float ms = block_sum(part == 0 ? o * o : 0.f, red) / (float)dv;
        if (part == 0) {
            const float z = __bfloat162float(x[row * x_stride + c + h * dv + j]);
            out[row * (size_t)(hv * dv) + h * dv + j] = __float2bfloat16(o * rsqrtf(ms + eps) * wn * silu_f(z));
        }
        __syncthreads();                                   // sq / sk / sc are rewritten by the next token
    }
#pragma unroll
    for (int i = 0; i < ROWS; ++i) sp[(size_t)i * dv] = S[i];
}

// Mamba-2 state update: grid (requests, heads), block = head_dim threads; thread p holds S[p, :] (NS values)
// in registers. conv: [N, inner + 2 * groups * NS] (x | B | C after the convolution); x: the projection
// [N, z | x B C | dt] for dt; y: [N, inner] fp32 (gate and norm follow outside: they span all heads).
template <int NS>
__global__ void __launch_bounds__(256)
mamba2_ssm_kernel(const float* __restrict__ conv, const bf16* __restrict__ x, int x_stride,
                  const float* __restrict__ a_log, const float* __restrict__ dt_bias, const float* __restrict__ d_skip,
                  float* __restrict__ rec_state, const int* __restrict__ qo_indptr, const int* __restrict__ slots,
                  const int* __restrict__ reset, float* __restrict__ y, int heads, int head_dim, int groups) {
    __shared__ float sb[NS], scv[NS], sc[1];
    const int r = blockIdx.x, h = blockIdx.y, p = threadIdx.x;
    const int first = qo_indptr[r], len = qo_indptr[r + 1] - first;
    if (len <= 0 || slots[r] < 0) return;
    const int inner = heads * head_dim, c = inner + 2 * groups * NS;
    const int g = h / (heads / groups);
    float* sp = rec_state + (((size_t)slots[r] * heads + h) * head_dim + p) * NS;
    float S[NS];
    if (reset[r]) {
#pragma unroll
        for (int i = 0; i < NS; ++i) S[i] = 0.f;
    } else {
#pragma unroll
        for (int i = 0; i < NS; ++i) S[i] = sp[i];
    }
    const float a = -__expf(a_log[h]), bias = dt_bias[h], dsk = d_skip[h];
    for (int t = 0; t < len; ++t) {
        const size_t row = (size_t)(first + t);
        const float* cr = conv + row * c;
        for (int i = p; i < NS; i += blockDim.x) {
            sb[i] = cr[inner + g * NS + i];
            scv[i] = cr[inner + groups * NS + g * NS + i];
        }
        if (p == 0) sc[0] = softplus_f(__bfloat162float(x[row * x_stride + inner + c + h]) + bias);
        __syncthreads();
        const float dt = sc[0], xv = cr[h * head_dim + p];
        const float decay = __expf(dt * a), dx = dt * xv;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < NS; ++i) {
            S[i] = S[i] * decay + dx * sb[i];
            acc += S[i] * scv[i];
        }
        y[row * inner + h * head_dim + p] = acc + dsk * xv;
        __syncthreads();                                   // sb / scv / sc are rewritten by the next token
    }
#pragma unroll
    for (int i = 0; i < NS; ++i) sp[i] = S[i];
}

// dst slot <- src slot in both caches of every linear layer (fork of a context).
__global__ void gdn_copy_slot_kernel(float* __restrict__ buf, size_t layer_stride, size_t slot_elems, int layers,
                                     int src, int dst) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= slot_elems) return;
    for (int l = 0; l < layers; ++l) {
        float* base = buf + (size_t)l * layer_stride;
        base[(size_t)dst * slot_elems + i] = base[(size_t)src * slot_elems + i];
    }
}

}  // namespace pie

PIE_API int pie_gdn_mixer(const void* x, int x_stride, const void* conv_w, const float* a_log, const float* dt_bias,
                          const void* norm_w, float* conv_state, float* rec_state, const int* qo_indptr,
                          const int* tok_req, const int* slots, const int* reset, float* conv_scratch, void* out,
                          int n, int r, int hk, int hv, int dk, int dv, int kernel, float eps, cudaStream_t st) {
    using namespace pie;
    if (n <= 0 || r <= 0) return 0;
    if (kernel != 4) return (int)cudaErrorInvalidValue;
    if (dv % 32 != 0 || dv > 256 || (dk == 128 && dv > 128) || hv % hk != 0) return (int)cudaErrorInvalidValue;
    const int c = 2 * hk * dk + hv * dv;
    const bf16* xb = static_cast<const bf16*>(x);
    dim3 cg((c + 127) / 128, n);
    gdn_conv_kernel<4><<<cg, 128, 0, st>>>(xb, x_stride, static_cast<const bf16*>(conv_w), nullptr, conv_state,
                                           qo_indptr, tok_req, slots, reset, conv_scratch, n, c);
    dim3 sg((c + 127) / 128, r);
    gdn_conv_state_kernel<4><<<sg, 128, 0, st>>>(xb, x_stride, conv_state, qo_indptr, slots, reset, c);
    dim3 rg(r, hv);
#define PIE_GDN_LAUNCH(DKV, SP)                                                                                  \
    gdn_recurrent_kernel<DKV, SP><<<rg, SP * dv, 0, st>>>(conv_scratch, xb, x_stride, a_log, dt_bias,            \
                                                 static_cast<const bf16*>(norm_w), rec_state, qo_indptr, slots, \
                                                 reset, static_cast<bf16*>(out), hk, hv, dv, eps)
    if (dk == 32) PIE_GDN_LAUNCH(32, 1);
    else if (dk == 64) PIE_GDN_LAUNCH(64, 1);
    else if (dk == 128) PIE_GDN_LAUNCH(128, 2);
    else return (int)cudaErrorInvalidValue;
#undef PIE_GDN_LAUNCH
    return (int)cudaGetLastError();
}

PIE_API int pie_mamba2_mixer(const void* x, int x_stride, const void* conv_w, const void* conv_b, const float* a_log,
                             const float* dt_bias, const float* d_skip, float* conv_state, float* rec_state,
                             const int* qo_indptr, const int* tok_req, const int* slots, const int* reset,
                             float* conv_scratch, float* y, int n, int r, int heads, int head_dim, int state, int groups,
                             cudaStream_t st) {
    using namespace pie;
    if (n <= 0 || r <= 0) return 0;
    if (head_dim > 256 || heads % groups != 0) return (int)cudaErrorInvalidValue;
    const int inner = heads * head_dim, c = inner + 2 * groups * state;
    const bf16* xb = static_cast<const bf16*>(x) + inner;          // the convolved channels follow the gate
    dim3 cg((c + 127) / 128, n);
    gdn_conv_kernel<4><<<cg, 128, 0, st>>>(xb, x_stride, static_cast<const bf16*>(conv_w), static_cast<const bf16*>(conv_b),
                                           conv_state, qo_indptr, tok_req, slots, reset, conv_scratch, n, c);
    dim3 sg((c + 127) / 128, r);
    gdn_conv_state_kernel<4><<<sg, 128, 0, st>>>(xb, x_stride, conv_state, qo_indptr, slots, reset, c);
    dim3 rg(r, heads);
    const bf16* x0 = static_cast<const bf16*>(x);
#define PIE_MAMBA_LAUNCH(NSV)                                                                                   \
    mamba2_ssm_kernel<NSV><<<rg, head_dim, 0, st>>>(conv_scratch, x0, x_stride, a_log, dt_bias, d_skip, rec_state, \
                                                    qo_indptr, slots, reset, y, heads, head_dim, groups)
    if (state == 16) PIE_MAMBA_LAUNCH(16);
    else if (state == 64) PIE_MAMBA_LAUNCH(64);
    else if (state == 128) PIE_MAMBA_LAUNCH(128);
    else return (int)cudaErrorInvalidValue;
#undef PIE_MAMBA_LAUNCH
    return (int)cudaGetLastError();
}

PIE_API int pie_gdn_copy_slot(float* buf, long layer_stride, long slot_elems, int layers, int src, int dst,
                              cudaStream_t st) {
    if (slot_elems <= 0 || layers <= 0 || src == dst) return 0;
    pie::gdn_copy_slot_kernel<<<(unsigned)((slot_elems + 255) / 256), 256, 0, st>>>(buf, (size_t)layer_stride,
                                                                                    (size_t)slot_elems, layers, src, dst);
    return (int)cudaGetLastError();
}
