// Token sampling and probe kernels over bf16 logits.
//
// pie_sample: per row temperature, top-k, top-p, min-p, a seeded counter-based
// random stream and an optional vocabulary bitmask (constrained decoding), all
// on the device. The kept set is found exactly on the 16-bit order key of the
// bf16 logits with a two-level radix select (two histogram passes), then one
// token is drawn from the renormalised kept set with the Gumbel-max trick, so
// no sort, no probability row in memory and no host round trip is needed.
// Temperature <= 0 selects the arg-max (lowest index on ties).
//
// Reference behaviour: driver/cuda/src/kernels/sample_temp.cu:30-180 (Gumbel-max
// with hash noise, min-p), driver/cuda/src/kernels/sample_flashinfer.cu:19,86
// (top-k / top-p), driver/cuda/src/executor/executor.cpp:2741-2756 (logit masks
// are applied on the host there; here the sampler consumes them),
// driver/cuda/src/kernels/{logprobs,entropy}.cu (probes from unscaled logits).
#include "common.cuh"

namespace pie {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_WARPS = SAMPLE_THREADS / 32;

__device__ __forceinline__ uint32_t bf16_key(uint16_t bits) {
    return (bits & 0x8000u) ? (uint32_t)(uint16_t)~bits : (uint32_t)(bits | 0x8000u);
}
__device__ __forceinline__ uint32_t f32_key(float f) {
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long x = __shfl_xor_sync(0xffffffffu, v, o);
        v = x > v ? x : v;
    }
    return v;
}
// Block-wide max of a packed (key << 32 | ~index) value.
__device__ __forceinline__ unsigned long long block_max_u64(unsigned long long v,
                                                            unsigned long long* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    v = warp_max_u64(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    unsigned long long t = lane < SAMPLE_WARPS ? red[lane] : 0ull;
    return warp_max_u64(t);
}

struct RowView {
    const uint4* vec;       // row as 16-byte vectors of 8 bf16
    const uint32_t* mask;   // vocabulary bitmask of the row or null
    int nvec;
    __device__ __forceinline__ bool allowed(int idx) const {
        return !mask || ((mask[idx >> 5] >> (idx & 31)) & 1u);
    }
};

// Visit every 8-element vector of the row: f(vector index, 8 bf16). Four loads are in flight per
// thread before the first is consumed (a single dependent load per thread leaves the pass
// latency-bound on L2).
template <typename F>
__device__ __forceinline__ void scan_row(const RowView& rv, F&& f) {
    constexpr int U = 4;
    for (int v0 = threadIdx.x; v0 < rv.nvec; v0 += SAMPLE_THREADS * U) {
        uint4 pk[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int v = v0 + u * SAMPLE_THREADS;
            if (v < rv.nvec) pk[u] = rv.vec[v];
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int v = v0 + u * SAMPLE_THREADS;
            if (v < rv.nvec) f(v, pk[u]);
        }
    }
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const bf16* __restrict__ logits, long row_stride, int vocab,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p,
              const unsigned long long* __restrict__ seeds, const uint32_t* __restrict__ mask_bits,
              const int* __restrict__ mask_row, int mask_words, int* __restrict__ out_tokens) {
    extern __shared__ __align__(16) uint8_t dyn[];
    int* h_cnt = reinterpret_cast<int*>(dyn);                          // [W][256]
    float* h_mass = reinterpret_cast<float*>(dyn) + SAMPLE_WARPS * 256;  // [W][256]
    __shared__ unsigned long long red64[32];
    __shared__ float redf[32];
    __shared__ int s_cnt[256];
    __shared__ float s_mass[256];
    __shared__ int s_sel[6];
    __shared__ float s_self[4];

    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    RowView rv;
    rv.vec = reinterpret_cast<const uint4*>(logits + (size_t)row * row_stride);
    rv.nvec = vocab >> 3;
    const int mr = mask_row ? mask_row[row] : -1;
    rv.mask = (mask_bits && mr >= 0) ? mask_bits + (size_t)mr * mask_words : nullptr;

    // ---- pass 1: arg-max over the allowed entries
    unsigned long long best = 0ull;
    scan_row(rv, [&](int v, const uint4& pk) {
        const uint16_t* e = reinterpret_cast<const uint16_t*>(&pk);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int idx = v * 8 + k;
            if (!rv.allowed(idx)) continue;
            const unsigned long long cand =
                ((unsigned long long)(bf16_key(e[k]) + 1u) << 32) | (0xffffffffu - (uint32_t)idx);
            best = cand > best ? cand : best;
        }
    });
    best = block_max_u64(best, red64);
    const float T = temperature[row];
    if (best == 0ull) {  // nothing allowed: emit token 0
        if (threadIdx.x == 0) out_tokens[row] = 0;
        return;
    }
    const int arg = (int)(0xffffffffu - (uint32_t)(best & 0xffffffffu));
    if (T <= 0.f) {
        if (threadIdx.x == 0) out_tokens[row] = arg;
        return;
    }
    const uint32_t kmax = (uint32_t)(best >> 32) - 1u;
    float xmax;
    {
        const uint16_t b = (kmax & 0x8000u) ? (uint16_t)(kmax & 0x7fffu) : (uint16_t)~kmax;
        xmax = __bfloat162float(__ushort_as_bfloat16(b));
    }
    const float inv_t = 1.f / T;
    const int K = top_k[row];
    const float P = top_p[row];
    const float MP = min_p[row];
    const bool need_k = K > 0 && K < vocab;
    const bool need_p = P < 1.f;
    uint32_t thr_key = 0;  // keep entries whose key >= thr_key
    // min-p: keep p_i >= min_p * p_max  <=>  x_i >= xmax + T * ln(min_p)
    const float x_floor = (MP > 0.f) ? xmax + T * __logf(MP) : -INFINITY;
    // per-row stream keys from the 64-bit seed; per-element noise is one 32-bit mix of the index
    const unsigned long long seed = splitmix64(seeds[row]);
    const uint32_t s0 = (uint32_t)seed, s1 = (uint32_t)(seed >> 32);

    // Gumbel-max over the entries with key >= lo (and the min-p floor, and the mask); `salt`
    // separates the noise streams of different rounds. Returns (score key << 32 | ~index) or 0.
    auto gumbel_pass = [&](uint32_t lo, uint32_t salt) -> unsigned long long {
        unsigned long long pick = 0ull;
        scan_row(rv, [&](int v, const uint4& pk) {
            const uint16_t* e = reinterpret_cast<const uint16_t*>(&pk);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int idx = v * 8 + k;
                const uint32_t key = bf16_key(e[k]);
                if (key < lo) continue;
                const float x = __bfloat162float(__ushort_as_bfloat16(e[k]));
                if (x < x_floor) continue;
                if (!rv.allowed(idx)) continue;
                uint32_t hsh = ((uint32_t)idx + s0 + salt * 0x632BE5ABu) * 0x9E3779B1u ^ s1;
                hsh ^= hsh >> 16; hsh *= 0x85EBCA6Bu; hsh ^= hsh >> 13; hsh *= 0xC2B2AE35u; hsh ^= hsh >> 16;
                const float u = ((float)(hsh >> 8) + 0.5f) * (1.0f / 16777216.0f);
                const float score = (x - xmax) * inv_t - __logf(-__logf(u));
                const unsigned long long cand =
                    ((unsigned long long)f32_key(score) << 32) | (0xffffffffu - (uint32_t)idx);
                pick = cand > pick ? cand : pick;
            }
        });
        return block_max_u64(pick, red64);
    };

    if (need_k || need_p) {
        // Rejection rounds (no histogram, no atomics): draw a candidate from the distribution
        // restricted to keys >= lo, then measure how much probability mass / how many entries lie
        // strictly above its key. It belongs to the kept set iff that is below top-p * Z and below
        // top-k (ties at the threshold are kept, as in the radix select below). A rejected candidate
        // proves that every key <= its key is outside the kept set, so the next round draws above it.
        // With top-p = 0.9 a round accepts with probability >= 0.9; after three rejections, and for
        // top-k or a small top-p (where a round rarely accepts), the exact radix select takes over.
        uint32_t lo = 0;
        bool accepted = false;
        // rejection pays when a round is likely to accept: top-p alone with a large nucleus
        const int rounds = (need_p && !need_k && P >= 0.5f) ? 3 : 0;
        for (int round = 0; round < rounds && !accepted; ++round) {
            const unsigned long long pick = gumbel_pass(lo, (uint32_t)round);
            if (pick == 0ull) {                       // nothing left above lo: fall back to the arg-max
                if (threadIdx.x == 0) out_tokens[row] = arg;
                return;
            }
            const int cand = (int)(0xffffffffu - (uint32_t)(pick & 0xffffffffu));
            const uint16_t cb = reinterpret_cast<const uint16_t*>(rv.vec)[cand];
            const uint32_t ckey = bf16_key(cb);
            float z = 0.f, above = 0.f, n_above = 0.f;
            scan_row(rv, [&](int v, const uint4& pk) {
                const uint16_t* e = reinterpret_cast<const uint16_t*>(&pk);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int idx = v * 8 + k;
                    if (!rv.allowed(idx)) continue;
                    const uint32_t key = bf16_key(e[k]);
                    const float w = __expf((__bfloat162float(__ushort_as_bfloat16(e[k])) - xmax) * inv_t);
                    z += w;
                    if (key > ckey) { above += w; n_above += 1.f; }
                }
            });
            z = block_sum(z, redf);
            above = block_sum(above, redf);
            n_above = block_sum(n_above, redf);
            const bool ok_p = !need_p || above < P * z;
            const bool ok_k = !need_k || n_above < (float)K;
            if (ok_p && ok_k) {
                if (threadIdx.x == 0) out_tokens[row] = cand;
                return;
            }
            lo = ckey + 1u;
        }
    }
    if (need_k || need_p) {
        // ---- pass 2: histogram of the key's high byte (count and softmax mass)
        for (int i = threadIdx.x; i < SAMPLE_WARPS * 256; i += SAMPLE_THREADS) {
            h_cnt[i] = 0;
            h_mass[i] = 0.f;
        }
        __syncthreads();
        scan_row(rv, [&](int v, const uint4& pk) {
            const uint16_t* e = reinterpret_cast<const uint16_t*>(&pk);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int idx = v * 8 + k;
                if (!rv.allowed(idx)) continue;
                const uint32_t key = bf16_key(e[k]);
                const float x = __bfloat162float(__ushort_as_bfloat16(e[k]));
                atomicAdd(&h_cnt[wid * 256 + (key >> 8)], 1);
                atomicAdd(&h_mass[wid * 256 + (key >> 8)], __expf((x - xmax) * inv_t));
            }
        });
        __syncthreads();
        if (threadIdx.x < 256) {
            int c = 0;
            float m = 0.f;
            for (int w = 0; w < SAMPLE_WARPS; ++w) {
                c += h_cnt[w * 256 + threadIdx.x];
                m += h_mass[w * 256 + threadIdx.x];
            }
            s_cnt[threadIdx.x] = c;
            s_mass[threadIdx.x] = m;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            float Z = 0.f;
            for (int b = 0; b < 256; ++b) Z += s_mass[b];
            int binK = -1, cBefore = 0, binP = -1;
            float mBefore = 0.f;
            int c = 0;
            float m = 0.f;
            for (int b = 255; b >= 0; --b) {
                if (need_k && binK < 0 && c + s_cnt[b] >= K) { binK = b; cBefore = c; }
                if (need_p && binP < 0 && m + s_mass[b] >= P * Z) { binP = b; mBefore = m; }
                c += s_cnt[b];
                m += s_mass[b];
            }
            s_sel[0] = binK; s_sel[1] = cBefore; s_sel[2] = binP;
            s_self[0] = mBefore; s_self[1] = Z;
        }
        __syncthreads();
        const int binK = s_sel[0], cBefore = s_sel[1], binP = s_sel[2];
        const float mBefore = s_self[0], Z = s_self[1];
        // ---- pass 3: histogram of the low byte inside the selected bins
        if (binK >= 0 || binP >= 0) {
            for (int i = threadIdx.x; i < SAMPLE_WARPS * 256; i += SAMPLE_THREADS) {
                h_cnt[i] = 0;
                h_mass[i] = 0.f;
            }
            __syncthreads();
            scan_row(rv, [&](int v, const uint4& pk) {
                const uint16_t* e = reinterpret_cast<const uint16_t*>(&pk);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int idx = v * 8 + k;
                    const uint32_t key = bf16_key(e[k]);
                    const int hi = (int)(key >> 8);
                    if (hi != binK && hi != binP) continue;
                    if (!rv.allowed(idx)) continue;
                    if (hi == binK) atomicAdd(&h_cnt[wid * 256 + (key & 255u)], 1);
                    if (hi == binP) {
                        const float x = __bfloat162float(__ushort_as_bfloat16(e[k]));
                        atomicAdd(&h_mass[wid * 256 + (key & 255u)], __expf((x - xmax) * inv_t));
                    }
                }
            });
            __syncthreads();
            if (threadIdx.x < 256) {
                int c = 0;
                float m = 0.f;
                for (int w = 0; w < SAMPLE_WARPS; ++w) {
                    c += h_cnt[w * 256 + threadIdx.x];
                    m += h_mass[w * 256 + threadIdx.x];
                }
                s_cnt[threadIdx.x] = c;
                s_mass[threadIdx.x] = m;
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                int keyK = 0, keyP = 0;
                if (binK >= 0) {
                    int c = cBefore, lo = 0;
                    for (int b = 255; b >= 0; --b) {
                        c += s_cnt[b];
                        if (c >= K) { lo = b; break; }
                    }
                    keyK = (binK << 8) | lo;
                }
                if (binP >= 0) {
                    float m = mBefore;
                    int lo = 0;
                    for (int b = 255; b >= 0; --b) {
                        m += s_mass[b];
                        if (m >= P * Z) { lo = b; break; }
                    }
                    keyP = (binP << 8) | lo;
                }
                s_sel[3] = max(keyK, keyP);
            }
            __syncthreads();
            thr_key = (uint32_t)s_sel[3];
        }
    }
    // ---- final pass: Gumbel-max over the kept set
    const unsigned long long pick = gumbel_pass(thr_key, 7u);
    if (threadIdx.x == 0)
        out_tokens[row] = pick ? (int)(0xffffffffu - (uint32_t)(pick & 0xffffffffu)) : arg;
}

// Per-row max, log-sum-exp and Shannon entropy of the unscaled distribution.
// stats[row] = {max, lse, entropy}.
__global__ void __launch_bounds__(SAMPLE_THREADS)
row_stats_kernel(const bf16* __restrict__ logits, long row_stride, int vocab,
                 float* __restrict__ stats) {
    __shared__ float red[32];
    const int row = blockIdx.x;
    const uint4* vec = reinterpret_cast<const uint4*>(logits + (size_t)row * row_stride);
    const int nvec = vocab >> 3;
    float mx = -INFINITY;
    for (int v = threadIdx.x; v < nvec; v += SAMPLE_THREADS) {
        const uint4 pk = vec[v];
        float f[8];
        unpack8(*reinterpret_cast<const bf16x8*>(&pk), f);
#pragma unroll
        for (int k = 0; k < 8; ++k) mx = fmaxf(mx, f[k]);
    }
    mx = block_max(mx, red);
    float z = 0.f, a = 0.f;  // z = sum e^(x-m), a = sum (x-m) e^(x-m)
    for (int v = threadIdx.x; v < nvec; v += SAMPLE_THREADS) {
        const uint4 pk = vec[v];
        float f[8];
        unpack8(*reinterpret_cast<const bf16x8*>(&pk), f);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float d = f[k] - mx;
            const float e = __expf(d);
            z += e;
            a += d * e;
        }
    }
    z = block_sum(z, red);
    a = block_sum(a, red);
    if (threadIdx.x == 0) {
        const float lz = logf(z);
        stats[row * 3 + 0] = mx;
        stats[row * 3 + 1] = mx + lz;
        stats[row * 3 + 2] = lz - a / z;  // H = log Z - E[x - m]
    }
}

}  // namespace pie

using namespace pie;

PIE_API int pie_sample(const void* logits, long row_stride, int rows, int vocab,
                       const float* temperature, const int* top_k, const float* top_p,
                       const float* min_p, const unsigned long long* seeds,
                       const uint32_t* mask_bits, const int* mask_row, int mask_words,
                       int* out_tokens, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (vocab % 8 || row_stride % 8) return (int)cudaErrorInvalidValue;
    const int smem = SAMPLE_WARPS * 256 * 8;
    cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    sample_kernel<<<rows, SAMPLE_THREADS, smem, st>>>((const bf16*)logits, row_stride, vocab,
                                                      temperature, top_k, top_p, min_p, seeds,
                                                      mask_bits, mask_row, mask_words, out_tokens);
    return (int)cudaGetLastError();
}

PIE_API int pie_row_stats(const void* logits, long row_stride, int rows, int vocab, float* stats,
                          cudaStream_t st) {
    if (rows <= 0) return 0;
    if (vocab % 8 || row_stride % 8) return (int)cudaErrorInvalidValue;
    row_stats_kernel<<<rows, SAMPLE_THREADS, 0, st>>>((const bf16*)logits, row_stride, vocab, stats);
    return (int)cudaGetLastError();
}
