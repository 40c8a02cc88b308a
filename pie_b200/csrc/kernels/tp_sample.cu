// Token sampling over a vocabulary-sharded lm_head (tensor parallelism): every rank holds the
// logits of its own vocabulary slice [rows, V / world] and all ranks arrive at the same token
// without ever gathering the logits. The algorithm is the one of sampling.cu (arg-max, Gumbel-max
// rejection rounds for top-p, two-level radix select for top-k / small top-p, final Gumbel-max
// over the kept set) with every block-wide reduction followed by a cross-rank combine: a few
// words per row travel through peer memory instead of rows * V logits (131 MB per 512-row step at
// V = 128 256). Noise and tie-breaks are functions of the GLOBAL vocabulary index, so the result
// equals the single-GPU sampler's on the concatenated logits.
//
// Exchange protocol (plain peer stores / loads over NVLink, no multimem): a CTA owns one row at a
// time and a mailbox [cta][parity][src rank] of 64-bit words on every rank. To exchange, it stores
// each of its 32-bit words, paired with the exchange's sequence number in the upper half, into its
// slot of every rank's mailbox, then polls (bounded) the slots of all source ranks in its own mailbox
// until every word carries the sequence number. An aligned 8-byte store is never torn, so a word
// that shows the sequence number also shows its data: no fence and no separate flag are needed.
// Slots alternate by the parity of the sequence number: a rank can run at most one exchange ahead of
// a peer, so the slot it overwrites has been read by everybody. All ranks launch the same grid and
// walk rows in the same order, so CTA c of every rank works on the same row. Every CTA of the grid
// is resident (the launcher bounds the grid by the occupancy), so no CTA waits for one that cannot run.
//
// Reference behaviour replaced: under tensor parallelism the reference vocabulary-shards lm_head
// only for greedy sampling (arg-max pairs + all-gather: driver/cuda/src/model/llama_like.cpp:764-813,
// driver/cuda/src/kernels/sample_temp.cu:185-340); for any other sampler rank 0 alone computes the
// full logits (driver/cuda/src/entry.cpp:961) while the other ranks idle.
#include "common.cuh"

namespace pie {

#ifndef TS_MIN_BLOCKS
#define TS_MIN_BLOCKS 4
#endif
#ifndef TS_UNROLL
#define TS_UNROLL 1
#endif
constexpr int TS_THREADS = 256;
constexpr int TS_WARPS = TS_THREADS / 32;
constexpr int TS_MAX_RANKS = 8;
constexpr int TS_SLOT_WORDS = 528;      // 512 histogram words + header room, 16-byte multiple

struct TpSampleRank {
    const bf16* logits;     // this rank's [rows, vocab_local] slice
    int* out_tokens;        // [rows]
    int* seq;               // [grid_max] exchange counters of this rank's CTAs (persist across launches)
};

struct TpSampleArgs {
    unsigned long long* peer_xbuf[TS_MAX_RANKS];   // mailbox of rank i: [grid_max][2][world][TS_SLOT_WORDS]
    TpSampleRank r[TS_MAX_RANKS];        // real launch: r[0] is this rank; emulation: one entry per rank
    int* status;
    int world, rank_base, vocab_local, grid_max;
    long long wait_cycles;
};

__device__ __forceinline__ uint32_t ts_bf16_key(uint16_t bits) {
    return (bits & 0x8000u) ? (uint32_t)(uint16_t)~bits : (uint32_t)(bits | 0x8000u);
}
__device__ __forceinline__ uint32_t ts_f32_key(float f) {
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ unsigned long long ts_warp_max_u64(unsigned long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long x = __shfl_xor_sync(0xffffffffu, v, o);
        v = x > v ? x : v;
    }
    return v;
}
__device__ __forceinline__ unsigned long long ts_block_max_u64(unsigned long long v, unsigned long long* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    v = ts_warp_max_u64(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    unsigned long long t = lane < TS_WARPS ? red[lane] : 0ull;
    return ts_warp_max_u64(t);
}

// One CTA's view of the exchange machinery.
struct TsLink {
    const TpSampleArgs* a;
    int rank;              // this CTA's rank
    int cta;               // mailbox index
    int seq;               // exchanges done so far (same in every thread)
    uint32_t* gathered;    // shared memory [world][TS_SLOT_WORDS]
    int* s_fail;           // shared flag
};

// Sends `nw` words (shared memory) to every rank and gathers every rank's words into
// link.gathered[src * TS_SLOT_WORDS + w]. Returns false when a wait ran out.
__device__ __forceinline__ bool ts_exchange(TsLink& L, const uint32_t* mine, int nw) {
    const TpSampleArgs& a = *L.a;
    const int world = a.world;
    L.seq += 1;
    const uint32_t seq = (uint32_t)L.seq;
    const size_t slot0 = ((size_t)L.cta * 2 + (seq & 1u)) * world;       // slot index of source rank 0
    for (int i = threadIdx.x; i < world * nw; i += TS_THREADS) {
        const int p = i / nw, w = i - p * nw;
        volatile unsigned long long* dst = a.peer_xbuf[p] + (slot0 + L.rank) * TS_SLOT_WORDS + w;
        *dst = ((unsigned long long)seq << 32) | mine[w];
    }
    const volatile unsigned long long* box = a.peer_xbuf[L.rank] + slot0 * TS_SLOT_WORDS;
    const long long t0 = clock64();
    for (int i = threadIdx.x; i < world * nw; i += TS_THREADS) {
        const int p = i / nw, w = i - p * nw;
        const volatile unsigned long long* src = box + (size_t)p * TS_SLOT_WORDS + w;
        unsigned long long v = *src;
        while ((uint32_t)(v >> 32) != seq) {
            if (*reinterpret_cast<volatile int*>(a.status) != 0 || clock64() - t0 > a.wait_cycles) {
                atomicCAS(a.status, 0, PIE_ERR_WAIT_PEER);
                *L.s_fail = 1;
                break;
            }
            v = *src;
        }
        L.gathered[p * TS_SLOT_WORDS + w] = (uint32_t)v;
    }
    __syncthreads();
    return *L.s_fail == 0;
}

struct TsRow {
    const uint4* vec;
    const uint32_t* mask;   // bitmask over the GLOBAL vocabulary or null
    int nvec, vocab_start;
    __device__ __forceinline__ bool allowed(int gidx) const {
        return !mask || ((mask[gidx >> 5] >> (gidx & 31)) & 1u);
    }
};

template <typename F>
__device__ __forceinline__ void ts_scan(const TsRow& rv, F&& f) {
    constexpr int U = TS_UNROLL;
    for (int v0 = threadIdx.x; v0 < rv.nvec; v0 += TS_THREADS * U) {
        uint4 pk[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int v = v0 + u * TS_THREADS;
            if (v < rv.nvec) pk[u] = rv.vec[v];
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int v = v0 + u * TS_THREADS;
            if (v < rv.nvec) f(v, pk[u]);
        }
    }
}

// four resident CTAs per SM: 592 mailboxes on a 148-SM part, one row per CTA for up to 592 rows
__global__ void __launch_bounds__(TS_THREADS, TS_MIN_BLOCKS)
tp_sample_kernel(const __grid_constant__ TpSampleArgs a, long row_stride, int rows,
                 const float* __restrict__ temperature, const int* __restrict__ top_k,
                 const float* __restrict__ top_p, const float* __restrict__ min_p,
                 const unsigned long long* __restrict__ seeds, const uint32_t* __restrict__ mask_bits,
                 const int* __restrict__ mask_row, int mask_words) {
    __shared__ __align__(16) uint32_t s_mine[TS_SLOT_WORDS];
    __shared__ __align__(16) uint32_t s_gath[TS_MAX_RANKS * TS_SLOT_WORDS];
    __shared__ int h_cnt[TS_WARPS * 256];
    __shared__ float h_mass[TS_WARPS * 256];
    __shared__ unsigned long long red64[32];
    __shared__ float redf[32];
    __shared__ int s_cnt[256];
    __shared__ float s_mass[256];
    __shared__ int s_sel[6];
    __shared__ float s_self[4];
    __shared__ int s_fail;

    const int slot = blockIdx.y;
    const TpSampleRank R = a.r[slot];
    const int wid = threadIdx.x >> 5;
    const int world = a.world;
    if (threadIdx.x == 0) s_fail = 0;
    __syncthreads();
    TsLink L{&a, a.rank_base + slot, (int)blockIdx.x, R.seq[blockIdx.x], s_gath, &s_fail};
    const int vocab_start = L.rank * a.vocab_local;
    const int vocab_total = world * a.vocab_local;

    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        TsRow rv;
        rv.vec = reinterpret_cast<const uint4*>(R.logits + (size_t)row * row_stride);
        rv.nvec = a.vocab_local >> 3;
        rv.vocab_start = vocab_start;
        const int mr = mask_row ? mask_row[row] : -1;
        rv.mask = (mask_bits && mr >= 0) ? mask_bits + (size_t)mr * mask_words : nullptr;
        const uint16_t* row16 = reinterpret_cast<const uint16_t*>(rv.vec);

        // ---- pass 1: arg-max over the allowed entries of all shards
        unsigned long long best = 0ull;
        ts_scan(rv, [&](int v, const uint4& pk) {
            const uint16_t* e = reinterpret_cast<const uint16_t*>(&pk);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const int gidx = vocab_start + v * 8 + k;
                if (!rv.allowed(gidx)) continue;
                const unsigned long long cand =
                    ((unsigned long long)(ts_bf16_key(e[k]) + 1u) << 32) | (0xffffffffu - (uint32_t)gidx);
                best = cand > best ? cand : best;
            }
        });
        best = ts_block_max_u64(best, red64);
        if (threadIdx.x == 0) {
            s_mine[0] = (uint32_t)best; s_mine[1] = (uint32_t)(best >> 32); s_mine[2] = 0; s_mine[3] = 0;
        }
        __syncthreads();
        if (!ts_exchange(L, s_mine, 4)) break;
        best = 0ull;
        for (int p = 0; p < world; ++p) {
            const unsigned long long c = ((unsigned long long)s_gath[p * TS_SLOT_WORDS + 1] << 32) | s_gath[p * TS_SLOT_WORDS];
            best = c > best ? c : best;
        }
        const float T = temperature[row];
        if (best == 0ull) {  // nothing allowed: emit token 0
            if (threadIdx.x == 0) R.out_tokens[row] = 0;
            continue;
        }
        const int arg = (int)(0xffffffffu - (uint32_t)(best & 0xffffffffu));
        if (T <= 0.f) {
            if (threadIdx.x == 0) R.out_tokens[row] = arg;
            continue;
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
        const bool need_k = K > 0 && K < vocab_total;
        const bool need_p = P < 1.f;
        uint32_t thr_key = 0;
        const float x_floor = (MP > 0.f) ? xmax + T * __logf(MP) : -INFINITY;
        const unsigned long long seed = splitmix64(seeds[row]);
        const uint32_t s0 = (uint32_t)seed, s1 = (uint32_t)(seed >> 32);

        // Gumbel-max over the entries of all shards with key >= lo; returns false on a failed wait.
        // pick = (score key << 32 | ~global index) or 0; ckey = bf16 key of the picked entry.
        auto gumbel_pick = [&](uint32_t lo, uint32_t salt, unsigned long long& pick, uint32_t& ckey) -> bool {
            unsigned long long mine = 0ull;
            ts_scan(rv, [&](int v, const uint4& pk) {
                const uint16_t* e = reinterpret_cast<const uint16_t*>(&pk);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int gidx = vocab_start + v * 8 + k;
                    const uint32_t key = ts_bf16_key(e[k]);
                    if (key < lo) continue;
                    const float x = __bfloat162float(__ushort_as_bfloat16(e[k]));
                    if (x < x_floor) continue;
                    if (!rv.allowed(gidx)) continue;
                    uint32_t hsh = ((uint32_t)gidx + s0 + salt * 0x632BE5ABu) * 0x9E3779B1u ^ s1;
                    hsh ^= hsh >> 16; hsh *= 0x85EBCA6Bu; hsh ^= hsh >> 13; hsh *= 0xC2B2AE35u; hsh ^= hsh >> 16;
                    const float u = ((float)(hsh >> 8) + 0.5f) * (1.0f / 16777216.0f);
                    const float score = (x - xmax) * inv_t - __logf(-__logf(u));
                    const unsigned long long cand =
                        ((unsigned long long)ts_f32_key(score) << 32) | (0xffffffffu - (uint32_t)gidx);
                    mine = cand > mine ? cand : mine;
                }
            });
            mine = ts_block_max_u64(mine, red64);
            if (threadIdx.x == 0) {
                uint32_t k = 0;
                if (mine) k = ts_bf16_key(row16[(int)(0xffffffffu - (uint32_t)(mine & 0xffffffffu)) - vocab_start]);
                s_mine[0] = (uint32_t)mine; s_mine[1] = (uint32_t)(mine >> 32); s_mine[2] = k; s_mine[3] = 0;
            }
            __syncthreads();
            if (!ts_exchange(L, s_mine, 4)) return false;
            pick = 0ull;
            ckey = 0;
            for (int p = 0; p < world; ++p) {
                const uint32_t* g = s_gath + p * TS_SLOT_WORDS;
                const unsigned long long c = ((unsigned long long)g[1] << 32) | g[0];
                if (c > pick) { pick = c; ckey = g[2]; }
            }
            return true;
        };

        bool failed = false, done = false;
        if (need_k || need_p) {
            uint32_t lo = 0;
            const int rounds = (need_p && !need_k && P >= 0.5f) ? 3 : 0;
            for (int round = 0; round < rounds && !done; ++round) {
                unsigned long long pick;
                uint32_t ckey;
                if (!gumbel_pick(lo, (uint32_t)round, pick, ckey)) { failed = true; break; }
                if (pick == 0ull) {
                    if (threadIdx.x == 0) R.out_tokens[row] = arg;
                    done = true;
                    break;
                }
                const int cand = (int)(0xffffffffu - (uint32_t)(pick & 0xffffffffu));
                float z = 0.f, above = 0.f, n_above = 0.f;
                ts_scan(rv, [&](int v, const uint4& pk) {
                    const uint16_t* e = reinterpret_cast<const uint16_t*>(&pk);
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const int gidx = vocab_start + v * 8 + k;
                        if (!rv.allowed(gidx)) continue;
                        const uint32_t key = ts_bf16_key(e[k]);
                        const float w = __expf((__bfloat162float(__ushort_as_bfloat16(e[k])) - xmax) * inv_t);
                        z += w;
                        if (key > ckey) { above += w; n_above += 1.f; }
                    }
                });
                z = block_sum(z, redf);
                above = block_sum(above, redf);
                n_above = block_sum(n_above, redf);
                if (threadIdx.x == 0) {
                    s_mine[0] = __float_as_uint(z); s_mine[1] = __float_as_uint(above);
                    s_mine[2] = __float_as_uint(n_above); s_mine[3] = 0;
                }
                __syncthreads();
                if (!ts_exchange(L, s_mine, 4)) { failed = true; break; }
                z = above = n_above = 0.f;
                for (int p = 0; p < world; ++p) {
                    z += __uint_as_float(s_gath[p * TS_SLOT_WORDS]);
                    above += __uint_as_float(s_gath[p * TS_SLOT_WORDS + 1]);
                    n_above += __uint_as_float(s_gath[p * TS_SLOT_WORDS + 2]);
                }
                const bool ok_p = !need_p || above < P * z;
                const bool ok_k = !need_k || n_above < (float)K;
                if (ok_p && ok_k) {
                    if (threadIdx.x == 0) R.out_tokens[row] = cand;
                    done = true;
                    break;
                }
                lo = ckey + 1u;
            }
        }
        if (failed) break;
        if (done) continue;

        if (need_k || need_p) {
            // ---- exact radix select on the 16-bit order key, histograms summed over the ranks
            int binK = -1, cBefore = 0, binP = -1;
            float mBefore = 0.f, Z = 0.f;
            for (int level = 0; level < 2; ++level) {
                if (level == 1 && binK < 0 && binP < 0) break;
                for (int i = threadIdx.x; i < TS_WARPS * 256; i += TS_THREADS) {
                    h_cnt[i] = 0;
                    h_mass[i] = 0.f;
                }
                __syncthreads();
                ts_scan(rv, [&](int v, const uint4& pk) {
                    const uint16_t* e = reinterpret_cast<const uint16_t*>(&pk);
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const int gidx = vocab_start + v * 8 + k;
                        const uint32_t key = ts_bf16_key(e[k]);
                        const int hi = (int)(key >> 8);
                        if (level == 1 && hi != binK && hi != binP) continue;
                        if (!rv.allowed(gidx)) continue;
                        const float w = __expf((__bfloat162float(__ushort_as_bfloat16(e[k])) - xmax) * inv_t);
                        if (level == 0) {
                            atomicAdd(&h_cnt[wid * 256 + hi], 1);
                            atomicAdd(&h_mass[wid * 256 + hi], w);
                        } else {
                            if (hi == binK) atomicAdd(&h_cnt[wid * 256 + (key & 255u)], 1);
                            if (hi == binP) atomicAdd(&h_mass[wid * 256 + (key & 255u)], w);
                        }
                    }
                });
                __syncthreads();
                {
                    int c = 0;
                    float m = 0.f;
                    for (int w = 0; w < TS_WARPS; ++w) {
                        c += h_cnt[w * 256 + threadIdx.x];
                        m += h_mass[w * 256 + threadIdx.x];
                    }
                    s_mine[threadIdx.x] = (uint32_t)c;
                    s_mine[256 + threadIdx.x] = __float_as_uint(m);
                }
                __syncthreads();
                if (!ts_exchange(L, s_mine, 512)) { failed = true; break; }
                {
                    int c = 0;
                    float m = 0.f;
                    for (int p = 0; p < world; ++p) {
                        c += (int)s_gath[p * TS_SLOT_WORDS + threadIdx.x];
                        m += __uint_as_float(s_gath[p * TS_SLOT_WORDS + 256 + threadIdx.x]);
                    }
                    s_cnt[threadIdx.x] = c;
                    s_mass[threadIdx.x] = m;
                }
                __syncthreads();
                if (threadIdx.x == 0) {
                    if (level == 0) {
                        float z = 0.f;
                        for (int b = 0; b < 256; ++b) z += s_mass[b];
                        int bk = -1, cb = 0, bp = -1;
                        float mb = 0.f;
                        int c = 0;
                        float m = 0.f;
                        for (int b = 255; b >= 0; --b) {
                            if (need_k && bk < 0 && c + s_cnt[b] >= K) { bk = b; cb = c; }
                            if (need_p && bp < 0 && m + s_mass[b] >= P * z) { bp = b; mb = m; }
                            c += s_cnt[b];
                            m += s_mass[b];
                        }
                        s_sel[0] = bk; s_sel[1] = cb; s_sel[2] = bp;
                        s_self[0] = mb; s_self[1] = z;
                    } else {
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
                }
                __syncthreads();
                if (level == 0) {
                    binK = s_sel[0]; cBefore = s_sel[1]; binP = s_sel[2];
                    mBefore = s_self[0]; Z = s_self[1];
                } else {
                    thr_key = (uint32_t)s_sel[3];
                }
            }
            if (failed) break;
        }
        // ---- final pass: Gumbel-max over the kept set
        unsigned long long pick;
        uint32_t ckey;
        if (!gumbel_pick(thr_key, 7u, pick, ckey)) break;
        if (threadIdx.x == 0)
            R.out_tokens[row] = pick ? (int)(0xffffffffu - (uint32_t)(pick & 0xffffffffu)) : arg;
    }
    __syncthreads();
    if (threadIdx.x == 0) R.seq[blockIdx.x] = L.seq;
}

}  // namespace pie

using namespace pie;

PIE_API int pie_tp_sample_args_size() { return (int)sizeof(TpSampleArgs); }
PIE_API int pie_tp_sample_slot_words() { return TS_SLOT_WORDS; }

// Bytes of mailbox every rank must provide (zero-initialised, 8-byte aligned) for `grid_max` CTAs.
PIE_API long pie_tp_sample_mailbox_bytes(int grid_max, int world) {
    return (long)grid_max * 2 * world * TS_SLOT_WORDS * 8;
}

// Largest grid whose CTAs are all resident on a device with `num_sms` SMs.
PIE_API int pie_tp_sample_max_grid(int num_sms) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, tp_sample_kernel, TS_THREADS, 0) != cudaSuccess)
        return 0;
    return per_sm * num_sms;
}

// peer_xbuf[i]: rank i's mailbox as mapped on THIS GPU. seq: this rank's [grid_max] int32 counters
// (zero-initialised once, then owned by the kernel).
PIE_API int pie_tp_sample_fill_args(void* blob, void* const* peer_xbuf, int* seq,
                                    int* status, int world, int rank, int vocab_local, int grid_max,
                                    long long wait_cycles) {
    if (world < 1 || world > TS_MAX_RANKS || rank < 0 || rank >= world || vocab_local % 8 || grid_max < 1)
        return (int)cudaErrorInvalidValue;
    TpSampleArgs a{};
    for (int i = 0; i < world; ++i) a.peer_xbuf[i] = (unsigned long long*)peer_xbuf[i];
    a.r[0].seq = seq;
    a.status = status; a.world = world; a.rank_base = rank; a.vocab_local = vocab_local; a.grid_max = grid_max;
    a.wait_cycles = wait_cycles > 0 ? wait_cycles : 1500000000ll;
    *reinterpret_cast<TpSampleArgs*>(blob) = a;
    return 0;
}

// Sample one token per row from logits sharded over the ranks' vocabulary slices. Every rank calls
// it with the same rows / sampler parameters / seeds / masks and gets the same tokens.
PIE_API int pie_tp_sample(const void* blob, const void* logits, long row_stride, int rows,
                          const float* temperature, const int* top_k, const float* top_p, const float* min_p,
                          const unsigned long long* seeds, const uint32_t* mask_bits, const int* mask_row,
                          int mask_words, int* out_tokens, int num_sms, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (row_stride % 8) return (int)cudaErrorInvalidValue;
    TpSampleArgs a = *reinterpret_cast<const TpSampleArgs*>(blob);
    a.r[0].logits = (const bf16*)logits;
    a.r[0].out_tokens = out_tokens;
    int grid = pie_tp_sample_max_grid(num_sms);
    if (grid <= 0) return (int)cudaErrorLaunchOutOfResources;
    if (grid > a.grid_max) grid = a.grid_max;
    if (grid > rows) grid = rows;
    tp_sample_kernel<<<dim3(grid, 1), TS_THREADS, 0, st>>>(a, row_stride, rows, temperature, top_k, top_p, min_p,
                                                           seeds, mask_bits, mask_row, mask_words);
    return (int)cudaGetLastError();
}

// All `world` ranks in ONE cooperative launch on one GPU (blockIdx.y = rank): the multi-rank path
// on a machine with fewer GPUs than ranks. xbuf / seq: [world] local buffers sized as above.
PIE_API int pie_tp_sample_emulated(void* const* xbuf, int* const* seq, int* status,
                                   int world, int vocab_local, int grid_max, long long wait_cycles,
                                   const void* const* logits, long row_stride, int rows,
                                   const float* temperature, const int* top_k, const float* top_p,
                                   const float* min_p, const unsigned long long* seeds,
                                   const uint32_t* mask_bits, const int* mask_row, int mask_words,
                                   int* const* out_tokens, int num_sms, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (world < 1 || world > TS_MAX_RANKS || vocab_local % 8 || row_stride % 8) return (int)cudaErrorInvalidValue;
    TpSampleArgs a{};
    for (int i = 0; i < world; ++i) {
        a.peer_xbuf[i] = (unsigned long long*)xbuf[i];
        a.r[i].logits = (const bf16*)logits[i];
        a.r[i].out_tokens = out_tokens[i];
        a.r[i].seq = seq[i];
    }
    a.status = status; a.world = world; a.rank_base = 0; a.vocab_local = vocab_local; a.grid_max = grid_max;
    a.wait_cycles = wait_cycles > 0 ? wait_cycles : 1500000000ll;
    int grid = pie_tp_sample_max_grid(num_sms) / world;
    if (grid > grid_max) grid = grid_max;
    if (grid > rows) grid = rows;
    if (grid <= 0) return (int)cudaErrorLaunchOutOfResources;
    void* params[] = {(void*)&a, (void*)&row_stride, (void*)&rows, (void*)&temperature, (void*)&top_k, (void*)&top_p,
                      (void*)&min_p, (void*)&seeds, (void*)&mask_bits, (void*)&mask_row, (void*)&mask_words};
    return (int)cudaLaunchCooperativeKernel((const void*)tp_sample_kernel, dim3(grid, world), dim3(TS_THREADS),
                                            params, 0, st);
}
