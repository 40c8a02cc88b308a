// Definitions shared by the single-CTA and CTA-pair tcgen05 GEMM kernels: epilogue modes, the
// tensor-parallel side channel, stream-K work walking and the epilogue store.
#pragma once
#include "tcgen05.cuh"

namespace pie {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;

enum GemmEpilogue : int {
    EPI_STORE = 0,     // C = acc
    EPI_RESIDUAL = 1,  // C = acc + R
    EPI_SWIGLU = 2,    // C[:, j] = silu(acc[:, 2j]) * acc[:, 2j+1]   (C is [M, N/2])
    EPI_RS = 3,        // reduce-scatter: rows go to their owner rank's receive buffer (peer stores)
    // Swapped operands (small batches): the kernel computes C^T = W * A^T, so its rows are output
    // features and its columns tokens; these epilogues write the tile back transposed.
    EPI_STORE_T = 4,
    EPI_RESIDUAL_T = 5,
    EPI_SWIGLU_T = 6,
};

constexpr int TP_MAX_RANKS = 8;

// Tensor-parallel side channel of the fused kernels. All pointers are device addresses valid
// on THIS GPU; peer_* entries are peer-mapped (NVLink) addresses of the same buffer on rank i.
//   gated loads : before the TMA load of an activation tile the producer waits until the ranks that
//                 own the tile's rows have pushed them (ag_flags[src] >= *ag_epoch, written by peers);
//                 with rows_per_rank == 0 (an activation that is not the gathered buffer) every rank.
//   EPI_RS      : the epilogue stores each accumulator row into the receive buffer of the rank
//                 that owns the row (rows_per_rank consecutive rows per rank, a multiple of 32),
//                 at [this rank][row within owner][col]; the last epilogue warp of the grid
//                 bumps the local epoch and writes it into every owner's flag word for this rank.
struct TpArgs {
    const int* ag_flags;          // [world] local, written by peers
    const int* ag_epoch;          // local expected value
    bf16* peer_recv[TP_MAX_RANKS];
    int* peer_rs_flags[TP_MAX_RANKS];  // word [rank] of rank i's flag array is at peer_rs_flags[i] + rank
    int* rs_done;                 // local arrival counter of the epilogue warps
    int* rs_epoch;                // local count of reduce-scatter ops issued
    int world, rank, rows_per_rank, gated;
};

// Stream-K side of the kernel. With `enabled`, the (tile, k-block) units of the whole problem are
// split evenly over the CTAs instead of whole tiles, so skinny problems (few tiles, long K) keep
// every SM busy. A CTA whose share covers only part of a tile's K range writes its fp32 partial
// tile to `ws` and bumps the tile's arrival counter; the last warp to arrive for a 32-row quarter
// adds the other partials and runs the real epilogue. Nobody waits for anybody.
//   ws  : [(grid + num_tiles)][128][BN] floats, slot = cta + tile
//   cnt : [num_tiles][4] ints, zero before the launch; the last arriver resets its counter
struct StreamKArgs {
    float* ws;
    int* cnt;
    int enabled;
    // Diagnostics, compiled in only with -DPIE_GEMM_DIAG (a production build ignores both fields):
    int dbg;   // 1 skip the MMAs, 2 skip the loads, 4 relay instead of direct signalling (results are meaningless)
    unsigned long long* trace;   // [grid][8] globaltimer stamps of the kernel's phases
};

#ifdef PIE_GEMM_DIAG
#define PIE_DIAG(expr) (expr)
__device__ __forceinline__ void trace_stamp(unsigned long long* trace, int slot) {
    if (trace) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        trace[blockIdx.x * 8 + slot] = t;
    }
}
#else
#define PIE_DIAG(expr) 0
__device__ __forceinline__ void trace_stamp(unsigned long long*, int) {}
#endif

struct Segment {
    int tile, kb0, kb1;
};

// Walks the work of one CTA; every role of the CTA walks the same sequence.
struct SegmentWalk {
    long long u, u_end;
    int t, t_step, num_tiles, num_kb;
    bool sk;
    // worker = CTA (or CTA pair) index, workers = how many share the problem
    __device__ SegmentWalk(bool streamk, int num_tiles_, int num_kb_, int worker, int workers)
        : num_tiles(num_tiles_), num_kb(num_kb_), sk(streamk) {
        if (sk) {
            const long long total = (long long)num_tiles * num_kb;
            u = total * worker / workers;
            u_end = total * (worker + 1) / workers;
        } else {
            t = worker;
            t_step = workers;
        }
    }
    __device__ bool next(Segment& s) {
        if (sk) {
            if (u >= u_end) return false;
            s.tile = (int)(u / num_kb);
            s.kb0 = (int)(u - (long long)s.tile * num_kb);
            const long long left = u_end - u;
            s.kb1 = (int)min((long long)num_kb, s.kb0 + left);
            u += s.kb1 - s.kb0;
            return true;
        }
        if (t >= num_tiles) return false;
        s.tile = t;
        s.kb0 = 0;
        s.kb1 = num_kb;
        t += t_step;
        return true;
    }
};

// CTA whose unit range contains unit `unit` (ranges are [c*total/grid, (c+1)*total/grid)).
__device__ __forceinline__ int streamk_cta_of(long long unit, long long total, int grid) {
    return (int)(((unit + 1) * grid + total - 1) / total - 1);
}


// Final epilogue of 32 accumulator columns [col0, col0+32) of one output row held by a thread.
template <int EPI>
__device__ __forceinline__ void epilogue_store_chunk(const uint32_t (&v)[32], int row, int col0, int M, int N,
                                                     bf16* __restrict__ C, int ldc, const bf16* __restrict__ R,
                                                     int ldr, const TpArgs& tp) {
    if (row >= M || col0 >= N) return;
    if (EPI == EPI_RS) {
        const int owner = row / tp.rows_per_rank;
        const int local = row - owner * tp.rows_per_rank;
        bf16* dst = tp.peer_recv[owner] + ((size_t)tp.rank * tp.rows_per_rank + local) * (size_t)N + col0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (col0 + 8 * j >= N) break;
            float o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(v[8 * j + e]);
            *reinterpret_cast<bf16x8*>(dst + 8 * j) = pack8(o);
        }
    } else if (EPI == EPI_SWIGLU) {
        bf16* dst = C + (size_t)row * ldc + (col0 >> 1);
        float o[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float g = __uint_as_float(v[2 * j]);
            const float u = __uint_as_float(v[2 * j + 1]);
            o[j] = g / (1.f + __expf(-g)) * u;
        }
#pragma unroll
        for (int j = 0; j < 2; ++j)
            if (col0 + 16 * j < N) *reinterpret_cast<bf16x8*>(dst + 8 * j) = pack8(o + 8 * j);
    } else {
        bf16* dst = C + (size_t)row * ldc + col0;
        const bf16* res = (EPI == EPI_RESIDUAL) ? R + (size_t)row * ldr + col0 : nullptr;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (col0 + 8 * j >= N) break;
            float o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(v[8 * j + e]);
            if (EPI == EPI_RESIDUAL) {
                float rr[8];
                unpack8(*reinterpret_cast<const bf16x8*>(res + 8 * j), rr);
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] += rr[e];
            }
            *reinterpret_cast<bf16x8*>(dst + 8 * j) = pack8(o);
        }
    }
}

// Epilogue of 64 accumulator columns [col0, col0+64) for the 32 rows of one warp, with coalesced
// global accesses. Thread `lane` holds row (row0 + lane): v0 = columns col0..+31, v1 = +32..+63.
// The values go through a per-warp staging tile in shared memory (32 rows x 128 B, 16-byte
// chunks XOR-swizzled by row) so that one store instruction of the warp covers 4 rows x 128 B
// (8 rows x 64 B for SwiGLU) instead of 32 rows x 16 B.
//   stage : this warp's 4 KB staging tile (shared memory)
//   n_end : columns at or past n_end are not stored (end of this tile or of the matrix); N itself
//           stays the row pitch of the reduce-scatter receive buffers
template <int EPI>
__device__ __forceinline__ void epilogue_store_64(const uint32_t (&v0)[32], const uint32_t (&v1)[32],
                                                  uint8_t* stage, int row0, int col0, int M, int N,
                                                  bf16* __restrict__ C, int ldc, const bf16* __restrict__ R,
                                                  int ldr, const TpArgs& tp, int n_end) {
    const int lane = threadIdx.x & 31;
    auto slot = [&](int r, int c) { return reinterpret_cast<bf16x8*>(stage + r * 128 + ((c ^ (r & 7)) << 4)); };
    if (EPI == EPI_SWIGLU) {
        // 64 accumulator columns -> 32 outputs (64 B) per row
        float o[32];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const float g0 = __uint_as_float(v0[2 * j]), u0 = __uint_as_float(v0[2 * j + 1]);
            const float g1 = __uint_as_float(v1[2 * j]), u1 = __uint_as_float(v1[2 * j + 1]);
            o[j] = g0 / (1.f + __expf(-g0)) * u0;
            o[16 + j] = g1 / (1.f + __expf(-g1)) * u1;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) *slot(lane, c) = pack8(o + 8 * c);
        __syncwarp();
        const int oc0 = col0 >> 1;   // first output column
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = i * 8 + (lane >> 2), c = lane & 3;
            const int row = row0 + r, oc = oc0 + c * 8;
            if (row < M && 2 * oc < n_end) *reinterpret_cast<bf16x8*>(C + (size_t)row * ldc + oc) = *slot(r, c);
        }
        __syncwarp();
        return;
    }
    if (EPI == EPI_RESIDUAL) {
        // bring the residual tile in with coalesced loads, add in fp32 on the owning thread
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int r = i * 4 + (lane >> 3), c = lane & 7;
            const int row = row0 + r, col = col0 + c * 8;
            bf16x8 t;
#pragma unroll
            for (int e = 0; e < 4; ++e) t.v[e] = __floats2bfloat162_rn(0.f, 0.f);
            if (row < M && col < n_end) t = *reinterpret_cast<const bf16x8*>(R + (size_t)row * ldr + col);
            *slot(r, c) = t;
        }
        __syncwarp();
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(c < 4 ? v0[8 * c + e] : v1[8 * (c - 4) + e]);
        if (EPI == EPI_RESIDUAL) {
            float rr[8];
            unpack8(*slot(lane, c), rr);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] += rr[e];
        }
        *slot(lane, c) = pack8(o);
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = i * 4 + (lane >> 3), c = lane & 7;
        const int row = row0 + r, col = col0 + c * 8;
        if (row >= M || col >= n_end) continue;
        bf16* dst;
        if (EPI == EPI_RS) {
            const int owner = row / tp.rows_per_rank;
            const int local = row - owner * tp.rows_per_rank;
            dst = tp.peer_recv[owner] + ((size_t)tp.rank * tp.rows_per_rank + local) * (size_t)N + col;
        } else {
            dst = C + (size_t)row * ldc + col;
        }
        *reinterpret_cast<bf16x8*>(dst) = *slot(r, c);
    }
    __syncwarp();
}

// Transposed epilogue of the swapped-operand launch: thread `lane` holds output feature
// (feat0 + lane), v0 / v1 its values for tokens tok0..+31 / +32..+63. The output is C[token][feature].
// Values are staged as bf16 in the warp's 4 KB tile as [64 tokens][32 features] (64 B per token; for
// SwiGLU [64 tokens][16 outputs]) and leave in 16-byte stores, 8 (16) token rows per warp store.
//   F       : number of output features of the GEMM (rows of the swapped problem)
//   tok_end : tokens at or past tok_end are not stored
template <int EPI>
__device__ __forceinline__ void epilogue_store_64_t(const uint32_t (&v0)[32], const uint32_t (&v1)[32],
                                                    uint8_t* stage, int feat0, int tok0, int F, int tok_end,
                                                    bf16* __restrict__ C, int ldc, const bf16* __restrict__ R,
                                                    int ldr) {
    const int lane = threadIdx.x & 31;
    bf16* st = reinterpret_cast<bf16*>(stage);
    const int feat = feat0 + lane;
    if (EPI == EPI_SWIGLU_T) {
        // even lanes hold gate_j, odd lanes up_j of output j = feat / 2
#pragma unroll
        for (int t = 0; t < 64; ++t) {
            const float mine = __uint_as_float(t < 32 ? v0[t] : v1[t - 32]);
            const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
            if (!(lane & 1)) st[t * 16 + (lane >> 1)] = __float2bfloat16(mine / (1.f + __expf(-mine)) * other);
        }
        __syncwarp();
        const int oc0 = feat0 >> 1;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int t = i * 16 + (lane >> 1), c = lane & 1;
            const int tok = tok0 + t;
            if (tok < tok_end && 2 * (oc0 + c * 8) < F)
                *reinterpret_cast<bf16x8*>(C + (size_t)tok * ldc + oc0 + c * 8) = *reinterpret_cast<const bf16x8*>(st + t * 16 + c * 8);
        }
        __syncwarp();
        return;
    }
#pragma unroll
    for (int t = 0; t < 64; ++t) {
        float o = __uint_as_float(t < 32 ? v0[t] : v1[t - 32]);
        if (EPI == EPI_RESIDUAL_T) {
            const int tok = tok0 + t;
            if (tok < tok_end && feat < F) o += __bfloat162float(R[(size_t)tok * ldr + feat]);
        }
        st[t * 32 + lane] = __float2bfloat16(o);
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int t = i * 8 + (lane >> 2), c = lane & 3;
        const int tok = tok0 + t;
        if (tok < tok_end && feat0 + c * 8 < F)
            *reinterpret_cast<bf16x8*>(C + (size_t)tok * ldc + feat0 + c * 8) = *reinterpret_cast<const bf16x8*>(st + t * 32 + c * 8);
    }
    __syncwarp();
}

// Reduce-scatter publication: called by lane 0 of an epilogue warp after its rows of a tile
// reached their owners. The `total`-th arrival bumps the epoch and raises this rank's flag on
// every owner.
__device__ __forceinline__ void rs_publish_arrival(const TpArgs& tp, int total) {
    if (atomicAdd(tp.rs_done, 1) + 1 == total) {
        *tp.rs_done = 0;
        const int e = *reinterpret_cast<volatile int*>(tp.rs_epoch) + 1;
        *reinterpret_cast<volatile int*>(tp.rs_epoch) = e;
        __threadfence_system();
        for (int p = 0; p < tp.world; ++p) *reinterpret_cast<volatile int*>(tp.peer_rs_flags[p] + tp.rank) = e;
    }
}

// All-gather gate for the rows [row0, row0 + nrows) of the gathered activation: spin (bounded) until
// the ranks that own those rows (rows_per_rank consecutive rows each; every rank when rows_per_rank
// is 0) have pushed for this rank's epoch. `seen` is the caller's bit set of owners already confirmed,
// so a tile whose owners were seen costs nothing and rank p's rows are consumed as soon as p pushed.
__device__ __forceinline__ bool ag_gate_wait_rows(const TpArgs& tp, int* status, int row0, int nrows, uint32_t& seen) {
    int o0 = 0, o1 = tp.world - 1;
    if (tp.rows_per_rank > 0) {
        o0 = min(tp.world - 1, row0 / tp.rows_per_rank);
        o1 = min(tp.world - 1, (row0 + nrows - 1) / tp.rows_per_rank);
    }
    const uint32_t need = ((2u << o1) - 1u) & ~((1u << o0) - 1u);
    if ((need & ~seen) == 0u) return true;
    const int e = *reinterpret_cast<const volatile int*>(tp.ag_epoch);
    const long long t0 = clock64();
    const unsigned long long tg = blockIdx.x == 0 ? global_ns() : 0ull;
    for (int src = o0; src <= o1; ++src) {
        if (seen & (1u << src)) continue;
        while (*reinterpret_cast<const volatile int*>(tp.ag_flags + src) < e) {
            if (*reinterpret_cast<volatile int*>(status) != 0 || clock64() - t0 > 1500000000ll) {
                atomicCAS(status, 0, PIE_ERR_WAIT_PEER);
                return false;
            }
        }
    }
    if (blockIdx.x == 0) status_add_wait(status, 0, tg);
    seen |= need;
    __threadfence_system();
    asm volatile("fence.proxy.async;\n" ::: "memory");
    return true;
}

// All-gather gate: spin (bounded) until every rank's push flag reached this rank's epoch.
__device__ __forceinline__ bool ag_gate_wait(const TpArgs& tp, int* status) {
    const int e = *reinterpret_cast<const volatile int*>(tp.ag_epoch);
    const long long t0 = clock64();
    bool ok = true;
    for (int src = 0; src < tp.world && ok; ++src) {
        while (*reinterpret_cast<const volatile int*>(tp.ag_flags + src) < e) {
            if (*reinterpret_cast<volatile int*>(status) != 0 || clock64() - t0 > 1500000000ll) {
                atomicCAS(status, 0, PIE_ERR_WAIT_PEER);
                ok = false;
                break;
            }
        }
    }
    __threadfence_system();
    asm volatile("fence.proxy.async;\n" ::: "memory");
    return ok;
}

}  // namespace pie
