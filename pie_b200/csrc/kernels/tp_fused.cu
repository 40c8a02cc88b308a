// Tensor-parallel glue kernels over NVLink peer memory (plain peer loads/stores, no multimem):
//
//  tp_reduce_norm_push   the owner side of the fused GEMM -> reduce-scatter: waits for every
//                        rank's partial rows (flags written by the GEMM epilogues), sums them
//                        with the residual in fp32, stores the new residual, applies RMSNorm
//                        and PUSHES the normalised rows into every rank's full activation
//                        buffer (the all-gather half), then raises this rank's flag on every peer.
//  tp_wait_ag            gate for consumers of the gathered activation that are not the GEMM.
//  tp_allreduce_small    one-shot all-reduce of a small bf16 tensor: every rank stores its data into
//                        its slot on every peer, raises a flag, waits for the others' flags and sums
//                        the slots in rank order (replaces ncclAllReduce for sub-MiB sums; the
//                        reference's P2P all-reduce, driver/cuda/src/custom_all_reduce.cu:137-199,
//                        is not built for sm_100).
//
// Together with the EPI_RS epilogue and the gated loads of gemm_tcgen05.cu this replaces the
// reference's GEMM + ncclAllReduce + residual_add_rmsnorm sequence
// (driver/cuda/src/model/llama_like.cpp:626-647, 703-733): the residual stream stays
// row-sharded between blocks, one reduce-scatter and one all-gather cross NVLink instead of
// an all-reduce, and neither is a separate collective call.
// Every spin has an iteration/time bound; on a time-out the kernel records PIE_ERR_WAIT_PEER
// in the status word and finishes without touching peer data.
#include "common.cuh"

namespace pie {

constexpr int TPN_MAX_RANKS = 8;

struct TpNormArgs {
    const bf16* recv;                 // local [world][rows_per_rank][H] partial rows from each rank
    const int* rs_flags;              // local [world], written by peers' GEMM epilogues
    const int* rs_epoch;              // local expected value (bumped by this rank's own GEMM)
    bf16* residual;                   // local [rows_per_rank][H]
    const bf16* weight;               // RMSNorm weight [H]
    bf16* peer_xfull[TPN_MAX_RANKS];  // full activation [world*rows_per_rank][H] on every rank
    int* peer_ag_flags[TPN_MAX_RANKS];
    int* ag_done;                     // local CTA arrival counter
    int* ag_epoch;                    // local count of pushes issued
    int* status;
    int world, rank, rows_per_rank, hidden, valid_rows, reduce;
    float eps;
};

template <int MAXV>
__global__ void __launch_bounds__(256)
tp_reduce_norm_push_kernel(const __grid_constant__ TpNormArgs a) {
    __shared__ float red[32];
    __shared__ int s_ok;
    const int row = blockIdx.x;
    const int nvec = a.hidden >> 3;
    // Launched with programmatic stream serialisation: the block may be resident while the GEMM that
    // feeds it drains (no launch gap), but the epoch it compares the flags with is bumped by that GEMM,
    // so nothing is read before the grid dependency resolves.
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x == 0) {
        int ok = 1;
        if (a.reduce) {
            const int e = *reinterpret_cast<const volatile int*>(a.rs_epoch);
            const long long t0 = clock64();
            const unsigned long long tg = row == 0 ? global_ns() : 0ull;
            for (int src = 0; src < a.world && ok; ++src) {
                while (*reinterpret_cast<const volatile int*>(a.rs_flags + src) < e) {
                    if (*reinterpret_cast<volatile int*>(a.status) != 0 || clock64() - t0 > 1500000000ll) {
                        atomicCAS(a.status, 0, PIE_ERR_WAIT_PEER);
                        ok = 0;
                        break;
                    }
                }
            }
            if (row == 0) status_add_wait(a.status, 1, tg);
            __threadfence_system();
        }
        s_ok = ok;
    }
    __syncthreads();
    const bool ok = s_ok != 0;
    if (ok && row < a.valid_rows) {
        bf16x8* res = reinterpret_cast<bf16x8*>(a.residual + (size_t)row * a.hidden);
        float cache[MAXV][8];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            const int i = threadIdx.x + j * 256;
            if (i < nvec) {
                unpack8(res[i], cache[j]);
                if (a.reduce) {
                    for (int src = 0; src < a.world; ++src) {
                        const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(
                            a.recv + ((size_t)src * a.rows_per_rank + row) * a.hidden) + i);
                        float p[8];
                        unpack8(*reinterpret_cast<const bf16x8*>(&raw), p);
#pragma unroll
                        for (int k = 0; k < 8; ++k) cache[j][k] += p[k];
                    }
                    bf16x8 packed = pack8(cache[j]);
                    unpack8(packed, cache[j]);
                    res[i] = packed;
                }
#pragma unroll
                for (int k = 0; k < 8; ++k) ss += cache[j][k] * cache[j][k];
            }
        }
        ss = block_sum(ss, red);
        const float inv = rsqrtf(ss / (float)a.hidden + a.eps);
        const bf16x8* wr = reinterpret_cast<const bf16x8*>(a.weight);
        const size_t grow = (size_t)a.rank * a.rows_per_rank + row;
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            const int i = threadIdx.x + j * 256;
            if (i < nvec) {
                float wv[8], o[8];
                unpack8(wr[i], wv);
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = cache[j][k] * inv * wv[k];
                const bf16x8 packed = pack8(o);
                for (int p = 0; p < a.world; ++p)
                    reinterpret_cast<bf16x8*>(a.peer_xfull[p] + grow * a.hidden)[i] = packed;
            }
        }
    }
    // publish once per kernel: the last CTA to finish raises this rank's flag on every peer
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(a.ag_done, 1) + 1 == (int)gridDim.x) {
            *a.ag_done = 0;
            const int e = *reinterpret_cast<volatile int*>(a.ag_epoch) + 1;
            *reinterpret_cast<volatile int*>(a.ag_epoch) = e;
            __threadfence_system();
            if (ok)
                for (int p = 0; p < a.world; ++p)
                    *reinterpret_cast<volatile int*>(a.peer_ag_flags[p] + a.rank) = e;
        }
    }
}

__global__ void tp_wait_ag_kernel(const int* ag_flags, const int* ag_epoch, int world, int* status) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    const int e = *reinterpret_cast<const volatile int*>(ag_epoch);
    const long long t0 = clock64();
    for (int src = 0; src < world; ++src) {
        while (*reinterpret_cast<const volatile int*>(ag_flags + src) < e) {
            if (*reinterpret_cast<volatile int*>(status) != 0 || clock64() - t0 > 1500000000ll) {
                atomicCAS(status, 0, PIE_ERR_WAIT_PEER);
                return;
            }
        }
    }
    __threadfence_system();
}

struct TpArArgs {
    bf16* peer_slots[TPN_MAX_RANKS];   // [2 parities][world][cap] bf16 on every rank
    int* peer_flags[TPN_MAX_RANKS];    // [world] on every rank (word [src] written by rank src)
    const int* flags;                  // local flags
    int* done;                         // local CTA arrival counter
    int* epoch;                        // local count of all-reduces issued
    int* status;
    int world, rank;
    long cap;                          // elements per slot
};

// Cooperative across ranks (each GPU runs its own launch); grid <= number of SMs so that every
// block is resident while it waits. Waits are bounded.
__global__ void __launch_bounds__(256)
tp_allreduce_small_kernel(const __grid_constant__ TpArArgs a, const bf16* __restrict__ in, bf16* __restrict__ out,
                          long n) {
    __shared__ int s_epoch, s_ok;
    const long nvec = n >> 3;
    const int e_next = *reinterpret_cast<volatile int*>(a.epoch) + 1;     // the same in every block until bumped
    const int par = e_next & 1;
    // 1. push this rank's data into slot [par][rank] of every rank (own included)
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
        const bf16x8 v = reinterpret_cast<const bf16x8*>(in)[i];
        for (int p = 0; p < a.world; ++p)
            reinterpret_cast<bf16x8*>(a.peer_slots[p] + ((size_t)par * a.world + a.rank) * a.cap)[i] = v;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        // 2. last block of this rank raises the flag on every peer
        if (atomicAdd(a.done, 1) + 1 == (int)gridDim.x) {
            *a.done = 0;
            __threadfence_system();
            for (int p = 0; p < a.world; ++p) *reinterpret_cast<volatile int*>(a.peer_flags[p] + a.rank) = e_next;
            *reinterpret_cast<volatile int*>(a.epoch) = e_next;
        }
        // 3. wait for every rank's flag
        int ok = 1;
        const long long t0 = clock64();
        for (int src = 0; src < a.world && ok; ++src) {
            while (*reinterpret_cast<const volatile int*>(a.flags + src) < e_next) {
                if (*reinterpret_cast<volatile int*>(a.status) != 0 || clock64() - t0 > 1500000000ll) {
                    atomicCAS(a.status, 0, PIE_ERR_WAIT_PEER);
                    ok = 0;
                    break;
                }
            }
        }
        __threadfence_system();
        s_ok = ok;
        s_epoch = e_next;
    }
    __syncthreads();
    if (!s_ok) return;
    // 4. sum the slots in rank order
    const bf16* base = a.peer_slots[a.rank] + (size_t)par * a.world * a.cap;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int src = 0; src < a.world; ++src) {
            float v[8];
            unpack8(reinterpret_cast<const bf16x8*>(base + (size_t)src * a.cap)[i], v);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += v[j];
        }
        reinterpret_cast<bf16x8*>(out)[i] = pack8(acc);
    }
}

}  // namespace pie

using namespace pie;

PIE_API int pie_tp_ar_args_size() { return (int)sizeof(TpArArgs); }

PIE_API int pie_tp_fill_ar_args(void* blob, void* const* peer_slots, int* const* peer_flags, const int* flags,
                                int* done, int* epoch, int* status, int world, int rank, long cap) {
    if (world > TPN_MAX_RANKS || world < 1) return (int)cudaErrorInvalidValue;
    TpArArgs a{};
    for (int i = 0; i < world; ++i) {
        a.peer_slots[i] = (bf16*)peer_slots[i];
        a.peer_flags[i] = peer_flags[i];
    }
    a.flags = flags; a.done = done; a.epoch = epoch; a.status = status; a.world = world; a.rank = rank; a.cap = cap;
    *reinterpret_cast<TpArArgs*>(blob) = a;
    return 0;
}

// out = sum over ranks of in (n bf16 elements, n % 8 == 0, n <= cap). Every rank must call it the
// same number of times; `in` may equal `out`.
PIE_API int pie_tp_allreduce_small(const void* blob, const void* in, void* out, long n, int num_sms, cudaStream_t st) {
    if (n <= 0) return 0;
    const TpArArgs a = *reinterpret_cast<const TpArArgs*>(blob);
    if (n % 8 || n > a.cap) return (int)cudaErrorInvalidValue;
    long blocks = (n / 8 + 255) / 256;
    if (blocks > num_sms) blocks = num_sms;
    tp_allreduce_small_kernel<<<(int)blocks, 256, 0, st>>>(a, (const bf16*)in, (bf16*)out, n);
    return (int)cudaGetLastError();
}

PIE_API int pie_tp_norm_args_size() { return (int)sizeof(TpNormArgs); }

PIE_API int pie_tp_fill_norm_args(void* blob, const void* recv, const int* rs_flags, const int* rs_epoch,
                                  void* const* peer_xfull, int* const* peer_ag_flags, int* ag_done,
                                  int* ag_epoch, int* status, int world, int rank) {
    if (world > TPN_MAX_RANKS || world < 1) return (int)cudaErrorInvalidValue;
    TpNormArgs a{};
    a.recv = (const bf16*)recv; a.rs_flags = rs_flags; a.rs_epoch = rs_epoch;
    for (int i = 0; i < world; ++i) {
        a.peer_xfull[i] = (bf16*)peer_xfull[i];
        a.peer_ag_flags[i] = peer_ag_flags[i];
    }
    a.ag_done = ag_done; a.ag_epoch = ag_epoch; a.status = status; a.world = world; a.rank = rank;
    *reinterpret_cast<TpNormArgs*>(blob) = a;
    return 0;
}

// residual[rows_per_rank, H] (+= sum of partial rows when `reduce`), then RMSNorm(weight) of the
// valid rows pushed to every rank's gathered activation buffer.
PIE_API int pie_tp_reduce_norm_push(const void* blob, void* residual, const void* weight,
                                    int rows_per_rank, int hidden, int valid_rows, int reduce, float eps,
                                    cudaStream_t st) {
    if (rows_per_rank <= 0) return 0;
    if (hidden % 8 || hidden > 256 * 8 * 8) return (int)cudaErrorInvalidValue;
    TpNormArgs a = *reinterpret_cast<const TpNormArgs*>(blob);
    a.residual = (bf16*)residual; a.weight = (const bf16*)weight;
    a.rows_per_rank = rows_per_rank; a.hidden = hidden; a.valid_rows = valid_rows; a.reduce = reduce; a.eps = eps;
    const int per = (hidden / 8 + 255) / 256;
    cudaError_t e;
    if (per <= 1) e = launch_pdl(tp_reduce_norm_push_kernel<1>, dim3(rows_per_rank), dim3(256), 0, st, a);
    else if (per <= 2) e = launch_pdl(tp_reduce_norm_push_kernel<2>, dim3(rows_per_rank), dim3(256), 0, st, a);
    else if (per <= 4) e = launch_pdl(tp_reduce_norm_push_kernel<4>, dim3(rows_per_rank), dim3(256), 0, st, a);
    else e = launch_pdl(tp_reduce_norm_push_kernel<8>, dim3(rows_per_rank), dim3(256), 0, st, a);
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

PIE_API int pie_tp_wait_ag(const int* ag_flags, const int* ag_epoch, int world, int* status,
                           cudaStream_t st) {
    tp_wait_ag_kernel<<<1, 32, 0, st>>>(ag_flags, ag_epoch, world, status);
    return (int)cudaGetLastError();
}
