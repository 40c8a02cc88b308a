// Shared device helpers for the sm_100a kernel library.
//
// Every launcher in this library is an `extern "C"` function that takes raw
// device pointers plus the CUDA stream to launch on and returns the value of
// cudaGetLastError() after the launch. Python calls them through ctypes with
// `tensor.data_ptr()` and the current torch stream, so launches are capturable
// in CUDA graphs and no torch headers are needed to build the library.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define PIE_API extern "C" __attribute__((visibility("default")))

// Status words written by kernels that can give up on a bounded wait.
enum PieKernelStatus : int {
    PIE_OK = 0,
    PIE_ERR_WAIT_TMA = 1,      // producer/consumer mbarrier wait ran out
    PIE_ERR_WAIT_MMA = 2,      // accumulator-ready wait ran out
    PIE_ERR_WAIT_EPILOGUE = 3, // accumulator-free wait ran out
    PIE_ERR_WAIT_PEER = 4,     // peer flag wait ran out
    PIE_ERR_BOUNDS = 5,        // index outside its table (debug checks)
};

// Layout of the status block (8 int32, 8-byte aligned) that the kernels with peer waits are given:
//   [0]    first PieKernelStatus error code, 0 while healthy
//   [1]    for PIE_ERR_BOUNDS from the index validator: table code << 24 | position of the first bad entry
//   [2..3] nanoseconds (u64) that CTA 0 of the gated GEMMs spent waiting for all-gather flags, [6] waits counted
//   [4..5] nanoseconds (u64) that CTA 0 of the reduce + norm + push kernel spent waiting for reduce-scatter
//          flags, [7] waits counted
// The wait counters are a profiling aid (one atomic per kernel); nothing reads them on the hot path.
constexpr int PIE_STATUS_WORDS = 8;

// Programmatic dependent launch (off unless pie_set_pdl(1)): a kernel launched through
// pie::launch_pdl may start while its predecessor in the stream is still draining. It must call
// pdl_wait() before it reads anything the predecessor wrote or writes anything the predecessor
// may still read; work that touches only constants (weights) may run before that.
// pdl_trigger() lets the successor's blocks start as soon as resources free up.
extern int g_pie_pdl;

namespace pie {

__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_pie_pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void status_add_wait(int* status, int slot, unsigned long long t0) {
    atomicAdd(reinterpret_cast<unsigned long long*>(status + 2 + 2 * slot), global_ns() - t0);
    atomicAdd(status + 6 + slot, 1);
}

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum for blocks of up to 1024 threads. `red` is >= 32 floats of
// shared memory. Every thread gets the total.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : 0.f;
    t = warp_sum(t);
    return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}

struct __align__(16) bf16x8 {
    bf162 v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float* f) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __bfloat1622float2(p.v[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ bf16x8 pack8(const float* f) {
    bf16x8 p;
#pragma unroll
    for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return p;
}

// 64-bit mix used for counter-based random numbers (SplitMix64 finaliser).
__device__ __host__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
// Uniform in (0,1) from (seed, row, index).
__device__ __forceinline__ float uniform01(uint64_t seed, uint32_t row, uint32_t idx) {
    uint64_t h = splitmix64(seed ^ splitmix64(((uint64_t)row << 32) | idx));
    return ((float)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

}  // namespace pie
