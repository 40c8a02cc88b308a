/* Allocation-free entry point of the kernel library.
 *
 * This function has no counterpart in the reference engine; it exists for
 * embedders of this library only.
 *
 * Who needs it: a serving process hands almost all free device memory to the
 * KV-page pool when it starts, and from then on a late cudaMalloc can fail,
 * and even when it succeeds it synchronises the whole device and stalls the
 * pipelined decode loop. The same holds for a host that loads this library as
 * a plug-in into a process whose device memory is a fixed arena it does not
 * own. Such callers can pass inputs and outputs that they already hold, but
 * they cannot create the split-KV scratch buffer that pie_paged_decode_attn
 * expects from its caller.
 *
 * pie_paged_decode_attn_noalloc is pie_paged_decode_attn with that scratch
 * taken from a fixed array inside the library instead:
 *
 *   - the array is PIE_NOALLOC_SCRATCH_FLOATS floats (16 MiB) of device
 *     memory per GPU; every GPU that loads the library holds it until the
 *     process exits;
 *   - a call needs max_items * hq * (head_dim + 1) floats; a call that needs
 *     more is rejected with PIE_NOALLOC_ERR_TOO_LARGE (a line on stderr says
 *     how much was asked for) and launches nothing;
 *   - the function calls no cudaMalloc, cudaFree or other allocating routine;
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current). Make that first call
 *     outside of any stream capture;
 *   - all calls share the one array and it keeps whatever the last call left
 *     in it. Nothing in it has to start at zero: every partial result that the
 *     merge pass reads was written by the first pass of the same call. Two
 *     calls whose kernels overlap on the GPU (different streams, or different
 *     host threads) race on the array - serialise them.
 *
 * Arguments are those of pie_paged_decode_attn without `scratch`; q, the KV
 * layer, the index arrays and `out` stay caller-owned device memory.
 * Returns 0, a cudaError_t value, or one of the codes below.
 */
#pragma once
#include <cuda_runtime.h>

#define PIE_NOALLOC_SCRATCH_FLOATS (4u * 1024u * 1024u)
#define PIE_NOALLOC_ERR_TOO_LARGE (-1001)
#define PIE_NOALLOC_ERR_SETUP (-1002)

#ifdef __cplusplus
extern "C" {
#endif

int pie_paged_decode_attn_noalloc(const void* q, const void* kv_layer, const int* page_indices,
                                  const int* kv_page_indptr, const int* item_req,
                                  const int* item_start, const int* item_end,
                                  const int* req_item_indptr, const int* num_items_ptr, void* out,
                                  int max_items, int num_reqs, int hq, int hkv, int head_dim,
                                  int page_size, float sm_scale, int num_ctas, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
