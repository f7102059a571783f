// Decode attention for callers that must not allocate.  This entry point has no counterpart in the reference
// (laik/vllm-cpp): it exists for hosts that embed this library.
//
// Who needs it: a caller that has already handed every byte of free device memory to its own pools (an engine
// that sized its cache to fill the GPU, a host application with a memory manager of its own), or one that runs
// in a phase where a device allocation is not acceptable because cudaMalloc and cudaFree take driver locks and
// may synchronise the whole device (a serving loop with a latency bound, a callback of another runtime).  The
// regular entry points vcb_attn_paged + vcb_attn_merge need two buffers for the partial results of the key
// slices, which such a caller has nowhere to get from.
//
// What it does instead: the partials live in a file-scope __device__ array of VCB_NO_ALLOC_SCRATCH_FLOATS floats
// (32 MiB) that is part of the library image.  Every GPU that loads the library holds that array until the
// process exits.  The function calls no cudaMalloc, cudaFree or allocating library routine; inputs and outputs
// are still the caller's.
//
// Rules for callers:
//  * n_dec * nh * nslices * (hd + 2) must not exceed VCB_NO_ALLOC_SCRATCH_FLOATS; larger calls are refused with
//    an error text (vcb_last_error), nothing is launched.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
//    current).  Make that first call outside any stream capture.
//  * All calls on a device share the one array and it keeps the last call's contents.  Calls whose kernels may
//    overlap on the GPU (different streams without an ordering between them) race on it: order them.
//  * Arguments as vcb_attn_paged with rows_max 8 (one item per (decoded token, key slice), item[5] = index of
//    the token among the n_dec), plus dec_rows[n_dec]: the output row of each token, or -1 to skip it.
//  * An entry without tokens (q_len <= 0 or ctx_len <= 0) gets zeros in its output row; give it dec_rows = -1
//    if that row must stay as it is.
//  * Every item must name a token index below n_dec (item[5]), a slice below nslices (item[3]) and the same
//    slice count as the call (item[4] == nslices).  An item that does not is left out, nothing of the built-in
//    array is touched for it, bit 32 is set in *status (which must not be null), and the output row of its token
//    is not valid.
#pragma once
#include <cuda_runtime.h>

#define VCB_NO_ALLOC_SCRATCH_FLOATS (8 * 1024 * 1024)

extern "C" int vcb_attn_decode_no_alloc(const void* q, void* out, int dtype, const void* pages, long long page_stride,
                                        const int* block_table, const int* table_row, int max_blocks,
                                        const int* q_start, const int* q_len, const int* ctx_len, const int* items,
                                        const int* dec_rows, int n_dec, int nslices, int nh, int nkv, int hd,
                                        int page_size, int num_pages, int window, float scale, int* status,
                                        cudaStream_t stream);
