// The TMA view of one layer's pages, shared by the attention kernels: a matrix
// [num_pages * 2 * num_kv_heads * page_size rows, head_dim] of bfloat16 with boxes of
// [page_size rows, 64 lanes] and 128-byte swizzle.  Maps are cached by (pointer, rows, head_dim, page_size).
// Returns false, with the error text set, when the driver refuses.  Defined in attention_mma.cu.
#pragma once
#include <cuda.h>

bool vcb_kv_tensor_map(const void* pages, long long rows, int hd, int page_size, CUtensorMap* out);
