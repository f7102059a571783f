// The TMA views of one layer's pages, shared by the attention kernels.  Plain: a matrix
// [num_pages * 2 * num_kv_heads * page_size rows, head_dim] of bfloat16 with boxes of [page_size rows, 64 lanes]
// and 128-byte swizzle.  Grouped: the same memory as [rows / 8][head_dim / 64][8 rows][64 lanes] with a box of a
// whole page, [page_size / 8][head_dim / 64][8][64], which lands as 1 KB swizzle atoms of 8 rows, a group's halves of
// head_dim side by side.  Maps are cached by (pointer, rows, head_dim, page_size, kind).
// Returns false, with the error text set, when the driver refuses.  Defined in attention_mma.cu.
#pragma once
#include <cuda.h>

bool vcb_kv_tensor_map(const void* pages, long long rows, int hd, int page_size, CUtensorMap* out, bool grouped = false);
