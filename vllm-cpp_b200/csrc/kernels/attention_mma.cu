// bfloat16 attention over the paged cache on tensor cores (head_dim 64 or 128).
//
// Same contract and work items as attention.cu (one item = an entry, a run of
// query tokens, one slice of the key range; rows = tokens x the query heads that
// share a KV head), same math in 32-bit: scores (q.k)/sqrt(head_dim), keys in
// (pos - window, pos], streaming softmax, sum_j w_j v_j
// (src/model.cpp:1000-1052 of the reference).  What differs is how the work is
// laid on the SM:
//  * K and V tiles of 64 keys are gathered from their pages into shared memory
//    with cp.async, 16 bytes a thread, double buffered, so HBM reads stay in
//    flight while the previous tile is multiplied;
//  * Q.K^T and P.V are mma.sync m16n8k16 products (bf16 in, f32 accumulate) fed by
//    ldmatrix from a 16-byte XOR-swizzled layout;
//  * the four warps either take four different row groups and all keys of a tile
//    (prompt portions: 128 rows a block on eight warps) or the same 16 rows and a quarter of the
//    tile's keys each (single decoded tokens: few rows, long key ranges), their
//    partial softmax states merged through shared memory at the end.
// Rows beyond the item's real rows and keys beyond the slice are zero-filled and
// masked, never read from memory that is not theirs.
//
// Two loaders feed the same multiply code.  With pages of 8, 16, 32 or 64 tokens a fifth warp issues TMA
// tile loads (cp.async.bulk.tensor with 128-byte swizzle, one box per page and 64 lanes of head_dim) into a
// ring of three stages guarded by full/empty mbarriers, so the four multiplying warps spend no instructions
// on addresses; every wait is bounded and reports through the status word.  Other page sizes use cp.async
// from all threads with two stages.
#include "common.cuh"
#include "mbarrier.cuh"
#include "kv_tensor_map.h"

#include <cuda.h>
#include <math_constants.h>

#include <mutex>
#include <unordered_map>

namespace {

constexpr int BN = 64;        // keys per tile
constexpr int ITEM_INTS = 6;  // entry, q0, nq, slice, nslices, decode index

// Decoding straight from the stacked q, k, v projection (single-token items only): the block makes its own query
// rows -- k-slice partial sums added in slice order, per-head RMSNorm, rotation by the token's position, exactly
// the arithmetic of qknorm_rope_kvwrite_kernel -- and the blocks whose key slice holds the token's own position
// make its key and value likewise and store them in the token's cache slot before they load that page.  One kernel
// and one kernel boundary less per layer.  qkv == null: queries come from q, keys and values are in the cache.
struct FusedQkv {
    const float* qkv;          // [slices][tokens][(nh + 2 nkv) * HD] 32-bit partial sums
    int slices;
    long long slice_stride;    // elements between slices
    const void* q_gain;        // [HD] gains of the per-head norms (null with use_norm 0)
    const void* k_gain;
    int gain_dtype, use_norm;
    float eps;
    const float* cos_sin;      // [max_pos][HD]: HD/2 cosines, then HD/2 sines
    int max_pos;
    const int* slot_map;       // [tokens]: page * page_size + offset of the token's cache entry, -1: none
    __nv_bfloat16* pages_w;    // the same pages, to write
};

struct AttnArgs {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    const __nv_bfloat16* pages;
    long long page_stride;
    const int* block_table;
    const int* table_row;
    int max_blocks;
    const int* q_start;
    const int* q_len;
    const int* ctx_len;
    const int* items;
    float* part_o;
    float* part_ml;
    int* slice_counters;   // one per (decoded token, KV head group): slices finished; null: a separate kernel merges
    const int* dec_rows;   // output row of each decoded token (for the merging block)
    int nh, nkv, page_size, num_pages, window;
    float scale;
    int* status;
    FusedQkv f;
    int cluster;   // > 1: the blocks of a token's key slices form a cluster of that many and merge through shared memory
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `c` of row `r` in a tile of ROWS rows: the tile is stored as head_dim/64 blocks of
// [ROWS][128 bytes], each 128-byte row XOR-swizzled by its row index -- the layout a 128-byte-swizzled TMA box
// of 64 lanes produces, and conflict-free for ldmatrix.
template <int ROWS> __device__ __forceinline__ int swz(int r, int c) {
    return (c >> 3) * (ROWS * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4);
}

// The same for a K or V tile: [groups of 8 keys][head_dim/64 halves][8 rows][128 bytes], every 1 KB piece of 8 rows
// swizzled like the above.  It is what ONE TMA box per page produces, whatever head_dim, from the cache seen as
// [groups of 8 tokens][halves][8 tokens][64 lanes] (kv_tensor_map, grouped): a copy per page and half of head_dim
// cost the loading warp about 100 clocks each, 1,600 a tile -- more than the tile's share of the HBM time.
template <int HALVES> __device__ __forceinline__ int swz_kv(int key, int c) {
    return (key >> 3) * (HALVES * 1024) + (c >> 3) * 1024 + (key & 7) * 128 + (((c & 7) ^ (key & 7)) << 4);
}

// a box of whole groups of 8 tokens, all lanes: coordinates (lane 0, token 0, half 0, group)
__device__ __forceinline__ void tma_load_groups(uint32_t dst, const CUtensorMap* map, uint32_t bar, int group) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %3, %3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(0), "r"(group) : "memory");
}

// Blocks of a cluster: rank, the common barrier (arrive with release, wait with acquire), and reads of another
// block's shared memory.
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float2 ld_cluster_f2(const void* local, uint32_t rank) {
    uint32_t remote;
    float2 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(remote) : "memory");
    return v;
}

// WR row groups x WK key groups multiplying warps, MR tiles of 16 rows each; TMA adds one warp that only issues
// tile loads.
// DEEP: a ring of six stages instead of three, for launches whose blocks have an SM each anyway (one or two requests
// decoding): a short key slice is then all on its way before the block's wait is over, where a ring of three brought
// the second half one memory latency after the first.
template <int HD, int WR, int WK, int MR, bool TMA, bool DEEP = false>
__global__ __launch_bounds__(WR * WK * 32 + (TMA ? 32 : 0)) void attn_mma_kernel(const __grid_constant__ CUtensorMap kv_map,
                                                                        AttnArgs a) {
    static_assert(HD % 64 == 0 && BN % (16 * WK) == 0, "layout");
    constexpr int NW = WR * WK;     // multiplying warps
    constexpr int NT = NW * 32;     // their threads
    constexpr int RMAX = 16 * WR * MR;   // rows a block holds: WR warp groups x MR tiles of 16 rows each
    constexpr int CH = HD / 8;      // 16-byte chunks per row
    constexpr int ROWB = HD * 2;
    constexpr int KW = BN / WK;     // keys of a tile that one warp multiplies
    constexpr int NS = KW / 8;      // score n-tiles per warp
    constexpr int ND = HD / 8;      // output n-tiles
    constexpr int STAGES = (TMA && WK == 4) ? (DEEP ? 6 : 3) : 2;   // decoding streams keys: a deeper ring; prompt portions multiply more
    constexpr int TILE_BYTES = BN * ROWB;   // one K or V tile
    constexpr float LOG2E = 1.4426950408889634f;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base_u32 = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzle atoms are 1024-byte aligned
    uint8_t* smem = smem_raw + (base_u32 - smem_u32(smem_raw));
    uint8_t* k_s = smem;                              // STAGES tiles
    uint8_t* v_s = k_s + STAGES * TILE_BYTES;         // STAGES tiles
    uint8_t* q_s = v_s + STAGES * TILE_BYTES;         // RMAX rows
    uint8_t* bar_s = q_s + RMAX * ROWB;               // 2 * STAGES mbarriers, then the abort flag
    auto full_bar = [&](int st) { return smem_u32(bar_s) + 8u * st; };
    auto empty_bar = [&](int st) { return smem_u32(bar_s) + 8u * (STAGES + st); };
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_s + 16 * STAGES);

    pdl_trigger();
    tl_mark(VCB_TL_ATTN_DEC, 0);
    // The queries and the newest keys come from the kernel before this one.  With TMA loads the wait is put off:
    // what describes the work (items, lengths and block tables are in place before the step's first model kernel
    // starts: the copy of the step's integers is an ordinary stream operation and the kernel that updates the tables
    // triggers no early launch) and the keys and values of earlier steps can be read before it.
    if (!TMA) pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wr = (warp % NW) / WK, wk = (warp % NW) % WK;
    const int* item = a.items + (size_t)blockIdx.x * ITEM_INTS;
    const int e = item[0], q0 = item[1], slice = item[3], nslices = item[4], dec_index = item[5];
    const int qlen = a.q_len[e], ctx = a.ctx_len[e];
    // an item of a captured step is laid out for the largest portion the step serves: fewer tokens may be there
    const int nq = min(item[2], qlen - q0);
    if (qlen <= 0 || ctx <= 0 || nq <= 0) {
        if (TMA) pdl_wait();
        return;
    }

    const int g = a.nh / a.nkv;
    const int gq_max = g < RMAX ? g : RMAX;
    const int hchunks = (g + gq_max - 1) / gq_max;
    const int kvh = blockIdx.y / hchunks, hc = blockIdx.y % hchunks;
    const int head0 = kvh * g + hc * gq_max;
    const int gq = min(gq_max, g - hc * gq_max);
    const int R = nq * gq;

    const int row0 = a.q_start[e] + q0;
    const int pos0 = ctx - qlen + q0;
    const int pos_last = pos0 + nq - 1;
    const int W = a.window;
    const int ps = a.page_size;
    const int lo = W > 0 ? max(0, pos0 - W + 1) : 0;
    const int hi = pos_last + 1;
    const int pb_lo = lo / ps, pb_hi = (hi + ps - 1) / ps;
    const int pps = (pb_hi - pb_lo + nslices - 1) / nslices;
    const int my_pb_lo = pb_lo + slice * pps, my_pb_hi = min(pb_hi, my_pb_lo + pps);
    const int k_begin = max(lo, my_pb_lo * ps), k_end = min(hi, my_pb_hi * ps);
    // tiles start on a page boundary when TMA loads whole pages
    const int t_first = TMA ? my_pb_lo * ps : k_begin;
    const int n_tiles = k_end > k_begin ? (k_end - t_first + BN - 1) / BN : 0;

    const int* bt = a.block_table + (size_t)(a.table_row ? a.table_row[e] : e) * a.max_blocks;

    if (TMA && tid == 0) {
        for (int st = 0; st < STAGES; ++st) {
            mbar_init(full_bar(st), 1);
            mbar_init(empty_bar(st), NW);   // one arrival per multiplying warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }

    // ---- TMA producer state: one box per page for K and one for V.  The boxes of a tile (up to 16) are issued by
    // as many lanes at once, each with its page id read ahead: one thread issuing them in turn, each behind its own
    // block-table read, took about as long as the tile's share of HBM time. ----
    const int pages_per_tile = BN / ps;
    const int groups_page = ps / 8;
    const int groups_kv = a.nkv * groups_page;   // groups of 8 rows from a page's K to its V
    const int my_pg = lane >> 1, my_v = lane & 1;
    auto page_of = [&](int it) {
        const int pb = my_pb_lo + it * pages_per_tile + my_pg;
        return (it < n_tiles && my_pg < pages_per_tile && pb < my_pb_hi) ? bt[pb] : -1;
    };
    // page ids of the next AHEAD tiles, read that far ahead: each is a load from the block table, and read only one
    // tile ahead they made the tiles of a short key range (a few tiles, nothing else to wait for) follow each other
    // at one round trip to memory apiece
#ifndef VCB_AHEAD
#define VCB_AHEAD 4
#endif
    constexpr int AHEAD = VCB_AHEAD;
    int ahead_page[AHEAD];
#pragma unroll
    for (int k = 0; k < AHEAD; ++k) ahead_page[k] = -1;
    // asks for tile `it` once its stage is free (the producer warp, all lanes); false: give up
    auto issue_tile = [&](int it) {
        const int st = it % STAGES;
        bool ok = true;
        if (lane == 0) ok = mbar_wait(empty_bar(st), ((it / STAGES) & 1) ^ 1u, abort_flag, a.status);
        if (!__shfl_sync(0xffffffffu, ok, 0)) return false;
        const int pb0 = my_pb_lo + it * pages_per_tile;
        const int np = min(pages_per_tile, my_pb_hi - pb0);
        if (lane == 0) mbar_expect_tx(full_bar(st), (uint32_t)(np * ps * ROWB * 2));
        __syncwarp();
        if (my_pg < np) {
            int page = ahead_page[0];
            if (page < 0 || page >= a.num_pages) {
                atomicOr(a.status, VCB_STATUS_BAD_PAGE);
                page = 0;   // keep the byte count whole; the status word reports the fault
            }
            const int group = (page * 2 * a.nkv + kvh) * groups_page + (my_v ? groups_kv : 0);
            const uint32_t dst = smem_u32((my_v ? v_s : k_s) + st * TILE_BYTES) + my_pg * ps * ROWB;
            tma_load_groups(dst, &kv_map, full_bar(st), group);
        }
#pragma unroll
        for (int k = 0; k + 1 < AHEAD; ++k) ahead_page[k] = ahead_page[k + 1];
        ahead_page[AHEAD - 1] = page_of(it + AHEAD);
        return true;
    };
    int pre_tiles = 0;
    constexpr int FPJ = HD / 64;   // lanes of half a head that one thread owns
    float f_cos[FPJ], f_sin[FPJ], f_g1[FPJ], f_g2[FPJ];
    long long f_slot = -1;
    if (TMA) {
        __syncthreads();   // the barriers are initialised
        if (warp == NW) {
            // Tiles whose pages hold only tokens of earlier steps are asked for before the wait: up to a ring's worth.
            const int first_new = ctx - qlen;
#pragma unroll
            for (int k = 0; k < AHEAD; ++k) ahead_page[k] = page_of(k);
            while (pre_tiles < n_tiles && pre_tiles < STAGES &&
                   min(my_pb_hi, my_pb_lo + (pre_tiles + 1) * pages_per_tile) * ps <= first_new) {
                if (!issue_tile(pre_tiles)) break;
                ++pre_tiles;
            }
        }
        // What the fused form needs beside the projection -- the token's position, its cosines and sines, the gains of
        // this warp's heads (queries for the multiplying warps, keys for the loading warp), its cache slot -- is written
        // by no kernel of the step and read before the wait, so that one round trip to memory follows it.
        if constexpr (WR == 1 && MR == 1) {
            if (a.f.qkv != nullptr) {
                int pos = pos0;   // a decoded token's position is its context length less one: no load to wait for
                if (pos < 0 || pos >= a.f.max_pos) {
                    if (tid == 0) atomicOr(a.status, VCB_STATUS_BAD_POSITION);
                    pos = 0;
                }
                const float* cs = a.f.cos_sin + (size_t)pos * HD;
                const void* gain = warp < NW ? a.f.q_gain : a.f.k_gain;
#pragma unroll
                for (int j = 0; j < FPJ; ++j) {
                    const int p = lane + 32 * j;
                    f_cos[j] = cs[p];
                    f_sin[j] = cs[HD / 2 + p];
                    f_g1[j] = a.f.use_norm ? load_as_f32(gain, a.f.gain_dtype, p) : 1.f;
                    f_g2[j] = a.f.use_norm ? load_as_f32(gain, a.f.gain_dtype, p + HD / 2) : 1.f;
                }
                if (warp == NW) f_slot = a.f.slot_map[row0];
            }
        }
        pdl_wait();
    }
    tl_mark(VCB_TL_ATTN_DEC, 1);

    bool fused = false;
    if constexpr (TMA && WR == 1 && MR == 1) fused = a.f.qkv != nullptr;
    if (fused) {
        if constexpr (TMA && WR == 1 && MR == 1) {
            // ---- the token's heads from the stacked projection: warp per head, lane l owns lanes l + 32 j and their
            // partners half a head further on ----
            constexpr int HALF = HD / 2, PJ = HALF / 32;
            const int tok = row0;
            const size_t row_w = (size_t)(a.nh + 2 * a.nkv) * HD;
            // sums of the k-slice partials of one head, four slices' loads in flight at a time
            auto head_sums = [&](int head_col, float (&x1)[PJ], float (&x2)[PJ]) {
                const float* src = a.f.qkv + (size_t)tok * row_w + (size_t)head_col * HD;
#pragma unroll
                for (int j = 0; j < PJ; ++j) x1[j] = x2[j] = 0.f;
                for (int s0 = 0; s0 < a.f.slices; s0 += 4) {
                    float t1[4][PJ], t2[4][PJ];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (s0 + k < a.f.slices) {
#pragma unroll
                            for (int j = 0; j < PJ; ++j) {
                                t1[k][j] = src[(size_t)(s0 + k) * a.f.slice_stride + lane + 32 * j];
                                t2[k][j] = src[(size_t)(s0 + k) * a.f.slice_stride + lane + 32 * j + HALF];
                            }
                        }
                    }
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        if (s0 + k < a.f.slices) {
#pragma unroll
                            for (int j = 0; j < PJ; ++j) { x1[j] += t1[k][j]; x2[j] += t2[k][j]; }
                        }
                    }
                }
            };
            // norm and rotation of one head in place (the order of operations of qknorm_rope_kvwrite_kernel)
            auto norm_rotate = [&](float (&x1)[PJ], float (&x2)[PJ]) {
                float inv = 1.f;
                if (a.f.use_norm) {
                    float ss = 0.f;
#pragma unroll
                    for (int j = 0; j < PJ; ++j) ss += x1[j] * x1[j] + x2[j] * x2[j];
                    ss = warp_sum(ss);
                    inv = 1.0f / sqrtf(ss / (float)HD + a.f.eps);
                }
#pragma unroll
                for (int j = 0; j < PJ; ++j) {
                    float u = x1[j], w = x2[j];
                    if (a.f.use_norm) {
                        u = f_g1[j] * u * inv;
                        w = f_g2[j] * w * inv;
                    }
                    x1[j] = u * f_cos[j] - w * f_sin[j];
                    x2[j] = w * f_cos[j] + u * f_sin[j];
                }
            };
            // rows beyond the token's heads are zero
            for (int idx = tid; idx < (RMAX - R) * CH; idx += blockDim.x)
                *reinterpret_cast<uint4*>(q_s + swz<RMAX>(R + idx / CH, idx % CH)) = make_uint4(0, 0, 0, 0);
            if (warp < NW) {
                for (int r = warp; r < R; r += NW) {
                    float x1[PJ], x2[PJ];
                    head_sums(head0 + r, x1, x2);
                    norm_rotate(x1, x2);
#pragma unroll
                    for (int j = 0; j < PJ; ++j) {
                        const int p = lane + 32 * j, p2 = p + HALF;
                        *reinterpret_cast<__nv_bfloat16*>(q_s + swz<RMAX>(r, p >> 3) + (p & 7) * 2) = __float2bfloat16_rn(x1[j]);
                        *reinterpret_cast<__nv_bfloat16*>(q_s + swz<RMAX>(r, p2 >> 3) + (p2 & 7) * 2) = __float2bfloat16_rn(x2[j]);
                    }
                }
            } else if (k_end == hi && k_end > k_begin) {
                // The loading warp of a block whose slice ends with the token's own position: key and value of the
                // token go into its cache slot, and only then does this warp ask for the page that holds them.
                // (Blocks of several head chunks of one KV head each write the same values.)
                const long long slot = f_slot;
                if (slot >= 0) {
                    if (slot / ps >= a.num_pages) {
                        if (lane == 0) atomicOr(a.status, VCB_STATUS_BAD_PAGE);
                    } else {
                        __nv_bfloat16* page = a.f.pages_w + (slot / ps) * a.page_stride;
                        float x1[PJ], x2[PJ], v1[PJ], v2[PJ];
                        head_sums(a.nh + a.nkv + kvh, v1, v2);     // (the compiler issues these loads with the key's)
                        head_sums(a.nh + kvh, x1, x2);
                        norm_rotate(x1, x2);
                        __nv_bfloat16* kd = page + ((size_t)kvh * ps + slot % ps) * HD;
#pragma unroll
                        for (int j = 0; j < PJ; ++j) {
                            kd[lane + 32 * j] = __float2bfloat16_rn(x1[j]);
                            kd[lane + 32 * j + HALF] = __float2bfloat16_rn(x2[j]);
                        }
#pragma unroll
                        for (int j = 0; j < PJ; ++j) { x1[j] = v1[j]; x2[j] = v2[j]; }
                        __nv_bfloat16* vd = page + ((size_t)(a.nkv + kvh) * ps + slot % ps) * HD;
#pragma unroll
                        for (int j = 0; j < PJ; ++j) {
                            vd[lane + 32 * j] = __float2bfloat16_rn(x1[j]);
                            vd[lane + 32 * j + HALF] = __float2bfloat16_rn(x2[j]);
                        }
                        // the stores above are ordinary ones, the page loads that follow go through the async proxy
                        asm volatile("fence.proxy.async;" ::: "memory");
                        __syncwarp();
                    }
                }
            }
        }
    } else {
        // ---- Q rows -> shared memory (rows beyond R are zero) ----
        for (int idx = tid; idx < RMAX * CH; idx += blockDim.x) {
            const int r = idx / CH, c = idx % CH;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < R) {
                const int iq = r / gq, ih = r % gq;
                v = *reinterpret_cast<const uint4*>(a.q + ((size_t)(row0 + iq) * a.nh + head0 + ih) * HD + c * 8);
            }
            *reinterpret_cast<uint4*>(q_s + swz<RMAX>(r, c)) = v;
        }
    }

    // ---- cp.async loader (all threads): 64 keys x HD of K and of V, gathered page by page ----
    auto load_tile = [&](int stage, int t0) {
        uint8_t* kd = k_s + stage * TILE_BYTES;
        uint8_t* vd = v_s + stage * TILE_BYTES;
#pragma unroll
        for (int i = 0; i < BN * CH / NT; ++i) {
            const int idx = tid + i * NT;
            const int j = idx / CH, c = idx % CH;
            const int kidx = t0 + j;
            const __nv_bfloat16* src = a.pages;
            int bytes = 0;
            if (kidx < k_end) {
                const int page = bt[kidx / ps];
                if (page < 0 || page >= a.num_pages) {
                    atomicOr(a.status, VCB_STATUS_BAD_PAGE);
                } else {
                    src = a.pages + (size_t)page * a.page_stride + ((size_t)kvh * ps + kidx % ps) * HD + c * 8;
                    bytes = 16;
                }
            }
            const int off = swz_kv<HD / 64>(j, c);
            cp_async16(smem_u32(kd + off), src, bytes);
            cp_async16(smem_u32(vd + off), bytes ? src + (size_t)a.nkv * ps * HD : src, bytes);
        }
    };

    if (!TMA) {
        if (n_tiles > 0) load_tile(0, t_first);
        cp_async_commit();
    }
    __syncthreads();   // Q and the barriers are in shared memory

    if (TMA && warp == NW) {
        // ---- TMA producer: the tiles after the ones asked for before the wait ----
        int armed = pre_tiles;
        for (int it = pre_tiles; it < n_tiles; ++it) {
            if (!issue_tile(it)) break;
            armed = it + 1;
        }
        if (lane == 0 && *abort_flag) {   // let copies in flight land before the block goes away
            for (int i = max(0, armed - STAGES); i < armed; ++i) {
                const long long t0 = clock64();
                while (!mbar_try(full_bar(i % STAGES), (i / STAGES) & 1) && clock64() - t0 < VCB_WAIT_CLOCKS) {}
            }
        }
    }

    float o[MR][ND][4];
    float m_run[MR][2], l_run[MR][2];   // rows lane/4 and lane/4 + 8 of each of this warp's 16-row tiles
    int r_a[MR], pos_a[MR], pos_b[MR];
    bool ok_a[MR], ok_b[MR];
#pragma unroll
    for (int mr = 0; mr < MR; ++mr) {
#pragma unroll
        for (int i = 0; i < ND; ++i) o[mr][i][0] = o[mr][i][1] = o[mr][i][2] = o[mr][i][3] = 0.f;
        m_run[mr][0] = m_run[mr][1] = -CUDART_INF_F;
        l_run[mr][0] = l_run[mr][1] = 0.f;   // per-thread partial sums (reduced over the quad at the end)
        r_a[mr] = (wr * MR + mr) * 16 + (lane >> 2);
        pos_a[mr] = pos0 + r_a[mr] / gq;
        pos_b[mr] = pos0 + (r_a[mr] + 8) / gq;
        ok_a[mr] = r_a[mr] < R;
        ok_b[mr] = r_a[mr] + 8 < R;
    }

    if (warp < NW) {
        // ---- one 16-row tile per warp: its Q fragments stay in registers; two: they are re-read per key tile ----
        uint32_t qf[MR == 1 ? HD / 16 : 1][4];
        if (MR == 1) {
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks)
                ldmatrix_x4(qf[MR == 1 ? ks : 0], smem_u32(q_s + swz<RMAX>(wr * 16 + (lane & 15), ks * 2 + (lane >> 4))));
        }

        for (int it = 0; it < n_tiles; ++it) {
            const int st = it % STAGES;
            const int t0 = t_first + it * BN;
            if (TMA) {
                if (!mbar_wait(full_bar(st), (it / STAGES) & 1, abort_flag, a.status)) break;
                if (t0 + BN > k_end) {
                    // the last page may hold slots beyond the sequence (and rows of pages not loaded are stale):
                    // their V must be finite, because a zero weight times NaN is NaN.  Each warp clears what it reads.
                    for (int idx = lane; idx < KW * CH; idx += 32) {
                        const int j = wk * KW + idx / CH, c = idx % CH;
                        if (t0 + j >= k_end) *reinterpret_cast<uint4*>(v_s + st * TILE_BYTES + swz_kv<HD / 64>(j, c)) = make_uint4(0, 0, 0, 0);
                    }
                    __syncwarp();
                }
            } else {
                if (it + 1 < n_tiles) {
                    load_tile((it + 1) & 1, t0 + BN);
                    cp_async_commit();
                    cp_async_wait<1>();
                } else {
                    cp_async_wait<0>();
                }
                __syncthreads();
            }
            const uint8_t* kt = k_s + st * TILE_BYTES;
            const uint8_t* vt = v_s + st * TILE_BYTES;
            const int key0 = t0 + wk * KW;   // first key this warp multiplies

            // S = Q K^T
            float s[MR][NS][4];
#pragma unroll
            for (int mr = 0; mr < MR; ++mr)
#pragma unroll
                for (int i = 0; i < NS; ++i) s[mr][i][0] = s[mr][i][1] = s[mr][i][2] = s[mr][i][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < HD / 16; ++ks) {
                uint32_t qk[MR][4];
#pragma unroll
                for (int mr = 0; mr < MR; ++mr) {
                    if (MR == 1) {
                        qk[mr][0] = qf[MR == 1 ? ks : 0][0]; qk[mr][1] = qf[MR == 1 ? ks : 0][1];
                        qk[mr][2] = qf[MR == 1 ? ks : 0][2]; qk[mr][3] = qf[MR == 1 ? ks : 0][3];
                    } else {
                        ldmatrix_x4(qk[mr], smem_u32(q_s + swz<RMAX>((wr * MR + mr) * 16 + (lane & 15), ks * 2 + (lane >> 4))));
                    }
                }
#pragma unroll
                for (int np = 0; np < KW / 16; ++np) {
                    uint32_t b[4];
                    const int mi = lane >> 3;
                    const int krow = wk * KW + np * 16 + (mi >> 1) * 8 + (lane & 7);
                    ldmatrix_x4(b, smem_u32(kt + swz_kv<HD / 64>(krow, ks * 2 + (mi & 1))));
#pragma unroll
                    for (int mr = 0; mr < MR; ++mr) {
                        mma_16816(s[mr][2 * np], qk[mr], b[0], b[1]);
                        mma_16816(s[mr][2 * np + 1], qk[mr], b[2], b[3]);
                    }
                }
            }
            // mask (only where the tile touches an edge of some row's key range), running maximum
            // rows beyond R hold zero queries and are never written, so they need no mask of their own
            const bool inner = key0 >= k_begin && key0 + KW <= k_end && key0 + KW - 1 <= pos0 && (W <= 0 || key0 > pos_last - W);
            const bool all_inner = __all_sync(0xffffffffu, inner);
            uint32_t pa[MR][KW / 16][4];
#pragma unroll
            for (int mr = 0; mr < MR; ++mr) {
                float mx_a = -CUDART_INF_F, mx_b = -CUDART_INF_F;
                if (all_inner) {
#pragma unroll
                    for (int i = 0; i < NS; ++i) {
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            s[mr][i][c] *= a.scale;
                            s[mr][i][2 + c] *= a.scale;
                            mx_a = fmaxf(mx_a, s[mr][i][c]);
                            mx_b = fmaxf(mx_b, s[mr][i][2 + c]);
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < NS; ++i) {
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const int kidx = key0 + i * 8 + 2 * (lane & 3) + c;
                            const bool in = kidx >= k_begin && kidx < k_end;
                            const bool sa = ok_a[mr] && in && kidx <= pos_a[mr] && (W <= 0 || kidx > pos_a[mr] - W);
                            const bool sb = ok_b[mr] && in && kidx <= pos_b[mr] && (W <= 0 || kidx > pos_b[mr] - W);
                            s[mr][i][c] = sa ? s[mr][i][c] * a.scale : -CUDART_INF_F;
                            s[mr][i][2 + c] = sb ? s[mr][i][2 + c] * a.scale : -CUDART_INF_F;
                            mx_a = fmaxf(mx_a, s[mr][i][c]);
                            mx_b = fmaxf(mx_b, s[mr][i][2 + c]);
                        }
                    }
                }
                mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
                mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
                mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
                mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
                const float mn_a = fmaxf(m_run[mr][0], mx_a), mn_b = fmaxf(m_run[mr][1], mx_b);
                const float use_a = mn_a == -CUDART_INF_F ? 0.f : mn_a, use_b = mn_b == -CUDART_INF_F ? 0.f : mn_b;
                const bool moved = mn_a != m_run[mr][0] || mn_b != m_run[mr][1];
                const float al_a = exp2f((m_run[mr][0] - use_a) * LOG2E), al_b = exp2f((m_run[mr][1] - use_b) * LOG2E);
                m_run[mr][0] = mn_a;
                m_run[mr][1] = mn_b;
                float sum_a = 0.f, sum_b = 0.f;
                const float off_a = use_a * LOG2E, off_b = use_b * LOG2E;
#pragma unroll
                for (int i = 0; i < NS; ++i) {
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        s[mr][i][c] = exp2f(fmaf(s[mr][i][c], LOG2E, -off_a));
                        s[mr][i][2 + c] = exp2f(fmaf(s[mr][i][2 + c], LOG2E, -off_b));
                        sum_a += s[mr][i][c];
                        sum_b += s[mr][i][2 + c];
                    }
                }
                l_run[mr][0] = l_run[mr][0] * al_a + sum_a;
                l_run[mr][1] = l_run[mr][1] * al_b + sum_b;
                if (__any_sync(0xffffffffu, moved)) {   // the running maximum seldom moves after the first tiles
#pragma unroll
                    for (int i = 0; i < ND; ++i) {
                        o[mr][i][0] *= al_a; o[mr][i][1] *= al_a; o[mr][i][2] *= al_b; o[mr][i][3] *= al_b;
                    }
                }
#pragma unroll
                for (int kk = 0; kk < KW / 16; ++kk) {
                    pa[mr][kk][0] = pack_bf16(s[mr][2 * kk][0], s[mr][2 * kk][1]);
                    pa[mr][kk][1] = pack_bf16(s[mr][2 * kk][2], s[mr][2 * kk][3]);
                    pa[mr][kk][2] = pack_bf16(s[mr][2 * kk + 1][0], s[mr][2 * kk + 1][1]);
                    pa[mr][kk][3] = pack_bf16(s[mr][2 * kk + 1][2], s[mr][2 * kk + 1][3]);
                }
            }
            // O += P V
#pragma unroll
            for (int kk = 0; kk < KW / 16; ++kk) {
#pragma unroll
                for (int dp = 0; dp < HD / 16; ++dp) {
                    uint32_t b[4];
                    const int mi = lane >> 3;
                    const int vrow = wk * KW + kk * 16 + (mi & 1) * 8 + (lane & 7);
                    ldmatrix_x4_trans(b, smem_u32(vt + swz_kv<HD / 64>(vrow, dp * 2 + (mi >> 1))));
#pragma unroll
                    for (int mr = 0; mr < MR; ++mr) {
                        mma_16816(o[mr][2 * dp], pa[mr][kk], b[0], b[1]);
                        mma_16816(o[mr][2 * dp + 1], pa[mr][kk], b[2], b[3]);
                    }
                }
            }
            if (TMA) {
                if (t0 + BN > k_end) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the clearing stores above
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar(st));   // this warp is done with the stage
            } else {
                __syncthreads();   // the stage may be overwritten by the load issued in the next iteration
            }
        }
    }
    __syncthreads();   // every tile has been multiplied; the stages and the Q rows are free
    tl_mark(VCB_TL_ATTN_DEC, 3);

    // ---- partial states -> shared memory: o_s[wk][row][HD], ml_s[wk][row][2] ----
    float* o_s = reinterpret_cast<float*>(k_s);             // WK * RMAX x HD floats, over the K and V stages
    float* ml_s = o_s + WK * RMAX * HD;                     // WK * RMAX x 2 floats
    float* cl_o = ml_s + WK * RMAX * 2;                     // RMAX x HD floats: the block's own result, for its cluster
    float* cl_ml = cl_o + RMAX * HD;                        // RMAX x 2 floats
    const bool in_cluster = a.cluster > 1 && nslices > 1;   // the same for all blocks of a cluster
    if (warp < NW) {
#pragma unroll
        for (int mr = 0; mr < MR; ++mr) {
            l_run[mr][0] += __shfl_xor_sync(0xffffffffu, l_run[mr][0], 1);
            l_run[mr][0] += __shfl_xor_sync(0xffffffffu, l_run[mr][0], 2);
            l_run[mr][1] += __shfl_xor_sync(0xffffffffu, l_run[mr][1], 1);
            l_run[mr][1] += __shfl_xor_sync(0xffffffffu, l_run[mr][1], 2);
            const int ra = wk * RMAX + r_a[mr], rb = ra + 8;
#pragma unroll
            for (int i = 0; i < ND; ++i) {
                const int d = i * 8 + 2 * (lane & 3);
                *reinterpret_cast<float2*>(o_s + (size_t)ra * HD + d) = make_float2(o[mr][i][0], o[mr][i][1]);
                *reinterpret_cast<float2*>(o_s + (size_t)rb * HD + d) = make_float2(o[mr][i][2], o[mr][i][3]);
            }
            if ((lane & 3) == 0) {
                ml_s[ra * 2] = m_run[mr][0]; ml_s[ra * 2 + 1] = l_run[mr][0];
                ml_s[rb * 2] = m_run[mr][1]; ml_s[rb * 2 + 1] = l_run[mr][1];
            }
        }
    }
    __syncthreads();

    // ---- merge the key groups and write ----
    for (int idx = tid; idx < R * (HD / 2); idx += blockDim.x) {
        const int r = idx / (HD / 2), d = (idx % (HD / 2)) * 2;
        float m = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < WK; ++w) m = fmaxf(m, ml_s[(w * RMAX + r) * 2]);
        float l = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll
        for (int w = 0; w < WK; ++w) {
            const float mw = ml_s[(w * RMAX + r) * 2];
            if (mw == -CUDART_INF_F) continue;
            const float f = exp2f((mw - m) * LOG2E);
            l += ml_s[(w * RMAX + r) * 2 + 1] * f;
            const float2 ov = *reinterpret_cast<const float2*>(o_s + (size_t)(w * RMAX + r) * HD + d);
            o0 += ov.x * f;
            o1 += ov.y * f;
        }
        const int iq = r / gq, ih = r % gq;
        if (nslices == 1) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            *reinterpret_cast<__nv_bfloat162*>(a.out + ((size_t)(row0 + iq) * a.nh + head0 + ih) * HD + d) =
                __floats2bfloat162_rn(o0 * inv, o1 * inv);
        } else if (in_cluster) {
            *reinterpret_cast<float2*>(cl_o + (size_t)r * HD + d) = make_float2(o0, o1);
            if (d == 0) *reinterpret_cast<float2*>(cl_ml + r * 2) = make_float2(m, l);
        } else {
            const size_t prow = ((size_t)dec_index * a.nh + head0 + r) * nslices + slice;
            *reinterpret_cast<float2*>(a.part_o + prow * HD + d) = make_float2(o0, o1);
            if (d == 0) {
                a.part_ml[prow * 2] = m;
                a.part_ml[prow * 2 + 1] = l;
            }
        }
    }

    // ---- the blocks of a token's key slices, a cluster: each merges its share of the lanes from all the blocks' results
    // in shared memory (two barriers of the cluster and one round of reads between SMs, where the way through global
    // memory below is a fence, a counter and a round trip of the last block, three to six microseconds a launch) ----
    if (in_cluster) {
        cluster_barrier();          // every block's result is in its shared memory (the barrier orders the block's threads too)
        const int out_row = a.dec_rows[dec_index];
        const uint32_t me = cluster_rank();
        if (out_row >= 0) {
            for (int idx = (int)me * (int)blockDim.x + tid; idx < gq * (HD / 2); idx += nslices * (int)blockDim.x) {
                const int ih = idx / (HD / 2), d = (idx % (HD / 2)) * 2;
                constexpr int MC = 8;     // a cluster has at most eight blocks
                float2 mlv[MC], ov[MC];
#pragma unroll
                for (int j = 0; j < MC; ++j) {
                    if (j < nslices) {
                        mlv[j] = ld_cluster_f2(cl_ml + ih * 2, (uint32_t)j);
                        ov[j] = ld_cluster_f2(cl_o + (size_t)ih * HD + d, (uint32_t)j);
                    }
                }
                float m = -CUDART_INF_F, l = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll
                for (int j = 0; j < MC; ++j)
                    if (j < nslices) m = fmaxf(m, mlv[j].x);
#pragma unroll
                for (int j = 0; j < MC; ++j) {     // slice order (a block's rank in its cluster is its slice)
                    if (j < nslices && mlv[j].x != -CUDART_INF_F) {
                        const float w = expf(mlv[j].x - m);
                        l += mlv[j].y * w;
                        o0 += ov[j].x * w;
                        o1 += ov[j].y * w;
                    }
                }
                const float inv = l > 0.f ? 1.f / l : 0.f;
                *reinterpret_cast<__nv_bfloat162*>(a.out + ((size_t)out_row * a.nh + head0 + ih) * HD + d) =
                    __floats2bfloat162_rn(o0 * inv, o1 * inv);
            }
        }
        cluster_barrier();          // nobody leaves while its result may still be read
    }
    // ---- else the block that finishes the last slice of a (token, head group) merges the slices ----
    if (!in_cluster && nslices > 1 && a.slice_counters != nullptr) {
        __shared__ int is_last;
        __threadfence();            // this block's partials are visible before its arrival is counted
        __syncthreads();
        int* counter = a.slice_counters + (size_t)dec_index * gridDim.y + blockIdx.y;
        if (tid == 0) {
            const int prev = atomicAdd(counter, 1);
            is_last = prev == nslices - 1;
            if (is_last) *counter = 0;   // ready for the next launch
        }
        __syncthreads();
        tl_mark(VCB_TL_ATTN_DEC, 4);
        if (is_last) {
            __threadfence();        // the other slices' partials are visible to this block
            const int out_row = a.dec_rows[dec_index];
            if (out_row >= 0) {
                // Everything the merge reads -- every slice's (maximum, sum) and output of this thread's head and pair of
                // lanes -- is asked for at once and then combined in slice order: one round trip to memory.  One load
                // behind the other, the merge of twelve slices took the block as long as its keys had.
#ifndef VCB_MS
#define VCB_MS 12
#endif
                constexpr int MS = VCB_MS;     // slices merged per batch (more run through the loop again)
                for (int idx = tid; idx < gq * (HD / 2); idx += blockDim.x) {
                    const int ih = idx / (HD / 2), d = (idx % (HD / 2)) * 2;
                    const size_t prow0 = ((size_t)dec_index * a.nh + head0 + ih) * nslices;
                    float m = -CUDART_INF_F, l = 0.f, o0 = 0.f, o1 = 0.f;
                    if (nslices <= MS) {
                        float2 mlv[MS], ov[MS];
#pragma unroll
                        for (int j = 0; j < MS; ++j) {
                            if (j < nslices) {
                                mlv[j] = __ldcg(reinterpret_cast<const float2*>(a.part_ml + (prow0 + j) * 2));
                                ov[j] = __ldcg(reinterpret_cast<const float2*>(a.part_o + (prow0 + j) * HD + d));
                            }
                        }
#pragma unroll
                        for (int j = 0; j < MS; ++j)
                            if (j < nslices) m = fmaxf(m, mlv[j].x);
#pragma unroll
                        for (int j = 0; j < MS; ++j) {     // slice order, as the separate merge kernel does
                            if (j < nslices && mlv[j].x != -CUDART_INF_F) {
                                const float w = expf(mlv[j].x - m);
                                l += mlv[j].y * w;
                                o0 += ov[j].x * w;
                                o1 += ov[j].y * w;
                            }
                        }
                    } else {
                        for (int sl = 0; sl < nslices; ++sl) m = fmaxf(m, __ldcg(a.part_ml + (prow0 + sl) * 2));
                        for (int sl0 = 0; sl0 < nslices; sl0 += MS) {
                            float2 mlv[MS], ov[MS];
#pragma unroll
                            for (int j = 0; j < MS; ++j) {
                                if (sl0 + j < nslices) {
                                    mlv[j] = __ldcg(reinterpret_cast<const float2*>(a.part_ml + (prow0 + sl0 + j) * 2));
                                    ov[j] = __ldcg(reinterpret_cast<const float2*>(a.part_o + (prow0 + sl0 + j) * HD + d));
                                }
                            }
#pragma unroll
                            for (int j = 0; j < MS; ++j) {
                                if (sl0 + j < nslices && mlv[j].x != -CUDART_INF_F) {
                                    const float w = expf(mlv[j].x - m);
                                    l += mlv[j].y * w;
                                    o0 += ov[j].x * w;
                                    o1 += ov[j].y * w;
                                }
                            }
                        }
                    }
                    const float inv = l > 0.f ? 1.f / l : 0.f;
                    *reinterpret_cast<__nv_bfloat162*>(a.out + ((size_t)out_row * a.nh + head0 + ih) * HD + d) =
                        __floats2bfloat162_rn(o0 * inv, o1 * inv);
                }
            }
        }
    }
    tl_mark(VCB_TL_ATTN_DEC, 2);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// The pages of one layer seen as a matrix [num_pages * 2 * nkv * page_size, HD]; boxes of [page_size rows, 64 lanes].
bool kv_tensor_map(const void* pages, long long rows, int hd, int page_size, CUtensorMap* out, bool grouped = false) {
    struct Key {
        const void* p; long long rows; int hd, ps;
        bool operator==(const Key& o) const { return p == o.p && rows == o.rows && hd == o.hd && ps == o.ps; }
    };
    struct Hash {
        size_t operator()(const Key& k) const {
            return std::hash<const void*>()(k.p) ^ (std::hash<long long>()(k.rows) * 31) ^ (size_t)(k.hd * 131 + k.ps);
        }
    };
    static std::mutex mu;
    static std::unordered_map<Key, CUtensorMap, Hash> cache;
    const Key key{pages, rows, hd, grouped ? -page_size : page_size};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        vcb_set_error("attn_mma: the driver does not offer cuTensorMapEncodeTiled");
        return false;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)page_size};
    const cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    CUresult r;
    if (!grouped) {
        r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, elem,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        // [groups of 8 rows][halves of head_dim][8 rows][64 lanes], innermost first
        const cuuint64_t dims4[4] = {64, 8, (cuuint64_t)(hd / 64), (cuuint64_t)(rows / 8)};
        const cuuint64_t strides4[3] = {(cuuint64_t)hd * 2, 128, (cuuint64_t)hd * 2 * 8};
        const cuuint32_t box4[4] = {64u, 8u, (cuuint32_t)(hd / 64), (cuuint32_t)(page_size / 8)};
        const cuuint32_t elem4[4] = {1, 1, 1, 1};
        r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(pages), dims4, strides4, box4, elem4,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) {
        vcb_set_error("attn_mma: cuTensorMapEncodeTiled failed with %d (rows %lld, head_dim %d, page %d)", (int)r, rows, hd, page_size);
        return false;
    }
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int HD, int WR, int WK, int MR, bool TMA, bool DEEP = false>
int launch(const AttnArgs& a, int n_items, cudaStream_t stream) {
    constexpr int RMAX = 16 * WR * MR;
    constexpr int STAGES = (TMA && WK == 4) ? (DEEP ? 6 : 3) : 2;
    if constexpr (TMA && WK == 4 && !DEEP) {
        // blocks that have an SM to themselves anyway take the deep ring
        const int g0 = a.nh / a.nkv, gq0 = g0 < RMAX ? g0 : RMAX;
        if ((long long)n_items * a.nkv * ((g0 + gq0 - 1) / gq0) <= sm_count()) return launch<HD, WR, WK, MR, TMA, true>(a, n_items, stream);
    }
    const int g = a.nh / a.nkv;
    const int gq_max = g < RMAX ? g : RMAX;
    const int hchunks = (g + gq_max - 1) / gq_max;
    const size_t stages = 2 * (size_t)STAGES * BN * HD * 2 + (size_t)RMAX * HD * 2 + 16 * STAGES + 16;
    const size_t merge = ((size_t)WK * RMAX * HD + (size_t)WK * RMAX * 2 + (size_t)RMAX * HD + (size_t)RMAX * 2) * sizeof(float);
    const size_t smem = (stages > merge ? stages : merge) + 1024;   // + alignment slack
    CUtensorMap map;
    memset(&map, 0, sizeof(map));
    if (TMA) {
        const long long rows = (long long)a.num_pages * 2 * a.nkv * a.page_size;
        if (a.page_stride != (long long)2 * a.nkv * a.page_size * HD) {
            vcb_set_error("attn_mma: the pages of a layer must be contiguous for TMA loads");
            return -1;
        }
        if (!kv_tensor_map(a.pages, rows, HD, a.page_size, &map, true)) return -3;
    }
    auto kern = attn_mma_kernel<HD, WR, WK, MR, TMA, DEEP>;
    static bool opted = false;
    if (!opted) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            vcb_set_error("attn_mma: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
            return -2;
        }
        opted = true;
    }
    if (a.cluster > 1) {
        if (a.cluster > 8 || n_items % a.cluster != 0 || a.slice_counters == nullptr || a.dec_rows == nullptr) {
            vcb_set_error("attn_mma: clusters of %d blocks for %d items (at most 8, a divisor of the items, with the merge's arrays)", a.cluster, n_items);
            return -1;
        }
        launch_pdl_clusters(kern, dim3(n_items, a.nkv * hchunks), dim3(WR * WK * 32 + (TMA ? 32 : 0)), smem, stream, (unsigned)a.cluster, map, a);
    } else {
        launch_pdl(kern, dim3(n_items, a.nkv * hchunks), dim3(WR * WK * 32 + (TMA ? 32 : 0)), smem, stream, map, a);
    }
    VCB_CHECK_LAUNCH("attn_mma");
    return 0;
}

template <int HD, bool TMA>
int launch_rows(const AttnArgs& a, int n_items, int rows_max, cudaStream_t stream) {
    return rows_max == 16 ? launch<HD, 1, 4, 1, TMA>(a, n_items, stream) : launch<HD, 8, 1, 1, TMA>(a, n_items, stream);
}

}  // namespace

VCB_TIMELINE_UNIT(attn_mma)

bool vcb_kv_tensor_map(const void* pages, long long rows, int hd, int page_size, CUtensorMap* out, bool grouped) {
    return kv_tensor_map(pages, rows, hd, page_size, out, grouped);
}

// cluster: 0, or the number of key slices per decoded token (2 to 8) when their blocks are to run as a cluster and
// merge through shared memory (with slice_counters and dec_rows given, as for the merge by the last block).
// rows_max: 16 (single decoded tokens; four warps split each tile's keys) or 128 (prompt portions; eight warps of
// 16 rows each share the K and V tiles, enough independent MMA chains per SM to keep the tensor pipe fed).
// Only bfloat16 and head_dim 64 or 128; the caller falls back to vcb_attn_paged otherwise.
VCB_API int vcb_attn_mma_supported(int dtype, int hd) { return dtype == VCB_BF16 && (hd == 64 || hd == 128); }

VCB_API int vcb_attn_mma(const void* q, void* out, const void* pages, long long page_stride, const int* block_table,
                         const int* table_row, int max_blocks, const int* q_start, const int* q_len,
                         const int* ctx_len, const int* items, int n_items, int rows_max, float* part_o,
                         float* part_ml, int* slice_counters, const int* dec_rows, int nh, int nkv, int hd,
                         int page_size, int num_pages, int window, float scale, int* status, int allow_tma,
                         int cluster, cudaStream_t stream) {
    if (n_items == 0) return 0;
    VCB_CHECK_ARG(nh > 0 && nkv > 0 && nh % nkv == 0, "attn_mma: %d query heads are not a multiple of %d KV heads", nh, nkv);
    VCB_CHECK_ARG(hd == 64 || hd == 128, "attn_mma: head_dim %d is not 64 or 128", hd);
    VCB_CHECK_ARG(rows_max == 16 || rows_max == 128, "attn_mma: rows_max must be 16 or 128");
    VCB_CHECK_ARG(page_size > 0 && window >= 0, "attn_mma: bad page_size %d or window %d", page_size, window);
    AttnArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)pages, page_stride, block_table,
               table_row, max_blocks, q_start, q_len, ctx_len, items, part_o, part_ml, slice_counters, dec_rows, nh, nkv,
               page_size, num_pages, window, scale, status, FusedQkv{}, cluster};
    const bool tma = allow_tma && (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64) &&
                     ((uintptr_t)pages % 16 == 0) && page_stride == (long long)2 * nkv * page_size * hd;
    if (hd == 64) return tma ? launch_rows<64, true>(a, n_items, rows_max, stream) : launch_rows<64, false>(a, n_items, rows_max, stream);
    return tma ? launch_rows<128, true>(a, n_items, rows_max, stream) : launch_rows<128, false>(a, n_items, rows_max, stream);
}

// How many clusters of `cluster` blocks of the decode kernel (TMA loads, head_dim hd; the ring of six stages if `deep`)
// the device runs at once: what a caller needs to choose a number of key slices whose clusters all fit.  -1: unknown.
template <int HD, bool DEEP> int max_clusters_of(int cluster) {
    constexpr int WR = 1, WK = 4, MR = 1, RMAX = 16;
    constexpr int STAGES = DEEP ? 6 : 3;
    const size_t stages = 2 * (size_t)STAGES * BN * HD * 2 + (size_t)RMAX * HD * 2 + 16 * STAGES + 16;
    const size_t merge = ((size_t)WK * RMAX * HD + (size_t)WK * RMAX * 2 + (size_t)RMAX * HD + (size_t)RMAX * 2) * sizeof(float);
    const size_t smem = (stages > merge ? stages : merge) + 1024;
    auto kern = attn_mma_kernel<HD, WR, WK, MR, true, DEEP>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)cluster * 64, 1);
    cfg.blockDim = dim3(WR * WK * 32 + 32);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return n;
}
VCB_API int vcb_attn_mma_max_clusters(int hd, int cluster, int deep) {
    if (cluster < 1 || cluster > 8 || (hd != 64 && hd != 128)) return -1;
    if (hd == 64) return deep ? max_clusters_of<64, true>(cluster) : max_clusters_of<64, false>(cluster);
    return deep ? max_clusters_of<128, true>(cluster) : max_clusters_of<128, false>(cluster);
}

// Whether vcb_attn_mma_decode_fused takes these sizes: the page sizes whose pages the TMA loader brings in whole.
VCB_API int vcb_attn_mma_fused_supported(int dtype, int hd, int page_size) {
    return dtype == VCB_BF16 && (hd == 64 || hd == 128) && (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64);
}

// Decoded tokens straight from the stacked q, k, v projection (see FusedQkv): items of one token each (rows_max 16).
// qkv: [slices][tokens][(nh + 2 nkv) * hd] float; gains bfloat16 or float (gain_dtype), may be null with use_norm 0.
VCB_API int vcb_attn_mma_decode_fused(const float* qkv, int slices, long long slice_stride, const void* q_gain,
                                      const void* k_gain, int gain_dtype, int use_norm, float eps, const float* cos_sin,
                                      int max_pos, const int* slot_map, void* out, void* pages,
                                      long long page_stride, const int* block_table, const int* table_row, int max_blocks,
                                      const int* q_start, const int* q_len, const int* ctx_len, const int* items, int n_items,
                                      float* part_o, float* part_ml, int* slice_counters, const int* dec_rows, int nh, int nkv,
                                      int hd, int page_size, int num_pages, int window, float scale, int* status,
                                      int cluster, cudaStream_t stream) {
    if (n_items == 0) return 0;
    VCB_CHECK_ARG(nh > 0 && nkv > 0 && nh % nkv == 0, "attn_mma_decode_fused: %d query heads are not a multiple of %d KV heads", nh, nkv);
    VCB_CHECK_ARG(vcb_attn_mma_fused_supported(VCB_BF16, hd, page_size), "attn_mma_decode_fused: head_dim %d with pages of %d tokens is not supported", hd, page_size);
    VCB_CHECK_ARG(((uintptr_t)pages % 16 == 0) && page_stride == (long long)2 * nkv * page_size * hd,
                  "attn_mma_decode_fused: the pages of a layer must be contiguous and 16-byte aligned");
    VCB_CHECK_ARG(qkv != nullptr && slices >= 1 && cos_sin != nullptr && slot_map != nullptr && status != nullptr,
                  "attn_mma_decode_fused: missing operand");
    VCB_CHECK_ARG(!use_norm || (q_gain != nullptr && k_gain != nullptr), "attn_mma_decode_fused: the per-head norms need their gains");
    VCB_CHECK_ARG(window >= 0, "attn_mma_decode_fused: bad window %d", window);
    AttnArgs a{nullptr, (__nv_bfloat16*)out, (const __nv_bfloat16*)pages, page_stride, block_table, table_row, max_blocks,
               q_start, q_len, ctx_len, items, part_o, part_ml, slice_counters, dec_rows, nh, nkv, page_size, num_pages, window,
               scale, status,
               FusedQkv{qkv, slices, slice_stride, q_gain, k_gain, gain_dtype, use_norm, eps, cos_sin, max_pos,
                        slot_map, (__nv_bfloat16*)pages},
               cluster};
    return hd == 64 ? launch<64, 1, 4, 1, true>(a, n_items, stream) : launch<128, 1, 4, 1, true>(a, n_items, stream);
}
