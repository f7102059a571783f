// Decode attention for steps of many single tokens (bfloat16, head_dim 64 or 128, pages of 8 to 64 tokens): the
// same math as attention_mma.cu's decode form -- scores (q.k)/sqrt(head_dim) over the keys in (pos - window, pos],
// streaming softmax in 32-bit, sum_j w_j v_j (src/model.cpp:1000-1052 of the reference) -- on persistent blocks.
//
// attention_mma.cu gives every (token, KV head, key slice) a block of its own.  Over a few long contexts that is
// right; over hundreds of short ones each block lives for one round trip to memory (its lengths, its block table,
// its pages, its queries, each behind the other) and the SMs wait more than they stream: 44 % of the copy bandwidth
// for 256 requests of 128 keys.  Here a block walks (token, KV head) pairs, blockIdx.x, + gridDim.x, ..., and its
// loading warp runs ahead of the four multiplying warps across the pairs: it reads what describes the next 32 pairs
// (one lane a pair: lengths, the block-table row, the first page ids) while the present ones are streamed, and keeps
// the ring of K and V tiles full from one pair into the next, the pair's query rows in a ring of their own.  Tiles
// that hold only keys of earlier steps are asked for before the wait for the kernel that writes this step's.  The multiplying warps split each tile's 64 keys four ways, as in attention_mma.cu, and merge their
// partial results through shared memory once per pair.  No key slices: this form is for launches with more pairs
// than blocks.
//
// Every mbarrier wait is bounded by the clock and reports through the status word; page ids outside the pool are
// reported and replaced by page 0.
#include "common.cuh"
#include "mbarrier.cuh"
#include "kv_tensor_map.h"

#include <cuda.h>
#include <math_constants.h>

namespace {

constexpr int BN = 64;          // keys per tile
constexpr int ITEM_INTS = 6;    // entry, q0, nq, slice, nslices, decode index (as in attention_mma.cu)
constexpr int NW = 4;           // multiplying warps: each takes 16 keys of a tile
constexpr int KW = BN / NW;
constexpr int NS = KW / 8;
constexpr int BATCH = 32;       // pairs described at a time, one per lane of the loading warp
constexpr int META_INTS = 16;   // per pair: see enum Meta; then the first META_PAGES page ids of its key range
constexpr int META_PAGES = 8;
enum Meta { M_TILES = 0, M_TABLE, M_PB_LO, M_PB_HI, M_K_BEGIN, M_K_END, M_ROW, M_KVH, M_HEAD };
constexpr int AHEAD = 4;        // tiles whose page ids are read ahead beyond those the description holds

struct StreamArgs {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    const int* block_table;
    const int* table_row;
    int max_blocks;
    const int* q_len;
    const int* ctx_len;
    const int* items;       // [n_dec][ITEM_INTS]: entry and decode index are used
    const int* dec_rows;    // [n_dec]: the token's row of q and out
    int n_dec, nh, nkv, page_size, num_pages, window, stages;
    float scale;
    int* status;
};

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
// Byte offset of 16-byte chunk c of key `key` in a K or V tile as one TMA box per page leaves it:
// [groups of 8 keys][head_dim/64 halves][8 rows][128 bytes], each 1 KB piece swizzled by the row (see attention_mma.cu).
template <int HALVES> __device__ __forceinline__ int swz_kv(int key, int c) {
    return (key >> 3) * (HALVES * 1024) + (c >> 3) * 1024 + (key & 7) * 128 + (((c & 7) ^ (key & 7)) << 4);
}
__device__ __forceinline__ void tma_load_groups(uint32_t dst, const CUtensorMap* map, uint32_t bar, int group) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %3, %3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(0), "r"(group) : "memory");
}
// `bytes` (a multiple of 16) from global to shared memory, reported to the barrier
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

template <int HD>
__global__ __launch_bounds__(NW * 32 + 32) void attn_stream_kernel(const __grid_constant__ CUtensorMap kv_map, StreamArgs a) {
    constexpr int CH = HD / 8;          // 16-byte chunks per row
    constexpr int ROWB = HD * 2;
    constexpr int QROWB = ROWB + 16;    // query rows are 16 bytes apart from a multiple of 128: ldmatrix without conflicts
    constexpr int ND = HD / 8;
    constexpr int TILE_BYTES = BN * ROWB;
    constexpr float LOG2E = 1.4426950408889634f;
    const int STAGES = a.stages;
    const int g = a.nh / a.nkv;         // query heads of a KV head: the rows of a pair (at most 16)

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base_u32 = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzle atoms are 1024-byte aligned
    uint8_t* smem = smem_raw + (base_u32 - smem_u32(smem_raw));
    uint8_t* k_s = smem;                                   // STAGES tiles
    uint8_t* v_s = k_s + STAGES * TILE_BYTES;              // STAGES tiles
    uint8_t* q_s = v_s + STAGES * TILE_BYTES;              // STAGES x g query rows (slot: the pair's number modulo STAGES), then one row of zeros
    uint8_t* zero_s = q_s + STAGES * g * QROWB;
    float* o_s = reinterpret_cast<float*>(zero_s + QROWB);  // [NW][g][HD]: the warps' partial results of a pair
    float* ml_s = o_s + NW * g * HD;                       // [NW][g][2]
    int* meta_s = reinterpret_cast<int*>(ml_s + NW * g * 2);   // 2 x BATCH descriptions
    uint8_t* bar_s = reinterpret_cast<uint8_t*>(meta_s + 2 * BATCH * META_INTS);
    auto full_bar = [&](int st) { return smem_u32(bar_s) + 8u * st; };
    auto empty_bar = [&](int st) { return smem_u32(bar_s) + 8u * (STAGES + st); };
    auto meta_full = [&](int p) { return smem_u32(bar_s) + 8u * (2 * STAGES + p); };
    auto meta_empty = [&](int p) { return smem_u32(bar_s) + 8u * (2 * STAGES + 2 + p); };
    const uint32_t merge_full = smem_u32(bar_s) + 8u * (2 * STAGES + 4);    // the four warps' partial results are written
    const uint32_t merge_empty = smem_u32(bar_s) + 8u * (2 * STAGES + 5);   // and read
    auto q_bar = [&](int slot) { return smem_u32(bar_s) + 8u * (2 * STAGES + 6 + slot); };   // a pair's query rows are there
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_s + 8 * (3 * STAGES + 6));

    pdl_trigger();
    tl_mark(VCB_TL_ATTN_DEC, 0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ps = a.page_size;
    const int pages_per_tile = BN / ps;
    const int pre_tiles = META_PAGES / pages_per_tile;     // tiles whose page ids the description holds
    const long long pairs = (long long)a.n_dec * a.nkv;
    const int mine = (long long)blockIdx.x < pairs ? (int)((pairs - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
    const int batches = (mine + BATCH - 1) / BATCH;

    if (tid == 0) {
        for (int st = 0; st < STAGES; ++st) {
            mbar_init(full_bar(st), 1);
            mbar_init(empty_bar(st), NW);      // one arrival per multiplying warp
            mbar_init(q_bar(st), 1);
        }
        for (int p = 0; p < 2; ++p) {
            mbar_init(meta_full(p), 1);
            mbar_init(meta_empty(p), NW);
        }
        mbar_init(merge_full, NW);
        mbar_init(merge_empty, NW);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    for (int i = tid; i < QROWB / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(zero_s)[i] = 0u;
    __syncthreads();

    if (warp == NW) {
        // ================= the loading warp =================
        // describes pair k = BATCH * j + lane of this block (lengths, table row, page range, first page ids)
        auto describe = [&](int j) {
            int* m = meta_s + ((j & 1) * BATCH + lane) * META_INTS;
            const int k = j * BATCH + lane;
            int n_tiles = 0;
            if (k < mine) {
                const long long w = (long long)blockIdx.x + (long long)k * gridDim.x;
                const int n = (int)(w / a.nkv), kvh = (int)(w % a.nkv);
                const int e = a.items[(size_t)n * ITEM_INTS];
                const int qlen = a.q_len[e], ctx = a.ctx_len[e];
                if (qlen == 1 && ctx > 0) {
                    const int pos = ctx - 1;
                    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
                    const int pb_lo = lo / ps, pb_hi = (ctx + ps - 1) / ps;
                    const int table = (a.table_row ? a.table_row[e] : e) * a.max_blocks;
                    n_tiles = (ctx - pb_lo * ps + BN - 1) / BN;
                    m[M_TABLE] = table;
                    m[M_PB_LO] = pb_lo;
                    m[M_PB_HI] = pb_hi;
                    m[M_K_BEGIN] = lo;
                    m[M_K_END] = ctx;
                    m[M_ROW] = a.dec_rows[n];
                    m[M_KVH] = kvh;
                    int pg[META_PAGES];
#pragma unroll
                    for (int i = 0; i < META_PAGES; ++i) pg[i] = pb_lo + i < pb_hi ? a.block_table[(size_t)table + pb_lo + i] : -1;
#pragma unroll
                    for (int i = 0; i < META_PAGES; ++i) m[M_HEAD + i] = pg[i];
                } else if (qlen > 1) {
                    atomicOr(a.status, VCB_STATUS_BAD_ITEM);    // this kernel takes single tokens only
                }
            }
            m[M_TILES] = n_tiles;
        };
        bool ok = true;
        if (batches > 0) {
            describe(0);     // what describes the work is in place before the step's first kernel starts
            __syncwarp();
            if (lane == 0) mbar_arrive(meta_full(0));
        }
        const int my_pg = lane >> 1, my_v = lane & 1;
        // asks for the K and V pages of tile t of the pair described by m into stage st; `page`: this lane's page id
        auto issue_kv = [&](const int* m, int t, int st, int page) {
            const int pb0 = m[M_PB_LO] + t * pages_per_tile;
            const int np = min(pages_per_tile, m[M_PB_HI] - pb0);
            if (lane == 0) mbar_expect_tx(full_bar(st), (uint32_t)(np * ps * ROWB * 2));
            __syncwarp();
            if (my_pg < np) {
                if (page < 0 || page >= a.num_pages) {
                    atomicOr(a.status, VCB_STATUS_BAD_PAGE);
                    page = 0;   // keep the byte count whole; the status word reports the fault
                }
                const int groups_page = ps / 8;
                const int group = (page * 2 * a.nkv + m[M_KVH]) * groups_page + (my_v ? a.nkv * groups_page : 0);
                const uint32_t dst = smem_u32((my_v ? v_s : k_s) + st * TILE_BYTES) + my_pg * ps * ROWB;
                tma_load_groups(dst, &kv_map, full_bar(st), group);
            }
        };
        // Before the wait: the first tiles of the first batch as far as they hold keys of earlier steps only (their
        // page ids are in the descriptions), a ring's worth at most.
        int early = 0;
        for (int i = 0; i < min(BATCH, mine) && early < STAGES; ++i) {
            const int* m = meta_s + i * META_INTS;
            const int n_tiles = m[M_TILES];
            bool stop = false;
            for (int t = 0; t < n_tiles && early < STAGES; ++t) {
                const int end = min(m[M_PB_HI], m[M_PB_LO] + (t + 1) * pages_per_tile) * ps;
                if (t >= pre_tiles || end > m[M_K_END] - 1) { stop = true; break; }
                issue_kv(m, t, early, my_pg < pages_per_tile ? m[M_HEAD + t * pages_per_tile + my_pg] : -1);
                ++early;
            }
            if (stop) break;
        }
        pdl_wait();          // the queries and the newest keys come from the kernel before this one
        tl_mark(VCB_TL_ATTN_DEC, 1);
        int it = 0, armed = early, pseq = 0;      // tiles and pairs (with keys) of this block so far
        for (int j = 0; j < batches && ok; ++j) {
            const int in_batch = min(BATCH, mine - j * BATCH);
            for (int i = 0; i < in_batch && ok; ++i) {
                if (i == BATCH / 4 && j + 1 < batches) {
                    // the next 32 pairs, a quarter into this batch: the multiplying warps are through with the batch
                    // before this one (they are a ring of tiles behind), whose place the descriptions take
                    if (lane == 0) ok = mbar_wait(meta_empty((j + 1) & 1), ((((j + 1) >> 1) & 1) ^ 1u), abort_flag, a.status);
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (!ok) break;
                    describe(j + 1);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(meta_full((j + 1) & 1));
                }
                const int* m = meta_s + ((j & 1) * BATCH + i) * META_INTS;
                const int n_tiles = m[M_TILES];
                if (n_tiles == 0) continue;
                const int table = m[M_TABLE], pb_lo = m[M_PB_LO], pb_hi = m[M_PB_HI], kvh = m[M_KVH];
                const int* bt = a.block_table + (size_t)table;
                auto page_of = [&](int t) {
                    const int pb = pb_lo + t * pages_per_tile + my_pg;
                    return (t < n_tiles && my_pg < pages_per_tile && pb < pb_hi) ? bt[pb] : -1;
                };
                int ahead_page[AHEAD];
#pragma unroll
                for (int k = 0; k < AHEAD; ++k) ahead_page[k] = n_tiles > pre_tiles ? page_of(pre_tiles + k) : -1;
                for (int t = 0; t < n_tiles; ++t, ++it) {
                    const int st = it % STAGES;
                    if (it >= early) {      // (the tiles asked for before the wait are on their way)
                        if (lane == 0) ok = mbar_wait(empty_bar(st), ((it / STAGES) & 1) ^ 1u, abort_flag, a.status);
                        ok = __shfl_sync(0xffffffffu, ok, 0);
                        if (!ok) break;
                        int page;
                        if (t < pre_tiles) {
                            page = my_pg < pages_per_tile ? m[M_HEAD + t * pages_per_tile + my_pg] : -1;
                        } else {
                            page = ahead_page[0];
#pragma unroll
                            for (int k = 0; k + 1 < AHEAD; ++k) ahead_page[k] = ahead_page[k + 1];
                            ahead_page[AHEAD - 1] = page_of(t + AHEAD);
                        }
                        issue_kv(m, t, st, page);
                        armed = it + 1;
                    }
                    if (t == 0) {
                        // The pair's query rows, into the slot of the pair's number: the pair that had it before is
                        // STAGES pairs back, so its first tile, before whose release its rows were read, is at least
                        // STAGES tiles back and released, or this tile's stage would not be free.
                        const int slot = pseq % STAGES;
                        if (lane == 0) mbar_expect_tx(q_bar(slot), (uint32_t)(g * ROWB));
                        __syncwarp();
                        if (lane < g) {
                            const __nv_bfloat16* src = a.q + ((size_t)m[M_ROW] * a.nh + (size_t)kvh * g + lane) * HD;
                            bulk_load(smem_u32(q_s + (slot * g + lane) * QROWB), src, ROWB, q_bar(slot));
                        }
                        ++pseq;
                    }
                }
            }
        }
        if (lane == 0 && *abort_flag) {   // let copies in flight land before the block goes away
            for (int i = max(0, armed - STAGES); i < armed; ++i) {
                const long long t0 = clock64();
                while (!mbar_try(full_bar(i % STAGES), (i / STAGES) & 1) && clock64() - t0 < VCB_WAIT_CLOCKS) {}
            }
            for (int i = max(0, pseq - STAGES); i < pseq; ++i) {
                const long long t0 = clock64();
                while (!mbar_try(q_bar(i % STAGES), (i / STAGES) & 1) && clock64() - t0 < VCB_WAIT_CLOCKS) {}
            }
        }
    } else {
        // ================= the multiplying warps =================
        const int wk = warp;
        int it = 0, done = 0;       // tiles and pairs (with keys) of this block so far
        bool ok = true;
        for (int j = 0; j < batches && ok; ++j) {
            ok = mbar_wait(meta_full(j & 1), (j >> 1) & 1, abort_flag, a.status);
            if (!ok) break;
            const int in_batch = min(BATCH, mine - j * BATCH);
            for (int i = 0; i < in_batch && ok; ++i) {
                const int* m = meta_s + ((j & 1) * BATCH + i) * META_INTS;
                const int n_tiles = m[M_TILES];
                if (n_tiles == 0) continue;
                const int k_begin = m[M_K_BEGIN], k_end = m[M_K_END], t_first = m[M_PB_LO] * ps;
                float o[ND][4];
#pragma unroll
                for (int d = 0; d < ND; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
                float m_a = -CUDART_INF_F, m_b = -CUDART_INF_F, l_a = 0.f, l_b = 0.f;   // rows lane/4 and lane/4 + 8
                const int r_a = lane >> 2;
                const bool ok_a = r_a < g, ok_b = r_a + 8 < g;
                uint32_t qf[HD / 16][4];
                for (int t = 0; t < n_tiles; ++t, ++it) {
                    const int st = it % STAGES;
                    ok = mbar_wait(full_bar(st), (it / STAGES) & 1, abort_flag, a.status);
                    if (!ok) break;
                    const int t0 = t_first + t * BN;
                    if (t == 0) {
                        // query fragments stay in registers for the pair; rows beyond its heads read the row of zeros
                        const int slot = done % STAGES;
                        ok = mbar_wait(q_bar(slot), (done / STAGES) & 1, abort_flag, a.status);
                        if (!ok) break;
                        const int r = lane & 15;
                        const uint32_t row = r < g ? smem_u32(q_s + (slot * g + r) * QROWB) : smem_u32(zero_s);
#pragma unroll
                        for (int ks = 0; ks < HD / 16; ++ks) ldmatrix_x4(qf[ks], row + (r < g ? (ks * 2 + (lane >> 4)) * 16 : 0));
                    }
                    if (t0 + BN > k_end) {
                        // the last page may hold slots beyond the sequence (and rows of pages not loaded are stale):
                        // their V must be finite, because a zero weight times NaN is NaN.  Each warp clears what it reads.
                        for (int idx = lane; idx < KW * CH; idx += 32) {
                            const int kk = wk * KW + idx / CH, c = idx % CH;
                            if (t0 + kk >= k_end) *reinterpret_cast<uint4*>(v_s + st * TILE_BYTES + swz_kv<HD / 64>(kk, c)) = make_uint4(0, 0, 0, 0);
                        }
                        __syncwarp();
                    }
                    const uint8_t* kt = k_s + st * TILE_BYTES;
                    const uint8_t* vt = v_s + st * TILE_BYTES;
                    const int key0 = t0 + wk * KW;
                    // S = Q K^T
                    float s[NS][4];
#pragma unroll
                    for (int n = 0; n < NS; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ++ks) {
                        uint32_t b[4];
                        const int mi = lane >> 3;
                        const int krow = wk * KW + (mi >> 1) * 8 + (lane & 7);
                        ldmatrix_x4(b, smem_u32(kt + swz_kv<HD / 64>(krow, ks * 2 + (mi & 1))));
                        mma_16816(s[0], qf[ks], b[0], b[1]);
                        mma_16816(s[1], qf[ks], b[2], b[3]);
                    }
                    // mask only where the tile touches an edge of the key range
                    const bool inner = key0 >= k_begin && key0 + KW <= k_end;
                    float mx_a = -CUDART_INF_F, mx_b = -CUDART_INF_F;
#pragma unroll
                    for (int n = 0; n < NS; ++n) {
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const int kidx = key0 + n * 8 + 2 * (lane & 3) + c;
                            const bool in = inner || (kidx >= k_begin && kidx < k_end);
                            s[n][c] = (ok_a && in) ? s[n][c] * a.scale : -CUDART_INF_F;
                            s[n][2 + c] = (ok_b && in) ? s[n][2 + c] * a.scale : -CUDART_INF_F;
                            mx_a = fmaxf(mx_a, s[n][c]);
                            mx_b = fmaxf(mx_b, s[n][2 + c]);
                        }
                    }
                    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
                    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
                    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
                    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
                    const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
                    const float use_a = mn_a == -CUDART_INF_F ? 0.f : mn_a, use_b = mn_b == -CUDART_INF_F ? 0.f : mn_b;
                    const bool moved = mn_a != m_a || mn_b != m_b;
                    const float al_a = exp2f((m_a - use_a) * LOG2E), al_b = exp2f((m_b - use_b) * LOG2E);
                    m_a = mn_a;
                    m_b = mn_b;
                    float sum_a = 0.f, sum_b = 0.f;
                    const float off_a = use_a * LOG2E, off_b = use_b * LOG2E;
#pragma unroll
                    for (int n = 0; n < NS; ++n) {
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            s[n][c] = exp2f(fmaf(s[n][c], LOG2E, -off_a));
                            s[n][2 + c] = exp2f(fmaf(s[n][2 + c], LOG2E, -off_b));
                            sum_a += s[n][c];
                            sum_b += s[n][2 + c];
                        }
                    }
                    l_a = l_a * al_a + sum_a;
                    l_b = l_b * al_b + sum_b;
                    if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
                        for (int d = 0; d < ND; ++d) {
                            o[d][0] *= al_a; o[d][1] *= al_a; o[d][2] *= al_b; o[d][3] *= al_b;
                        }
                    }
                    uint32_t pa[4];
                    pa[0] = pack_bf16(s[0][0], s[0][1]);
                    pa[1] = pack_bf16(s[0][2], s[0][3]);
                    pa[2] = pack_bf16(s[1][0], s[1][1]);
                    pa[3] = pack_bf16(s[1][2], s[1][3]);
                    // O += P V
#pragma unroll
                    for (int dp = 0; dp < HD / 16; ++dp) {
                        uint32_t b[4];
                        const int mi = lane >> 3;
                        const int vrow = wk * KW + (mi & 1) * 8 + (lane & 7);
                        ldmatrix_x4_trans(b, smem_u32(vt + swz_kv<HD / 64>(vrow, dp * 2 + (mi >> 1))));
                        mma_16816(o[2 * dp], pa, b[0], b[1]);
                        mma_16816(o[2 * dp + 1], pa, b[2], b[3]);
                    }
                    if (t0 + BN > k_end) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the clearing stores above
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_bar(st));   // this warp is done with the stage
                }
                if (!ok) break;
                // ---- the four warps' partial results -> shared memory, merged, written ----
                float* po = o_s;      // [warp][row][HD] partial outputs, [warp][row][2] their maxima and sums
                float* pml = ml_s;
                // every warp has read the pair before (a wait that is over long since: that pair's tiles lie between)
                ok = mbar_wait(merge_empty, ((uint32_t)done & 1u) ^ 1u, abort_flag, a.status);
                if (!ok) break;
                l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
                l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
                l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
                l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
#pragma unroll
                for (int d = 0; d < ND; ++d) {
                    const int col = d * 8 + 2 * (lane & 3);
                    if (ok_a) *reinterpret_cast<float2*>(po + (size_t)(wk * g + r_a) * HD + col) = make_float2(o[d][0], o[d][1]);
                    if (ok_b) *reinterpret_cast<float2*>(po + (size_t)(wk * g + r_a + 8) * HD + col) = make_float2(o[d][2], o[d][3]);
                }
                if ((lane & 3) == 0) {
                    if (ok_a) { pml[(wk * g + r_a) * 2] = m_a; pml[(wk * g + r_a) * 2 + 1] = l_a; }
                    if (ok_b) { pml[(wk * g + r_a + 8) * 2] = m_b; pml[(wk * g + r_a + 8) * 2 + 1] = l_b; }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(merge_full);
                ok = mbar_wait(merge_full, (uint32_t)done & 1u, abort_flag, a.status);
                if (!ok) break;
                const int out_row = m[M_ROW], head0 = m[M_KVH] * g;
                for (int idx = tid; idx < g * (HD / 2); idx += NW * 32) {
                    const int r = idx / (HD / 2), d = (idx % (HD / 2)) * 2;
                    float mm = -CUDART_INF_F;
#pragma unroll
                    for (int w = 0; w < NW; ++w) mm = fmaxf(mm, pml[(w * g + r) * 2]);
                    float l = 0.f, o0 = 0.f, o1 = 0.f;
#pragma unroll
                    for (int w = 0; w < NW; ++w) {
                        const float mw = pml[(w * g + r) * 2];
                        if (mw == -CUDART_INF_F) continue;
                        const float f = exp2f((mw - mm) * LOG2E);
                        l += pml[(w * g + r) * 2 + 1] * f;
                        const float2 ov = *reinterpret_cast<const float2*>(po + (size_t)(w * g + r) * HD + d);
                        o0 += ov.x * f;
                        o1 += ov.y * f;
                    }
                    const float inv = l > 0.f ? 1.f / l : 0.f;
                    if (out_row >= 0)
                        *reinterpret_cast<__nv_bfloat162*>(a.out + ((size_t)out_row * a.nh + head0 + r) * HD + d) =
                            __floats2bfloat162_rn(o0 * inv, o1 * inv);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(merge_empty);
                ++done;
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(meta_empty(j & 1));     // this warp has read the batch's descriptions
        }
    }
    tl_mark(VCB_TL_ATTN_DEC, 2);
}

size_t stream_smem(int hd, int g, int stages) {
    const size_t tile = (size_t)BN * hd * 2, qrow = (size_t)hd * 2 + 16;
    return 2 * stages * tile + (size_t)stages * g * qrow + qrow + (size_t)NW * g * (hd + 2) * 4 +
           2 * (size_t)BATCH * META_INTS * 4 + 8 * (3 * (size_t)stages + 6) + 16 + 1024;
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

template <int HD>
int launch(const StreamArgs& a0, const void* pages, int blocks, cudaStream_t stream) {
    StreamArgs a = a0;
    const int g = a.nh / a.nkv;
    // two blocks an SM with rings of three stages where they fit (head groups of up to eight rows), else one with five
    int per_sm = 2;
    a.stages = 3;
    if (2 * (stream_smem(HD, g, 3) + 1024) > 228 * 1024) {
        per_sm = 1;
        a.stages = 5;
    }
    const size_t smem = stream_smem(HD, g, a.stages);
    CUtensorMap map;
    const long long rows = (long long)a.num_pages * 2 * a.nkv * a.page_size;
    if (!vcb_kv_tensor_map(pages, rows, HD, a.page_size, &map, true)) return -3;
    auto kern = attn_stream_kernel<HD>;
    static size_t opted = 0;
    if (smem > opted) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            vcb_set_error("attn_stream: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
            return -2;
        }
        opted = smem;
    }
    const long long pairs = (long long)a.n_dec * a.nkv;
    const long long most = blocks > 0 ? blocks : (long long)per_sm * sm_count();
    launch_pdl(kern, dim3((unsigned)(pairs < most ? pairs : most)), dim3(NW * 32 + 32), smem, stream, map, a);
    VCB_CHECK_LAUNCH("attn_stream");
    return 0;
}

}  // namespace

VCB_TIMELINE_UNIT(attn_stream)

// Whether vcb_attn_stream takes these sizes.
VCB_API int vcb_attn_stream_supported(int dtype, int hd, int page_size, int nh, int nkv) {
    return dtype == VCB_BF16 && (hd == 64 || hd == 128) && (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64) &&
           nkv > 0 && nh % nkv == 0 && nh / nkv <= 16;
}

// Single decoded tokens, every key of a token by one block: items [n_dec][6] as for vcb_attn_mma with one slice
// (entry, 0, 1, 0, 1, decode index); dec_rows[n]: the token's row of q [rows, nh * hd] and out.  Entries whose
// q_len is 0 are skipped.  blocks: 0, or the number of blocks to run on (tests, measurements).
VCB_API int vcb_attn_stream(const void* q, void* out, const void* pages, long long page_stride, const int* block_table,
                            const int* table_row, int max_blocks, const int* q_len, const int* ctx_len, const int* items,
                            int n_dec, const int* dec_rows, int nh, int nkv, int hd, int page_size, int num_pages,
                            int window, float scale, int* status, int blocks, cudaStream_t stream) {
    if (n_dec == 0) return 0;
    VCB_CHECK_ARG(vcb_attn_stream_supported(VCB_BF16, hd, page_size, nh, nkv),
                  "attn_stream: head_dim %d, pages of %d tokens, %d query heads on %d KV heads are not supported", hd, page_size, nh, nkv);
    VCB_CHECK_ARG(((uintptr_t)pages % 16 == 0) && page_stride == (long long)2 * nkv * page_size * hd,
                  "attn_stream: the pages of a layer must be contiguous and 16-byte aligned");
    VCB_CHECK_ARG((uintptr_t)q % 16 == 0 && dec_rows != nullptr && status != nullptr && window >= 0, "attn_stream: bad operand");
    StreamArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, block_table, table_row, max_blocks, q_len, ctx_len, items, dec_rows,
                 n_dec, nh, nkv, page_size, num_pages, window, 3, scale, status};
    return hd == 64 ? launch<64>(a, pages, blocks, stream) : launch<128>(a, pages, blocks, stream);
}
