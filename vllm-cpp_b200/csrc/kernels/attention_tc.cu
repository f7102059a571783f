// bfloat16 attention of prompt portions over the paged cache on the fifth-generation tensor cores
// (tcgen05.mma with accumulators in TMEM), head_dim 64 or 128, pages of 8, 16, 32 or 64 tokens.
//
// Same contract, work items and math as attention_mma.cu (one item = an entry and a run of its query tokens;
// rows = tokens x the query heads that share a KV head, at most 128; scores (q.k)/sqrt(head_dim) in 32-bit, keys
// in (pos - window, pos], streaming softmax, sum_j w_j v_j: src/model.cpp:1000-1052 of the reference).  What
// differs is where the products run.  Per block of 128 rows and per tile of 64 keys:
//
//   S = Q . K^T     one MMA chain, M = 128 rows (TMEM lanes), N = 64 keys, K = head_dim; Q and the K tile are
//                   K-major operands in 128-byte-swizzled shared memory, S lands in TMEM (two buffers);
//   softmax         four warps, one thread per row (= per TMEM lane): tcgen05.ld of the row's 64 scores, mask,
//                   running maximum and sum in 32-bit, P = exp2(s - m) rounded to bfloat16 and written back over the
//                   row's scores in TMEM (tcgen05.st, two weights a column), where the next product reads it as
//                   its A operand;
//   O += P . V      M = 128, N = head_dim, K = 64 keys; the V tile is used as it lies in the cache (keys x
//                   head_dim, head_dim contiguous), i.e. as an MN-major B operand; O stays in TMEM over all
//                   tiles.  A row's weights are taken against a reference maximum that is only moved, and O
//                   and the sum rescaled with it (tcgen05.ld, multiply, tcgen05.st), when the row's true maximum
//                   has outgrown it by more than 2^8 -- the weights then stay below 256, exact in the end because
//                   numerator and denominator carry the same reference.
//
// Two blocks share an SM (112 KB of shared memory and 256 TMEM columns each), so one block's softmax overlaps
// the other's products.  K tiles have a ring of three stages and V tiles one of two: a K stage is free again
// as soon as its scores are computed, and the next keys must be asked for two tiles ahead to arrive in time.
// Roles (192 threads): warp 0 issues TMA loads of K and V pages (cp.async.bulk.tensor, 128-byte swizzle; no
// multicast) into a ring of stages; warp 1 allocates TMEM and issues every MMA; warps 2-5 are the softmax rows.
//
// A page comes in with ONE copy, whatever head_dim: the cache is described to the TMA unit as a four-dimensional
// tensor [groups of 8 tokens][halves of head_dim][8 tokens][64 lanes], and a box of a page's groups lands as
// [group][half][8 rows of 128 bytes] -- every 1 KB piece a swizzle atom of 8 rows.  The descriptors of both products
// step from one group of 8 keys to the next by the same stride (halves x 1 KB) and from one half of head_dim to the
// other by 1 KB, so the keys keep their order in a tile whatever the page size.  (One copy per page and half, the
// obvious way, made the copying warp the slowest role of the block: about 100 clocks a copy, 16 copies a tile.)
// All hand-offs are mbarriers; every wait is bounded by the clock, and a wait that runs out sets a bit in the
// status word and an abort flag that the other roles see, after which the block frees its TMEM and returns.
#include "common.cuh"
#include "mbarrier.cuh"
#include "kv_tensor_map.h"

#include <cuda.h>
#include <math_constants.h>

namespace {

constexpr int BNK = 64;       // keys per tile
constexpr int ROWS = 128;     // rows per block = TMEM lanes
constexpr int ITEM_INTS = 6;  // entry, q0, nq, slice, nslices, decode index (as in attention_mma.cu)
constexpr int NTHREADS = 192;
// Marks of the roles inside a block in a timeline build (TlRole; the block-wide marks are phases 0 to 2): the
// loading warp asks for a stage, has it, has sent the copies; the thread that issues the products asks for a K tile,
// has it, has issued Q.K^T, has the tile's weights (and values), has issued P.V; the first softmax row asks for a
// tile's scores, has them, has loaded them, has computed its weights, has handed them over.
enum : int { TL_LOAD_ASKS = 10, TL_LOAD_FREE, TL_LOAD_SENT, TL_QK_ASKS = 20, TL_QK_KEYS, TL_QK_ISSUED, TL_PV_WEIGHTS, TL_PV_ISSUED,
             TL_ROW_ASKS = 30, TL_ROW_SCORES, TL_ROW_LOADED, TL_ROW_COMPUTED, TL_ROW_HANDED };
constexpr int UNIT_RING = 8;   // units a block's loader may know of before its slowest role has taken them up

struct TcArgs {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    const int* block_table;
    const int* table_row;
    int max_blocks;
    const int* q_start;
    const int* q_len;
    const int* ctx_len;
    const int* items;
    int nh, nkv, page_size, num_pages, window;
    float scale;
    int* status;
    int n_units;   // items x KV heads x chunks of the query heads that share one
    int* work;     // two counters, zero between launches: units handed out after the first of each block; blocks done
};

// a box of whole groups of 8 tokens, all lanes: coordinates (lane 0, token 0, half 0, group)
__device__ __forceinline__ void tma_load_groups(uint32_t dst, const CUtensorMap* map, uint32_t bar, int group) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %3, %3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(0), "r"(group) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// the same with the A operand in TMEM (lane = row, two bfloat16 of consecutive k per 32-bit column)
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptors (version 1, 128-byte swizzle = layout 2 in bits 61-63; addresses and offsets
// in units of 16 bytes).  K-major tile (rows of 128 bytes along the inner dimension): 8-row groups `group_bytes`
// apart (stride offset, bits 32-45); the leading offset is unused.  MN-major tile (rows of 128 bytes = 64
// elements along M or N, one row per inner index): groups of 8 inner indices `group_bytes` apart (stride offset),
// groups of 64 outer elements `outer_bytes` apart (leading offset, bits 16-29).
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr, uint32_t group_bytes) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(group_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t outer_bytes, uint32_t group_bytes) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(outer_bytes >> 4) << 16) | ((uint64_t)(group_bytes >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: f32 accumulate (bits 4-5 = 1), A and B bfloat16 (bits 7-9, 10-12 = 1),
// A K-major (bit 15 = 0), B K-major or MN-major (bit 16), N / 8 in bits 17-22, M / 16 in bits 24-28.
__host__ __device__ constexpr uint32_t instr_desc(int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(ROWS >> 4) << 24);
}

// Byte offset of 16-byte chunk c of row r in a tile of NROWS rows stored as head_dim/64 blocks of [NROWS][128
// bytes], each row XOR-swizzled by its index: what a 128-byte-swizzled TMA box of 64 lanes produces and what
// the descriptors above describe.
template <int NROWS> __device__ __forceinline__ int swz(int r, int c) {
    return (c >> 3) * (NROWS * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4);
}
// The same for a K or V tile as the page copies lay it out: [groups of 8 keys][halves of head_dim][8 rows][128 bytes].
template <int HALVES> __device__ __forceinline__ int swz_groups(int key, int c) {
    return (key >> 3) * (HALVES * 1024) + (c >> 3) * 1024 + (key & 7) * 128 + (((c & 7) ^ (key & 7)) << 4);
}
// 2^x to 2^-22 relative; -inf gives 0
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// What halves the instructions of a row's softmax: the maximum of three numbers in one instruction, and the
// scaling and the summation on pairs of 32-bit numbers (two results an instruction, each rounded as alone).
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint64_t pair_f32(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpair_f32(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_pair(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add_pair(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// What a block works on: one unit = a work item (an entry and a run of its query tokens) for one KV head and one
// chunk of the query heads that share it.
struct Unit {
    int nq, kvh, head0, gq, R, row0, pos0, pos_last, k_end, pb_lo, pb_hi, t_first, n_tiles, bt_row;
};
constexpr int UNIT_INTS = sizeof(Unit) / sizeof(int);

template <int HD, int KS, int VS>
struct Layout {
    static constexpr int Q_BYTES = ROWS * HD * 2;
    static constexpr int KV_BYTES = BNK * HD * 2;       // one K or V tile
    static constexpr int K_OFF = Q_BYTES;
    static constexpr int V_OFF = K_OFF + KS * KV_BYTES;
    static constexpr int BAR_OFF = V_OFF + VS * KV_BYTES;
    static constexpr int NUM_BARS = 2 * KS + VS + 7;
    static_assert(VS == 2, "a V stage is given back by the barrier of the score buffer its tile used");
    static constexpr int TOTAL = BAR_OFF + NUM_BARS * 8 + 16 + 4 * UNIT_RING * (UNIT_INTS + 2);   // + TMEM address, abort flag, the units to come
    static constexpr uint32_t TMEM_COLS = 256;                  // S, S (64 each; P over the first half of its S), O (head_dim)
    static_assert(2 * BNK + HD <= 256, "TMEM columns");
    static_assert(2 * (TOTAL + 1024) <= 228 * 1024, "two blocks per SM");
};

constexpr float RESCALE_STEP = 8.0f;   // log2 of how far a row's maximum may outgrow its reference

// false: the unit has nothing to do (an item laid out for a longer portion than is there)
__device__ __forceinline__ bool read_unit(const TcArgs& a, int unit, Unit& u) {
    const int g = a.nh / a.nkv;
    const int gq_max = g < ROWS ? g : ROWS;
    const int hchunks = (g + gq_max - 1) / gq_max;
    const int per_item = a.nkv * hchunks;
    const int* item = a.items + (size_t)(unit / per_item) * ITEM_INTS;
    const int e = item[0], q0 = item[1];
    const int qlen = a.q_len[e], ctx = a.ctx_len[e];
    // an item of a captured step is laid out for the largest portion the step serves: fewer tokens may be there
    u.nq = min(item[2], qlen - q0);
    if (qlen <= 0 || ctx <= 0 || u.nq <= 0) return false;
    const int hc = (unit % per_item) % hchunks;
    u.kvh = (unit % per_item) / hchunks;
    u.head0 = u.kvh * g + hc * gq_max;
    u.gq = min(gq_max, g - hc * gq_max);
    u.R = u.nq * u.gq;
    u.row0 = a.q_start[e] + q0;
    u.pos0 = ctx - qlen + q0;
    u.pos_last = u.pos0 + u.nq - 1;
    const int ps = a.page_size;
    const int lo = a.window > 0 ? max(0, u.pos0 - a.window + 1) : 0;
    u.k_end = u.pos_last + 1;
    u.pb_lo = lo / ps;
    u.pb_hi = (u.k_end + ps - 1) / ps;
    u.t_first = u.pb_lo * ps;     // tiles start on a page boundary: whole pages are loaded
    u.n_tiles = (u.k_end - u.t_first + BNK - 1) / BNK;   // >= 1: every query sees itself
    u.bt_row = a.table_row ? a.table_row[e] : e;
    return true;
}

// The grid is two blocks per SM at most, and a block works through several units: first the one of its own index,
// then whichever is next in line when it is through (a counter in global memory that the launch's last block sets
// back).  Units are numbered item by item, the KV heads of an item side by side, and the items come longest first, so
// the long units start at once and the short ones fill the gaps.  (One block per unit, left to the hardware's
// scheduler, kept a third of the SMs with one block or none over the second half of a 2,048-token launch: a new
// block was placed a microsecond and a half after one had left, and not beside a block of the launch's first wave.)
// The block's loader takes the next unit from the counter when the current one has four tiles to go, reads what the
// unit is (its entry's lengths, its rows, its key range) two tiles before the end, and hands all of that to the other
// roles through a small ring in shared memory, so that none of them waits for global memory between two units; it
// cannot be more than the K ring and the two score buffers ahead of them.
// Barrier phases, ring stages and score buffers go on counting from unit to unit, so `t0` below is the number of
// tiles of the units before.
template <int HD, int KS, int VS>
__global__ __launch_bounds__(NTHREADS, 2) void attn_tc_kernel(const __grid_constant__ CUtensorMap kv_map, TcArgs a) {
    using L = Layout<HD, KS, VS>;
    constexpr int CH = HD / 8;          // 16-byte chunks per row of head_dim
    constexpr int ROWB = HD * 2;
    constexpr int HALVES = HD / 64;
    constexpr float LOG2E = 1.4426950408889634f;

    extern __shared__ __align__(1024) uint8_t smem_raw[];   // swizzle atoms are 1024-byte aligned
    uint8_t* gen = smem_raw;
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t bars = base + L::BAR_OFF;
    auto k_full = [&](int s) { return bars + 8u * s; };
    auto k_empty = [&](int s) { return bars + 8u * (KS + s); };
    auto v_full = [&](int s) { return bars + 8u * (2 * KS + s); };
    auto s_full = [&](int b) { return bars + 8u * (2 * KS + VS + b); };
    // Every row has written its weights of a tile.  One barrier per score buffer: a warp may finish tile j + 1
    // before another has finished tile j (its scores are ready early), and with a single barrier its second
    // arrival would be counted into the phase of tile j.  Tile j + 2 cannot begin before that phase is over.
    auto p_ready = [&](int b) { return bars + 8u * (2 * KS + VS + 2 + b); };
    // P . V of a tile has been added to O: tile j completes phase j / 2 of barrier j % 2.  Two barriers, because those
    // who ask (a row that must rescale O, the loader that wants the tile's V stage back) ask by parity and may be a
    // tile behind the products; with one phase per tile on a single barrier an old phase would pass for the new one.
    auto pv_done = [&](int b) { return bars + 8u * (2 * KS + VS + 4 + b); };
    const uint32_t q_ready = bars + 8u * (2 * KS + VS + 6);   // one phase per unit: its queries are in shared memory
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(gen + L::BAR_OFF + L::NUM_BARS * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::BAR_OFF + L::NUM_BARS * 8 + 8);

    tl_mark(VCB_TL_ATTN_TC, 0);
    pdl_trigger();
    pdl_wait();   // the queries and the newest keys come from the kernel before this one
    tl_mark(VCB_TL_ATTN_TC, 1);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (base & 1023u) {                  // the layout below needs the alignment asked for above
        if (tid == 0) atomicOr(a.status, VCB_STATUS_BAD_LAYOUT);
        return;
    }
    const int W = a.window;
    const int ps = a.page_size;
    volatile int* ring_tag = reinterpret_cast<volatile int*>(gen + L::BAR_OFF + L::NUM_BARS * 8 + 16);
    volatile int* ring_index = ring_tag + UNIT_RING;
    volatile int* ring_unit = ring_index + UNIT_RING;   // UNIT_INTS numbers a slot
    // the unit that follows the block's seq-th one, as soon as the loader has made it known; -1: none, or gave up
    auto next_unit = [&](int seq, Unit& w) {
        const int slot = (seq + 1) % UNIT_RING;
        if (ring_tag[slot] != seq + 1) {
            const long long c0 = clock64();
            while (ring_tag[slot] != seq + 1) {
                if (*abort_flag) return -1;
                if (clock64() - c0 > VCB_WAIT_CLOCKS) {
                    *abort_flag = 1;
                    atomicOr(a.status, VCB_STATUS_WAIT_TIMEOUT);
                    return -1;
                }
            }
        }
        __threadfence_block();
        int* wi = reinterpret_cast<int*>(&w);
#pragma unroll
        for (int i = 0; i < UNIT_INTS; ++i) wi[i] = ring_unit[slot * UNIT_INTS + i];
        return (int)ring_index[slot];
    };

    if (tid == 0) {
        for (int s = 0; s < KS; ++s) {
            mbar_init(k_full(s), 1);
            mbar_init(k_empty(s), 1);
        }
        for (int s = 0; s < VS; ++s) mbar_init(v_full(s), 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(s_full(b), 1);
            mbar_init(p_ready(b), ROWS);    // one arrival per row
            mbar_init(pv_done(b), 1);
        }
        mbar_init(q_ready, ROWS);
        *abort_flag = 0;
        for (int i = 0; i < UNIT_RING; ++i) ring_tag[i] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void*)tmem_holder)), "r"(L::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 2 * BNK;   // S, S, O

    if (warp == 0) {
        // ---- TMA producer: one box per page.  Lanes 0-7 copy the pages of a K tile, lanes 8-15 those of a V tile, in
        // one go: the K tile two ahead of the V tile, so that one wait, one round of byte counts and one divergent
        // copy instruction serve both (a call of its own per tile cost this warp 1,000 clocks, of which the copies
        // themselves were a third, and made it the slowest role of the block). ----
        const int pages_per_tile = BNK / ps;
        const int groups_page = ps / 8;
        const int groups_kv = a.nkv * groups_page;   // groups of 8 rows from a page's K to its V
        const bool copies_v = lane >= 8;
        const int pl = lane & 7;
        int armed[2] = {0, 0};
        bool ok = true;
        int t0 = 0;
        TlRole tl;
        tl.begin(VCB_TL_ATTN_TC, 0, lane == 0);
        Unit u;
        int unit = (int)blockIdx.x;
        bool has = read_unit(a, unit, u);
        // this lane's page id for the first tile of the unit (see page_of below)
        auto first_page = [&](const Unit& w) {
            const int pb = w.pb_lo + pl;
            return (lane < 16 && pl < pages_per_tile && pb < w.pb_hi) ? a.block_table[(size_t)w.bt_row * a.max_blocks + pb] : -1;
        };
        int next_page = has ? first_page(u) : -1;
        for (int seq = 0; unit >= 0 && ok; ++seq) {
            // The unit after this one.  Its number is asked for when this one has four tiles to go -- not earlier, or
            // the blocks that start first would take the whole queue while they still have their long first units
            // to do -- and looked up and made known two tiles later, when the counter's answer is there.  Units with
            // nothing to do (an item laid out for a longer portion than is there) are passed over: every unit that the
            // other roles hear of has a tile, and so the K ring keeps this warp from getting further ahead of them
            // than the ring of units is long.
            int raw = 0, after = -1, after_page = -1;
            bool asked = false, known = false;
            Unit un;
            auto ask = [&]() {
                if (lane == 0) raw = atomicAdd(a.work, 1);
                asked = true;
            };
            auto make_known = [&]() {
                if (!asked) ask();
                for (;;) {
                    after = (int)gridDim.x + __shfl_sync(0xffffffffu, raw, 0);
                    if (after >= a.n_units) {
                        after = -1;
                        break;
                    }
                    if (read_unit(a, after, un)) break;
                    if (lane == 0) raw = atomicAdd(a.work, 1);
                }
                if (after >= 0) after_page = first_page(un);
                if (lane == 0) {
                    const int slot = (seq + 1) % UNIT_RING;
                    const int* wi = reinterpret_cast<const int*>(&un);
                    if (after >= 0)
                        for (int i = 0; i < UNIT_INTS; ++i) ring_unit[slot * UNIT_INTS + i] = wi[i];
                    ring_index[slot] = after;
                    __threadfence_block();
                    ring_tag[slot] = seq + 1;
                    if (after < 0 && atomicAdd(a.work + 1, 1) == (int)gridDim.x - 1) {   // the last block of the launch
                        a.work[0] = 0;
                        a.work[1] = 0;
                    }
                }
                known = true;
            };
            if (has) {
                const int* bt = a.block_table + (size_t)u.bt_row * a.max_blocks;
                // This lane's page id for its next tile, read one call ahead: a block-table read that misses L1 costs
                // about as long as a whole tile's products, and it stood between the stage's release and the load.
                // Tiles of one kind are loaded in order, so the next tile is known.
                auto page_of = [&](int it) {
                    const int pb = u.pb_lo + it * pages_per_tile + pl;
                    return (lane < 16 && it < u.n_tiles && pl < pages_per_tile && pb < u.pb_hi) ? bt[pb] : -1;
                };
                // loads K tile itk and V tile itv of the unit (either may be -1: none) once their stages are free;
                // false: give up
                auto load_tiles = [&](int itk, int itv) {
                    const int gk = t0 + itk, gv = t0 + itv;
                    bool free = true;
                    tl.mark(TL_LOAD_ASKS, gv);
                    if (lane == 0) {
                        // a K stage is free when its scores are there; a V stage when the product of the tile that
                        // used it (VS = 2 tiles ago, so on the same score buffer) has been added
                        if (itk >= 0) free = mbar_wait(k_empty(gk % KS), ((gk / KS) & 1) ^ 1u, abort_flag, a.status);
                        if (free && itv >= 0 && gv >= VS) free = mbar_wait(pv_done(gv & 1), (((gv - VS) >> 1) & 1), abort_flag, a.status);
                    }
                    tl.mark(TL_LOAD_FREE, gv);
                    if (!__shfl_sync(0xffffffffu, free, 0)) return false;
                    const int it = copies_v ? itv : itk;
                    const bool mine = lane < 16 && it >= 0;
                    const int st = mine ? (t0 + it) % (copies_v ? VS : KS) : 0;
                    const uint32_t fullb = copies_v ? v_full(st) : k_full(st);
                    const int np = mine ? min(pages_per_tile, u.pb_hi - (u.pb_lo + it * pages_per_tile)) : 0;
                    if (mine && pl == 0) mbar_expect_tx(fullb, (uint32_t)(np * ps * ROWB));
                    __syncwarp();
                    if (pl < np) {   // at most 8 pages a tile: one box a lane
                        int page = next_page;
                        if (page < 0 || page >= a.num_pages) {
                            atomicOr(a.status, VCB_STATUS_BAD_PAGE);
                            page = 0;   // keep the byte count whole; the status word reports the fault
                        }
                        const int group = (page * 2 * a.nkv + u.kvh) * groups_page + (copies_v ? groups_kv : 0);
                        const uint32_t dst = base + (copies_v ? L::V_OFF : L::K_OFF) + st * L::KV_BYTES;
                        tma_load_groups(dst + pl * ps * ROWB, &kv_map, fullb, group);
                    }
                    tl.mark(TL_LOAD_SENT, gv);
                    if (mine) next_page = page_of(it + 1);
                    if (itk >= 0) armed[0] = gk + 1;
                    if (itv >= 0) armed[1] = gv + 1;
                    return true;
                };
                ok = load_tiles(0, -1);
                if (ok && u.n_tiles > 1) ok = load_tiles(1, -1);
                for (int it = 0; it < u.n_tiles && ok; ++it) {
                    if (it == max(0, u.n_tiles - 4)) ask();
                    if (it == max(0, u.n_tiles - 2)) make_known();
                    ok = load_tiles(it + 2 < u.n_tiles ? it + 2 : -1, it);   // keys two tiles ahead of the values
                }
                t0 += u.n_tiles;
            }
            if (!known) make_known();
            unit = after;
            u = un;
            has = after >= 0;
            next_page = after_page;
        }
        if (lane == 0 && *abort_flag) {   // let copies in flight land before the block goes away
            for (int is_v = 0; is_v < 2; ++is_v) {
                const int ns = is_v ? VS : KS;
                for (int i = max(0, armed[is_v] - ns); i < armed[is_v]; ++i) {
                    const long long c0 = clock64();
                    const uint32_t fullb = is_v ? v_full(i % ns) : k_full(i % ns);
                    while (!mbar_try(fullb, (i / ns) & 1) && clock64() - c0 < VCB_WAIT_CLOCKS) {}
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            constexpr uint32_t idesc_qk = instr_desc(BNK, false);
            constexpr uint32_t idesc_pv = instr_desc(HD, true);
            bool ok = true;
            int t0 = 0, done = 0;
            TlRole tl;
            tl.begin(VCB_TL_ATTN_TC, 1, true);
            Unit u;
            int unit = (int)blockIdx.x;
            bool has = read_unit(a, unit, u);
            for (int seq = 0; unit >= 0 && ok; unit = next_unit(seq, u), has = unit >= 0, ++seq) {
                if (!has) continue;
                // The rows have read the output of the unit before and written this unit's queries.
                ok = mbar_wait(q_ready, done & 1, abort_flag, a.status);
                // S[j & 1] = Q . K_j^T once the tile has landed.  The buffer's last user was P . V of tile j - 2, issued
                // before this by the same thread, and the tensor cores work through their queue in order.
                auto issue_qk = [&](int j) {
                    const int gj = t0 + j, st = gj % KS, b = gj & 1;
                    tl.mark(TL_QK_ASKS, gj);
                    if (!mbar_wait(k_full(st), (gj / KS) & 1, abort_flag, a.status)) return false;
                    tl.mark(TL_QK_KEYS, gj);
                    tc_fence_after();
                    const uint32_t qa = base, ka = base + L::K_OFF + st * L::KV_BYTES;
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ++ks) {
                        // 16 lanes of head_dim = 32 bytes along the 128-byte rows; the second 64 lanes are the next block
                        const uint64_t da = desc_k_major(qa + (ks / 4) * (ROWS * 128) + (ks % 4) * 32, 1024);
                        const uint64_t db = desc_k_major(ka + (ks / 4) * 1024 + (ks % 4) * 32, HALVES * 1024);
                        tc_mma(tmem_s + b * BNK, da, db, idesc_qk, ks > 0);
                    }
                    tc_commit(s_full(b));   // the row that sees it first gives the K stage back (a commit less for this thread)
                    tl.mark(TL_QK_ISSUED, gj);
                    return true;
                };
                if (ok) ok = issue_qk(0);
                for (int j = 0; j < u.n_tiles && ok; ++j) {
                    const int gj = t0 + j, st = gj % VS, b = gj & 1;
                    if (j + 1 < u.n_tiles) {
                        ok = issue_qk(j + 1);   // runs while the rows work on tile j
                        if (!ok) break;
                    }
                    // the values first: they have long landed when the rows hand over their weights
                    ok = mbar_wait(v_full(st), (gj / VS) & 1, abort_flag, a.status) && mbar_wait(p_ready(b), (gj >> 1) & 1, abort_flag, a.status);
                    if (!ok) break;
                    tl.mark(TL_PV_WEIGHTS, gj);
                    tc_fence_after();
                    const uint32_t va = base + L::V_OFF + st * L::KV_BYTES;
#pragma unroll
                    for (int ks = 0; ks < BNK / 16; ++ks) {
                        // 16 keys = two groups of 8 rows; the second 64 lanes of head_dim lie 1 KB after the first.
                        // P: 16 keys = 8 columns of the scores' buffer.
                        const uint64_t db = desc_mn_major(va + ks * 2 * (HALVES * 1024), 1024, HALVES * 1024);
                        tc_mma_ts(tmem_o, tmem_s + b * BNK + ks * 8, db, idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
                    }
                    tc_commit(pv_done(b));   // also gives the V stage back
                    tl.mark(TL_PV_ISSUED, gj);
                }
                t0 += u.n_tiles;
                ++done;
            }
        }
    } else {
        // ---- softmax rows: warp w reads TMEM lanes 32 (w % 4) .. + 31 ----
        const int qtr = warp & 3;
        const int r = qtr * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(qtr * 32) << 16;
        const float scale_log2 = a.scale * LOG2E;
        bool ok = true;
        int t0 = 0;
        TlRole tl;
        tl.begin(VCB_TL_ATTN_TC, 2, tid == 64);
        // This row's query of the unit to come is asked for before the row finishes the unit it is on (the loader
        // names the next unit two or three tiles early), so that the load's latency passes behind the last product
        // and the output of the old unit; it goes to shared memory when that is done.
        uint4 qv[CH];
        auto ask_query = [&](const Unit& w, bool there) {   // writes all of qv in any case: what it held is dead
            const bool mine = there && r < w.R;
            const int wq = mine ? r / w.gq : 0, wh = mine ? r % w.gq : 0;
            const __nv_bfloat16* src = a.q + (mine ? ((size_t)(w.row0 + wq) * a.nh + w.head0 + wh) * HD : 0);
#pragma unroll
            for (int c = 0; c < CH; ++c) qv[c] = mine ? *reinterpret_cast<const uint4*>(src + c * 8) : make_uint4(0, 0, 0, 0);
        };
        Unit u;
        int unit = (int)blockIdx.x, seq = 0;
        bool has = read_unit(a, unit, u);
        ask_query(u, has);
        while (unit >= 0 && ok) {
            if (!has) {
                unit = next_unit(seq++, u);
                has = unit >= 0;
                ask_query(u, has);
                continue;
            }
            const bool row_ok = r < u.R;
            const int iq = r / u.gq, ih = r % u.gq;
            const int pos_r = u.pos0 + iq;
            const int lo_r = W > 0 ? max(0, pos_r - W + 1) : 0;

            // The row's query -> shared memory (rows beyond R are zero).  The products of the unit before have all
            // been waited for (its last P . V, and with it everything issued earlier), so nothing reads the old rows.
            {
#pragma unroll
                for (int c = 0; c < CH; ++c) *reinterpret_cast<uint4*>(gen + swz<ROWS>(r, c)) = qv[c];
                fence_async_smem();
                tc_fence_before();   // this row's reads of O for the unit before come before the products to follow
                mbar_arrive(q_ready);
            }

            float m_ref = -CUDART_INF_F, l_run = 0.f;   // reference maximum (scaled, log2 domain) and sum against it

            for (int j = 0; j < u.n_tiles; ++j) {
                const int gj = t0 + j, b = gj & 1, st = gj % VS;
                const int k0 = u.t_first + j * BNK;
                tl.mark(TL_ROW_ASKS, gj);
                ok = mbar_wait(s_full(b), (gj >> 1) & 1, abort_flag, a.status);
                if (!ok) break;
                tl.mark(TL_ROW_SCORES, gj);
                if (tid == 64) mbar_arrive(k_empty(gj % KS));   // the scores are there: the keys of this stage have been read
                tc_fence_after();
                uint32_t sv[4][16];
#pragma unroll
                for (int i = 0; i < 4; ++i) tc_ld16(tmem_s + lane_addr + (uint32_t)(b * BNK + 16 * i), sv[i]);
                tc_wait_ld();
                tl.mark(TL_ROW_LOADED, gj);

                // Scores stay unscaled in sv; only tiles that touch a row's own position or the window's edge mask.
                const bool plain_tile = k0 + BNK - 1 <= u.pos0 && (W == 0 || k0 >= u.pos_last - W + 1);   // uniform over the block
                float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
                if (!plain_tile) {
#pragma unroll
                    for (int c = 0; c < BNK; ++c) {
                        const int kidx = k0 + c;
                        const bool valid = row_ok && kidx >= lo_r && kidx <= pos_r;
                        sv[c / 16][c % 16] = valid ? sv[c / 16][c % 16] : __float_as_uint(-CUDART_INF_F);
                    }
                }
#pragma unroll
                for (int c = 0; c < BNK; c += 2)
                    mx4[(c >> 1) & 3] = max3(mx4[(c >> 1) & 3], __uint_as_float(sv[c / 16][c % 16]), __uint_as_float(sv[c / 16][c % 16 + 1]));
                // the scale is positive: the maximum of the scaled scores is the scaled maximum
                const float m_new = fmaxf(fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2, m_ref);
                // Move the reference when the maximum has outgrown it.  O (in TMEM) holds the sum so far against the
                // old reference: the warp rescales its 32 rows together, rows that keep theirs by a factor of one.
                const bool first_keys = m_ref == -CUDART_INF_F && m_new != -CUDART_INF_F;   // nothing summed yet
                const bool grow = m_ref != -CUDART_INF_F && m_new > m_ref + RESCALE_STEP;
                if (__any_sync(0xffffffffu, grow)) {
                    ok = mbar_wait(pv_done((gj - 1) & 1), ((gj - 1) >> 1) & 1, abort_flag, a.status);   // grow implies j > 0
                    if (!ok) break;
                    tc_fence_after();
                    const float alpha = grow ? exp2f(m_ref - m_new) : 1.f;
#pragma unroll
                    for (int c0 = 0; c0 < HD; c0 += 32) {
                        uint32_t v[2][16];
                        tc_ld16(tmem_o + lane_addr + (uint32_t)c0, v[0]);
                        tc_ld16(tmem_o + lane_addr + (uint32_t)(c0 + 16), v[1]);
                        tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i / 16][i % 16] = __float_as_uint(__uint_as_float(v[i / 16][i % 16]) * alpha);
                        tc_st16(tmem_o + lane_addr + (uint32_t)c0, v[0]);
                        tc_st16(tmem_o + lane_addr + (uint32_t)(c0 + 16), v[1]);
                    }
                    tc_wait_st();
                    tc_fence_before();
                    l_run *= alpha;
                }
                if (grow || first_keys) m_ref = m_new;
                const float m_sub = m_ref == -CUDART_INF_F ? 0.f : m_ref;   // no key yet: every weight is exp2(-inf) = 0

                uint64_t sum4[4] = {0ull, 0ull, 0ull, 0ull};   // four pairs of partial sums, all +0
                uint32_t pk[BNK / 2];
                const uint64_t scale2 = pair_f32(scale_log2, scale_log2), shift2 = pair_f32(-m_sub, -m_sub);
#pragma unroll
                for (int c = 0; c < BNK; c += 2) {
                    float x0, x1;
                    unpair_f32(fma_pair(pair_f32(__uint_as_float(sv[c / 16][c % 16]), __uint_as_float(sv[c / 16][c % 16 + 1])), scale2, shift2), x0, x1);
                    const float p0 = ex2_fast(x0), p1 = ex2_fast(x1);
                    sum4[(c >> 1) & 3] = add_pair(sum4[(c >> 1) & 3], pair_f32(p0, p1));
                    pk[c / 2] = pack_bf16(p0, p1);
                }
                {
                    float lo4, hi4;
                    unpair_f32(add_pair(add_pair(sum4[0], sum4[1]), add_pair(sum4[2], sum4[3])), lo4, hi4);
                    l_run += lo4 + hi4;
                }

                if (k0 + BNK > u.k_end) {
                    // The last page may hold slots beyond the sequence, and rows of pages that were not loaded are
                    // stale: their V must be finite, because a zero weight times NaN is NaN.
                    ok = mbar_wait(v_full(st), (gj / VS) & 1, abort_flag, a.status);
                    if (!ok) break;
                    const int first = u.k_end - k0;
                    for (int idx = r; idx < (BNK - first) * CH; idx += ROWS) {
                        const int jj = first + idx / CH, c = idx % CH;
                        *reinterpret_cast<uint4*>(gen + L::V_OFF + st * L::KV_BYTES + swz_groups<HALVES>(jj, c)) = make_uint4(0, 0, 0, 0);
                    }
                    fence_async_smem();   // before the arrival below, which the product that reads these rows awaits
                }
                tl.mark(TL_ROW_COMPUTED, gj);
                // The row of P over the first half of its scores: column c holds the weights of keys 2c and 2c + 1.
                // (P of tile j - 2 lay here; its product was issued before the scores of this tile were computed.)
                {
                    uint32_t (*pk16)[16] = reinterpret_cast<uint32_t (*)[16]>(pk);
                    tc_st16(tmem_s + lane_addr + (uint32_t)(b * BNK), pk16[0]);
                    tc_st16(tmem_s + lane_addr + (uint32_t)(b * BNK + 16), pk16[1]);
                    tc_wait_st();
                }
                tc_fence_before();
                mbar_arrive(p_ready(b));
                tl.mark(TL_ROW_HANDED, gj);
            }
            const int g_last = t0 + u.n_tiles - 1;
            t0 += u.n_tiles;
            const float l_end = l_run;
            const int out_row = u.row0 + iq, out_head = u.head0 + ih;
            // the unit to come, and this row's query of it on its way
            unit = ok ? next_unit(seq++, u) : -1;
            has = unit >= 0;
            ask_query(u, has);
            if (ok) ok = mbar_wait(pv_done(g_last & 1), (g_last >> 1) & 1, abort_flag, a.status);

            if (ok) {
                tc_fence_after();
                const float inv = l_end > 0.f ? 1.f / l_end : 0.f;
                __nv_bfloat16* dst = a.out + ((size_t)out_row * a.nh + out_head) * HD;
#pragma unroll
                for (int c0 = 0; c0 < HD; c0 += 16) {   // 16 columns at a time: the query of the unit to come is in registers too
                    uint32_t v[16];
                    tc_ld16(tmem_o + lane_addr + (uint32_t)c0, v);
                    tc_wait_ld();
                    if (row_ok) {
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            float f[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[8 * c + i]) * inv;
                            *reinterpret_cast<uint4*>(dst + c0 + 8 * c) =
                                make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
                        }
                    }
                }
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    tl_mark(VCB_TL_ATTN_TC, 2);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::TMEM_COLS) : "memory");
    }
}

template <int HD>
int launch(const CUtensorMap& map, const TcArgs& a, int n_items, cudaStream_t stream) {
    constexpr int KS = 3, VS = 2;
    using L = Layout<HD, KS, VS>;
    auto kern = attn_tc_kernel<HD, KS, VS>;
    static bool opted = false;
    if (!opted) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) {
            vcb_set_error("attn_tc: %d bytes of shared memory refused: %s", L::TOTAL, cudaGetErrorString(e));
            return -2;
        }
        opted = true;
    }
    static int resident = 0;   // blocks that run at once: two an SM
    if (resident == 0) {
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
            vcb_set_error("attn_tc: the device does not say how many SMs it has");
            return -2;
        }
        resident = 2 * sms;
    }
    launch_pdl(kern, dim3((unsigned)(a.n_units < resident ? a.n_units : resident)), dim3(NTHREADS), (size_t)L::TOTAL, stream, map, a);
    VCB_CHECK_LAUNCH("attn_tc");
    return 0;
}

}  // namespace

VCB_TIMELINE_UNIT(attn_tc)

// What the tcgen05 kernel takes; the caller uses vcb_attn_mma (or vcb_attn_paged) for everything else.
VCB_API int vcb_attn_tc_supported(int dtype, int hd, int page_size) {
    return dtype == VCB_BF16 && (hd == 64 || hd == 128) &&
           (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64);
}

// Prompt portions only: every item has slice 0 of 1 and at most 128 rows (tokens x query heads per KV head).
// work: two ints that are zero when the kernel starts and zero again when it ends (the blocks' queue of units); the
// launches that share them must not overlap.
VCB_API int vcb_attn_tc(const void* q, void* out, const void* pages, long long page_stride, const int* block_table,
                        const int* table_row, int max_blocks, const int* q_start, const int* q_len, const int* ctx_len,
                        const int* items, int n_items, int nh, int nkv, int hd, int page_size, int num_pages, int window,
                        float scale, int* status, int* work, cudaStream_t stream) {
    if (n_items == 0) return 0;
    VCB_CHECK_ARG(nh > 0 && nkv > 0 && nh % nkv == 0, "attn_tc: %d query heads are not a multiple of %d KV heads", nh, nkv);
    VCB_CHECK_ARG(vcb_attn_tc_supported(VCB_BF16, hd, page_size), "attn_tc: head_dim %d with pages of %d tokens is not supported", hd, page_size);
    VCB_CHECK_ARG(window >= 0, "attn_tc: bad window %d", window);
    VCB_CHECK_ARG((long long)n_items * nh < (1ll << 31), "attn_tc: %d items of %d heads are more blocks than a grid holds", n_items, nh);
    VCB_CHECK_ARG(((uintptr_t)pages % 16 == 0) && page_stride == (long long)2 * nkv * page_size * hd,
                  "attn_tc: the pages of a layer must be contiguous and 16-byte aligned for TMA loads");
    VCB_CHECK_ARG(((uintptr_t)q % 16 == 0) && ((uintptr_t)out % 16 == 0), "attn_tc: q and out must be 16-byte aligned");
    VCB_CHECK_ARG(work != nullptr, "attn_tc: no work counters");
    CUtensorMap map;
    if (!vcb_kv_tensor_map(pages, (long long)num_pages * 2 * nkv * page_size, hd, page_size, &map, true)) return -3;
    const int g = nh / nkv;
    const int hchunks = (g + ROWS - 1) / ROWS;
    TcArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, block_table, table_row, max_blocks, q_start, q_len, ctx_len,
             items, nh, nkv, page_size, num_pages, window, scale, status, n_items * nkv * hchunks, work};
    return hd == 64 ? launch<64>(map, a, n_items, stream) : launch<128>(map, a, n_items, stream);
}
