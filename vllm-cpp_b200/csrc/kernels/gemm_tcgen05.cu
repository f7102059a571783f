// bfloat16 projections on the fifth-generation tensor cores:
//     out[z][t][m] = sum over the z-th slice of k of  W[m][k] * X[t][k]
// i.e. y = x . W^T with W stored [out_features, in_features] as in the checkpoint
// (src/model.cpp:932-944 of the reference; its CUDA sketch calls cublasGemmEx for
// this, cuda/tp_model.cu:259-269).
//
// Orientation.  The weight matrix is the M operand of the MMA (tiles of 128 output
// features = 128 TMEM lanes), the tokens are the N operand (16 to 256 per tile).
// One orientation serves a 2,048-token prompt portion and a single decoded token:
// with few tokens the kernel is a pipeline that streams weights from HBM at full
// rate into MMAs of small N; with many it is a 128x256 tile kernel.  The
// accumulator D[feature][token] lives in TMEM; each epilogue thread owns one
// feature (lane) and walks the tokens, so a warp's store of one token covers 32
// consecutive features of the row-major output: coalesced.
//
// Blocks are persistent (one per SM) and walk work units (feature tiles x token tiles x k-slices) round
// robin.  Roles (192 threads): warp 0 issues TMA loads (cp.async.bulk.tensor, 128-byte
// swizzle, zero fill beyond the matrix edges) into a ring of stages guarded by
// full/empty mbarriers; warp 1 allocates TMEM and issues tcgen05.mma
// (kind::f16, bf16 x bf16 -> f32) from shared-memory descriptors, releasing each
// stage with tcgen05.commit; warps 2-5 read the accumulator with tcgen05.ld once
// the last commit lands and store it.  Split-K: blockIdx.z takes a slice of K and
// writes an f32 partial; the consumer (the next norm or element-wise kernel) adds
// the partials in slice order, so results do not depend on timing.
//
// Every mbarrier wait is bounded by the clock; a wait that runs out sets a bit in
// the status word, raises an abort flag that the other roles see, and the block
// still frees its TMEM and returns.  No cluster multicast anywhere.
#include "common.cuh"
#include "mbarrier.cuh"

#include <cuda.h>

#include <stdlib.h>
#include <string.h>

#include <algorithm>

#include <mutex>
#include <unordered_map>

namespace {

constexpr int BM = 128;   // output features per tile (TMEM lanes)
constexpr int BK = 64;    // k per stage: 64 bf16 = 128 bytes = one swizzle span
constexpr int UMMA_K = 16;
constexpr int NTHREADS = 192;
constexpr int VCB_GEMM_AFTER_SMALL_KERNEL = 1;


__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
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

__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzled:
// start address / 16 in bits 0-13, leading byte offset (unused for this layout, 1) in 16-29, stride
// between 8-row groups (1024 bytes) / 16 in 32-45, descriptor version 1 in 46-47, layout 2 = SWIZZLE_128B in 61-63.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor of kind::f16: f32 accumulate (bits 4-5 = 1), A and B bfloat16 (bits 7-9, 10-12 = 1),
// both K-major (bits 15, 16 = 0), N / 8 in bits 17-22, M / 16 in bits 24-28.
__host__ __device__ constexpr uint32_t instr_desc(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// What the epilogue of the stacked q, k, v projection needs to do the work of the norm-rotate-store kernel itself (prompt
// portions, head_dim 128: a 128-feature unit is one head).  q_out null: an ordinary product.
struct QkvEpilogue {
    __nv_bfloat16* q_out;        // [tokens][nh * 128]
    __nv_bfloat16* pages;        // the layer's pages [page][2][nkv][page_size][128]; null: no keys and values to store
    long long page_stride;
    const int* slot_map;         // per token: slot in the cache, -1: store nowhere
    const int* positions;        // per token
    const float* cos_sin;        // [max_pos][128]: 64 cosines, 64 sines
    const void* q_gain;          // per-head norm gains [128] (gain_dtype), unused without use_norm
    const void* k_gain;
    int max_pos, gain_dtype, use_norm, nh, nkv, page_size, num_pages;
    float eps;
};

struct GemmArgs {
    void* out;
    int out_dtype;            // VCB_F32 or VCB_BF16
    int M, N, K;              // features, tokens, inner size
    long long ldc;            // elements between output rows (tokens)
    long long split_stride;   // elements between the partials of consecutive k-slices
    int kb_per_split;         // 64-wide k-blocks per slice
    int splits;               // k-slices
    int swiglu;               // 1: rows 2i and 2i+1 of W are gate_i and up_i, and the output is silu(gate) * up, [tokens, M/2] bfloat16
    int* status;
    QkvEpilogue qe;
    int pf_tiles, pf_delay_ns;   // weight tiles asked into L2 beyond the first ring, that long after the block's start (0: none)
};

// MT = 128-feature tiles per work unit that share one token tile (2 halves the bytes that cross L2 per flop);
// ACC = accumulator buffers in TMEM (2: the epilogue of one unit overlaps the MMAs of the next).
template <int BN, int STAGES, int MT, int ACC>
struct Smem {
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = MT * A_BYTES + B_BYTES;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int NUM_BARS = 2 * STAGES + 2 * ACC;
    // where the q, k, v epilogue passes a head's values between its four warps: 128 features x 32 tokens (rows padded
    // to 33 words), the warps' partial sums of squares, the tokens' factors, positions and slots
    static constexpr int EPI_OFFSET = (BAR_OFFSET + NUM_BARS * 8 + 16 + 15) / 16 * 16;
    static constexpr int EPI_BYTES = (MT == 1 && BN >= 128) ? (128 * 33 + 4 * 32 + 4 * 32) * 4 : 0;
    static constexpr int TOTAL = EPI_OFFSET + EPI_BYTES + 1024;   // + alignment slack
};


// silu(z) = z / (1 + exp(-z)) with the fast exponential and division (a few ulp; the result is rounded to
// bfloat16).  The exponent is capped so that the divisor stays where the fast division is defined; below
// z = -87 the result is about -1e-36 instead of a smaller denormal.
__device__ __forceinline__ float silu_fast(float z) { return __fdividef(z, 1.0f + __expf(fminf(-z, 87.0f))); }

// Epilogue of a product whose weight rows alternate gate_i, up_i: lane 2i holds gate_i, lane 2i+1 up_i of the
// same token, so one shuffle brings them together.  v: CHUNK token columns of this lane's row m; writes
// out[token][m / 2] for even m.  Every lane of the warp must call it.
template <int CHUNK>
__device__ __forceinline__ void swiglu_store(uint32_t (*v)[16], __nv_bfloat16* out, long long ldc, int m, int M, int n_first,
                                             int N, int lane) {
    // All values first, without a branch in sight, so that the shuffles' and the exponentials' latencies overlap
    // across the columns; a branch per column made this epilogue slower than the unit's MMAs.
    float r[CHUNK];
#pragma unroll
    for (int jj = 0; jj < CHUNK; ++jj) {
        const float mine = __uint_as_float(v[jj / 16][jj % 16]);
        const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
        r[jj] = silu_fast(mine) * other;
    }
    if (!(lane & 1) && m + 1 < M) {
        __nv_bfloat16* o = out + (size_t)n_first * ldc + (m >> 1);
#pragma unroll
        for (int jj = 0; jj < CHUNK; ++jj)
            if (n_first + jj < N) o[(size_t)jj * ldc] = __float2bfloat16_rn(r[jj]);
    }
}

// Epilogue of the stacked q, k, v projection for prompt portions with head_dim 128: the unit's 128 features are one
// head.  Called by the four epilogue warps together for 32 token columns at a time (thread = feature f = 32 q + lane,
// x = its 32 values): a query or key head is normed over its 128 features (sum of squares through shared memory),
// scaled by its gains, rotated with the partner feature 64 away (half-split pairs: out_i = a_i cos_i - a_{i+64} sin_i,
// out_{i+64} = a_{i+64} cos_i + a_i sin_i), rounded to bfloat16 and stored -- queries to q_out, keys to the token's
// slot of the cache; a value head is stored as it is.  All in 32-bit, from the product's 32-bit sums (the separate
// kernel reads them rounded to bfloat16).  Named barrier 1 is the four warps'.
__device__ __forceinline__ void epilogue_warps_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void qkv_head_store(const float (&x)[32], const QkvEpilogue& e, int head, int f, int q, int lane,
                                               int tok0, int N, float* stage, int* status) {
    float* part = stage + 128 * 33;                       // [4][32] partial sums of squares
    float* factor = part + 4 * 32;                        // [32]
    int* pos_s = reinterpret_cast<int*>(factor + 32);     // [32]
    long long* where_s = reinterpret_cast<long long*>(pos_s + 32);   // [32]: where in the pages the token's row of K head 0 begins; -1: nowhere
    const bool is_q = head < e.nh, is_v = head >= e.nh + e.nkv;
    const int kvh = is_q ? 0 : (is_v ? head - e.nh - e.nkv : head - e.nh);
    // this chunk's positions and places in the cache, looked up and checked once
    if (q == 0) {
        int pos = tok0 + lane < N ? e.positions[tok0 + lane] : 0;
        if (pos < 0 || pos >= e.max_pos) {
            atomicOr(status, VCB_STATUS_BAD_POSITION);
            pos = 0;
        }
        pos_s[lane] = pos;
    } else if (q == 1) {
        int slot = (!is_q && e.pages != nullptr && tok0 + lane < N) ? e.slot_map[tok0 + lane] : -1;
        if (slot >= 0 && slot / e.page_size >= e.num_pages) {
            atomicOr(status, VCB_STATUS_BAD_PAGE);
            slot = -1;
        }
        where_s[lane] = slot < 0 ? -1ll : (long long)(slot / e.page_size) * e.page_stride + (long long)(slot % e.page_size) * 128;
    }
    // this thread's feature of this head within a token's row of the pages
    const long long head_at = ((long long)((is_v ? e.nkv : 0) + kvh) * e.page_size) * 128 + f;
    if (!is_v) {
#pragma unroll
        for (int t = 0; t < 32; ++t) stage[f * 33 + t] = x[t];
    }
    epilogue_warps_sync();
    if (is_v) {
#pragma unroll
        for (int t = 0; t < 32; ++t) {
            const long long at = where_s[t];
            if (at >= 0) e.pages[at + head_at] = __float2bfloat16_rn(x[t]);
        }
        epilogue_warps_sync();      // the places are read; the next chunk may write its own
        return;
    }
    float n[32];
    if (e.use_norm) {
        // token = lane: the squares of this warp's 32 features, then the four warps' sums
        float ss = 0.f;
#pragma unroll
        for (int ff = 0; ff < 32; ++ff) {
            const float y = stage[(q * 32 + ff) * 33 + lane];
            ss += y * y;
        }
        part[q * 32 + lane] = ss;
        epilogue_warps_sync();
        if (q == 0) factor[lane] = 1.0f / sqrtf((part[lane] + part[32 + lane] + part[64 + lane] + part[96 + lane]) / 128.f + e.eps);
        epilogue_warps_sync();
        const float gain = load_as_f32(is_q ? e.q_gain : e.k_gain, e.gain_dtype, f);
#pragma unroll
        for (int t = 0; t < 32; ++t) n[t] = gain * x[t] * factor[t];
#pragma unroll
        for (int t = 0; t < 32; ++t) stage[f * 33 + t] = n[t];      // every read of the raw values is behind the barriers above
        epilogue_warps_sync();
    } else {
#pragma unroll
        for (int t = 0; t < 32; ++t) n[t] = x[t];
    }
    const int fi = f & 63;
    const float sign = f < 64 ? -1.f : 1.f;
    // all the cosines and sines first (read-only loads: none waits behind a store), then all the stores
#pragma unroll
    for (int t = 0; t < 32; ++t) {
        const float partner = stage[(f ^ 64) * 33 + t];
        const float* cs = e.cos_sin + (size_t)pos_s[t] * 128;
        n[t] = n[t] * __ldg(cs + fi) + sign * partner * __ldg(cs + 64 + fi);
    }
    if (is_q) {
        __nv_bfloat16* dst = e.q_out + ((size_t)tok0 * e.nh + head) * 128 + f;
#pragma unroll
        for (int t = 0; t < 32; ++t)
            if (tok0 + t < N) dst[(size_t)t * e.nh * 128] = __float2bfloat16_rn(n[t]);
    } else {
#pragma unroll
        for (int t = 0; t < 32; ++t) {
            const long long at = where_s[t];
            if (at >= 0) e.pages[at + head_at] = __float2bfloat16_rn(n[t]);
        }
    }
    epilogue_warps_sync();          // the partners, positions and places are read; the next chunk may write its own
}

// Order of the (feature tile, token tile) pairs: token tiles fastest, in groups of up to TOKEN_TILE_GROUP, so
// that the units in flight at one time (one per SM) share few feature tiles -- every weight tile is then
// fetched from HBM once and read by its group's blocks from L2 -- while the group's tokens stay in L2 too.
// (With feature tiles fastest a round touched every weight row, and 2,048 tokens read the weights five times.)
constexpr int TOKEN_TILE_GROUP = 8;
__device__ __forceinline__ void tile_of(int idx, int m_tiles, int n_tiles, int& mi, int& ni) {
    const int per_group = m_tiles * TOKEN_TILE_GROUP;
    const int grp = idx / per_group, r = idx - grp * per_group;
    const int gsize = min(TOKEN_TILE_GROUP, n_tiles - grp * TOKEN_TILE_GROUP);
    mi = r / gsize;
    ni = grp * TOKEN_TILE_GROUP + (r - mi * gsize);
}

// Persistent: each block walks the work units blockIdx.x, blockIdx.x + gridDim.x, ...; a unit is
// (feature tile group, token tile, k-slice).  The stage ring and the accumulator ring run on across units, so
// the loads of the next unit are in flight while the current one is multiplied and the one before is stored.
template <int BN, int STAGES, int MT, int ACC>
__global__ __launch_bounds__(NTHREADS, 1) void gemm_bf16_tn_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                    const __grid_constant__ CUtensorMap map_x,
                                                                    GemmArgs g) {
    using L = Smem<BN, STAGES, MT, ACC>;
    constexpr uint32_t ACC_COLS = BN < 32 ? 32 : BN;            // columns of one 128-feature accumulator
    constexpr int CHUNK = BN % 64 == 0 ? 64 : (BN % 32 == 0 ? 32 : 16);   // accumulator columns read per wait in the epilogue
    constexpr uint32_t USED_COLS = ACC * MT * ACC_COLS;
    constexpr uint32_t TMEM_COLS = USED_COLS <= 32 ? 32 : USED_COLS <= 64 ? 64 : USED_COLS <= 128 ? 128 : USED_COLS <= 256 ? 256 : 512;
    static_assert(USED_COLS <= 512, "TMEM columns");   // allocations are powers of two in [32, 512]
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + L::BAR_OFFSET;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * STAGES + ACC + a); };
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(gen + L::BAR_OFFSET + L::NUM_BARS * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::BAR_OFFSET + L::NUM_BARS * 8 + 8);

    pdl_trigger();
    tl_mark(VCB_TL_GEMM, 0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_kb = (g.K + BK - 1) / BK;
    const int unit_rows = BM * MT;   // rows of W per unit
    const int m_tiles = (g.M + unit_rows - 1) / unit_rows;
    const int n_tiles = (g.N + BN - 1) / BN;
    const int units = m_tiles * n_tiles * g.splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < ACC; ++a) {
            mbar_init(acc_full_bar(a), 1);
            mbar_init(acc_empty_bar(a), 4);   // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void*)tmem_holder)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    // unit -> (first feature, first token, first k-block, k-blocks)
    auto unit_at = [&](int u, int& m0, int& n0, int& kb0, int& nkb, int& z) {
        z = u / (m_tiles * n_tiles);
        int mi, ni;
        tile_of(u % (m_tiles * n_tiles), m_tiles, n_tiles, mi, ni);
        n0 = ni * BN;
        m0 = mi * unit_rows;
        kb0 = z * g.kb_per_split;
        nkb = min(total_kb, kb0 + g.kb_per_split) - kb0;
    };

    if (warp == 0) {
        // ---- TMA producer ----
        if (lane == 0) {
            int it = 0, armed = 0;
            bool ok = true;
            // The weights are written by no kernel of the step, so the first ring of weight tiles is requested
            // before waiting for the kernel that produces the activations: the weight stream is already in
            // flight while that kernel drains.  The activation tiles of those stages follow after the wait.
            int early = 0;
            {
                int m0, n0, kb0, nkb, z;
                if ((int)blockIdx.x < units) {
                    unit_at(blockIdx.x, m0, n0, kb0, nkb, z);
                    early = min(nkb, STAGES);
                    for (int i = 0; i < early; ++i) {
                        mbar_expect_tx(full_bar(i), L::STAGE_BYTES);
                        const uint32_t a_dst = base + i * L::STAGE_BYTES;
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt)
                            tma_load_2d(a_dst + mt * L::A_BYTES, &map_w, full_bar(i), (kb0 + i) * BK,
                                        m0 + mt * BM);
                    }
                    armed = early;
                    if (g.pf_tiles > 0) {
                        // A decode product that follows a small kernel (norm, SiLU-gate) waits several microseconds
                        // with only its ring on the way while the memory system idles.  Its next weight tiles are
                        // asked into L2 meanwhile -- but not at once: the small kernel's one round trip to memory
                        // would queue behind them (asked at the block's start they cost more than they save); a
                        // little later that kernel has its operands and the requests fill the rest of the gap.
                        const unsigned long long t0 = global_ns();
                        while (global_ns() - t0 < (unsigned long long)g.pf_delay_ns) {}
                        // the k-blocks after the ring, on into this block's next units
                        int left = g.pf_tiles, i = early;
                        for (int u = blockIdx.x; u < units && left > 0; u += gridDim.x) {
                            unit_at(u, m0, n0, kb0, nkb, z);
                            for (; i < nkb && left > 0; ++i, --left)
#pragma unroll
                                for (int mt = 0; mt < MT; ++mt) tma_prefetch_2d(&map_w, (kb0 + i) * BK, m0 + mt * BM);
                            i = 0;
                        }
                    }
                }
            }
            pdl_wait();
            tl_mark(VCB_TL_GEMM, 1);
            for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
                int m0, n0, kb0, nkb, z;
                unit_at(u, m0, n0, kb0, nkb, z);
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    const uint32_t a_dst = base + s * L::STAGE_BYTES;
                    if (it < early) {   // its weight tiles are already on their way
                        tma_load_2d(a_dst + MT * L::A_BYTES, &map_x, full_bar(s), (kb0 + i) * BK, n0);
                        continue;
                    }
                    if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, g.status)) { ok = false; break; }
                    mbar_expect_tx(full_bar(s), L::STAGE_BYTES);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
                        tma_load_2d(a_dst + mt * L::A_BYTES, &map_w, full_bar(s), (kb0 + i) * BK,
                                    m0 + mt * BM);
                    tma_load_2d(a_dst + MT * L::A_BYTES, &map_x, full_bar(s), (kb0 + i) * BK, n0);
                    armed = it + 1;
                }
            }
            if (*abort_flag) {
                // let the copies already in flight land before the block goes away
                for (int i = max(0, armed - STAGES); i < armed; ++i) {
                    const long long t0 = clock64();
                    while (!mbar_try(full_bar(i % STAGES), (i / STAGES) & 1) && clock64() - t0 < VCB_WAIT_CLOCKS) {}
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BN);
            int it = 0, j = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < units && ok; u += gridDim.x, ++j) {
                int m0, n0, kb0, nkb, z;
                unit_at(u, m0, n0, kb0, nkb, z);
                const int a = j % ACC;
                ok = mbar_wait(acc_empty_bar(a), ((j / ACC) & 1) ^ 1u, abort_flag, g.status);   // drained by the epilogue
                if (!ok) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + a * (MT * ACC_COLS);
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(full_bar(s), (it / STAGES) & 1, abort_flag, g.status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_addr = base + s * L::STAGE_BYTES;
                    const uint64_t db = smem_desc(a_addr + MT * L::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // 16 k = 32 bytes further along the 128-byte rows: +2 in the descriptor's 16-byte units
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt)
                            tc_mma(tmem_d + mt * ACC_COLS, smem_desc(a_addr + mt * L::A_BYTES) + 2 * k, db + 2 * k, idesc,
                                   (i > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(empty_bar(s));   // arrives when these MMAs have read the stage
                }
                if (ok) tc_commit(acc_full_bar(a));
            }
        }
    } else {
        // ---- epilogue: warps 2..5 own TMEM lane quarters 2, 3, 0, 1 ----
        const int q = warp & 3;
        int j = 0;
        for (int u = blockIdx.x; u < units; u += gridDim.x, ++j) {
            int m0, n0, kb0, nkb, z;
            unit_at(u, m0, n0, kb0, nkb, z);
            const int a = j % ACC;
            if (!mbar_wait(acc_full_bar(a), (j / ACC) & 1, abort_flag, g.status)) break;
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + a * (MT * ACC_COLS);
            const size_t zoff = (size_t)z * g.split_stride;
#pragma unroll 1
            for (int cc = 0; cc < MT * BN; cc += CHUNK) {
                const int mt = cc / BN, c0 = cc % BN;
                if (n0 + c0 >= g.N) continue;   // uniform over the warp
                const int m = m0 + mt * BM + q * 32 + lane;
                // several TMEM loads in flight before one wait: their latencies overlap
                uint32_t v[CHUNK / 16][16];
#pragma unroll
                for (int b = 0; b < CHUNK / 16; ++b)
                    tc_ld16(tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)(mt * ACC_COLS + c0 + 16 * b), v[b]);
                tc_wait_ld();
                if constexpr (L::EPI_BYTES > 0) {
                    if (g.qe.q_out != nullptr) {     // uniform over the block: every warp takes part in the barriers
                        float* stage = reinterpret_cast<float*>(gen + L::EPI_OFFSET);
#pragma unroll
                        for (int hh = 0; hh < CHUNK / 32; ++hh) {
                            float x[32];
#pragma unroll
                            for (int t = 0; t < 32; ++t) x[t] = __uint_as_float(v[(32 * hh + t) / 16][(32 * hh + t) % 16]);
                            qkv_head_store(x, g.qe, m0 / BM, q * 32 + lane, q, lane, n0 + c0 + 32 * hh, g.N, stage, g.status);
                        }
                        continue;
                    }
                }
                if (g.swiglu) {
                    swiglu_store<CHUNK>(v, reinterpret_cast<__nv_bfloat16*>(g.out), g.ldc, m, g.M, n0 + c0, g.N, lane);
                } else if (m < g.M) {
                    if (g.out_dtype == VCB_F32) {
                        float* o = reinterpret_cast<float*>(g.out) + zoff;
#pragma unroll
                        for (int jj = 0; jj < CHUNK; ++jj)
                            if (n0 + c0 + jj < g.N) o[(size_t)(n0 + c0 + jj) * g.ldc + m] = __uint_as_float(v[jj / 16][jj % 16]);
                    } else {
                        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(g.out) + zoff;
#pragma unroll
                        for (int jj = 0; jj < CHUNK; ++jj)
                            if (n0 + c0 + jj < g.N)
                                o[(size_t)(n0 + c0 + jj) * g.ldc + m] = __float2bfloat16_rn(__uint_as_float(v[jj / 16][jj % 16]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(a));   // this warp has read its quarter of the accumulator
        }
        tc_fence_before();
    }
    __syncthreads();
    tl_mark(VCB_TL_GEMM, 2);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------
// Two blocks on two SMs working as a pair (cta_group::2) for prompt portions.
//
// One MMA of the pair covers 256 features (128 TMEM lanes in each block) x 256 tokens; each block loads only its own
// 128 features of the weights and its own 128-token half of the token tile, which the tensor cores of both read:
// 32 KB per block and k-step of 64 where the single-block kernel draws 48 KB for the same 128 x 256 x 64 products,
// and what an SM can draw from L2 (about 70 bytes a clock) is what bounds that kernel.  A pair's unit is 256
// features x 256 tokens; each block holds two accumulators of 256 columns, so the epilogue of one unit overlaps the
// MMAs of the next.
//
// Block 0 of the pair issues every MMA.  Both blocks' TMA loads report to block 0's "full" barrier
// (cp.async.bulk.tensor with .cta_group::2 lets a load signal the peer's barrier; no multicast load is used);
// tcgen05.commit with a two-block arrival mask releases the stage, and hands over the accumulators, in both
// blocks; the epilogue warps of both report the drained accumulators to block 0.
// ---------------------------------------------------------------------------
constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;   // a shared::cluster address with this bit cleared names block 0 of the pair

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_block0, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar_block0), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this shared-memory offset in both blocks of the pair once the MMAs issued so far are done
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_block0(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & PEER_BIT_MASK) : "memory");
}

template <int STAGES>
struct SmemPair {
    static constexpr int BN = 256;
    static constexpr int A_BYTES = BM * BK * 2;           // one 128-feature tile
    static constexpr int B_BYTES = (BN / 2) * BK * 2;     // this block's half of the token tile
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
    static constexpr int NUM_BARS = 2 * STAGES + 4;
    static constexpr int EPI_OFFSET = (BAR_OFFSET + NUM_BARS * 8 + 16 + 15) / 16 * 16;    // as in Smem: the q, k, v epilogue's exchange
    static constexpr int EPI_BYTES = (128 * 33 + 4 * 32 + 4 * 32) * 4;
    static constexpr int TOTAL = EPI_OFFSET + EPI_BYTES + 1024;
};

template <int STAGES>
__global__ __launch_bounds__(NTHREADS, 1) void gemm_bf16_tn_pair_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                         const __grid_constant__ CUtensorMap map_x,
                                                                         GemmArgs g) {
    using L = SmemPair<STAGES>;
    constexpr int BN = 256;
    constexpr uint32_t TMEM_COLS = 512;   // two accumulators of 256 token columns, used in turn
    constexpr int CHUNK = 64;             // accumulator columns read per wait in the epilogue
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + L::BAR_OFFSET;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto acc_full_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(gen + L::BAR_OFFSET + L::NUM_BARS * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::BAR_OFFSET + L::NUM_BARS * 8 + 8);

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();          // 0 issues the MMAs
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int total_kb = (g.K + BK - 1) / BK;
    const int unit_rows = 2 * BM;   // rows of W per pair unit: 128 in each block
    const int m_tiles = (g.M + unit_rows - 1) / unit_rows;
    const int n_tiles = (g.N + BN - 1) / BN;
    const int units = m_tiles * n_tiles * g.splits;
    // unit -> (feature tile, token tile, k-slice): the k-slices of a tile are units of their own, each with a
    // 32-bit partial output, as in the single-block kernel
    auto unit_at = [&](int u, int& m0, int& n0, int& kb0, int& nkb, int& z) {
        z = u / (m_tiles * n_tiles);
        int mi, ni;
        tile_of(u % (m_tiles * n_tiles), m_tiles, n_tiles, mi, ni);
        m0 = mi * unit_rows;
        n0 = ni * BN;
        kb0 = z * g.kb_per_split;
        nkb = min(total_kb, kb0 + g.kb_per_split) - kb0;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(acc_full_bar(a), 1);
            mbar_init(acc_empty_bar(a), 8);   // four epilogue warps in each block of the pair
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void*)tmem_holder)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();   // the peer's barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        // ---- TMA producer (in both blocks): its feature tile and its half of the token tile ----
        if (lane == 0) {
            pdl_wait();
            int it = 0, armed = 0;
            bool ok = true;
            for (int u = pair; u < units && ok; u += pairs) {
                int m0, n0, kb0, nkb, z;
                unit_at(u, m0, n0, kb0, nkb, z);
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1) ^ 1u, abort_flag, g.status)) { ok = false; break; }
                    if (rank == 0) mbar_expect_tx(full_bar(s), 2 * L::STAGE_BYTES);   // both blocks' bytes land on block 0's barrier
                    const uint32_t dst = base + s * L::STAGE_BYTES;
                    const uint32_t bar0 = full_bar(s) & PEER_BIT_MASK;
                    tma_load_2d_pair(dst, &map_w, bar0, (kb0 + i) * BK, m0 + (int)rank * BM);
                    tma_load_2d_pair(dst + L::A_BYTES, &map_x, bar0, (kb0 + i) * BK, n0 + (int)rank * (BN / 2));
                    armed = it + 1;
                }
            }
            if (*abort_flag && rank == 0) {
                for (int i = max(0, armed - STAGES); i < armed; ++i) {
                    const long long t0 = clock64();
                    while (!mbar_try(full_bar(i % STAGES), (i / STAGES) & 1) && clock64() - t0 < VCB_WAIT_CLOCKS) {}
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: block 0 only ----
        if (lane == 0 && rank == 0) {
            // M = 256 (both blocks' lanes), N = 256
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            int it = 0, j = 0;
            bool ok = true;
            for (int u = pair; u < units && ok; u += pairs, ++j) {
                int m0, n0, kb0, nkb, z;
                unit_at(u, m0, n0, kb0, nkb, z);
                const int a = j & 1;
                ok = mbar_wait(acc_empty_bar(a), ((j >> 1) & 1) ^ 1u, abort_flag, g.status);   // both epilogues drained it
                if (!ok) break;
                tc_fence_after();
                for (int i = 0; i < nkb; ++i, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(full_bar(s), (it / STAGES) & 1, abort_flag, g.status);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_addr = base + s * L::STAGE_BYTES;
                    const uint64_t da = smem_desc(a_addr), db = smem_desc(a_addr + L::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        tc_mma_pair(tmem_base + a * BN, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    tc_commit_pair(empty_bar(s));   // frees the stage in both blocks
                }
                if (ok) tc_commit_pair(acc_full_bar(a));
            }
        }
    } else {
        // ---- epilogue (both blocks): each owns its 128 lanes of the accumulator ----
        const int q = warp & 3;
        int j = 0;
        for (int u = pair; u < units; u += pairs, ++j) {
            int m0, n0, kb0, nkb, z;
            unit_at(u, m0, n0, kb0, nkb, z);
            const size_t zoff = (size_t)z * g.split_stride;
            const int a = j & 1;
            if (!mbar_wait(acc_full_bar(a), (j >> 1) & 1, abort_flag, g.status)) break;
            tc_fence_after();
            const int m = m0 + (int)rank * BM + q * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += CHUNK) {
                if (n0 + c0 >= g.N) continue;   // uniform over the warp
                uint32_t v[CHUNK / 16][16];
#pragma unroll
                for (int b = 0; b < CHUNK / 16; ++b)
                    tc_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(a * BN + c0 + 16 * b), v[b]);
                tc_wait_ld();
                if (g.qe.q_out != nullptr) {     // uniform over the block: every warp takes part in the barriers
                    float* stage = reinterpret_cast<float*>(gen + L::EPI_OFFSET);
                    const int head = m0 / BM + (int)rank;
                    if (head * BM < g.M) {
#pragma unroll
                        for (int hh = 0; hh < CHUNK / 32; ++hh) {
                            float x[32];
#pragma unroll
                            for (int t = 0; t < 32; ++t) x[t] = __uint_as_float(v[(32 * hh + t) / 16][(32 * hh + t) % 16]);
                            qkv_head_store(x, g.qe, head, q * 32 + lane, q, lane, n0 + c0 + 32 * hh, g.N, stage, g.status);
                        }
                    }
                    continue;
                }
                if (g.swiglu) {
                    swiglu_store<CHUNK>(v, reinterpret_cast<__nv_bfloat16*>(g.out), g.ldc, m, g.M, n0 + c0, g.N, lane);
                } else if (m < g.M) {
                    if (g.out_dtype == VCB_F32) {
                        float* o = reinterpret_cast<float*>(g.out) + zoff;
#pragma unroll
                        for (int jj = 0; jj < CHUNK; ++jj)
                            if (n0 + c0 + jj < g.N) o[(size_t)(n0 + c0 + jj) * g.ldc + m] = __uint_as_float(v[jj / 16][jj % 16]);
                    } else {
                        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(g.out) + zoff;
#pragma unroll
                        for (int jj = 0; jj < CHUNK; ++jj)
                            if (n0 + c0 + jj < g.N)
                                o[(size_t)(n0 + c0 + jj) * g.ldc + m] = __float2bfloat16_rn(__uint_as_float(v[jj / 16][jj % 16]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_block0(acc_empty_bar(a));
        }
        tc_fence_before();
    }
    __syncthreads();
    cluster_sync();   // neither block leaves while the other may still signal its barriers or read its tiles
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------
// host side: tensor maps (cached) and launch
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

struct MapKey {
    const void* ptr;
    long long rows, cols, ld;
    int box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.ptr);
        for (long long v : {k.rows, k.cols, k.ld, (long long)k.box_rows}) h = h * 1000003u ^ std::hash<long long>()(v);
        return h;
    }
};

// A [rows, cols] bfloat16 matrix with `ld` elements between rows; boxes of box_rows x 64, 128-byte swizzle.
bool tensor_map(const void* ptr, long long rows, long long cols, long long ld, int box_rows, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{ptr, rows, cols, ld, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        vcb_set_error("gemm_bf16_tn: the driver does not offer cuTensorMapEncodeTiled");
        return false;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    const CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        vcb_set_error("gemm_bf16_tn: cuTensorMapEncodeTiled failed with %d (rows %lld, cols %lld, ld %lld, box %d)",
                      (int)r, rows, cols, ld, box_rows);
        return false;
    }
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

// VLLM_CPP_B200_GEMM_PREFETCH = "tiles,nanoseconds" (default 12,2000; 0 switches it off): what a decode product of
// up to 16 tokens that follows a small kernel asks into L2 before its wait, and how long after its block's start.
// 8B sizes, 36 layers, captured steps: batch 8 4.21 -> 4.12 ms with 12 tiles (4.11 with 20), one request 3.55 -> 3.45,
// batch 8 at context 2,176 3.88 -> 3.79; the 14B sizes 7.23 -> 7.16 with 12 tiles, 7.21 with 20, and 7.37 with 32.
// Asked at the block's start instead of 2 us later: 1.606 -> 1.629 ms for 12 layers.  Not behind attention (the output
// projection's blocks become resident as the attention's leave and hardly wait: the delay would hold them up) and
// not at 64 tokens (10.20 -> 10.36 ms).
int g_pf_tiles = -1, g_pf_delay = 2000;
void pf_settings(int* tiles, int* delay) {
    if (g_pf_tiles < 0) {
        g_pf_tiles = 12;
        const char* e = getenv("VLLM_CPP_B200_GEMM_PREFETCH");
        if (e) {
            g_pf_tiles = atoi(e);
            const char* c = strchr(e, ',');
            if (c) g_pf_delay = atoi(c + 1);
            if (g_pf_tiles < 0) g_pf_tiles = 0;
            if (g_pf_delay < 0 || g_pf_delay > 20000) g_pf_delay = 2000;     // never a long spin
        }
    }
    *tiles = g_pf_tiles;
    *delay = g_pf_delay;
}

int num_sms() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int BN, int STAGES, int MT, int ACC>
int launch_maps(const void* W, long long w_rows, const void* X, const GemmArgs& g, long long ldw, long long ldx, int splits,
                cudaStream_t stream) {
    using L = Smem<BN, STAGES, MT, ACC>;
    CUtensorMap mw, mx;
    if (!tensor_map(W, w_rows, g.K, ldw, BM, &mw) || !tensor_map(X, g.N, g.K, ldx, BN, &mx)) return -3;
    auto kern = gemm_bf16_tn_kernel<BN, STAGES, MT, ACC>;
    static bool opted = false;
    if (!opted) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) {
            vcb_set_error("gemm_bf16_tn: %d bytes of shared memory refused: %s", L::TOTAL, cudaGetErrorString(e));
            return -2;
        }
        opted = true;
    }
    const int unit_rows = BM * MT;
    const long long units = (long long)((g.M + unit_rows - 1) / unit_rows) * ((g.N + BN - 1) / BN) * splits;
    const int grid = (int)(units < num_sms() ? units : num_sms());
    launch_pdl(kern, dim3(grid), dim3(NTHREADS), L::TOTAL, stream, mw, mx, g);
    VCB_CHECK_LAUNCH("gemm_bf16_tn");
    return 0;
}

template <int BN, int STAGES, int MT, int ACC>
int launch(const void* W, const void* X, const GemmArgs& g, long long ldw, long long ldx, int splits, cudaStream_t stream) {
    return launch_maps<BN, STAGES, MT, ACC>(W, g.M, X, g, ldw, ldx, splits, stream);
}

// Which products of more than 128 tokens without k-slices run on the two-block kernel: 0 none, 1 (the default) those
// whose 256 x 256 units fill the rounds of the 74 pairs no worse than the single-block kernel's best shape fills
// those of the 148 SMs -- round for round the pairs measured about 4 % faster (2,048 tokens: qkv 79.4 -> 75.9 us,
// o 54.4 -> 52.6, gate_up 294 -> 288; 4,096 tokens: 158 -> 147, 106.5 -> 99.9, 600 -> 575, down 330 -> 297) --
// 2 all of them (tests).  VLLM_CPP_B200_GEMM_PAIRS sets the default.
int g_pairs = -1;
int pairs_mode() {
    if (g_pairs < 0) {
        const char* e = getenv("VLLM_CPP_B200_GEMM_PAIRS");
        g_pairs = (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 1;
    }
    return g_pairs;
}

int launch_pair(const void* W, long long w_rows, const void* X, const GemmArgs& g, long long ldw, long long ldx,
                cudaStream_t stream) {
    constexpr int STAGES = 6;
    using L = SmemPair<STAGES>;
    CUtensorMap mw, mx;
    if (!tensor_map(W, w_rows, g.K, ldw, BM, &mw) || !tensor_map(X, g.N, g.K, ldx, 128, &mx)) return -3;
    auto kern = gemm_bf16_tn_pair_kernel<STAGES>;
    static bool opted = false;
    if (!opted) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        if (e != cudaSuccess) {
            vcb_set_error("gemm_bf16_tn: %d bytes of shared memory refused: %s", L::TOTAL, cudaGetErrorString(e));
            return -2;
        }
        opted = true;
    }
    const int unit_rows = 2 * BM;
    const long long units = (long long)((g.M + unit_rows - 1) / unit_rows) * ((g.N + 255) / 256) * g.splits;
    const long long max_pairs = num_sms() / 2;
    const int pairs = (int)(units < max_pairs ? units : max_pairs);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = L::TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = vcb_pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, mw, mx, g);
    if (e != cudaSuccess) {
        vcb_set_error("gemm_bf16_tn (pairs): launch failed: %s", cudaGetErrorString(e));
        return -2;
    }
    return 0;
}

}  // namespace

VCB_TIMELINE_UNIT(gemm)

// out[z][t][m] (z < splits) = sum over k-slice z of W[m][k] X[t][k];  W [M,K], X [N,K] bfloat16, K contiguous.
// out_dtype bfloat16 needs splits == 1.  The number of slices actually used is vcb_gemm_effective_splits(K, splits).
VCB_API int vcb_gemm_effective_splits(int K, int splits) {
    const int total_kb = (K + BK - 1) / BK;
    if (splits < 1) splits = 1;
    if (splits > total_kb) splits = total_kb;
    const int kb_per_split = (total_kb + splits - 1) / splits;
    return (total_kb + kb_per_split - 1) / kb_per_split;
}

// The unit shapes that are built: tokens per tile (BN), stages of the ring, 128-feature tiles per unit, accumulators.
enum GemmShape { SHAPE_N16 = 0, SHAPE_N32, SHAPE_N64, SHAPE_N128, SHAPE_N256, SHAPE_M256_N192, SHAPE_M256_N256, SHAPE_PAIR, SHAPE_M256_N160,
                 SHAPE_COUNT };

namespace {
int launch_shape(int shape, const void* W, const void* X, const GemmArgs& g, long long ldw, long long ldx, int splits,
                 cudaStream_t stream) {
    switch (shape) {
        case SHAPE_N16: return launch<16, 8, 1, 2>(W, X, g, ldw, ldx, splits, stream);
        case SHAPE_N32: return launch<32, 8, 1, 2>(W, X, g, ldw, ldx, splits, stream);
        case SHAPE_N64: return launch<64, 8, 1, 2>(W, X, g, ldw, ldx, splits, stream);
        case SHAPE_N128: return launch<128, 6, 1, 2>(W, X, g, ldw, ldx, splits, stream);
        case SHAPE_N256: return launch<256, 4, 1, 2>(W, X, g, ldw, ldx, splits, stream);
        case SHAPE_M256_N192: return launch<192, 3, 2, 1>(W, X, g, ldw, ldx, splits, stream);
        case SHAPE_M256_N160: return launch<160, 3, 2, 1>(W, X, g, ldw, ldx, splits, stream);
        case SHAPE_M256_N256: return launch<256, 3, 2, 1>(W, X, g, ldw, ldx, splits, stream);
        case SHAPE_PAIR:
            if (g.M < 2 * BM) { vcb_set_error("gemm_bf16_tn: pairs of blocks need at least 256 features"); return -1; }
            return launch_pair(W, g.M, X, g, ldw, ldx, stream);
    }
    vcb_set_error("gemm_bf16_tn: no unit shape %d (0..%d)", shape, SHAPE_COUNT - 1);
    return -1;
}

// time of a product on pairs of blocks in the units of pick_shape's costs (token columns a block works through)
long long pair_cost(int M, int N) {
    const long long units = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
    const long long pairs = num_sms() / 2;
    return ((units + pairs - 1) / pairs) * 256;
}

int pick_shape(int M, int N, int K, int splits, long long* cost_out = nullptr) {
    if (cost_out) *cost_out = -1;
    if (N <= 16) return SHAPE_N16;
    if (N <= 32) return SHAPE_N32;
    if (N <= 64) return SHAPE_N64;
    if (N <= 128) return SHAPE_N128;
    // a sliced product has too few units for the SMs: the smallest units with 256 tokens measured fastest
    // at every size from 160 to 1,024 tokens
    if (M <= 128 || splits > 1) return SHAPE_N256;
    // Units of 128 x 256 (two accumulator buffers: the epilogue of one unit overlaps the MMAs of the next),
    // 256 x 256 or 256 x 192 tokens: whichever needs the least time over the SMs, counting whole rounds.
    // Measured at 2,048 tokens the 128 x 256 units are as fast per flop as the 256-feature ones at an inner size
    // of 4096, so ties go to them; at 12288 the 256 x 256 units, which read the token tile half as often, are
    // 7 to 9 % faster (down_proj 156 -> 146 us), so there ties go the other way.
    auto cost = [&](int mt, int bn) {
        const long long units = (long long)((M + mt * BM - 1) / (mt * BM)) * ((N + bn - 1) / bn);
        return ((units + num_sms() - 1) / num_sms()) * (long long)(mt * bn);
    };
    const long long c1 = cost(1, 256), c2 = cost(2, 256), c3 = cost(2, 192);
    // 256 x 160 units where they alone fill one round (2,560 features at 2,048 tokens: 130 units for 148 SMs, where
    // 192-token units make 110 and 256-token units of 128 features make 160, two rounds)
    const long long c4 = cost(2, 160);
    // 128 x 128 units draw more from L2 per flop: a k-block of theirs takes 0.29 us where one of 128 x 256 takes 0.36,
    // four fifths of the time for half the work.  They pay where they fill one round and 256-token units leave a
    // third of the SMs idle (qkv_proj at 384 tokens: 30.5 -> 24.5 us).
    const long long c0 = cost(1, 128) * 8 / 5;
    if (cost_out) *cost_out = std::min(std::min(std::min(c0, c1), std::min(c2, c3)), c4);
    if (c4 < c0 && c4 < c1 && c4 < c2 && c4 < c3) return SHAPE_M256_N160;
    if (c0 < c1 && c0 < c2 && c0 < c3) return SHAPE_N128;
    if (c1 == c2 && c2 <= c3 && K >= 8192) return SHAPE_M256_N256;
    if (c1 <= c2 && c1 <= c3) return SHAPE_N256;
    return c3 < c2 ? SHAPE_M256_N192 : SHAPE_M256_N256;
}
bool use_pairs(int M, int N, int K, int splits) {
    const int mode = pairs_mode();
    if (mode == 0 || N <= 128 || M < 2 * BM) return false;
    if (mode == 2) return true;
    if (splits != 1) {
        // k-slices on pairs: a pair's unit is 256 x 256 where a single block's is 128 x 256, so there are half as many
        // units for half as many takers; the pairs draw a third less from L2 per k-block.  That pays for the long inner
        // sizes (down_proj, 12288: 5 to 7 % at 384 to 768 tokens) where the rounds come out no worse, and not for 4096
        // (qkv_proj at 256 tokens: 18.1 -> 19.7 us).
        if (K < 8192) return false;
        const long long pair_units = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256) * splits;
        const long long single_units = (long long)((M + BM - 1) / BM) * ((N + 255) / 256) * splits;
        const long long pairs = num_sms() / 2;
        return (pair_units + pairs - 1) / pairs <= (single_units + num_sms() - 1) / num_sms();
    }
    long long single = -1;
    pick_shape(M, N, K, 1, &single);
    return single > 0 && pair_cost(M, N) * 24 <= single * 25;
}
}  // namespace

// shape < 0: chosen from the sizes; otherwise one of GemmShape, whatever the sizes (tests and measurements).
// flags: VCB_GEMM_AFTER_SMALL_KERNEL (1) -- the kernel before this one in the stream is a small one (see pf_settings).
VCB_API int vcb_gemm_bf16_tn_shape(const void* W, const void* X, void* out, int out_dtype, int M, int N, int K,
                                   long long ldw, long long ldx, long long ldc, int splits, long long split_stride,
                                   int shape, int flags, int* status, cudaStream_t stream) {
    VCB_CHECK_ARG(M > 0 && N > 0 && K > 0, "gemm_bf16_tn: bad sizes M=%d N=%d K=%d", M, N, K);
    VCB_CHECK_ARG(K % 8 == 0 && ldw % 8 == 0 && ldx % 8 == 0,
                  "gemm_bf16_tn: inner size %d and row strides %lld, %lld must be multiples of 8 (16-byte rows for TMA)", K, ldw, ldx);
    VCB_CHECK_ARG(((uintptr_t)W % 16 == 0) && ((uintptr_t)X % 16 == 0), "gemm_bf16_tn: operands must be 16-byte aligned");
    VCB_CHECK_ARG(splits >= 1 && (splits == 1 || out_dtype == VCB_F32), "gemm_bf16_tn: k-slices need 32-bit partial outputs");
    const int total_kb = (K + BK - 1) / BK;
    if (splits > total_kb) splits = total_kb;
    const int kb_per_split = (total_kb + splits - 1) / splits;
    splits = (total_kb + kb_per_split - 1) / kb_per_split;
    GemmArgs g{out, out_dtype, M, N, K, ldc, split_stride, kb_per_split, splits, 0, status};
    if ((flags & VCB_GEMM_AFTER_SMALL_KERNEL) && N <= 16 && vcb_pdl_enabled()) pf_settings(&g.pf_tiles, &g.pf_delay_ns);
    if (shape < 0 && use_pairs(M, N, K, splits)) return launch_pair(W, M, X, g, ldw, ldx, stream);
    return launch_shape(shape < 0 ? pick_shape(M, N, K, splits) : shape, W, X, g, ldw, ldx, splits, stream);
}

// Fused feed-forward front half.  W [2I, K] holds gate_i in row 2i and up_i in row 2i+1; out[t][i] =
// silu(gate_i . x_t) * (up_i . x_t), bfloat16 [N, I].  The pairing is done in the epilogue (adjacent TMEM lanes),
// so every unit shape serves; shape < 0 chooses as for a plain product of 2I features; flags as for
// vcb_gemm_bf16_tn_shape.
VCB_API int vcb_gemm_bf16_swiglu(const void* W, const void* X, void* out, int I, int N, int K, long long ldw,
                                 long long ldx, long long ldc, int shape, int flags, int* status, cudaStream_t stream) {
    VCB_CHECK_ARG(I > 0 && N > 0 && K > 0, "gemm_bf16_swiglu: bad sizes I=%d N=%d K=%d", I, N, K);
    VCB_CHECK_ARG(K % 8 == 0 && ldw % 8 == 0 && ldx % 8 == 0,
                  "gemm_bf16_swiglu: inner size %d and row strides %lld, %lld must be multiples of 8 (16-byte rows for TMA)", K, ldw, ldx);
    VCB_CHECK_ARG(((uintptr_t)W % 16 == 0) && ((uintptr_t)X % 16 == 0), "gemm_bf16_swiglu: operands must be 16-byte aligned");
    const int total_kb = (K + BK - 1) / BK;
    GemmArgs g{out, VCB_BF16, 2 * I, N, K, ldc, 0, total_kb, 1, 1, status};
    if ((flags & VCB_GEMM_AFTER_SMALL_KERNEL) && N <= 16 && vcb_pdl_enabled()) pf_settings(&g.pf_tiles, &g.pf_delay_ns);
    if (shape < 0 && use_pairs(2 * I, N, K, 1)) return launch_pair(W, 2LL * I, X, g, ldw, ldx, stream);
    return launch_shape(shape < 0 ? pick_shape(2 * I, N, K, 1) : shape, W, X, g, ldw, ldx, 1, stream);
}

// The stacked q, k, v projection of prompt portions with the per-head norm, the rotation and the cache store in its
// epilogue (head_dim 128, half-split pairs rotated over the whole head; see qkv_head_store).  W [(nh + 2 nkv) * 128, K]
// (or [nh * 128, K] with pages null: a layer that stores no keys), X [N, K] bfloat16; q_out [N, nh * 128] bfloat16;
// pages: the layer's pages, bfloat16, `page_stride` elements apart.  No k-slices: for more than 128 tokens.
VCB_API int vcb_gemm_bf16_qkv(const void* W, const void* X, int N, int K, long long ldw, long long ldx, void* q_out,
                              void* pages, long long page_stride, int page_size, int num_pages, const int* slot_map,
                              const int* positions, const float* cos_sin, int max_pos, const void* q_gain,
                              const void* k_gain, int gain_dtype, int use_norm, float eps, int nh, int nkv, int* status,
                              cudaStream_t stream) {
    VCB_CHECK_ARG(N > 0 && K > 0 && nh > 0 && nkv > 0, "gemm_bf16_qkv: bad sizes N=%d K=%d nh=%d nkv=%d", N, K, nh, nkv);
    VCB_CHECK_ARG(K % 8 == 0 && ldw % 8 == 0 && ldx % 8 == 0,
                  "gemm_bf16_qkv: inner size %d and row strides %lld, %lld must be multiples of 8 (16-byte rows for TMA)", K, ldw, ldx);
    VCB_CHECK_ARG(((uintptr_t)W % 16 == 0) && ((uintptr_t)X % 16 == 0), "gemm_bf16_qkv: operands must be 16-byte aligned");
    VCB_CHECK_ARG(q_out != nullptr && positions != nullptr && cos_sin != nullptr && status != nullptr && max_pos > 0,
                  "gemm_bf16_qkv: missing operand");
    VCB_CHECK_ARG(pages == nullptr || (slot_map != nullptr && page_size > 0 && num_pages > 0), "gemm_bf16_qkv: pages without slots or sizes");
    VCB_CHECK_ARG(!use_norm || (q_gain != nullptr && (pages == nullptr || k_gain != nullptr)), "gemm_bf16_qkv: the per-head norms need their gains");
    const int M = (nh + (pages != nullptr ? 2 * nkv : 0)) * BM;
    const int total_kb = (K + BK - 1) / BK;
    GemmArgs g{nullptr, VCB_BF16, M, N, K, 0, 0, total_kb, 1, 0, status,
               QkvEpilogue{(__nv_bfloat16*)q_out, (__nv_bfloat16*)pages, page_stride, slot_map, positions, cos_sin, q_gain, k_gain,
                           max_pos, gain_dtype, use_norm, nh, nkv, page_size, num_pages, eps}};
    // units of one head: 128 features x 256 tokens, or x 128 where those fill the SMs' rounds better (as pick_shape counts)
    auto rounds = [&](int bn) { return (((long long)(M / BM) * ((N + bn - 1) / bn) + num_sms() - 1) / num_sms()) * bn; };
    const bool narrow = N <= 128 || rounds(128) * 8 / 5 < rounds(256);
    // pairs of blocks as for a plain product of these sizes (mode 2, tests: wherever they can run)
    if ((!narrow || pairs_mode() == 2) && use_pairs(M, N, K, 1)) return launch_pair(W, M, X, g, ldw, ldx, stream);
    return narrow ? launch<128, 6, 1, 2>(W, X, g, ldw, ldx, 1, stream) : launch<256, 4, 1, 2>(W, X, g, ldw, ldx, 1, stream);
}

VCB_API int vcb_gemm_bf16_tn(const void* W, const void* X, void* out, int out_dtype, int M, int N, int K,
                             long long ldw, long long ldx, long long ldc, int splits, long long split_stride,
                             int* status, cudaStream_t stream) {
    return vcb_gemm_bf16_tn_shape(W, X, out, out_dtype, M, N, K, ldw, ldx, ldc, splits, split_stride, -1, 0, status, stream);
}

// 0: no product runs on pairs of blocks; 1: those that the rule above sends there; 2: all that can.
VCB_API void vcb_gemm_set_pairs(int mode) { g_pairs = mode < 0 ? 0 : (mode > 2 ? 2 : mode); }
