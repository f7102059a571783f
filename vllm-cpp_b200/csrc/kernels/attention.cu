// Attention over the paged cache for one step's queries, any mixture of prompt
// portions and single decoded tokens.
//
// A work item is (entry, a run of nq consecutive query tokens of that entry, one
// slice of the key range).  One block takes one item and one group of query heads
// that share a KV head, so the K/V pages are read once for all those rows
// (rows = nq tokens x gq heads).  Scores, the running maximum and sum of the
// streaming softmax and the output accumulator are 32-bit; the math per row is
//   s_j = (q . k_j) / sqrt(head_dim),  j in (pos - window, pos],  softmax,  sum_j w_j v_j
// as in the reference's compute_attention (src/model.cpp:1000-1052) and its paged
// form (src/paged_attention.cpp:11-90), without the 1e-9 guard in the divisor.
// Items whose key range is sliced write (max, sum, unnormalised output) partials,
// merged by attn_merge_kernel in slice order.
#include "common.cuh"

#include <math_constants.h>

namespace {

constexpr int TK = 128;       // keys per tile = threads per block
constexpr int ITEM_INTS = 6;  // entry, q0, nq, slice, nslices, decode index

struct AttnArgs {
    const void* q;
    void* out;
    const void* pages;
    long long page_stride;
    const int* block_table;
    const int* table_row;  // entry -> row of block_table (a request's slot), or null: row = entry
    int max_blocks;
    const int* q_start;
    const int* q_len;
    const int* ctx_len;
    const int* items;
    float* part_o;
    float* part_ml;
    int nh, nkv, hd, page_size, num_pages, window;
    float scale;
    int* status;
    // bounds of the partial-result buffers, for callers whose buffers have a fixed size (0: not checked): decoded
    // tokens and key slices that part_o / part_ml were laid out for
    int part_tokens, part_slices;
};

template <typename T> struct Vec8;
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
        const float4 a = *reinterpret_cast<const float4*>(p);
        const float4 b = *reinterpret_cast<const float4*>(p + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
};
template <> struct Vec8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

template <typename T, int RMAX>
__global__ __launch_bounds__(TK) void attn_paged_kernel(AttnArgs a) {
    extern __shared__ float smem[];
    const int hd = a.hd;
    float* q_s = smem;                      // [RMAX][hd], pre-scaled
    float* p_s = q_s + RMAX * hd;           // [RMAX][TK]
    float* m_s = p_s + RMAX * TK;           // [RMAX] running maximum
    float* l_s = m_s + RMAX;                // [RMAX] running sum
    float* al_s = l_s + RMAX;               // [RMAX] rescale factor of the current tile
    long long* voff_s = reinterpret_cast<long long*>(al_s + RMAX);  // [TK] element offset of each key's V row

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int* item = a.items + (size_t)blockIdx.x * ITEM_INTS;
    const int e = item[0], q0 = item[1], slice = item[3], nslices = item[4], dec_index = item[5];
    const int qlen = a.q_len[e], ctx = a.ctx_len[e];
    // an item of a captured step is laid out for the largest portion the step serves: fewer tokens may be there
    const int nq = min(item[2], qlen - q0);
    if (a.part_tokens > 0 &&
        (dec_index < 0 || dec_index >= a.part_tokens || slice < 0 || slice >= nslices || nslices != a.part_slices)) {
        // the item's partial row would lie outside the fixed buffer: report it and touch nothing
        if (tid == 0) atomicOr(a.status, VCB_STATUS_BAD_ITEM);
        return;
    }

    const int g = a.nh / a.nkv;
    const int gq_max = g < RMAX ? g : RMAX;
    const int hchunks = (g + gq_max - 1) / gq_max;
    const int kvh = blockIdx.y / hchunks, hc = blockIdx.y % hchunks;
    const int head0 = kvh * g + hc * gq_max;
    const int gq = min(gq_max, g - hc * gq_max);
    if (qlen <= 0 || ctx <= 0 || nq <= 0) {
        // an empty entry: its slices still say "nothing here" (max = -inf, sum = 0), so that the merge writes zeros
        // rather than whatever the partial buffers held before
        if (nslices > 1 && a.part_ml != nullptr && tid < gq) {
            const size_t prow = ((size_t)dec_index * a.nh + head0 + tid) * nslices + slice;
            a.part_ml[prow * 2] = -CUDART_INF_F;
            a.part_ml[prow * 2 + 1] = 0.f;
        }
        return;
    }
    const int R = nq * gq;  // rows in use: r = iq * gq + ih

    const int row0 = a.q_start[e] + q0;       // flat token index of the first query
    const int pos0 = ctx - qlen + q0;         // its position
    const int pos_last = pos0 + nq - 1;
    const int W = a.window;

    // key range of the whole item, then of this slice (in pages)
    const int lo = W > 0 ? max(0, pos0 - W + 1) : 0;
    const int hi = pos_last + 1;
    const int ps = a.page_size;
    const int pb_lo = lo / ps, pb_hi = (hi + ps - 1) / ps;
    const int pps = (pb_hi - pb_lo + nslices - 1) / nslices;
    const int my_pb_lo = pb_lo + slice * pps, my_pb_hi = min(pb_hi, my_pb_lo + pps);
    const int k_begin = max(lo, my_pb_lo * ps), k_end = min(hi, my_pb_hi * ps);

    // queries -> shared memory, scaled
    const T* qg = reinterpret_cast<const T*>(a.q);
    for (int idx = tid; idx < R * hd; idx += TK) {
        const int r = idx / hd, d = idx % hd;
        const int iq = r / gq, ih = r % gq;
        q_s[r * hd + d] = to_f32(qg[((size_t)(row0 + iq) * a.nh + head0 + ih) * hd + d]) * a.scale;
    }
    if (tid < RMAX) {
        m_s[tid] = -CUDART_INF_F;
        l_s[tid] = 0.f;
    }
    constexpr int DPT = VCB_MAX_HEAD_DIM / TK;  // output dims per thread
    float acc_o[RMAX][DPT];
#pragma unroll
    for (int r = 0; r < RMAX; ++r)
#pragma unroll
        for (int i = 0; i < DPT; ++i) acc_o[r][i] = 0.f;
    __syncthreads();

    const T* pages = reinterpret_cast<const T*>(a.pages);
    const int* bt = a.block_table + (size_t)(a.table_row ? a.table_row[e] : e) * a.max_blocks;

    for (int t0 = k_begin; t0 < k_end; t0 += TK) {
        const int n_valid = min(TK, k_end - t0);
        // ---- phase 1: one key per thread, scores of all rows ----
        {
            const int kidx = t0 + tid;
            float s[RMAX];
#pragma unroll
            for (int r = 0; r < RMAX; ++r) s[r] = 0.f;
            bool valid = tid < n_valid;
            if (valid) {
                const int page = bt[kidx / ps];
                if (page < 0 || page >= a.num_pages) {
                    atomicOr(a.status, VCB_STATUS_BAD_PAGE);
                    valid = false;
                    voff_s[tid] = -1;
                } else {
                    const long long base = (long long)page * a.page_stride + ((long long)kvh * ps + kidx % ps) * hd;
                    voff_s[tid] = base + (long long)a.nkv * ps * hd;
                    const T* kp = pages + base;
                    for (int c = 0; c < hd; c += 8) {
                        float kf[8];
                        Vec8<T>::load(kp + c, kf);
#pragma unroll
                        for (int r = 0; r < RMAX; ++r) {
                            if (r < R) {
                                const float4 qa = *reinterpret_cast<const float4*>(q_s + r * hd + c);
                                const float4 qb = *reinterpret_cast<const float4*>(q_s + r * hd + c + 4);
                                s[r] = fmaf(kf[0], qa.x, s[r]); s[r] = fmaf(kf[1], qa.y, s[r]);
                                s[r] = fmaf(kf[2], qa.z, s[r]); s[r] = fmaf(kf[3], qa.w, s[r]);
                                s[r] = fmaf(kf[4], qb.x, s[r]); s[r] = fmaf(kf[5], qb.y, s[r]);
                                s[r] = fmaf(kf[6], qb.z, s[r]); s[r] = fmaf(kf[7], qb.w, s[r]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < RMAX; ++r) {
                if (r < R) {
                    const int pos = pos0 + r / gq;
                    const bool seen = valid && kidx <= pos && (W <= 0 || kidx > pos - W);
                    p_s[r * TK + tid] = seen ? s[r] : -CUDART_INF_F;
                }
            }
        }
        __syncthreads();
        // ---- phase 2: streaming softmax, rows dealt to warps ----
        for (int r = warp; r < R; r += TK / 32) {
            float v[TK / 32];
            float mx = -CUDART_INF_F;
#pragma unroll
            for (int i = 0; i < TK / 32; ++i) {
                v[i] = p_s[r * TK + lane + 32 * i];
                mx = fmaxf(mx, v[i]);
            }
            mx = warp_max(mx);
            const float m_old = m_s[r];
            const float m_new = fmaxf(m_old, mx);
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < TK / 32; ++i) {
                const float p = (v[i] == -CUDART_INF_F) ? 0.f : expf(v[i] - m_new);
                p_s[r * TK + lane + 32 * i] = p;
                sum += p;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float alpha = (m_old == -CUDART_INF_F) ? 0.f : expf(m_old - m_new);
                al_s[r] = alpha;
                m_s[r] = m_new;
                l_s[r] = l_s[r] * alpha + sum;
            }
        }
        __syncthreads();
        // ---- phase 3: output dims dealt to threads ----
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = tid + i * TK;
            if (d < hd) {
#pragma unroll
                for (int r = 0; r < RMAX; ++r)
                    if (r < R) acc_o[r][i] *= al_s[r];
                for (int j = 0; j < n_valid; ++j) {
                    const long long vo = voff_s[j];
                    if (vo < 0) continue;
                    const float v = to_f32(pages[vo + d]);
#pragma unroll
                    for (int r = 0; r < RMAX; ++r)
                        if (r < R) acc_o[r][i] = fmaf(p_s[r * TK + j], v, acc_o[r][i]);
                }
            }
        }
        __syncthreads();
    }

    // ---- write out ----
    if (nslices == 1) {
        T* og = reinterpret_cast<T*>(a.out);
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = tid + i * TK;
            if (d < hd) {
#pragma unroll
                for (int r = 0; r < RMAX; ++r) {
                    if (r < R) {
                        const float l = l_s[r];
                        const int iq = r / gq, ih = r % gq;
                        og[((size_t)(row0 + iq) * a.nh + head0 + ih) * hd + d] = from_f32<T>(l > 0.f ? acc_o[r][i] / l : 0.f);
                    }
                }
            }
        }
    } else {
        // decode items only (nq == 1): partial row = (decode index, head, slice)
#pragma unroll
        for (int r = 0; r < RMAX; ++r) {
            if (r < R) {
                const size_t prow = ((size_t)dec_index * a.nh + head0 + r) * nslices + slice;
#pragma unroll
                for (int i = 0; i < DPT; ++i) {
                    const int d = tid + i * TK;
                    if (d < hd) a.part_o[prow * hd + d] = acc_o[r][i];
                }
                if (tid == 0) {
                    a.part_ml[prow * 2] = m_s[r];
                    a.part_ml[prow * 2 + 1] = l_s[r];
                }
            }
        }
    }
}

// merge the slices of sliced items: grid (decode tokens, heads)
template <typename T>
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                  const int* __restrict__ dec_rows, T* __restrict__ out, int nh, int hd, int nslices) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x, h = blockIdx.y;
    const size_t prow0 = ((size_t)n * nh + h) * nslices;
    float m = -CUDART_INF_F;
    for (int s = 0; s < nslices; ++s) m = fmaxf(m, part_ml[(prow0 + s) * 2]);
    const int row = dec_rows[n];
    if (row < 0) return;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float l = 0.f, o = 0.f;
        for (int s = 0; s < nslices; ++s) {
            const float ms = part_ml[(prow0 + s) * 2];
            if (ms == -CUDART_INF_F) continue;
            const float w = expf(ms - m);
            l += part_ml[(prow0 + s) * 2 + 1] * w;
            o += part_o[(prow0 + s) * hd + d] * w;
        }
        out[((size_t)row * nh + h) * hd + d] = from_f32<T>(l > 0.f ? o / l : 0.f);
    }
}

template <typename T, int RMAX>
int launch_attn(const AttnArgs& a, int n_items, cudaStream_t stream) {
    const int g = a.nh / a.nkv;
    const int gq_max = g < RMAX ? g : RMAX;
    const int hchunks = (g + gq_max - 1) / gq_max;
    const size_t smem = ((size_t)RMAX * a.hd + (size_t)RMAX * TK + 3 * RMAX) * sizeof(float) + TK * sizeof(long long);
    auto kern = attn_paged_kernel<T, RMAX>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            vcb_set_error("attn_paged: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
            return -2;
        }
    }
    kern<<<dim3(n_items, a.nkv * hchunks), TK, smem, stream>>>(a);
    VCB_CHECK_LAUNCH("attn_paged");
    return 0;
}

}  // namespace

// rows_max: 8 for items of single decoded tokens (key range may be sliced), 32 for prompt portions
VCB_API int vcb_attn_paged(const void* q, void* out, int dtype, const void* pages, long long page_stride,
                           const int* block_table, const int* table_row, int max_blocks, const int* q_start, const int* q_len,
                           const int* ctx_len, const int* items, int n_items, int rows_max, float* part_o,
                           float* part_ml, int nh, int nkv, int hd, int page_size, int num_pages, int window,
                           float scale, int* status, cudaStream_t stream) {
    if (n_items == 0) return 0;
    VCB_CHECK_ARG(nh > 0 && nkv > 0 && nh % nkv == 0, "attn_paged: %d query heads are not a multiple of %d KV heads", nh, nkv);
    VCB_CHECK_ARG(hd >= 16 && hd % 16 == 0 && hd <= VCB_MAX_HEAD_DIM, "attn_paged: head_dim %d must be a multiple of 16 in [16, %d]", hd, VCB_MAX_HEAD_DIM);
    VCB_CHECK_ARG(rows_max == 8 || rows_max == 32, "attn_paged: rows_max must be 8 or 32");
    VCB_CHECK_ARG(page_size > 0 && window >= 0, "attn_paged: bad page_size %d or window %d", page_size, window);
    AttnArgs a{q, out, pages, page_stride, block_table, table_row, max_blocks, q_start, q_len, ctx_len, items, part_o, part_ml,
               nh, nkv, hd, page_size, num_pages, window, scale, status, 0, 0};
    if (dtype == VCB_F32) return rows_max == 8 ? launch_attn<float, 8>(a, n_items, stream) : launch_attn<float, 32>(a, n_items, stream);
    return rows_max == 8 ? launch_attn<__nv_bfloat16, 8>(a, n_items, stream) : launch_attn<__nv_bfloat16, 32>(a, n_items, stream);
}

VCB_API int vcb_attn_merge(const float* part_o, const float* part_ml, const int* dec_rows, void* out, int dtype,
                           int n_dec, int nh, int hd, int nslices, cudaStream_t stream) {
    if (n_dec == 0) return 0;
    const int threads = hd <= 64 ? 64 : (hd <= 128 ? 128 : 256);
    if (dtype == VCB_F32)
        launch_pdl(attn_merge_kernel<float>, dim3(n_dec, nh), dim3(threads), 0, stream, part_o, part_ml, dec_rows, (float*)out, nh, hd, nslices);
    else
        launch_pdl(attn_merge_kernel<__nv_bfloat16>, dim3(n_dec, nh), dim3(threads), 0, stream, part_o, part_ml, dec_rows, (__nv_bfloat16*)out, nh, hd, nslices);
    VCB_CHECK_LAUNCH("attn_merge");
    return 0;
}

// ---------------------------------------------------------------------------
// Sliced decode attention that allocates nothing (declared in no_alloc_api.h).
//
// Same kernels as vcb_attn_paged + vcb_attn_merge, but the (max, sum, output) partials of the key slices live in
// a fixed array inside this library instead of buffers the caller allocates.  The array exists once per GPU that
// loads the library, from load until exit, whether or not this entry point is ever called.
// ---------------------------------------------------------------------------
#include "no_alloc_api.h"

#include <mutex>

static __device__ __align__(256) float g_decode_partials[VCB_NO_ALLOC_SCRATCH_FLOATS];

namespace {
constexpr int MAX_DEVICES = 64;
float* g_partials_addr[MAX_DEVICES];   // device address of g_decode_partials on each device, once looked up
bool g_partials_known[MAX_DEVICES];
std::mutex g_partials_mutex;

// In host code `g_decode_partials` is only a handle for the runtime; the address a kernel can use must be asked
// for, per device, with that device current.
int partials_address(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        vcb_set_error("attn_decode_no_alloc: cannot tell the current device (%s)", cudaGetErrorString(e));
        return -2;
    }
    std::lock_guard<std::mutex> lock(g_partials_mutex);
    if (!g_partials_known[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_decode_partials);
        if (e != cudaSuccess || p == nullptr) {
            vcb_set_error("attn_decode_no_alloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
            return -2;
        }
        g_partials_addr[dev] = static_cast<float*>(p);
        g_partials_known[dev] = true;
    }
    *out = g_partials_addr[dev];
    return 0;
}
}  // namespace

VCB_API int vcb_attn_decode_no_alloc(const void* q, void* out, int dtype, const void* pages, long long page_stride,
                                     const int* block_table, const int* table_row, int max_blocks,
                                     const int* q_start, const int* q_len, const int* ctx_len, const int* items,
                                     const int* dec_rows, int n_dec, int nslices, int nh, int nkv, int hd,
                                     int page_size, int num_pages, int window, float scale, int* status,
                                     cudaStream_t stream) {
    if (n_dec == 0) return 0;
    VCB_CHECK_ARG(n_dec > 0 && nslices >= 2, "attn_decode_no_alloc: needs at least one token and two key slices (got %d, %d)", n_dec, nslices);
    VCB_CHECK_ARG(nh > 0 && nkv > 0 && nh % nkv == 0, "attn_decode_no_alloc: %d query heads are not a multiple of %d KV heads", nh, nkv);
    VCB_CHECK_ARG(hd >= 16 && hd % 16 == 0 && hd <= VCB_MAX_HEAD_DIM, "attn_decode_no_alloc: head_dim %d must be a multiple of 16 in [16, %d]", hd, VCB_MAX_HEAD_DIM);
    VCB_CHECK_ARG(page_size > 0 && window >= 0, "attn_decode_no_alloc: bad page_size %d or window %d", page_size, window);
    const long long rows = (long long)n_dec * nh * nslices;
    const long long need = rows * (hd + 2);
    VCB_CHECK_ARG(need <= (long long)VCB_NO_ALLOC_SCRATCH_FLOATS,
                  "attn_decode_no_alloc: %d tokens x %d heads x %d slices x (head_dim %d + 2) = %lld floats of partials exceed "
                  "the built-in scratch of %lld floats; use fewer slices or the allocating entry points",
                  n_dec, nh, nslices, hd, need, (long long)VCB_NO_ALLOC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    if (int rc = partials_address(&scratch)) return rc;
    float* part_o = scratch;               // [rows, hd]
    float* part_ml = scratch + rows * hd;  // [rows, 2]
    // Every (token, head, slice) row is written by the block that owns it before the merge reads it -- an empty
    // slice and an entry without tokens write max = -inf, sum = 0 -- so nothing of an earlier call's contents is
    // read and nothing has to be cleared.  The one exception is an item the kernel refuses (see below): its rows
    // keep what they held, the status word says so, and the output of that token is not to be used.
    // The kernel checks every item against the layout the array was cut for (n_dec tokens, nslices slices): an item
    // naming a token or slice beyond it, or another slice count, sets VCB_STATUS_BAD_ITEM and writes nothing.
    VCB_CHECK_ARG(status != nullptr, "attn_decode_no_alloc: a status word is required (bad items are reported there)");
    AttnArgs a{q, out, pages, page_stride, block_table, table_row, max_blocks, q_start, q_len, ctx_len, items, part_o,
               part_ml, nh, nkv, hd, page_size, num_pages, window, scale, status, n_dec, nslices};
    const int rc = dtype == VCB_F32 ? launch_attn<float, 8>(a, n_dec * nslices, stream)
                                    : launch_attn<__nv_bfloat16, 8>(a, n_dec * nslices, stream);
    if (rc) return rc;
    const int threads = hd <= 64 ? 64 : (hd <= 128 ? 128 : 256);
    if (dtype == VCB_F32)
        launch_pdl(attn_merge_kernel<float>, dim3(n_dec, nh), dim3(threads), 0, stream, part_o, part_ml, dec_rows, (float*)out, nh, hd, nslices);
    else
        launch_pdl(attn_merge_kernel<__nv_bfloat16>, dim3(n_dec, nh), dim3(threads), 0, stream, part_o, part_ml, dec_rows, (__nv_bfloat16*)out, nh, hd, nslices);
    VCB_CHECK_LAUNCH("attn_decode_no_alloc merge");
    return 0;
}
