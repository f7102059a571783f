// Bandwidth-bound kernels of one model step: embedding gather, fused
// residual-add + RMSNorm, SiLU-gate product, and the fused per-head
// RMSNorm + rotary rotation + cache-page write.
//
// Statistics (sums of squares), rotation arithmetic and the residual stream are
// 32-bit in both precisions; only stored activations follow the engine dtype.
// Formulas: RMSNorm src/model.cpp:924-930 of the reference, per-head norm
// cuda/attention.cu:169-182, half-split rotation cuda/attention_kernels.cuh:275-287,
// SiLU src/model.cpp:964-966, page write src/paged_attention.cpp:127-142.
#include "common.cuh"

#include <stdarg.h>

// ---------------------------------------------------------------------------
// error text shared by all launchers of the library
// ---------------------------------------------------------------------------
static thread_local char g_last_error[512] = "";

void vcb_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
}

VCB_API const char* vcb_last_error() { return g_last_error; }

// ---------------------------------------------------------------------------
// embedding gather: out[t,:] = table[ids[t],:] widened to 32-bit
// ---------------------------------------------------------------------------
__global__ void embed_gather_kernel(const void* __restrict__ table, int table_dtype, const int* __restrict__ ids,
                                    float* __restrict__ out, int H, int V, int* status) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < V;
    if (!ok && threadIdx.x == 0) atomicOr(status, VCB_STATUS_BAD_TOKEN);
    float* dst = out + (size_t)t * H;
    for (int h = threadIdx.x; h < H; h += blockDim.x)
        dst[h] = ok ? load_as_f32(table, table_dtype, (size_t)id * H + h) : 0.f;
}

VCB_API int vcb_embed_gather(const void* table, int table_dtype, const int* ids, float* out, int T, int H, int V,
                             int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    VCB_CHECK_ARG(T > 0 && H > 0 && V > 0, "embed_gather: bad sizes T=%d H=%d V=%d", T, H, V);
    embed_gather_kernel<<<T, 256, 0, stream>>>(table, table_dtype, ids, out, H, V, status);
    VCB_CHECK_LAUNCH("embed_gather");
    return 0;
}

// ---------------------------------------------------------------------------
// fused residual add + RMSNorm
//   x = resid[r] + sum_s delta[s][r];  resid[r] = x (unless rows are gathered);
//   out[i] = w * x / sqrt(mean(x^2) + eps)
// ---------------------------------------------------------------------------
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const void* __restrict__ delta, int delta_dtype, int S,
                                   size_t delta_stride, const void* __restrict__ w, int w_dtype, float eps,
                                   void* __restrict__ out, int out_dtype, const int* __restrict__ rows, int H) {
    extern __shared__ float smem[];
    float* xs = smem;
    float* scratch = smem + H;
    const int i = blockIdx.x;
    const size_t r = rows ? (size_t)rows[i] : (size_t)i;
    const bool write_back = rows == nullptr && S > 0;
    float ss = 0.f;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float x = resid[r * H + h];
        for (int s = 0; s < S; ++s) x += load_as_f32(delta, delta_dtype, (size_t)s * delta_stride + r * H + h);
        xs[h] = x;
        ss += x * x;
        if (write_back) resid[r * H + h] = x;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    for (int h = threadIdx.x; h < H; h += blockDim.x)
        store_from_f32(out, out_dtype, (size_t)i * H + h, load_as_f32(w, w_dtype, h) * xs[h] * inv);
}

VCB_API int vcb_add_rmsnorm(float* resid, const void* delta, int delta_dtype, int S, long long delta_stride,
                            const void* w, int w_dtype, float eps, void* out, int out_dtype, const int* rows,
                            int n_out, int H, cudaStream_t stream) {
    if (n_out == 0) return 0;
    VCB_CHECK_ARG(n_out > 0 && H > 0 && S >= 0, "add_rmsnorm: bad sizes n=%d H=%d S=%d", n_out, H, S);
    const size_t smem = ((size_t)H + 40) * sizeof(float);
    VCB_CHECK_ARG(smem <= 200 * 1024, "add_rmsnorm: width %d needs %zu bytes of shared memory (limit 204800)", H, smem);
    static bool opted_in = false;
    if (smem > 48 * 1024 && !opted_in) {
        cudaFuncSetAttribute(add_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        opted_in = true;
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    add_rmsnorm_kernel<<<n_out, threads, smem, stream>>>(resid, delta, delta_dtype, S, (size_t)delta_stride, w, w_dtype,
                                                         eps, out, out_dtype, rows, H);
    VCB_CHECK_LAUNCH("add_rmsnorm");
    return 0;
}

// ---------------------------------------------------------------------------
// SiLU-gate product: out[t,i] = silu(gu[t,i]) * gu[t,I+i]
// ---------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I, i = idx % I;
        const float g = to_f32(gu[t * 2 * I + i]);
        const float u = to_f32(gu[t * 2 * I + I + i]);
        out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

VCB_API int vcb_swiglu(const void* gate_up, void* out, int dtype, int T, int I, cudaStream_t stream) {
    if (T == 0) return 0;
    VCB_CHECK_ARG(T > 0 && I > 0, "swiglu: bad sizes T=%d I=%d", T, I);
    const size_t total = (size_t)T * I;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (dtype == VCB_F32) swiglu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gate_up, (float*)out, I, total);
    else swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, I, total);
    VCB_CHECK_LAUNCH("swiglu");
    return 0;
}

// ---------------------------------------------------------------------------
// per-head RMSNorm of Q and K, rotary rotation by the token's position, Q store,
// and K/V scatter into the token's cache page.  One warp per (token, head).
//   qkv:     [T, (nh + 2 nkv) * hd]   (only [T, nh * hd] when has_kv == 0)
//   cos_sin: [max_pos, hd]  (hd/2 cosines then hd/2 sines, 32-bit)
//   pages:   [num_pages, 2, nkv, page_size, hd] of one layer
// ---------------------------------------------------------------------------
template <typename T>
__global__ void qknorm_rope_kvwrite_kernel(const T* __restrict__ qkv, const void* __restrict__ qw,
                                           const void* __restrict__ kw, int w_dtype, int use_norm, float eps,
                                           const float* __restrict__ cos_sin, int max_pos,
                                           const int* __restrict__ positions, const int* __restrict__ slot_map,
                                           T* __restrict__ q_out, T* __restrict__ pages, long long page_stride,
                                           int page_size, int num_pages, int nh, int nkv, int hd, int n_tokens,
                                           int has_kv, int* status) {
    const int lane = threadIdx.x & 31;
    const int heads_total = nh + (has_kv ? 2 * nkv : 0);
    const long long gw = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (gw >= (long long)n_tokens * heads_total) return;
    const int t = (int)(gw / heads_total), h = (int)(gw % heads_total);
    const T* src = qkv + (size_t)t * heads_total * hd + (size_t)h * hd;
    const int half = hd >> 1;

    long long slot = -1;
    if (h >= nh) {
        slot = slot_map[t];
        if (slot < 0) return;  // padded token: nothing to store
        if (slot / page_size >= num_pages) {
            if (lane == 0) atomicOr(status, VCB_STATUS_BAD_PAGE);
            return;
        }
    }

    if (h >= nh + nkv) {  // V head: stored as it is
        const int kvh = h - nh - nkv;
        T* dst = pages + (slot / page_size) * page_stride + ((size_t)(nkv + kvh) * page_size + slot % page_size) * hd;
        for (int i = lane; i < hd; i += 32) dst[i] = src[i];
        return;
    }

    int pos = positions[t];
    if (pos < 0 || pos >= max_pos) {
        if (lane == 0) atomicOr(status, VCB_STATUS_BAD_POSITION);
        pos = 0;
    }
    constexpr int MAXP = VCB_MAX_HEAD_DIM / 64;  // pairs per lane
    float x1[MAXP], x2[MAXP];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < MAXP; ++j) {
        const int p = lane + 32 * j;
        if (p < half) {
            x1[j] = to_f32(src[p]);
            x2[j] = to_f32(src[p + half]);
            ss += x1[j] * x1[j] + x2[j] * x2[j];
        }
    }
    const void* gain = h < nh ? qw : kw;
    float inv = 1.f;
    if (use_norm) {
        ss = warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)hd + eps);
    }
    T* dst;
    if (h < nh) dst = q_out + (size_t)t * nh * hd + (size_t)h * hd;
    else dst = pages + (slot / page_size) * page_stride + ((size_t)(h - nh) * page_size + slot % page_size) * hd;
    const float* cs = cos_sin + (size_t)pos * hd;
#pragma unroll
    for (int j = 0; j < MAXP; ++j) {
        const int p = lane + 32 * j;
        if (p < half) {
            float a = x1[j], b = x2[j];
            if (use_norm) {
                a = load_as_f32(gain, w_dtype, p) * a * inv;
                b = load_as_f32(gain, w_dtype, p + half) * b * inv;
            }
            const float c = cs[p], s = cs[half + p];
            dst[p] = from_f32<T>(a * c - b * s);
            dst[p + half] = from_f32<T>(b * c + a * s);
        }
    }
}

VCB_API int vcb_qknorm_rope_kvwrite(const void* qkv, int dtype, const void* qw, const void* kw, int w_dtype,
                                    int use_norm, float eps, const float* cos_sin, int max_pos, const int* positions,
                                    const int* slot_map, void* q_out, void* pages, long long page_stride,
                                    int page_size, int num_pages, int nh, int nkv, int hd, int T, int has_kv,
                                    int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    VCB_CHECK_ARG(hd > 0 && hd % 2 == 0 && hd <= VCB_MAX_HEAD_DIM,
                  "qknorm_rope_kvwrite: head_dim %d must be even and <= %d", hd, VCB_MAX_HEAD_DIM);
    VCB_CHECK_ARG(nh > 0 && nkv > 0 && page_size > 0, "qknorm_rope_kvwrite: bad sizes nh=%d nkv=%d page=%d", nh, nkv,
                  page_size);
    const long long warps = (long long)T * (nh + (has_kv ? 2 * nkv : 0));
    const int wpb = 4;
    const long long blocks = (warps + wpb - 1) / wpb;
    VCB_CHECK_ARG(blocks < (1ll << 31), "qknorm_rope_kvwrite: too many blocks");
    if (dtype == VCB_F32)
        qknorm_rope_kvwrite_kernel<float><<<(unsigned)blocks, wpb * 32, 0, stream>>>(
            (const float*)qkv, qw, kw, w_dtype, use_norm, eps, cos_sin, max_pos, positions, slot_map, (float*)q_out,
            (float*)pages, page_stride, page_size, num_pages, nh, nkv, hd, T, has_kv, status);
    else
        qknorm_rope_kvwrite_kernel<__nv_bfloat16><<<(unsigned)blocks, wpb * 32, 0, stream>>>(
            (const __nv_bfloat16*)qkv, qw, kw, w_dtype, use_norm, eps, cos_sin, max_pos, positions, slot_map,
            (__nv_bfloat16*)q_out, (__nv_bfloat16*)pages, page_stride, page_size, num_pages, nh, nkv, hd, T, has_kv,
            status);
    VCB_CHECK_LAUNCH("qknorm_rope_kvwrite");
    return 0;
}

// ---------------------------------------------------------------------------
// dst[idx[i]] = val[i]: how new block-table entries reach the device-resident tables
// ---------------------------------------------------------------------------
__global__ void scatter_i32_kernel(int* __restrict__ dst, const int* __restrict__ idx, const int* __restrict__ val,
                                   const int* __restrict__ count, int capacity, long long dst_size) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int n = min(*count, capacity);
    if (i < n && idx[i] >= 0 && idx[i] < dst_size) dst[idx[i]] = val[i];
}

// count lives on the device so that a captured launch can serve any number of updates up to capacity
VCB_API int vcb_scatter_i32(int* dst, const int* idx, const int* val, const int* count, int capacity,
                            long long dst_size, cudaStream_t stream) {
    if (capacity == 0) return 0;
    scatter_i32_kernel<<<(capacity + 255) / 256, 256, 0, stream>>>(dst, idx, val, count, capacity, dst_size);
    VCB_CHECK_LAUNCH("scatter_i32");
    return 0;
}
