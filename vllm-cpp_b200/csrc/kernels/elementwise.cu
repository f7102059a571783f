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
#include <stdlib.h>

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

// VLLM_CPP_B200_PDL=0 turns programmatic dependent launch off (every kernel then waits for the one before it)
bool vcb_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("VLLM_CPP_B200_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

// ---------------------------------------------------------------------------
// embedding gather: out[t,:] = table[ids[t],:] widened to 32-bit
// ---------------------------------------------------------------------------
__global__ void embed_gather_kernel(const void* __restrict__ table, int table_dtype, const int* __restrict__ ids,
                                    float* __restrict__ out, int H, int V, int* status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < V;
    if (!ok && threadIdx.x == 0) atomicOr(status, VCB_STATUS_BAD_TOKEN);
    float* dst = out + (size_t)t * H;
    for (int h = threadIdx.x; h < H; h += blockDim.x)
        dst[h] = ok ? load_as_f32(table, table_dtype, (size_t)id * H + h) : 0.f;
}

VCB_TIMELINE_UNIT(elementwise)

VCB_API int vcb_embed_gather(const void* table, int table_dtype, const int* ids, float* out, int T, int H, int V,
                             int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    VCB_CHECK_ARG(T > 0 && H > 0 && V > 0, "embed_gather: bad sizes T=%d H=%d V=%d", T, H, V);
    launch_pdl(embed_gather_kernel, dim3(T), dim3(256), 0, stream, table, table_dtype, ids, out, H, V, status);
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

// Same contract for the shapes serving uses (H a multiple of 4, 32-bit deltas, bfloat16 out): 16-byte loads, every
// load of a row issued before any is used, the row kept in registers.  VPT = float4s per thread.
template <int VPT>
__global__ __launch_bounds__(1024) void add_rmsnorm_vec_kernel(float* __restrict__ resid, const float* __restrict__ delta,
                                                               int S, size_t delta_stride, const void* __restrict__ w,
                                                               int w_dtype, float eps, __nv_bfloat16* __restrict__ out,
                                                               const int* __restrict__ rows, int H) {
    __shared__ float scratch[33];
    pdl_trigger();
    tl_mark(VCB_TL_NORM, 0);
    // What no kernel of the step writes -- the row index and the gains -- is read before waiting for the kernel
    // that produces the sums, so that only one round trip to memory follows the wait.
    const int i = blockIdx.x;
    const size_t r = rows ? (size_t)rows[i] : (size_t)i;
    const bool write_back = rows == nullptr && S > 0;
    const int H4 = H >> 2;
    float4 gain[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int c = threadIdx.x + v * blockDim.x;
        if (c < H4) {
            const int h = c * 4;
            gain[v] = make_float4(load_as_f32(w, w_dtype, h), load_as_f32(w, w_dtype, h + 1), load_as_f32(w, w_dtype, h + 2),
                                  load_as_f32(w, w_dtype, h + 3));
        }
    }
    pdl_wait();
    tl_mark(VCB_TL_NORM, 1);
    float4 x[VPT];
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int c = threadIdx.x + v * blockDim.x;
        if (c < H4) x[v] = reinterpret_cast<const float4*>(resid + r * H)[c];
    }
    // the slices' loads are issued several at a time before any is added: one round trip to memory for up to four
    // slices instead of one each (they are added in slice order all the same); wide rows, which hold more of a row
    // per thread, take fewer at a time to stay within the registers of a 1024-thread block
    constexpr int G = VPT == 1 ? 4 : (VPT == 2 ? 2 : 1);
    for (int s0 = 0; s0 < S; s0 += G) {
        float4 d[G][VPT];
#pragma unroll
        for (int j = 0; j < G; ++j) {
            if (s0 + j < S) {
                const float4* d4 = reinterpret_cast<const float4*>(delta + (size_t)(s0 + j) * delta_stride + r * H);
#pragma unroll
                for (int v = 0; v < VPT; ++v) {
                    const int c = threadIdx.x + v * blockDim.x;
                    if (c < H4) d[j][v] = d4[c];
                }
            }
        }
#pragma unroll
        for (int j = 0; j < G; ++j) {
            if (s0 + j < S) {
#pragma unroll
                for (int v = 0; v < VPT; ++v) {
                    const int c = threadIdx.x + v * blockDim.x;
                    if (c < H4) { x[v].x += d[j][v].x; x[v].y += d[j][v].y; x[v].z += d[j][v].z; x[v].w += d[j][v].w; }
                }
            }
        }
    }
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int c = threadIdx.x + v * blockDim.x;
        if (c < H4) {
            ss += x[v].x * x[v].x + x[v].y * x[v].y + x[v].z * x[v].z + x[v].w * x[v].w;
            if (write_back) reinterpret_cast<float4*>(resid + r * H)[c] = x[v];
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int c = threadIdx.x + v * blockDim.x;
        if (c < H4) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(gain[v].x * x[v].x * inv, gain[v].y * x[v].y * inv);
            __nv_bfloat162 hi = __floats2bfloat162_rn(gain[v].z * x[v].z * inv, gain[v].w * x[v].w * inv);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo);
            pk.y = *reinterpret_cast<uint32_t*>(&hi);
            reinterpret_cast<uint2*>(out + (size_t)i * H)[c] = pk;
        }
    }
    tl_mark(VCB_TL_NORM, 2);
}

// The same for many rows (prompt portions; at most one slice of deltas, every row in place): blocks walk the rows
// and ask for the next row's values before they reduce the current one, so that loads stay in flight across the
// block-wide sum.  One row a block left the memory system a third busy (24 us for 2,048 rows of 4096).
template <int VPT>
__global__ __launch_bounds__(1024) void add_rmsnorm_stream_kernel(float* __restrict__ resid, const float* __restrict__ delta,
                                                                  int S, const void* __restrict__ w, int w_dtype, float eps,
                                                                  __nv_bfloat16* __restrict__ out, int n_rows, int H) {
    __shared__ float scratch[33];
    pdl_trigger();
    const int H4 = H >> 2;
    float4 gain[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int c = threadIdx.x + v * blockDim.x;
        if (c < H4) {
            const int h = c * 4;
            gain[v] = make_float4(load_as_f32(w, w_dtype, h), load_as_f32(w, w_dtype, h + 1), load_as_f32(w, w_dtype, h + 2),
                                  load_as_f32(w, w_dtype, h + 3));
        }
    }
    pdl_wait();
    float4 xr[VPT], xd[VPT], nr[VPT], nd[VPT];
    auto fetch = [&](int row, float4* r4, float4* d4) {
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int c = threadIdx.x + v * blockDim.x;
            d4[v] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < H4) {
                r4[v] = reinterpret_cast<const float4*>(resid + (size_t)row * H)[c];
                if (S > 0) d4[v] = reinterpret_cast<const float4*>(delta + (size_t)row * H)[c];
            }
        }
    };
    int row = blockIdx.x;
    if (row < n_rows) fetch(row, xr, xd);
    for (; row < n_rows; row += gridDim.x) {
        const int next = row + gridDim.x;
        if (next < n_rows) fetch(next, nr, nd);
        float ss = 0.f;
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int c = threadIdx.x + v * blockDim.x;
            if (c < H4) {
                xr[v].x += xd[v].x; xr[v].y += xd[v].y; xr[v].z += xd[v].z; xr[v].w += xd[v].w;
                ss += xr[v].x * xr[v].x + xr[v].y * xr[v].y + xr[v].z * xr[v].z + xr[v].w * xr[v].w;
                if (S > 0) reinterpret_cast<float4*>(resid + (size_t)row * H)[c] = xr[v];
            }
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int c = threadIdx.x + v * blockDim.x;
            if (c < H4) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(gain[v].x * xr[v].x * inv, gain[v].y * xr[v].y * inv);
                __nv_bfloat162 hi = __floats2bfloat162_rn(gain[v].z * xr[v].z * inv, gain[v].w * xr[v].w * inv);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo);
                pk.y = *reinterpret_cast<uint32_t*>(&hi);
                reinterpret_cast<uint2*>(out + (size_t)row * H)[c] = pk;
            }
        }
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            xr[v] = nr[v];
            xd[v] = nd[v];
        }
    }
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
    const bool vec = H % 4 == 0 && out_dtype == VCB_BF16 && (S == 0 || delta_dtype == VCB_F32) && delta_stride % 4 == 0 &&
                     ((uintptr_t)resid % 16 == 0) && ((uintptr_t)delta % 16 == 0) && ((uintptr_t)out % 8 == 0) && H <= 16384;
    if (vec) {
        const int H4 = H / 4;
        int threads = H4 >= 1024 ? 1024 : ((H4 + 31) / 32) * 32;
        // More rows than SMs: blocks of 1024 threads are resident one an SM (registers), so 256 rows of 4096 ran as
        // two rounds of blocks (9 us in the step); with 512 threads and two float4s each, two are, and one round does.
        static int sms = 0;
        if (sms == 0 && (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0) != cudaSuccess || sms <= 0)) sms = 148;
        if (n_out > sms && threads == 1024 && H4 <= 2048) threads = 512;
        const int vpt = (H4 + threads - 1) / threads;
        const float* d = (const float*)delta;
        __nv_bfloat16* o = (__nv_bfloat16*)out;
        if (rows == nullptr && S <= 1 && n_out > 4 * 148 && vpt <= 2) {
            const int grid = 2 * 148;   // two blocks of 1024 threads fill an SM
            if (vpt == 1) launch_pdl(add_rmsnorm_stream_kernel<1>, dim3(grid), dim3(threads), 0, stream, resid, d, S, w, w_dtype, eps, o, n_out, H);
            else launch_pdl(add_rmsnorm_stream_kernel<2>, dim3(grid), dim3(threads), 0, stream, resid, d, S, w, w_dtype, eps, o, n_out, H);
            VCB_CHECK_LAUNCH("add_rmsnorm");
            return 0;
        }
        if (vpt == 1) launch_pdl(add_rmsnorm_vec_kernel<1>, dim3(n_out), dim3(threads), 0, stream, resid, d, S, (size_t)delta_stride, w, w_dtype, eps, o, rows, H);
        else if (vpt == 2) launch_pdl(add_rmsnorm_vec_kernel<2>, dim3(n_out), dim3(threads), 0, stream, resid, d, S, (size_t)delta_stride, w, w_dtype, eps, o, rows, H);
        else launch_pdl(add_rmsnorm_vec_kernel<4>, dim3(n_out), dim3(threads), 0, stream, resid, d, S, (size_t)delta_stride, w, w_dtype, eps, o, rows, H);
        VCB_CHECK_LAUNCH("add_rmsnorm");
        return 0;
    }
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    add_rmsnorm_kernel<<<n_out, threads, smem, stream>>>(resid, delta, delta_dtype, S, (size_t)delta_stride, w, w_dtype,
                                                         eps, out, out_dtype, rows, H);
    VCB_CHECK_LAUNCH("add_rmsnorm");
    return 0;
}

// ---------------------------------------------------------------------------
// SiLU-gate product: out[t,i] = silu(gu[t,2i]) * gu[t,2i+1]   (gate and up alternate along a row)
// ---------------------------------------------------------------------------
template <typename TIN, typename T>
__global__ void swiglu_kernel(const TIN* __restrict__ gu, int S, size_t s_stride, T* __restrict__ out, int I, size_t total) {
    pdl_trigger();
    tl_mark(VCB_TL_SWIGLU, 0);
    pdl_wait();
    tl_mark(VCB_TL_SWIGLU, 1);
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I, i = idx % I;
        float g = 0.f, u = 0.f;
        // k-slice partials of the product are added in slice order; their loads go out four slices at a time
        for (int s0 = 0; s0 < S; s0 += 4) {
            float gs[4], us[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (s0 + j < S) {
                    gs[j] = to_f32(gu[(s0 + j) * s_stride + t * 2 * I + 2 * i]);
                    us[j] = to_f32(gu[(s0 + j) * s_stride + t * 2 * I + 2 * i + 1]);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (s0 + j < S) { g += gs[j]; u += us[j]; }
            }
        }
        out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
    tl_mark(VCB_TL_SWIGLU, 2);
}

// 32-bit k-slice partial sums in, bfloat16 out, I a multiple of 4: a thread makes four outputs from two 16-byte loads a
// slice (g0 u0 g1 u1, g2 u2 g3 u3), all slices' loads of up to four slices in flight together, added in slice order.
__global__ void swiglu_partials_vec_kernel(const float* __restrict__ gu, int S, size_t s_stride, __nv_bfloat16* __restrict__ out,
                                           int I4, size_t total4) {
    pdl_trigger();
    tl_mark(VCB_TL_SWIGLU, 0);
    pdl_wait();
    tl_mark(VCB_TL_SWIGLU, 1);
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total4; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I4, i = idx % I4;
        const float4* src = reinterpret_cast<const float4*>(gu + t * 8 * (size_t)I4) + 2 * i;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
        for (int s0 = 0; s0 < S; s0 += 4) {
            float4 ta[4], tb[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (s0 + j < S) {
                    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src) + (size_t)(s0 + j) * s_stride);
                    ta[j] = p[0];
                    tb[j] = p[1];
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (s0 + j < S) {
                    a.x += ta[j].x; a.y += ta[j].y; a.z += ta[j].z; a.w += ta[j].w;
                    b.x += tb[j].x; b.y += tb[j].y; b.z += tb[j].z; b.w += tb[j].w;
                }
            }
        }
        __nv_bfloat162 lo = __floats2bfloat162_rn(a.x / (1.0f + expf(-a.x)) * a.y, a.z / (1.0f + expf(-a.z)) * a.w);
        __nv_bfloat162 hi = __floats2bfloat162_rn(b.x / (1.0f + expf(-b.x)) * b.y, b.z / (1.0f + expf(-b.z)) * b.w);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&lo);
        pk.y = *reinterpret_cast<uint32_t*>(&hi);
        reinterpret_cast<uint2*>(out)[idx] = pk;
    }
    tl_mark(VCB_TL_SWIGLU, 2);
}

// bfloat16 in and out, one slice, I a multiple of 8: 16-byte loads and stores
__global__ void swiglu_bf16_vec_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int I8, size_t total8) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I8, i = idx % I8;
        // 16 inputs (8 gate/up pairs) -> 8 outputs
        const uint4 a4 = reinterpret_cast<const uint4*>(gu + t * 16 * I8)[2 * i];
        const uint4 b4 = reinterpret_cast<const uint4*>(gu + t * 16 * I8)[2 * i + 1];
        const uint32_t w[8] = {a4.x, a4.y, a4.z, a4.w, b4.x, b4.y, b4.z, b4.w};   // each word: gate (low half), up (high half)
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float g0 = __uint_as_float(w[2 * k] << 16), u0 = __uint_as_float(w[2 * k] & 0xffff0000u);
            const float g1 = __uint_as_float(w[2 * k + 1] << 16), u1 = __uint_as_float(w[2 * k + 1] & 0xffff0000u);
            __nv_bfloat162 o = __floats2bfloat162_rn(g0 / (1.0f + expf(-g0)) * u0, g1 / (1.0f + expf(-g1)) * u1);
            ow[k] = *reinterpret_cast<uint32_t*>(&o);
        }
        reinterpret_cast<uint4*>(out + t * 8 * I8)[i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

// gate_up: [S, T, 2I] of in_dtype (S partial sums, s_stride elements apart), gate_i at 2i and up_i at 2i+1;
// out: [T, I] of out_dtype
VCB_API int vcb_swiglu(const void* gate_up, int in_dtype, int S, long long s_stride, void* out, int out_dtype, int T,
                       int I, cudaStream_t stream) {
    if (T == 0) return 0;
    VCB_CHECK_ARG(T > 0 && I > 0 && S >= 1, "swiglu: bad sizes T=%d I=%d S=%d", T, I, S);
    const size_t total = (size_t)T * I;
    if (in_dtype == VCB_BF16 && out_dtype == VCB_BF16 && S == 1 && I % 8 == 0 && ((uintptr_t)gate_up % 16 == 0) &&
        ((uintptr_t)out % 16 == 0)) {
        const size_t total8 = total / 8;
        const int nb = (int)((total8 + 255) / 256 < 148 * 32 ? (total8 + 255) / 256 : 148 * 32);
        swiglu_bf16_vec_kernel<<<nb, 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, I / 8, total8);
        VCB_CHECK_LAUNCH("swiglu");
        return 0;
    }
    if (in_dtype == VCB_F32 && out_dtype == VCB_BF16 && I % 4 == 0 && s_stride % 4 == 0 && ((uintptr_t)gate_up % 16 == 0) &&
        ((uintptr_t)out % 8 == 0)) {
        const size_t total4 = total / 4;
        const int nb = (int)((total4 + 255) / 256 < 148 * 8 ? (total4 + 255) / 256 : 148 * 8);   // all blocks resident at once
        launch_pdl(swiglu_partials_vec_kernel, dim3(nb), dim3(256), 0, stream, (const float*)gate_up, S, (size_t)s_stride,
                   (__nv_bfloat16*)out, I / 4, total4);
        VCB_CHECK_LAUNCH("swiglu");
        return 0;
    }
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    if (in_dtype == VCB_F32 && out_dtype == VCB_F32)
        launch_pdl(swiglu_kernel<float, float>, dim3(blocks), dim3(256), 0, stream, (const float*)gate_up, S, (size_t)s_stride, (float*)out, I, total);
    else if (in_dtype == VCB_F32)
        launch_pdl(swiglu_kernel<float, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const float*)gate_up, S, (size_t)s_stride, (__nv_bfloat16*)out, I, total);
    else if (out_dtype == VCB_BF16)
        launch_pdl(swiglu_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gate_up, S, (size_t)s_stride, (__nv_bfloat16*)out, I, total);
    else { vcb_set_error("swiglu: bfloat16 input with 32-bit output is not a combination the engine uses"); return -1; }
    VCB_CHECK_LAUNCH("swiglu");
    return 0;
}

// ---------------------------------------------------------------------------
// per-head RMSNorm of Q and K, rotary rotation by the token's position, Q store,
// and K/V scatter into the token's cache page.  One warp per (token, head).
//   qkv:     [T, (nh + 2 nkv) * hd]   (only [T, nh * hd] when has_kv == 0)
//   cos_sin: [max_pos, rot_dim]  (rot_dim/2 cosines then rot_dim/2 sines, 32-bit)
//   pages:   [num_pages, 2, nkv, page_size, hd] of one layer
// rot_dim <= hd lanes of a head are rotated, the rest pass (normed) as they are; the rotated lanes are paired
// (i, i + rot_dim/2), or (2i, 2i+1) with `interleaved` (the two pairings of the reference's back ends,
// src/mlx_backend.cpp:411-412 and src/model.cpp:983-985).  A thread owns pair i = lane + 32 j of a head: lanes
// (i, i + rot_dim/2) or (2i, 2i+1) while i < rot_dim/2, and the unrotated lanes (2i, 2i+1) beyond.
// ---------------------------------------------------------------------------
// MAXP: lane pairs a thread owns (2 serves heads of up to 128 lanes, 4 of up to 256): the serving models' heads
// keep the kernel at a register count that lets an SM hold enough warps when there are thousands of (token, head)s.
template <typename TIN, typename T, int MAXP>
__global__ void qknorm_rope_kvwrite_kernel(const TIN* __restrict__ qkv, int S, size_t s_stride, const void* __restrict__ qw,
                                           const void* __restrict__ kw, int w_dtype, int use_norm, float eps,
                                           const float* __restrict__ cos_sin, int max_pos,
                                           const int* __restrict__ positions, const int* __restrict__ slot_map,
                                           T* __restrict__ q_out, T* __restrict__ pages, long long page_stride,
                                           int page_size, int num_pages, int nh, int nkv, int hd, int n_tokens,
                                           int has_kv, int rot_dim, int interleaved, int* status) {
    pdl_trigger();
    tl_mark(VCB_TL_ROPE, 0);
    const int rot_half = rot_dim >> 1;
    auto e1_of = [&](int i) { return (interleaved || i >= rot_half) ? 2 * i : i; };
    auto e2_of = [&](int i) { return (interleaved || i >= rot_half) ? 2 * i + 1 : i + rot_half; };
    const int lane = threadIdx.x & 31;
    const int heads_total = nh + (has_kv ? 2 * nkv : 0);
    const long long gw = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const bool active = gw < (long long)n_tokens * heads_total;
    const int t = active ? (int)(gw / heads_total) : 0, h = active ? (int)(gw % heads_total) : 0;
    const TIN* src = qkv + (size_t)t * heads_total * hd + (size_t)h * hd;
    const int half = hd >> 1;

    // What no kernel of the step writes -- the token's slot and position, the gains, the angles -- is read before
    // waiting for the kernel that produces qkv, so that only one round trip to memory follows the wait.
    long long slot = -1;
    int pos = 0;
    bool bad_page = false, bad_pos = false;
    float g1[MAXP], g2[MAXP], cs1[MAXP], sn1[MAXP];
    if (active) {
        if (h >= nh) {
            slot = slot_map[t];
            bad_page = slot >= 0 && slot / page_size >= num_pages;
        }
        if (h < nh + nkv) {
            pos = positions[t];
            bad_pos = pos < 0 || pos >= max_pos;
            if (bad_pos) pos = 0;
            const void* gain = h < nh ? qw : kw;
            const float* cs = cos_sin + (size_t)pos * rot_dim;
#pragma unroll
            for (int j = 0; j < MAXP; ++j) {
                const int p = lane + 32 * j;
                if (p < half) {
                    g1[j] = use_norm ? load_as_f32(gain, w_dtype, e1_of(p)) : 1.f;
                    g2[j] = use_norm ? load_as_f32(gain, w_dtype, e2_of(p)) : 1.f;
                    cs1[j] = p < rot_half ? cs[p] : 1.f;
                    sn1[j] = p < rot_half ? cs[rot_half + p] : 0.f;
                }
            }
        }
    }
    pdl_wait();
    tl_mark(VCB_TL_ROPE, 1);
    if (!active) return;
    if (h >= nh) {
        if (slot < 0) return;  // padded token: nothing to store
        if (bad_page) {
            if (lane == 0) atomicOr(status, VCB_STATUS_BAD_PAGE);
            return;
        }
    }

    if (h >= nh + nkv) {  // V head: stored as it is
        const int kvh = h - nh - nkv;
        T* dst = pages + (slot / page_size) * page_stride + ((size_t)(nkv + kvh) * page_size + slot % page_size) * hd;
        for (int i = lane; i < hd; i += 32) {
            float v = 0.f;
            for (int s0 = 0; s0 < S; s0 += 4) {   // loads of four slices at a time, added in slice order
                float vs[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (s0 + j < S) vs[j] = to_f32(src[(s0 + j) * s_stride + i]);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (s0 + j < S) v += vs[j];
            }
            dst[i] = from_f32<T>(v);
        }
        return;
    }

    if (bad_pos && lane == 0) atomicOr(status, VCB_STATUS_BAD_POSITION);
    float x1[MAXP], x2[MAXP];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < MAXP; ++j) {
        const int p = lane + 32 * j;
        if (p < half) x1[j] = x2[j] = 0.f;
    }
    // k-slice partials of the projection are added in slice order; the loads of four slices go out together
    for (int s0 = 0; s0 < S; s0 += 4) {
        float a1[4][MAXP], a2[4][MAXP];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (s0 + k < S) {
#pragma unroll
                for (int j = 0; j < MAXP; ++j) {
                    const int p = lane + 32 * j;
                    if (p < half) {
                        a1[k][j] = to_f32(src[(s0 + k) * s_stride + e1_of(p)]);
                        a2[k][j] = to_f32(src[(s0 + k) * s_stride + e2_of(p)]);
                    }
                }
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (s0 + k < S) {
#pragma unroll
                for (int j = 0; j < MAXP; ++j) {
                    if (lane + 32 * j < half) { x1[j] += a1[k][j]; x2[j] += a2[k][j]; }
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < MAXP; ++j) {
        if (lane + 32 * j < half) ss += x1[j] * x1[j] + x2[j] * x2[j];
    }
    float inv = 1.f;
    if (use_norm) {
        ss = warp_sum(ss);
        inv = 1.0f / sqrtf(ss / (float)hd + eps);
    }
    T* dst;
    if (h < nh) dst = q_out + (size_t)t * nh * hd + (size_t)h * hd;
    else dst = pages + (slot / page_size) * page_stride + ((size_t)(h - nh) * page_size + slot % page_size) * hd;
#pragma unroll
    for (int j = 0; j < MAXP; ++j) {
        const int p = lane + 32 * j;
        if (p < half) {
            float a = x1[j], b = x2[j];
            if (use_norm) {
                a = g1[j] * a * inv;
                b = g2[j] * b * inv;
            }
            dst[e1_of(p)] = from_f32<T>(a * cs1[j] - b * sn1[j]);
            dst[e2_of(p)] = from_f32<T>(b * cs1[j] + a * sn1[j]);
        }
    }
}

// Same contract for the serving shape of prompt portions (head_dim 128, bfloat16 in and out, no partial sums):
// one block per token, its warps walk the heads; each lane owns lanes {2l, 2l+1} and their partners 64 further
// on, loads them as two 4-byte words, and keeps the token's cosines and sines in registers for all heads.
__global__ __launch_bounds__(256) void qknorm_rope_kvwrite_hd128_kernel(
    const __nv_bfloat16* __restrict__ qkv, const void* __restrict__ qw, const void* __restrict__ kw, int w_dtype,
    int use_norm, float eps, const float* __restrict__ cos_sin, int max_pos, const int* __restrict__ positions,
    const int* __restrict__ slot_map, __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ pages,
    long long page_stride, int page_size, int num_pages, int nh, int nkv, int has_kv, int* status) {
    constexpr int hd = 128, half = 64;
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int heads_total = nh + (has_kv ? 2 * nkv : 0);
    int pos = positions[t];
    if (pos < 0 || pos >= max_pos) {
        if (threadIdx.x == 0) atomicOr(status, VCB_STATUS_BAD_POSITION);
        pos = 0;
    }
    const float2 c = *reinterpret_cast<const float2*>(cos_sin + (size_t)pos * hd + 2 * lane);
    const float2 sn = *reinterpret_cast<const float2*>(cos_sin + (size_t)pos * hd + half + 2 * lane);
    int slot = has_kv ? slot_map[t] : -1;
    if (slot >= 0 && slot / page_size >= num_pages) {
        if (threadIdx.x == 0) atomicOr(status, VCB_STATUS_BAD_PAGE);
        slot = -1;
    }
    float gq[4] = {1.f, 1.f, 1.f, 1.f}, gk[4] = {1.f, 1.f, 1.f, 1.f};   // gains of this lane's four elements
    if (use_norm) {
        gq[0] = load_as_f32(qw, w_dtype, 2 * lane); gq[1] = load_as_f32(qw, w_dtype, 2 * lane + 1);
        gq[2] = load_as_f32(qw, w_dtype, half + 2 * lane); gq[3] = load_as_f32(qw, w_dtype, half + 2 * lane + 1);
        if (has_kv) {
            gk[0] = load_as_f32(kw, w_dtype, 2 * lane); gk[1] = load_as_f32(kw, w_dtype, 2 * lane + 1);
            gk[2] = load_as_f32(kw, w_dtype, half + 2 * lane); gk[3] = load_as_f32(kw, w_dtype, half + 2 * lane + 1);
        }
    }
    const __nv_bfloat16* row = qkv + (size_t)t * heads_total * hd;
    // six heads a round (the 48 heads of the 8B shape in one round of eight warps): their loads are all issued
    // before the first is used
    constexpr int U = 6;
    for (int h0 = warp; h0 < heads_total; h0 += U * nwarps) {
        __nv_bfloat162 lo[U], hi[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int h = h0 + u * nwarps;
            if (h < heads_total) {
                lo[u] = *reinterpret_cast<const __nv_bfloat162*>(row + (size_t)h * hd + 2 * lane);
                hi[u] = *reinterpret_cast<const __nv_bfloat162*>(row + (size_t)h * hd + half + 2 * lane);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int h = h0 + u * nwarps;
            if (h >= heads_total) break;
            __nv_bfloat16* dst;
            if (h < nh) {
                dst = q_out + ((size_t)t * nh + h) * hd;
            } else {
                if (slot < 0) continue;   // padded token: nothing to store
                const int kv = h >= nh + nkv, kvh = kv ? h - nh - nkv : h - nh;
                dst = pages + (size_t)(slot / page_size) * page_stride + ((size_t)(kv * nkv + kvh) * page_size + slot % page_size) * hd;
            }
            if (h >= nh + nkv) {   // V: stored as it is
                *reinterpret_cast<__nv_bfloat162*>(dst + 2 * lane) = lo[u];
                *reinterpret_cast<__nv_bfloat162*>(dst + half + 2 * lane) = hi[u];
                continue;
            }
            float a0 = __low2float(lo[u]), a1 = __high2float(lo[u]), b0 = __low2float(hi[u]), b1 = __high2float(hi[u]);
            if (use_norm) {
                const float ss = warp_sum(a0 * a0 + a1 * a1 + b0 * b0 + b1 * b1);
                const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
                const float* gw = h < nh ? gq : gk;
                a0 = gw[0] * a0 * inv; a1 = gw[1] * a1 * inv; b0 = gw[2] * b0 * inv; b1 = gw[3] * b1 * inv;
            }
            *reinterpret_cast<__nv_bfloat162*>(dst + 2 * lane) = __floats2bfloat162_rn(a0 * c.x - b0 * sn.x, a1 * c.y - b1 * sn.y);
            *reinterpret_cast<__nv_bfloat162*>(dst + half + 2 * lane) = __floats2bfloat162_rn(b0 * c.x + a0 * sn.x, b1 * c.y + a1 * sn.y);
        }
    }
}

// qkv: [S, T, width] of in_dtype (S partial sums, s_stride elements apart); q_out and pages of out_dtype
VCB_API int vcb_qknorm_rope_kvwrite(const void* qkv, int in_dtype, int S, long long s_stride, int out_dtype,
                                    const void* qw, const void* kw, int w_dtype, int use_norm, float eps,
                                    const float* cos_sin, int max_pos, const int* positions, const int* slot_map,
                                    void* q_out, void* pages, long long page_stride, int page_size, int num_pages,
                                    int nh, int nkv, int hd, int T, int has_kv, int rot_dim, int interleaved, int* status,
                                    cudaStream_t stream) {
    if (T == 0) return 0;
    VCB_CHECK_ARG(rot_dim >= 0 && rot_dim <= hd && rot_dim % 2 == 0,
                  "qknorm_rope_kvwrite: %d rotated lanes of a head of %d (an even number up to head_dim)", rot_dim, hd);
    VCB_CHECK_ARG(hd > 0 && hd % 2 == 0 && hd <= VCB_MAX_HEAD_DIM,
                  "qknorm_rope_kvwrite: head_dim %d must be even and <= %d", hd, VCB_MAX_HEAD_DIM);
    VCB_CHECK_ARG(nh > 0 && nkv > 0 && page_size > 0 && S >= 1, "qknorm_rope_kvwrite: bad sizes nh=%d nkv=%d page=%d S=%d",
                  nh, nkv, page_size, S);
    if (hd == 128 && rot_dim == hd && !interleaved && in_dtype == VCB_BF16 && out_dtype == VCB_BF16 && S == 1 && ((uintptr_t)qkv % 4 == 0) &&
        ((uintptr_t)q_out % 4 == 0) && ((uintptr_t)pages % 4 == 0)) {
        qknorm_rope_kvwrite_hd128_kernel<<<T, 256, 0, stream>>>(
            (const __nv_bfloat16*)qkv, qw, kw, w_dtype, use_norm, eps, cos_sin, max_pos, positions, slot_map,
            (__nv_bfloat16*)q_out, (__nv_bfloat16*)pages, page_stride, page_size, num_pages, nh, nkv, has_kv, status);
        VCB_CHECK_LAUNCH("qknorm_rope_kvwrite");
        return 0;
    }
    const long long warps = (long long)T * (nh + (has_kv ? 2 * nkv : 0));
    const int wpb = 4;
    const long long blocks = (warps + wpb - 1) / wpb;
    VCB_CHECK_ARG(blocks < (1ll << 31), "qknorm_rope_kvwrite: too many blocks");
#define VCB_QK_LAUNCH(TIN, TOUT)                                                                                      \
    if (hd <= 128)                                                                                                    \
    launch_pdl(qknorm_rope_kvwrite_kernel<TIN, TOUT, 2>, dim3((unsigned)blocks), dim3(wpb * 32), 0, stream,              \
        (const TIN*)qkv, S, (size_t)s_stride, qw, kw, w_dtype, use_norm, eps, cos_sin, max_pos, positions, slot_map,   \
        (TOUT*)q_out, (TOUT*)pages, page_stride, page_size, num_pages, nh, nkv, hd, T, has_kv, rot_dim, interleaved, status); \
    else                                                                                                              \
    launch_pdl(qknorm_rope_kvwrite_kernel<TIN, TOUT, VCB_MAX_HEAD_DIM / 64>, dim3((unsigned)blocks), dim3(wpb * 32), 0, stream, \
        (const TIN*)qkv, S, (size_t)s_stride, qw, kw, w_dtype, use_norm, eps, cos_sin, max_pos, positions, slot_map,   \
        (TOUT*)q_out, (TOUT*)pages, page_stride, page_size, num_pages, nh, nkv, hd, T, has_kv, rot_dim, interleaved, status)
    if (in_dtype == VCB_F32 && out_dtype == VCB_F32) VCB_QK_LAUNCH(float, float);
    else if (in_dtype == VCB_F32) VCB_QK_LAUNCH(float, __nv_bfloat16);
    else if (out_dtype == VCB_BF16) VCB_QK_LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else { vcb_set_error("qknorm_rope_kvwrite: bfloat16 input with 32-bit output is not a combination the engine uses"); return -1; }
#undef VCB_QK_LAUNCH
    VCB_CHECK_LAUNCH("qknorm_rope_kvwrite");
    return 0;
}

// ---------------------------------------------------------------------------
// dst[idx[i]] = val[i]: how new block-table entries reach the device-resident tables
// ---------------------------------------------------------------------------
__global__ void scatter_i32_kernel(int* __restrict__ dst, const int* __restrict__ idx, const int* __restrict__ val,
                                   const int* __restrict__ count, int capacity, long long dst_size) {
    // No early trigger here: the kernel after this one then starts only when this one has ended, and every later
    // kernel of the step after that, so all of them may read the block tables before their own dependency wait
    // (the attention kernel asks for old key tiles that early).
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int n = min(*count, capacity);
    if (i < n && idx[i] >= 0 && idx[i] < dst_size) dst[idx[i]] = val[i];
}

// count lives on the device so that a captured launch can serve any number of updates up to capacity
VCB_API int vcb_scatter_i32(int* dst, const int* idx, const int* val, const int* count, int capacity,
                            long long dst_size, cudaStream_t stream) {
    if (capacity == 0) return 0;
    launch_pdl(scatter_i32_kernel, dim3((capacity + 255) / 256), dim3(256), 0, stream, dst, idx, val, count, capacity, dst_size);
    VCB_CHECK_LAUNCH("scatter_i32");
    return 0;
}

// ---------------------------------------------------------------------------
// Fixed-size per-request state: the state of every request whose first tokens arrive in this step (its entry
// starts at position 0) is set to the state's initial value, in every cache of the group.  On the device, so that
// a captured step does it too.  state: [caches][slots][row] of 2- or 4-byte elements; grid (entries, caches).
// ---------------------------------------------------------------------------
template <typename E>
__global__ void state_reset_kernel(E* __restrict__ state, long long cache_stride, long long slot_stride, long long row,
                                   int num_slots, const int* __restrict__ slots, const int* __restrict__ q_len,
                                   const int* __restrict__ ctx_len, E value, int* status) {
    pdl_trigger();
    pdl_wait();
    const int e = blockIdx.x;
    if (q_len[e] <= 0 || ctx_len[e] != q_len[e]) return;     // empty, or a request that is further on than its start
    const int slot = slots[e];
    if (slot < 0 || slot >= num_slots) {
        if (threadIdx.x == 0) atomicOr(status, VCB_STATUS_BAD_ITEM);
        return;
    }
    E* dst = state + (size_t)blockIdx.y * cache_stride + (size_t)slot * slot_stride;
    for (long long i = threadIdx.x; i < row; i += blockDim.x) dst[i] = value;
}

VCB_API int vcb_state_reset(void* state, int elem_bytes, long long cache_stride, long long slot_stride, long long row,
                            int n_caches, int num_slots, const int* slots, const int* q_len, const int* ctx_len,
                            int n_entries, unsigned int value_bits, int* status, cudaStream_t stream) {
    if (n_entries == 0 || n_caches == 0 || row == 0) return 0;
    VCB_CHECK_ARG(elem_bytes == 2 || elem_bytes == 4, "state_reset: elements of %d bytes (2 or 4)", elem_bytes);
    VCB_CHECK_ARG(status != nullptr, "state_reset: a status word is required");
    const int threads = row >= 256 ? 256 : 64;
    if (elem_bytes == 4)
        launch_pdl(state_reset_kernel<unsigned int>, dim3(n_entries, n_caches), dim3(threads), 0, stream, (unsigned int*)state,
                   cache_stride, slot_stride, row, num_slots, slots, q_len, ctx_len, value_bits, status);
    else
        launch_pdl(state_reset_kernel<unsigned short>, dim3(n_entries, n_caches), dim3(threads), 0, stream, (unsigned short*)state,
                   cache_stride, slot_stride, row, num_slots, slots, q_len, ctx_len, (unsigned short)value_bits, status);
    VCB_CHECK_LAUNCH("state_reset");
    return 0;
}
