// Next-token choice from rows of 32-bit logits, one block per row.
//
// Order of operations as the reference's sample_token (src/model.cpp:1291-1352):
// repetition penalty once per earlier occurrence of a token (positive scores are
// divided, negative multiplied), division by the temperature, softmax, nucleus cut
// at top_p, draw.  temperature <= 0 takes the arg-max, lowest index on ties
// (src/mlx_backend.cpp:516-524).  The draw is argmax_i(score_i + Gumbel(u_i)) over
// the kept tokens, u_i a counter-based uniform of (seed, step, i): one pass, no
// sort, and the same token on any machine for equal logits.  The nucleus is the
// set {p_i >= c} for the largest c whose set has mass >= top_p (the shortest
// descending prefix, with ties at the cut all kept), found by bisection on the
// ordered bit pattern of the scores; masses are summed in 64-bit.
#include "common.cuh"

#include <math_constants.h>

namespace {

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float uniform01(unsigned long long key, unsigned int index) {
    const unsigned long long bits = mix64(key ^ (unsigned long long)index);
    return ((float)(bits >> 41) + 0.5f) * (1.0f / 8388608.0f);
}

// order-preserving map float -> uint32
__device__ __forceinline__ unsigned int ordered_key(float f) {
    const unsigned int u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ double block_sum_f64(double v, double* scratch /* 33 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        double t = lane < nwarps ? scratch[lane] : 0.0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// arg-max with lowest index on ties; every thread gets the result
__device__ __forceinline__ void block_argmax(float& v, int& idx, float* sv, int* si) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    __syncthreads();
    if (lane == 0) { sv[warp] = v; si[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        float tv = lane < nwarps ? sv[lane] : -CUDART_INF_F;
        int ti = lane < nwarps ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, tv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, ti, o);
            if (ov > tv || (ov == tv && oi < ti)) { tv = ov; ti = oi; }
        }
        if (lane == 0) { sv[32] = tv; si[32] = ti; }
    }
    __syncthreads();
    v = sv[32];
    idx = si[32];
}

struct RowParams {  // one per row, 32 bytes
    float temperature, top_p, repeat_penalty;
    int slot;              // row of the occurrence-count table, or -1
    unsigned int seed_lo, seed_hi, step, pad;
};

__device__ __forceinline__ float score_at(const float* logits, const int* counts, float penalty, float inv_t, int i) {
    float s = logits[i];
    if (counts) {
        const int c = counts[i];
        if (c > 0) {
            const float f = powf(penalty, (float)c);
            s = s > 0.f ? s / f : s * f;
        }
    }
    return s * inv_t;
}

__global__ __launch_bounds__(1024) void sample_kernel(const float* __restrict__ logits, long long row_stride, int V,
                                                      const RowParams* __restrict__ params,
                                                      const int* __restrict__ counts_table, int* __restrict__ out) {
    __shared__ float sv[33];
    __shared__ int si[33];
    __shared__ double sd[33];
    const int row = blockIdx.x;
    const RowParams p = params[row];
    const float* lg = logits + (size_t)row * row_stride;
    const int* counts = (counts_table && p.slot >= 0 && p.repeat_penalty != 1.0f) ? counts_table + (size_t)p.slot * V : nullptr;
    const bool greedy = !(p.temperature > 0.f);
    const float inv_t = greedy ? 1.f : 1.0f / p.temperature;

    // maximum of the scores (also the greedy answer)
    float best = -CUDART_INF_F;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float s = score_at(lg, counts, p.repeat_penalty, inv_t, i);
        if (s > best || (s == best && i < best_i)) { best = s; best_i = i; }
    }
    block_argmax(best, best_i, sv, si);
    if (greedy) {
        if (threadIdx.x == 0) out[row] = best_i;
        return;
    }
    const float m = best;

    unsigned int cut = 0;  // keep scores whose ordered key is >= cut
    if (p.top_p < 1.0f) {
        double z = 0.0;
        for (int i = threadIdx.x; i < V; i += blockDim.x) z += (double)expf(score_at(lg, counts, p.repeat_penalty, inv_t, i) - m);
        z = block_sum_f64(z, sd);
        const double need = (double)p.top_p * z;
        unsigned int lo = 0, hi = ordered_key(m);  // mass(lo) >= need holds; answer in [lo, hi]
        while (lo < hi) {
            const unsigned int mid = lo + (hi - lo + 1) / 2;
            double mass = 0.0;
            for (int i = threadIdx.x; i < V; i += blockDim.x) {
                const float s = score_at(lg, counts, p.repeat_penalty, inv_t, i);
                if (ordered_key(s) >= mid) mass += (double)expf(s - m);
            }
            mass = block_sum_f64(mass, sd);
            if (mass >= need) lo = mid; else hi = mid - 1;
        }
        cut = lo;
    }

    const unsigned long long key = mix64(((unsigned long long)p.seed_lo << 32) | (unsigned long long)p.step);
    float zbest = -CUDART_INF_F;
    int zi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float s = score_at(lg, counts, p.repeat_penalty, inv_t, i);
        if (ordered_key(s) < cut) continue;
        const float u = uniform01(key, (unsigned int)i);
        const float zv = s - logf(-logf(u));
        if (zv > zbest || (zv == zbest && i < zi)) { zbest = zv; zi = i; }
    }
    block_argmax(zbest, zi, sv, si);
    if (threadIdx.x == 0) out[row] = zi;
}

// Two-stage variant for rows that need no nucleus cut (top_p >= 1 or greedy): the vocabulary is dealt to
// `nb` blocks per row, each leaves its best (value, index), and the last stage picks among them with the same
// lowest-index rule, so the token equals the single-block kernel's.
__global__ __launch_bounds__(512) void sample_part_kernel(const float* __restrict__ logits, long long row_stride, int V,
                                                          const RowParams* __restrict__ params,
                                                          const int* __restrict__ counts_table, float* __restrict__ part_v,
                                                          int* __restrict__ part_i) {
    __shared__ float sv[33];
    __shared__ int si[33];
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x, nb = gridDim.y, b = blockIdx.y;
    const RowParams p = params[row];
    const float* lg = logits + (size_t)row * row_stride;
    const int* counts = (counts_table && p.slot >= 0 && p.repeat_penalty != 1.0f) ? counts_table + (size_t)p.slot * V : nullptr;
    const bool greedy = !(p.temperature > 0.f);
    const float inv_t = greedy ? 1.f : 1.0f / p.temperature;
    const unsigned long long key = mix64(((unsigned long long)p.seed_lo << 32) | (unsigned long long)p.step);
    const int chunk = (V + nb - 1) / nb;
    const int lo = b * chunk, hi = min(V, lo + chunk);
    float best = -CUDART_INF_F;
    int best_i = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        float s = score_at(lg, counts, p.repeat_penalty, inv_t, i);
        if (!greedy) s -= logf(-logf(uniform01(key, (unsigned int)i)));
        if (s > best || (s == best && i < best_i)) { best = s; best_i = i; }
    }
    block_argmax(best, best_i, sv, si);
    if (threadIdx.x == 0) {
        part_v[row * nb + b] = best;
        part_i[row * nb + b] = best_i;
    }
}

__global__ void sample_pick_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i, int nb,
                                   int* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    float best = -CUDART_INF_F;
    int best_i = 0x7fffffff;
    for (int b = threadIdx.x; b < nb; b += 32) {
        const float v = part_v[row * nb + b];
        const int i = part_i[row * nb + b];
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (threadIdx.x == 0) out[row] = best_i;
}

__global__ void count_tokens_kernel(const int* __restrict__ ids, const int* __restrict__ slots, int* __restrict__ counts,
                                    int n, int V, int slot_bias) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n) return;
    const int id = ids[t], slot = slots[t] - slot_bias;
    if (slot >= 0 && id >= 0 && id < V) atomicAdd(counts + (size_t)slot * V + id, 1);
}

}  // namespace

// params: n_rows records of 8 x 32-bit words: temperature, top_p, repeat_penalty (floats), count-table row or -1,
// seed (low 32 bits, high 32 bits, high unused), step, pad
VCB_API int vcb_sample(const float* logits, long long row_stride, int n_rows, int V, const void* params,
                       const int* counts_table, int* out, cudaStream_t stream) {
    if (n_rows == 0) return 0;
    VCB_CHECK_ARG(n_rows > 0 && V > 0 && row_stride >= V, "sample: bad sizes rows=%d V=%d stride=%lld", n_rows, V, row_stride);
    const int threads = V >= 8192 ? 1024 : 256;
    sample_kernel<<<n_rows, threads, 0, stream>>>(logits, row_stride, V, (const RowParams*)params, counts_table, out);
    VCB_CHECK_LAUNCH("sample");
    return 0;
}

// counts[slots[t] - slot_bias][ids[t]] += 1 for every token whose slot entry, less the bias, is >= 0
VCB_API int vcb_count_tokens(const int* ids, const int* slots, int* counts, int n, int V, int slot_bias, cudaStream_t stream) {
    if (n == 0) return 0;
    count_tokens_kernel<<<(n + 255) / 256, 256, 0, stream>>>(ids, slots, counts, n, V, slot_bias);
    VCB_CHECK_LAUNCH("count_tokens");
    return 0;
}

// For batches in which no row cuts a nucleus: `nb` blocks per row; part_v / part_i hold n_rows * nb entries.
VCB_API int vcb_sample_split(const float* logits, long long row_stride, int n_rows, int V, const void* params,
                             const int* counts_table, float* part_v, int* part_i, int nb, int* out,
                             cudaStream_t stream) {
    if (n_rows == 0) return 0;
    VCB_CHECK_ARG(n_rows > 0 && V > 0 && row_stride >= V && nb >= 1 && nb <= 1024, "sample_split: bad sizes");
    launch_pdl(sample_part_kernel, dim3(n_rows, nb), dim3(512), 0, stream, logits, row_stride, V, (const RowParams*)params,
               counts_table, part_v, part_i);
    VCB_CHECK_LAUNCH("sample_part");
    launch_pdl(sample_pick_kernel, dim3(n_rows), dim3(32), 0, stream, part_v, part_i, nb, out);
    VCB_CHECK_LAUNCH("sample_pick");
    return 0;
}
