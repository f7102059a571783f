// True 32-bit matrix product for the float32 path of the model:
//   C[M,N] = A[M,K] . B[N,K]^T   (both operands row-major with K contiguous)
// the orientation of every projection in the reference (src/model.cpp:932-944).
// Plain FFMA accumulation in K order: no tensor cores, no reduced-precision
// mode, and a summation order that does not depend on M or N, so a row's result
// is the same whatever else is in the batch.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TI, typename TO>
__global__ __launch_bounds__(256) void sgemm_tn_kernel(const TI* __restrict__ A, const TI* __restrict__ B,
                                                       TO* __restrict__ C, int M, int N, int K, long long lda,
                                                       long long ldb, long long ldc, int vec_ok) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lr = tid >> 2, lk = (tid & 3) * 4;  // this thread loads row lr, k-lanes lk..lk+3 of both tiles
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        float a[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
        const int k = k0 + lk;
        if (m0 + lr < M) {
            const TI* p = A + (long long)(m0 + lr) * lda + k;
            if (sizeof(TI) == 4 && vec_ok && k + 3 < K) {
                const float4 v = *reinterpret_cast<const float4*>(p);
                a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (k + i < K) a[i] = to_f32(p[i]);
            }
        }
        if (n0 + lr < N) {
            const TI* p = B + (long long)(n0 + lr) * ldb + k;
            if (sizeof(TI) == 4 && vec_ok && k + 3 < K) {
                const float4 v = *reinterpret_cast<const float4*>(p);
                b[0] = v.x; b[1] = v.y; b[2] = v.z; b[3] = v.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (k + i < K) b[i] = to_f32(p[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            As[lk + i][lr] = a[i];
            Bs[lk + i][lr] = b[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 av = *reinterpret_cast<const float4*>(&As[kk][ty * TM]);
            const float4 bv = *reinterpret_cast<const float4*>(&Bs[kk][tx * TN]);
            const float ar[4] = {av.x, av.y, av.z, av.w};
            const float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) C[(long long)m * ldc + n] = from_f32<TO>(acc[i][j]);
        }
    }
}
}  // namespace

VCB_API int vcb_sgemm_tn(const float* A, const float* B, float* C, int M, int N, int K, long long lda, long long ldb,
                         long long ldc, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    VCB_CHECK_ARG(M > 0 && N > 0 && K > 0, "sgemm_tn: bad sizes M=%d N=%d K=%d", M, N, K);
    VCB_CHECK_ARG(lda >= K && ldb >= K && ldc >= N, "sgemm_tn: a leading dimension is smaller than its row");
    const int gy = (M + BM - 1) / BM, gx = (N + BN - 1) / BN;
    VCB_CHECK_ARG(gy <= 65535, "sgemm_tn: M=%d exceeds %d rows per launch", M, 65535 * BM);
    const int vec_ok = (lda % 4 == 0) && (ldb % 4 == 0) && ((uintptr_t)A % 16 == 0) && ((uintptr_t)B % 16 == 0);
    sgemm_tn_kernel<float, float><<<dim3(gx, gy), 256, 0, stream>>>(A, B, C, M, N, K, lda, ldb, ldc, vec_ok);
    VCB_CHECK_LAUNCH("sgemm_tn");
    return 0;
}

// The same loop for bfloat16 operands whose rows are not 16-byte multiples (which the TMA kernel cannot
// address): bfloat16 in, 32-bit accumulation in k order, bfloat16 or 32-bit out.  Slow; exists so that no
// configuration is refused.
VCB_API int vcb_gemm_bf16_plain(const void* A, const void* B, void* C, int out_dtype, int M, int N, int K, long long lda,
                                long long ldb, long long ldc, cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    VCB_CHECK_ARG(M > 0 && N > 0 && K > 0, "gemm_bf16_plain: bad sizes M=%d N=%d K=%d", M, N, K);
    const int gy = (M + BM - 1) / BM, gx = (N + BN - 1) / BN;
    VCB_CHECK_ARG(gy <= 65535, "gemm_bf16_plain: M=%d exceeds %d rows per launch", M, 65535 * BM);
    if (out_dtype == VCB_F32)
        sgemm_tn_kernel<__nv_bfloat16, float><<<dim3(gx, gy), 256, 0, stream>>>((const __nv_bfloat16*)A, (const __nv_bfloat16*)B, (float*)C, M, N, K, lda, ldb, ldc, 0);
    else
        sgemm_tn_kernel<__nv_bfloat16, __nv_bfloat16><<<dim3(gx, gy), 256, 0, stream>>>((const __nv_bfloat16*)A, (const __nv_bfloat16*)B, (__nv_bfloat16*)C, M, N, K, lda, ldb, ldc, 0);
    VCB_CHECK_LAUNCH("gemm_bf16_plain");
    return 0;
}
