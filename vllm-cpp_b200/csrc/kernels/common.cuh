// Shared helpers of the sm_100a kernels: element types, conversions, reductions,
// launch-error plumbing.  Every exported launcher returns 0 or a negative code and
// leaves a message readable through vcb_last_error().
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define VCB_API extern "C" __attribute__((visibility("default")))

// largest head size the attention-side kernels take (steps of 16 below it)
#define VCB_MAX_HEAD_DIM 256

// element type codes shared with the Python side
enum VcbDtype : int { VCB_F32 = 0, VCB_BF16 = 1 };

// bits of the device status word that kernels set instead of trapping
enum VcbStatus : int {
    VCB_STATUS_OK = 0,
    VCB_STATUS_BAD_TOKEN = 1,      // token id outside the vocabulary
    VCB_STATUS_BAD_PAGE = 2,       // page id outside the pool
    VCB_STATUS_WAIT_TIMEOUT = 4,   // a bounded mbarrier wait gave up
    VCB_STATUS_BAD_POSITION = 8,   // position outside the rotary table
    VCB_STATUS_BAD_LAYOUT = 16,    // shared memory did not start on the boundary a kernel's tiles need
    VCB_STATUS_BAD_ITEM = 32,      // a work item names a partial-result row outside the buffer it was given
};

void vcb_set_error(const char* fmt, ...);

#define VCB_CHECK_ARG(cond, ...)                  \
    do {                                          \
        if (!(cond)) {                            \
            vcb_set_error(__VA_ARGS__);           \
            return -1;                            \
        }                                         \
    } while (0)

#define VCB_CHECK_LAUNCH(name)                                                   \
    do {                                                                         \
        cudaError_t e_ = cudaGetLastError();                                     \
        if (e_ != cudaSuccess) {                                                 \
            vcb_set_error("%s: launch failed: %s", name, cudaGetErrorString(e_)); \
            return -2;                                                           \
        }                                                                        \
    } while (0)

// Programmatic dependent launch: a kernel launched through launch_pdl may start while the kernel before it in
// the stream is still running.  It must call pdl_wait() -- in every block, before the block exits and before it
// touches anything the earlier kernel reads or writes; everything before that call (barrier set-up, fetching
// operands no kernel of the step writes) overlaps the earlier kernel's tail.  pdl_trigger() lets the next kernel
// start likewise.  Kernels launched the ordinary way keep full stream order.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool vcb_pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = vcb_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same with the grid's blocks in clusters of `cluster_x` along x (blocks of a cluster run at the same time on
// SMs of one GPC and can read one another's shared memory).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_clusters(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                       unsigned cluster_x, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = vcb_pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// A look at a step from inside (built only with -DVCB_TIMELINE; otherwise tl_mark is nothing).  Thread 0 of every
// block appends (time, kernel, phase, block, SM) records to a buffer that the host hands to each translation unit:
// word 0 counts the records, word 1 is the capacity, then four words a record.  Phases: 0 the block starts,
// 1 its wait for the kernel before it is over, 2 it ends.  This is how one sees, in a captured step with
// programmatic dependent launch, when blocks of the next kernel are really resident and how long they wait.
enum VcbTlKernel : int { VCB_TL_GEMM = 1, VCB_TL_ATTN_DEC = 2, VCB_TL_NORM = 3, VCB_TL_ROPE = 4, VCB_TL_SWIGLU = 5,
                         VCB_TL_ATTN_TC = 6, VCB_TL_OTHER = 7 };
#ifdef VCB_TIMELINE
static __device__ unsigned long long* vcb_tl;
__device__ __forceinline__ void tl_mark(int kernel, int phase) {
    if (threadIdx.x == 0 && vcb_tl != nullptr) {
        unsigned long long t, c;
        unsigned int sm;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        asm volatile("mov.u64 %0, %%clock64;" : "=l"(c));
        asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
        const unsigned long long i = atomicAdd(vcb_tl, 1ull);
        if (i < vcb_tl[1]) {
            unsigned long long* r = vcb_tl + 2 + 4 * i;
            r[0] = t;
            r[1] = c;
            r[2] = ((unsigned long long)kernel << 32) | ((unsigned long long)phase << 24) | (sm & 0xFFu);
            r[3] = ((unsigned long long)gridDim.x << 32) | (blockIdx.x + gridDim.x * blockIdx.y);
        }
    }
}
// The roles inside a block (a loading warp, a thread that issues products, rows of a softmax) mark their steps in
// logs of their own behind the records above: no counter to wait for, a clock read and two stores a mark.  Blocks
// 0, 37, 74, ... (eight at most) record, up to three roles each, each role through one thread.
constexpr int VCB_TL_ROLE_EVERY = 37, VCB_TL_ROLE_BLOCKS = 8, VCB_TL_ROLES = 3, VCB_TL_ROLE_MARKS = 2048;
struct TlRole {
    unsigned long long* log = nullptr;
    int n = 0;
    int kernel = 0;
    __device__ __forceinline__ void begin(int kernel_id, int role, bool this_thread) {
        log = nullptr;
        n = 0;
        kernel = kernel_id;
        if (this_thread && vcb_tl != nullptr && blockIdx.y == 0 && blockIdx.x % VCB_TL_ROLE_EVERY == 0 &&
            blockIdx.x / VCB_TL_ROLE_EVERY < VCB_TL_ROLE_BLOCKS)
            log = vcb_tl + 2 + 4 * vcb_tl[1] + (size_t)((blockIdx.x / VCB_TL_ROLE_EVERY) * VCB_TL_ROLES + role) * VCB_TL_ROLE_MARKS * 2;
    }
    __device__ __forceinline__ void mark(int phase, int tile) {
        if (log != nullptr && n < VCB_TL_ROLE_MARKS) {
            unsigned long long c;
            asm volatile("mov.u64 %0, %%clock64;" : "=l"(c) :: "memory");
            log[2 * n] = c;
            log[2 * n + 1] = (1ull << 63) | ((unsigned long long)kernel << 48) | ((unsigned long long)phase << 32) | (unsigned int)tile;
            ++n;
        }
    }
};
#define VCB_TIMELINE_UNIT(name)                                                             \
    VCB_API int vcb_timeline_set_##name(unsigned long long* p) {                            \
        return cudaMemcpyToSymbol(vcb_tl, &p, sizeof(p)) == cudaSuccess ? 0 : -1;           \
    }
#else
__device__ __forceinline__ void tl_mark(int, int) {}
struct TlRole {
    __device__ __forceinline__ void begin(int, int, bool) {}
    __device__ __forceinline__ void mark(int, int) {}
};
#define VCB_TIMELINE_UNIT(name)
#endif

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// load element i of an array whose element type is only known at run time
__device__ __forceinline__ float load_as_f32(const void* p, int dtype, size_t i) {
    return dtype == VCB_F32 ? ((const float*)p)[i] : __bfloat162float(((const __nv_bfloat16*)p)[i]);
}
__device__ __forceinline__ void store_from_f32(void* p, int dtype, size_t i, float v) {
    if (dtype == VCB_F32) ((float*)p)[i] = v;
    else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of
// the additions depends only on the block size, so equal inputs give equal sums.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
