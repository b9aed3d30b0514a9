// Shared helpers of the sm_100a kernels: element types, conversions, reductions
// and the launch-status convention.
//
// Every exported launcher has C linkage, takes raw device pointers plus a
// cudaStream_t (as void*), allocates nothing, and returns 0 or a positive
// cudaError_t from the launch; argument errors return a negative code and leave a
// message for kllm_last_error().  Element type codes: 0 = float32, 1 = bfloat16.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#define KLLM_F32 0
#define KLLM_BF16 1

#define KLLM_ERR_ARG (-2)

static thread_local char g_kllm_err[512];

#define KLLM_FAIL(...)                                         \
    do {                                                       \
        snprintf(g_kllm_err, sizeof(g_kllm_err), __VA_ARGS__); \
        return KLLM_ERR_ARG;                                   \
    } while (0)

#define KLLM_LAUNCH_STATUS()                                                   \
    do {                                                                       \
        cudaError_t e__ = cudaGetLastError();                                  \
        if (e__ != cudaSuccess) {                                              \
            snprintf(g_kllm_err, sizeof(g_kllm_err), "%s:%d: %s", __FILE__,    \
                     __LINE__, cudaGetErrorString(e__));                       \
            return (int)e__;                                                   \
        }                                                                      \
        return 0;                                                              \
    } while (0)

// ---- timeline (only with -DKLLM_TIMELINE) ---------------------------------------
// A build for looking at where a kernel's time goes inside a step: a kernel that is
// instrumented reads the GPU's nanosecond timer at up to 8 marks and, for three of its
// CTAs (first, middle, last), thread 0 stores them in a table in this library's device
// memory, one row per launch (rows are reused after KLLM_TL_LAUNCHES launches).  The
// host reads the table with kllm_timeline_<library>().  Without the definition all of
// this compiles to nothing.
#define KLLM_TL_LAUNCHES 512
#define KLLM_TL_MARKS 8
#ifdef KLLM_TIMELINE
__device__ unsigned long long g_kllm_tl[KLLM_TL_LAUNCHES][3][KLLM_TL_MARKS + 1];
static int g_kllm_tl_next = 0;
__device__ __forceinline__ unsigned long long kllm_gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define TL_BEGIN() unsigned long long tl_[KLLM_TL_MARKS] = {}; tl_[0] = kllm_gtime()
#define TL_MARK(i) tl_[i] = kllm_gtime()
#define TL_END(slot, tag)                                                                        \
    do {                                                                                         \
        const unsigned nb_ = gridDim.x * gridDim.y * gridDim.z;                                  \
        const unsigned b_ = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;      \
        const int w_ = b_ == 0 ? 0 : (b_ == nb_ / 2 ? 1 : (b_ == nb_ - 1 ? 2 : -1));             \
        if (w_ >= 0 && threadIdx.x == 0 && (slot) >= 0) {                                        \
            for (int i_ = 0; i_ < KLLM_TL_MARKS; i_++) g_kllm_tl[slot][w_][i_] = tl_[i_];        \
            g_kllm_tl[slot][w_][KLLM_TL_MARKS] = (tag);                                          \
        }                                                                                        \
    } while (0)
#define TL_SLOT() (g_kllm_tl_next++ % KLLM_TL_LAUNCHES)
#define KLLM_EXPORT_TIMELINE(libname)                                                            \
    extern "C" int kllm_timeline_##libname(unsigned long long* out) {                            \
        return (int)cudaMemcpyFromSymbol(out, g_kllm_tl, sizeof(g_kllm_tl));                     \
    }
#else
#define TL_BEGIN() do {} while (0)
#define TL_MARK(i) do {} while (0)
#define TL_END(slot, tag) do {} while (0)
#define TL_SLOT() (-1)
#define KLLM_EXPORT_TIMELINE(libname)
#endif

#define KLLM_EXPORT_LAST_ERROR(libname)                                 \
    extern "C" const char* kllm_last_error_##libname() { return g_kllm_err; } \
    KLLM_EXPORT_TIMELINE(libname)

// ---- programmatic dependent launch ------------------------------------------
// Kernels of one step form a chain in which each reads what the one before wrote.
// Launched with the "programmatic stream serialization" attribute, a kernel may be
// scheduled while its predecessor is still running; it calls griddep_wait() before
// its first access to anything a predecessor may write, and griddep_launch() once
// its successor may start to be scheduled.  What a kernel does before the wait
// (address arithmetic, prefetching weights or cache pages that no kernel of the
// chain writes) overlaps the predecessor's tail and the launch latency.  Without
// the attribute both calls do nothing.  KLLM_B200_PDL=0 in the environment turns
// the attribute off.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool kllm_pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("KLLM_B200_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// `early`: the grid may start before the kernel before it in the stream has ended (it
// then waits in griddep_wait for that kernel's results); without it the grid starts
// after that kernel as usual and griddep_wait returns at once.
template <typename... KArgs, typename... Args>
static inline cudaError_t kllm_launch_dep(bool early, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                          cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (early && kllm_pdl_enabled()) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
static inline cudaError_t kllm_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                      cudaStream_t stream, Args&&... args) {
    return kllm_launch_dep(true, kernel, grid, block, smem, stream, static_cast<Args&&>(args)...);
}

// ---- warming L2 for the kernel after this one ---------------------------------
// A decode step streams each weight matrix once, in kernels too short to keep the
// memory system full: each starts with empty queues and ends with a tail.  A kernel
// may therefore be handed the weights that a LATER kernel of the chain will stream;
// its CTAs ask for them to be brought into L2 (cp.async.bulk.prefetch.L2: no
// destination, no completion to wait for) before doing their own work, so that DRAM
// stays busy through this kernel's latency-bound phases and the later kernel reads
// from L2.  ptr must be 16-byte aligned; the last bytes % 16 are left out.
__device__ __forceinline__ void l2_prefetch_slice(const void* ptr, long long bytes, int threads) {
    if (!ptr || bytes < 16) return;
    constexpr long long CHUNK = 4096;
    const long long ctas = (long long)gridDim.x * gridDim.y * gridDim.z;
    const long long cta = ((long long)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    const long long per_cta = ((bytes / ctas + CHUNK) / CHUNK) * CHUNK;
    const long long lo = cta * per_cta;
    const long long hi = min(bytes & ~15LL, lo + per_cta);
    for (long long o = lo + (long long)threadIdx.x * CHUNK; o < hi; o += (long long)threads * CHUNK) {
        const unsigned sz = (unsigned)min(CHUNK, hi - o);
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"((const char*)ptr + o), "r"(sz) : "memory");
    }
}

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads; every thread gets the result.  The
// order of the additions is fixed by the thread count alone, so a row's result
// does not depend on which other rows are in the launch.
__device__ __forceinline__ float block_sum(float v, float* red /* [32] shared */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();  // protect red from a previous use
    if (lane == 0) red[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float t = (lane < nw) ? red[lane] : 0.f;
    t = warp_sum(t);
    return t;
}

__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float t = (lane < nw) ? red[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}
