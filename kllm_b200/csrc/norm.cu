// RMSNorm with the residual sum folded in.
//
//   x[r,:] (+)= res[r,:]          residual stream, float32, written back
//   out[r,:] = x[r,:] * rsqrt(mean(x^2) + eps) * gain[:]
//
// The sum of squares, the scale and the residual sum are float32 whatever the
// element types of `res` and `out` are (res may be float32 beside a bfloat16 out:
// a projection's float32 result goes into the residual stream unrounded).  One block per row; the order of the
// additions depends on the row width and the block size only.
// Formula: reference backend/model.cu:101-122 (norm) and :144-165 (sum + norm).
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(norm)

namespace {

constexpr int kThreads = 256;

// rows == nullptr: row r of x/res, x is written back.
// rows != nullptr: row rows[r] of x/res is read, nothing is written back (used to
// normalise only the rows whose logits are wanted).
template <typename T, typename R>
__global__ void __launch_bounds__(kThreads)
add_rmsnorm_kernel(float* __restrict__ x, const R* __restrict__ res, T* __restrict__ out,
                   const float* __restrict__ gain, const int* __restrict__ rows,
                   int d, float eps) {
    __shared__ float red[32];
    griddep_wait();
    griddep_launch();
    const int r = blockIdx.x;
    const int64_t src = rows ? (int64_t)rows[r] : (int64_t)r;
    float* xr = x + src * d;
    const R* rr = res ? res + src * d : nullptr;
    T* orow = out + (int64_t)r * d;
    const bool write_back = (rows == nullptr) && (res != nullptr);

    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += kThreads) {
        float v = xr[i];
        if (rr) {
            v += to_f32(rr[i]);
            if (write_back) xr[i] = v;
        }
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float scale = rsqrtf(ss / (float)d + eps);
    for (int i = threadIdx.x; i < d; i += kThreads) {
        float v = xr[i];
        if (rr && !write_back) v += to_f32(rr[i]);
        orow[i] = from_f32<T>(v * scale * gain[i]);
    }
}

// The common case of a step's rows (every row, float32 residual or none, bfloat16 out,
// width a multiple of 4 up to kThreads * 4 * kVec) in one pass: a thread keeps its
// elements in registers between the sum of squares and the scaling, 16-byte accesses.
// Same sums in the same order as the kernel above: thread k adds its elements i = k,
// k + kThreads, ... in that order (here four neighbours at a time, whose squares are
// added first; a rounding may differ from the scalar kernel's).
constexpr int kVec = 8;

__global__ void __launch_bounds__(kThreads)
add_rmsnorm_vec4_kernel(float* __restrict__ x, const float* __restrict__ res, bf16* __restrict__ out,
                        const float* __restrict__ gain, int d, float eps) {
    __shared__ float red[32];
    griddep_wait();
    griddep_launch();
    const int r = blockIdx.x;
    float4* xr = reinterpret_cast<float4*>(x + (int64_t)r * d);
    const float4* rr = res ? reinterpret_cast<const float4*>(res + (int64_t)r * d) : nullptr;
    const float4* g4 = reinterpret_cast<const float4*>(gain);
    const int n4 = d >> 2;
    float4 v[kVec];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kVec; k++) {
        const int i = threadIdx.x + k * kThreads;
        if (i < n4) {
            v[k] = xr[i];
            if (rr) {
                const float4 a = rr[i];
                v[k].x += a.x; v[k].y += a.y; v[k].z += a.z; v[k].w += a.w;
                xr[i] = v[k];
            }
            ss += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
        }
    }
    ss = block_sum(ss, red);
    const float scale = rsqrtf(ss / (float)d + eps);
    uint2* orow = reinterpret_cast<uint2*>(out + (int64_t)r * d);
#pragma unroll
    for (int k = 0; k < kVec; k++) {
        const int i = threadIdx.x + k * kThreads;
        if (i < n4) {
            const float4 g = g4[i];
            __nv_bfloat162 lo = __floats2bfloat162_rn(v[k].x * scale * g.x, v[k].y * scale * g.y);
            __nv_bfloat162 hi = __floats2bfloat162_rn(v[k].z * scale * g.z, v[k].w * scale * g.w);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo);
            pk.y = *reinterpret_cast<uint32_t*>(&hi);
            orow[i] = pk;
        }
    }
}

// One warp per row, the row in registers, no block-wide synchronisation; 8 rows per CTA.
// Width a multiple of 4 up to 32 * 4 * kWarpVec.  Lane l adds the squares of its float4 l,
// l + 32, ... in that order, then the lanes are added in a fixed tree.  Which of the two
// vectorised kernels runs is decided by the width alone, never by the number of rows, so
// a row is summed in the same order whatever else the step holds.
constexpr int kWarpVec = 16;

__global__ void __launch_bounds__(256)
add_rmsnorm_warp_kernel(float* __restrict__ x, const float* __restrict__ res, bf16* __restrict__ out,
                        const float* __restrict__ gain, int n_rows, int d, float eps) {
    griddep_wait();
    griddep_launch();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    float4* xr = reinterpret_cast<float4*>(x + (int64_t)r * d);
    const float4* rr = res ? reinterpret_cast<const float4*>(res + (int64_t)r * d) : nullptr;
    const float4* g4 = reinterpret_cast<const float4*>(gain);
    const int n4 = d >> 2;
    float4 v[kWarpVec];
#pragma unroll
    for (int k = 0; k < kWarpVec; k++) {
        const int i = lane + k * 32;
        if (i < n4) v[k] = xr[i];
    }
    if (rr) {
#pragma unroll
        for (int k = 0; k < kWarpVec; k++) {
            const int i = lane + k * 32;
            if (i < n4) {
                const float4 a = rr[i];
                v[k].x += a.x; v[k].y += a.y; v[k].z += a.z; v[k].w += a.w;
                xr[i] = v[k];
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kWarpVec; k++)
        if (lane + k * 32 < n4) ss += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
    ss = warp_sum(ss);
    const float scale = rsqrtf(ss / (float)d + eps);
    uint2* orow = reinterpret_cast<uint2*>(out + (int64_t)r * d);
#pragma unroll
    for (int k = 0; k < kWarpVec; k++) {
        const int i = lane + k * 32;
        if (i < n4) {
            const float4 g = g4[i];
            __nv_bfloat162 lo = __floats2bfloat162_rn(v[k].x * scale * g.x, v[k].y * scale * g.y);
            __nv_bfloat162 hi = __floats2bfloat162_rn(v[k].z * scale * g.z, v[k].w * scale * g.w);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo);
            pk.y = *reinterpret_cast<uint32_t*>(&hi);
            orow[i] = pk;
        }
    }
}

}  // namespace

// dtype: element type of out; res_dtype: element type of res (ignored when res is NULL).
extern "C" int kllm_add_rmsnorm(void* x, const void* res, void* out, const void* gain,
                                const int* rows, int n_rows, int d, float eps, int dtype,
                                int res_dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0) KLLM_FAIL("rmsnorm: width %d must be positive", d);
    cudaStream_t s = (cudaStream_t)stream;
    auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    if (dtype == KLLM_BF16 && (res == nullptr || res_dtype == KLLM_F32) && rows == nullptr && (d & 3) == 0 &&
        d <= kThreads * 4 * kVec && aligned(x) && aligned(res) && aligned(gain) && ((uintptr_t)out & 7) == 0) {
        if (d <= 32 * 4 * kWarpVec) {
            kllm_launch((add_rmsnorm_warp_kernel), dim3((n_rows + 7) / 8), dim3(256), 0, s, (float*)x, (const float*)res,
                        (bf16*)out, (const float*)gain, n_rows, d, eps);
            KLLM_LAUNCH_STATUS();
        }
        kllm_launch((add_rmsnorm_vec4_kernel), dim3(n_rows), dim3(kThreads), 0, s, (float*)x, (const float*)res, (bf16*)out,
                    (const float*)gain, d, eps);
        KLLM_LAUNCH_STATUS();
    }
    if (res == nullptr) res_dtype = dtype;
    if (dtype == KLLM_F32 && res_dtype == KLLM_F32) {
        kllm_launch((add_rmsnorm_kernel<float, float>), dim3(n_rows), dim3(kThreads), 0, s, 
            (float*)x, (const float*)res, (float*)out, (const float*)gain, rows, d, eps);
    } else if (dtype == KLLM_BF16 && res_dtype == KLLM_BF16) {
        kllm_launch((add_rmsnorm_kernel<bf16, bf16>), dim3(n_rows), dim3(kThreads), 0, s, 
            (float*)x, (const bf16*)res, (bf16*)out, (const float*)gain, rows, d, eps);
    } else if (dtype == KLLM_BF16 && res_dtype == KLLM_F32) {
        kllm_launch((add_rmsnorm_kernel<bf16, float>), dim3(n_rows), dim3(kThreads), 0, s, 
            (float*)x, (const float*)res, (bf16*)out, (const float*)gain, rows, d, eps);
    } else {
        KLLM_FAIL("rmsnorm: element types %d (out) and %d (res) are not supported together", dtype, res_dtype);
    }
    KLLM_LAUNCH_STATUS();
}
