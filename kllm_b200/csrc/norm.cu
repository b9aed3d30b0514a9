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

}  // namespace

// dtype: element type of out; res_dtype: element type of res (ignored when res is NULL).
extern "C" int kllm_add_rmsnorm(void* x, const void* res, void* out, const void* gain,
                                const int* rows, int n_rows, int d, float eps, int dtype,
                                int res_dtype, void* stream) {
    if (n_rows <= 0) return 0;
    if (d <= 0) KLLM_FAIL("rmsnorm: width %d must be positive", d);
    cudaStream_t s = (cudaStream_t)stream;
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
