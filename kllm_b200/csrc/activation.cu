// Gated activation of the feed-forward: out = act(gate) * up, act = SiLU,
// computed in float32 (reference backend/model.cu:477-483:
// g / (1 + expf(-g)) * u).  gate and up may be the two halves of one fused
// projection output: each has its own row stride.  They may be float32 beside a
// bfloat16 out, so that the activation sees the projection's unrounded result.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(activation)

namespace {

template <typename T, typename I>
__global__ void silu_mul_kernel(T* __restrict__ out, int64_t out_stride,
                                const I* __restrict__ gate, int64_t gate_stride,
                                const I* __restrict__ up, int64_t up_stride, int n, int f) {
    griddep_wait();
    griddep_launch();
    const int64_t total = (int64_t)n * f;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = idx / f;
        const int c = (int)(idx - r * f);
        const float g = to_f32(gate[r * gate_stride + c]);
        const float u = to_f32(up[r * up_stride + c]);
        out[r * out_stride + c] = from_f32<T>((g / (1.f + expf(-g))) * u);
    }
}

// Same arithmetic on 4 consecutive elements per thread: float32 gate/up rows read as
// float4, the bfloat16 result stored as 8 bytes.  Needs f % 4 == 0 and 16-byte
// aligned float32 rows (8-byte aligned bfloat16 rows).
__global__ void silu_mul_vec4_kernel(bf16* __restrict__ out, int64_t out_stride,
                                     const float* __restrict__ gate, int64_t gate_stride,
                                     const float* __restrict__ up, int64_t up_stride, int n, int f4) {
    griddep_wait();
    griddep_launch();
    const int64_t total = (int64_t)n * f4;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = idx / f4;
        const int c = (int)(idx - r * f4) * 4;
        const float4 g = *reinterpret_cast<const float4*>(gate + r * gate_stride + c);
        const float4 u = *reinterpret_cast<const float4*>(up + r * up_stride + c);
        __nv_bfloat162 lo = __floats2bfloat162_rn((g.x / (1.f + expf(-g.x))) * u.x, (g.y / (1.f + expf(-g.y))) * u.y);
        __nv_bfloat162 hi = __floats2bfloat162_rn((g.z / (1.f + expf(-g.z))) * u.z, (g.w / (1.f + expf(-g.w))) * u.w);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&lo);
        pk.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(out + r * out_stride + c) = pk;
    }
}

}  // namespace

// dtype: element type of out; in_dtype: element type of gate and up.
extern "C" int kllm_silu_mul(void* out, int64_t out_stride, const void* gate, int64_t gate_stride,
                             const void* up, int64_t up_stride, int n, int f, int dtype, int in_dtype,
                             void* stream) {
    if (n <= 0 || f <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t total = (int64_t)n * f;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == KLLM_F32 && in_dtype == KLLM_F32)
        kllm_launch((silu_mul_kernel<float, float>), dim3((unsigned)blocks), dim3(256), 0, s, 
            (float*)out, out_stride, (const float*)gate, gate_stride, (const float*)up, up_stride, n, f);
    else if (dtype == KLLM_BF16 && in_dtype == KLLM_BF16)
        kllm_launch((silu_mul_kernel<bf16, bf16>), dim3((unsigned)blocks), dim3(256), 0, s, 
            (bf16*)out, out_stride, (const bf16*)gate, gate_stride, (const bf16*)up, up_stride, n, f);
    else if (dtype == KLLM_BF16 && in_dtype == KLLM_F32 && f % 4 == 0 && gate_stride % 4 == 0 && up_stride % 4 == 0 &&
             out_stride % 4 == 0 && (((uintptr_t)gate | (uintptr_t)up) & 15) == 0 && ((uintptr_t)out & 7) == 0) {
        const int64_t work = (int64_t)n * (f / 4);
        int64_t b4 = (work + 255) / 256;
        if (b4 > 148 * 16) b4 = 148 * 16;
        kllm_launch((silu_mul_vec4_kernel), dim3((unsigned)b4), dim3(256), 0, s, (bf16*)out, out_stride,
                    (const float*)gate, gate_stride, (const float*)up, up_stride, n, f / 4);
    } else if (dtype == KLLM_BF16 && in_dtype == KLLM_F32)
        kllm_launch((silu_mul_kernel<bf16, float>), dim3((unsigned)blocks), dim3(256), 0, s, 
            (bf16*)out, out_stride, (const float*)gate, gate_stride, (const float*)up, up_stride, n, f);
    else
        KLLM_FAIL("silu_mul: element types %d (out) and %d (in) are not supported together", dtype, in_dtype);
    KLLM_LAUNCH_STATUS();
}
