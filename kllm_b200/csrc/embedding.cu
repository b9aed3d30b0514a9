// Token embedding lookup and row gathering.
//
//   x[t,:] = float32(E[ids[t],:])      (reference backend/model.cu:89-95)
//
// The residual stream that this fills is float32 whatever the table's element
// type is.  A negative id -(s + 1) stands for "the token that the sampling kernel chose
// for request slot s in the step before", which is still on the device in
// last_token[s]: the host may launch a step before it has read the previous one's
// tokens.  Any other id outside [0, vocab) never indexes the table: its row is filled
// with NaN so the fault shows in the logits (ids are validated on the host before).
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(embedding)

namespace {

template <typename T>
__global__ void embed_kernel(float* __restrict__ x, const T* __restrict__ table,
                             const int* __restrict__ ids, const int* __restrict__ last_token, int d, int vocab) {
    griddep_wait();
    griddep_launch();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 && last_token != nullptr) id = last_token[-id - 1];
    float* xr = x + (int64_t)t * d;
    if (id < 0 || id >= vocab) {
        for (int i = threadIdx.x; i < d; i += blockDim.x) xr[i] = __int_as_float(0x7fc00000);
        return;
    }
    const T* er = table + (int64_t)id * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) xr[i] = to_f32(er[i]);
}

// out[r,:] = in[rows[r],:] for rows of `width` elements of `elem` bytes each
// (role of gather_rows_kernel, reference backend/model.cu:411-417).
__global__ void gather_rows_kernel(char* __restrict__ out, const char* __restrict__ in,
                                   const int* __restrict__ rows, int64_t row_bytes) {
    griddep_wait();
    griddep_launch();
    const int r = blockIdx.x;
    const char* src = in + (int64_t)rows[r] * row_bytes;
    char* dst = out + (int64_t)r * row_bytes;
    if ((row_bytes & 3) == 0) {
        const int n4 = (int)(row_bytes >> 2);
        for (int i = threadIdx.x; i < n4; i += blockDim.x)
            ((uint32_t*)dst)[i] = ((const uint32_t*)src)[i];
    } else {
        for (int64_t i = threadIdx.x; i < row_bytes; i += blockDim.x) dst[i] = src[i];
    }
}

}  // namespace

// last_token: optional int32 table indexed by request slot (see above).
extern "C" int kllm_embed(void* x, const void* table, const int* ids, const int* last_token, int n, int d,
                          int vocab, int dtype, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = d >= 1024 ? 256 : 128;
    if (dtype == KLLM_F32)
        kllm_launch((embed_kernel<float>), dim3(n), dim3(threads), 0, s, (float*)x, (const float*)table, ids, last_token, d, vocab);
    else if (dtype == KLLM_BF16)
        kllm_launch((embed_kernel<bf16>), dim3(n), dim3(threads), 0, s, (float*)x, (const bf16*)table, ids, last_token, d, vocab);
    else
        KLLM_FAIL("embed: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}

extern "C" int kllm_gather_rows(void* out, const void* in, const int* rows, int n_rows,
                                int64_t row_bytes, void* stream) {
    if (n_rows <= 0) return 0;
    kllm_launch((gather_rows_kernel), dim3(n_rows), dim3(256), 0, (cudaStream_t)stream, (char*)out, (const char*)in, rows,
                                                                 row_bytes);
    KLLM_LAUNCH_STATUS();
}
