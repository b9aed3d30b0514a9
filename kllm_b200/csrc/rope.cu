// Rotary position encoding of q and k, fused with the write of k and v into the
// paged cache.
//
// rotate_half convention: within the first `rot` dims of a head, pair
// (j, j + rot/2) turns by the angle p * theta^(-2j/rot); cos and sin come from a
// float32 table [max_position, rot] (cos in the first half of a row, sin in the
// second) that the position-encoding part computes in float64 on the host, so the
// angle itself is never rounded to less than the reference's double precision
// (reference backend/model.cu:170-184).  The rotation is float32.  Keys are
// cached rotated, as in the reference (:1093-1100); the cache write follows
// kv_append_paged_kernel (:187-201) with the layout [page][kv head][slot][dim].
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(rope)

namespace {

template <typename T>
__global__ void rope_append_kernel(T* __restrict__ q, int64_t q_stride,
                                   const T* __restrict__ k, int64_t k_stride,
                                   const T* __restrict__ v, int64_t v_stride,
                                   const float* __restrict__ cos_sin,
                                   const int* __restrict__ positions,
                                   const int* __restrict__ token_req,
                                   const int* __restrict__ block_table, int max_blocks,
                                   T* __restrict__ kcache, T* __restrict__ vcache,
                                   int n_heads, int n_kv, int hd, int rot, int page_size) {
    griddep_wait();
    griddep_launch();
    const int t = blockIdx.x;
    const int p = positions[t];
    const int half = rot >> 1;
    const float* cs = cos_sin + (int64_t)p * rot;  // rot == 0: no rotation, cache write only

    // q in place
    T* qr = q + (int64_t)t * q_stride;
    for (int idx = threadIdx.x; idx < n_heads * half; idx += blockDim.x) {
        const int h = idx / half, j = idx - h * half;
        const float c = cs[j], s = cs[half + j];
        T* base = qr + h * hd;
        const float a = to_f32(base[j]), b = to_f32(base[j + half]);
        base[j] = from_f32<T>(a * c - b * s);
        base[j + half] = from_f32<T>(b * c + a * s);
    }
    if (kcache == nullptr) return;

    const int page = block_table[(int64_t)token_req[t] * max_blocks + p / page_size];
    if (page < 0) return;  // never for a validated step
    const int slot = p % page_size;
    const T* kr = k + (int64_t)t * k_stride;
    const T* vr = v + (int64_t)t * v_stride;
    const int64_t page_base = (int64_t)page * n_kv * page_size * hd;
    for (int idx = threadIdx.x; idx < n_kv * hd; idx += blockDim.x) {
        const int g = idx / hd, i = idx - g * hd;
        const int64_t dst = page_base + ((int64_t)g * page_size + slot) * hd + i;
        float kv;
        if (i < rot) {
            const int j = i < half ? i : i - half;
            const float c = cs[j], s = cs[half + j];
            const float a = to_f32(kr[g * hd + j]), b = to_f32(kr[g * hd + j + half]);
            kv = i < half ? a * c - b * s : b * c + a * s;
        } else {
            kv = to_f32(kr[g * hd + i]);
        }
        kcache[dst] = from_f32<T>(kv);
        vcache[dst] = vr[g * hd + i];
    }
}

}  // namespace

// q [n, n_heads*hd] is rotated in place.  k, v [n, n_kv*hd] are read; rotated k
// and v go to kcache/vcache [pages, n_kv, page_size, hd].  With kcache == NULL only
// q is rotated (a layer that reads another layer's cache).  With cos_sin == NULL
// nothing is rotated and k, v are only stored.  Strides in elements.
extern "C" int kllm_rope_append(void* q, int64_t q_stride, const void* k, int64_t k_stride,
                                const void* v, int64_t v_stride, const float* cos_sin,
                                const int* positions, const int* token_req,
                                const int* block_table, int max_blocks, void* kcache,
                                void* vcache, int n_tokens, int n_heads, int n_kv, int hd,
                                int rot, int page_size, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (cos_sin == nullptr) rot = 0;
    if (rot < 0 || rot > hd || (rot & 1) || (cos_sin && rot == 0))
        KLLM_FAIL("rope: rotary width %d invalid for head size %d", rot, hd);
    if (page_size <= 0) KLLM_FAIL("rope: page size %d", page_size);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 128;
    if (dtype == KLLM_F32)
        kllm_launch((rope_append_kernel<float>), dim3(n_tokens), dim3(threads), 0, s, 
            (float*)q, q_stride, (const float*)k, k_stride, (const float*)v, v_stride, cos_sin,
            positions, token_req, block_table, max_blocks, (float*)kcache, (float*)vcache, n_heads,
            n_kv, hd, rot, page_size);
    else if (dtype == KLLM_BF16)
        kllm_launch((rope_append_kernel<bf16>), dim3(n_tokens), dim3(threads), 0, s, 
            (bf16*)q, q_stride, (const bf16*)k, k_stride, (const bf16*)v, v_stride, cos_sin,
            positions, token_req, block_table, max_blocks, (bf16*)kcache, (bf16*)vcache, n_heads,
            n_kv, hd, rot, page_size);
    else
        KLLM_FAIL("rope: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}
