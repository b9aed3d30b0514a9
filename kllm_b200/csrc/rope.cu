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

// The same on 8 consecutive dims per thread, for bfloat16 with the whole head rotated:
// 16-byte loads and stores, cos and sin as float4.  Needs hd % 16 == 0, strides that are
// multiples of 8 elements and 16-byte aligned pointers.
__device__ __forceinline__ void rotate8(const uint4& va, const uint4& vb, const float* c, const float* s, uint4& oa,
                                        uint4& ob) {
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&va);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&vb);
    __nv_bfloat162* oa2 = reinterpret_cast<__nv_bfloat162*>(&oa);
    __nv_bfloat162* ob2 = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float a0 = __low2float(a2[i]), a1 = __high2float(a2[i]);
        const float b0 = __low2float(b2[i]), b1 = __high2float(b2[i]);
        oa2[i] = __floats2bfloat162_rn(a0 * c[2 * i] - b0 * s[2 * i], a1 * c[2 * i + 1] - b1 * s[2 * i + 1]);
        ob2[i] = __floats2bfloat162_rn(b0 * c[2 * i] + a0 * s[2 * i], b1 * c[2 * i + 1] + a1 * s[2 * i + 1]);
    }
}

__global__ void __launch_bounds__(128)
rope_append_vec8_kernel(bf16* __restrict__ q, int64_t q_stride, const bf16* __restrict__ k, int64_t k_stride,
                        const bf16* __restrict__ v, int64_t v_stride, const float* __restrict__ cos_sin,
                        const int* __restrict__ positions, const int* __restrict__ token_req,
                        const int* __restrict__ block_table, int max_blocks, bf16* __restrict__ kcache,
                        bf16* __restrict__ vcache, int n_heads, int n_kv, int hd, int page_size) {
    griddep_wait();
    griddep_launch();
    const int t = blockIdx.x;
    const int p = positions[t];
    const int half = hd >> 1, groups = half >> 3;            // groups of 8 pairs per head
    const float* cs = cos_sin + (int64_t)p * hd;
    int64_t page_base = -1;
    int slot = 0;
    if (kcache != nullptr) {
        const int page = block_table[(int64_t)token_req[t] * max_blocks + p / page_size];
        if (page >= 0) page_base = (int64_t)page * n_kv * page_size * hd;      // never negative for a validated step
        slot = p % page_size;
    }
    const int q_items = n_heads * groups, k_items = page_base >= 0 ? n_kv * groups : 0;
    const int v_items = page_base >= 0 ? n_kv * (hd >> 3) : 0;
    for (int idx = threadIdx.x; idx < q_items + k_items + v_items; idx += blockDim.x) {
        if (idx < q_items + k_items) {
            const bool is_q = idx < q_items;
            const int it = is_q ? idx : idx - q_items;
            const int h = it / groups, j = (it - h * groups) * 8;
            float c[8], sn[8];
            *reinterpret_cast<float4*>(c) = *reinterpret_cast<const float4*>(cs + j);
            *reinterpret_cast<float4*>(c + 4) = *reinterpret_cast<const float4*>(cs + j + 4);
            *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(cs + half + j);
            *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(cs + half + j + 4);
            const bf16* src = is_q ? q + (int64_t)t * q_stride + h * hd + j : k + (int64_t)t * k_stride + h * hd + j;
            const uint4 va = *reinterpret_cast<const uint4*>(src), vb = *reinterpret_cast<const uint4*>(src + half);
            uint4 oa, ob;
            rotate8(va, vb, c, sn, oa, ob);
            bf16* dst = is_q ? q + (int64_t)t * q_stride + h * hd + j
                             : kcache + page_base + ((int64_t)h * page_size + slot) * hd + j;
            *reinterpret_cast<uint4*>(dst) = oa;
            *reinterpret_cast<uint4*>(dst + half) = ob;
        } else {
            const int it = idx - q_items - k_items;
            const int g = it / (hd >> 3), i = (it - g * (hd >> 3)) * 8;
            *reinterpret_cast<uint4*>(vcache + page_base + ((int64_t)g * page_size + slot) * hd + i) =
                *reinterpret_cast<const uint4*>(v + (int64_t)t * v_stride + g * hd + i);
        }
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
    auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    if (dtype == KLLM_BF16 && rot == hd && hd % 16 == 0 && !((q_stride | k_stride | v_stride) & 7) && aligned(q) &&
        aligned(k) && aligned(v) && aligned(cos_sin) && aligned(kcache) && aligned(vcache)) {
        kllm_launch((rope_append_vec8_kernel), dim3(n_tokens), dim3(threads), 0, s, (bf16*)q, q_stride, (const bf16*)k,
                    k_stride, (const bf16*)v, v_stride, cos_sin, positions, token_req, block_table, max_blocks,
                    (bf16*)kcache, (bf16*)vcache, n_heads, n_kv, hd, page_size);
        KLLM_LAUNCH_STATUS();
    }
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
