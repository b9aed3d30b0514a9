// Causal grouped-query attention over the paged cache, generic form: any head
// size up to 256 (even), any number of heads and kv heads, any query length, an
// optional window, float32 arithmetic throughout.  It is the whole attention of
// the float32 path and the fallback of the bfloat16 path for head sizes that the
// tensor-core kernels do not take.
//
// One warp per (query token, head).  Keys are visited in chunks of 32 starting at
// the first visible key; lane i of the warp scores key i of the chunk, the running
// maximum and sum follow the online-softmax recurrence, and the lanes share the
// value accumulation by dimension.  A query at absolute position p sees keys
// [max(0, p + 1 - window), p]; the keys of its own step were appended before this
// kernel runs, so the loop bound is the whole mask (reference
// backend/model.cu:343-408: len = pos + 1, window start :361-362, scale after the
// dot :376, one division by the sum at the end :395-406).  The order of all sums
// depends on p and the window only, never on the batch or the cut of the prompt.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(attention_generic)

namespace {

constexpr int kWarps = 4;
constexpr int kMaxHd = 256;

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
attn_generic_kernel(T* __restrict__ out, const T* __restrict__ q, int64_t q_stride,
                    const T* __restrict__ kcache, const T* __restrict__ vcache,
                    const int* __restrict__ positions, const int* __restrict__ token_req,
                    const int* __restrict__ block_table, int max_blocks, int n_tokens,
                    int n_heads, int n_kv, int hd, int page_size, int window, float scale) {
    __shared__ float qs[kWarps][kMaxHd];
    griddep_wait();
    griddep_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * kWarps + warp;
    if (item >= (int64_t)n_tokens * n_heads) return;
    const int t = (int)(item / n_heads), h = (int)(item - (int64_t)t * n_heads);
    const int g = h / (n_heads / n_kv);
    const int p = positions[t];
    const int len = p + 1;
    const int start = (window > 0 && len > window) ? len - window : 0;
    const int* table = block_table + (int64_t)token_req[t] * max_blocks;

    const T* qr = q + (int64_t)t * q_stride + (int64_t)h * hd;
    for (int i = lane; i < hd; i += 32) qs[warp][i] = to_f32(qr[i]);
    __syncwarp();

    const int64_t head_off = (int64_t)g * page_size * hd;
    const int64_t page_elems = (int64_t)n_kv * page_size * hd;
    float acc[kMaxHd / 32];
#pragma unroll
    for (int i = 0; i < kMaxHd / 32; i++) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int base = start; base < len; base += 32) {
        const int key = base + lane;
        float sc = -INFINITY;
        int64_t row = 0;
        if (key < len) {
            const int page = table[key / page_size];
            row = (int64_t)page * page_elems + head_off + (int64_t)(key % page_size) * hd;
            const T* kr = kcache + row;
            float dot = 0.f;
            for (int d = 0; d < hd; d++) dot += qs[warp][d] * to_f32(kr[d]);
            sc = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(sc));
        const float corr = expf(m - m_new);  // 0 on the first chunk (m = -inf)
        const float pr = (key < len) ? expf(sc - m_new) : 0.f;
        l = l * corr + warp_sum(pr);
        m = m_new;
#pragma unroll
        for (int i = 0; i < kMaxHd / 32; i++) acc[i] *= corr;
        const int cnt = min(32, len - base);
        for (int j = 0; j < cnt; j++) {
            const float pj = __shfl_sync(0xffffffffu, pr, j);
            const int64_t rj = __shfl_sync(0xffffffffu, row, j);
            const T* vr = vcache + rj;
#pragma unroll
            for (int i = 0; i < kMaxHd / 32; i++) {
                const int d = lane + 32 * i;
                if (d < hd) acc[i] += pj * to_f32(vr[d]);
            }
        }
    }
    const float inv = 1.f / l;
    T* orow = out + (int64_t)t * n_heads * hd + (int64_t)h * hd;
#pragma unroll
    for (int i = 0; i < kMaxHd / 32; i++) {
        const int d = lane + 32 * i;
        if (d < hd) orow[d] = from_f32<T>(acc[i] * inv);
    }
}

}  // namespace

// out [n, n_heads*hd]; q rows of n_heads*hd at stride q_stride (elements);
// caches [pages, n_kv, page_size, hd]; block_table [requests, max_blocks].
extern "C" int kllm_attention_generic(void* out, const void* q, int64_t q_stride,
                                      const void* kcache, const void* vcache,
                                      const int* positions, const int* token_req,
                                      const int* block_table, int max_blocks, int n_tokens,
                                      int n_heads, int n_kv, int hd, int page_size, int window,
                                      float scale, int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (hd <= 0 || hd > kMaxHd) KLLM_FAIL("attention: head size %d not in 1..%d", hd, kMaxHd);
    if (n_kv <= 0 || n_heads % n_kv) KLLM_FAIL("attention: %d heads over %d kv heads", n_heads, n_kv);
    if (page_size <= 0) KLLM_FAIL("attention: page size %d", page_size);
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t items = (int64_t)n_tokens * n_heads;
    const unsigned grid = (unsigned)((items + kWarps - 1) / kWarps);
    if (dtype == KLLM_F32)
        kllm_launch((attn_generic_kernel<float>), dim3(grid), dim3(kWarps * 32), 0, s, 
            (float*)out, (const float*)q, q_stride, (const float*)kcache, (const float*)vcache,
            positions, token_req, block_table, max_blocks, n_tokens, n_heads, n_kv, hd, page_size,
            window, scale);
    else if (dtype == KLLM_BF16)
        kllm_launch((attn_generic_kernel<bf16>), dim3(grid), dim3(kWarps * 32), 0, s, 
            (bf16*)out, (const bf16*)q, q_stride, (const bf16*)kcache, (const bf16*)vcache,
            positions, token_req, block_table, max_blocks, n_tokens, n_heads, n_kv, hd, page_size,
            window, scale);
    else
        KLLM_FAIL("attention: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}
