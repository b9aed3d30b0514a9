// Next-token selection on the device, one block per row of float32 logits.
//
// temperature <= 0: greedy, the first index of the maximum with a strict '>'
//   comparison (reference engine/engine.go:216-224).
// temperature  > 0: p = softmax(z / temperature) in float32 and the inverse CDF at
//   a uniform number u in [0, 1) that the caller derives from (seed, request,
//   step), so a draw never depends on what else is in the batch (reference
//   docs/theory/02-autoregressive-decoding.md:122-124 describes the distribution;
//   it ships no sampler).  Thread k owns the contiguous slice k of the row, so the
//   order of all additions is fixed by the vocabulary size alone.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(sampling)

namespace {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, int64_t row_stride,
              int vocab, const float* __restrict__ temperature, const float* __restrict__ uniform) {
    __shared__ float red[32];
    __shared__ float s_val[kThreads];
    __shared__ int s_idx[kThreads];
    __shared__ float s_part[kThreads];
    __shared__ int s_choice;
    griddep_wait();
    griddep_launch();
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* z = logits + (int64_t)r * row_stride;
    const int seg = (vocab + kThreads - 1) / kThreads;
    const int lo = min(vocab, tid * seg), hi = min(vocab, lo + seg);

    // maximum and its first index: slices are in index order, so the first thread
    // holding the maximum holds its first occurrence
    float best = -INFINITY;
    int best_i = -1;
    for (int i = lo; i < hi; i++) {
        const float v = z[i];
        if (best_i < 0 || v > best) { best = v; best_i = i; }
    }
    s_val[tid] = best;
    s_idx[tid] = best_i;
    __syncthreads();
    if (tid == 0) {
        float b = s_val[0];
        int bi = s_idx[0];
        for (int k = 1; k < kThreads; k++)
            if (s_idx[k] >= 0 && s_val[k] > b) { b = s_val[k]; bi = s_idx[k]; }
        s_val[0] = b;
        s_choice = bi;
    }
    __syncthreads();
    const float tau = temperature ? temperature[r] : 0.f;
    if (!(tau > 0.f)) {
        if (tid == 0) out[r] = s_choice;
        return;
    }
    const float zmax = s_val[0];
    const float inv_tau = 1.f / tau;
    float part = 0.f;
    for (int i = lo; i < hi; i++) part += expf((z[i] - zmax) * inv_tau);
    s_part[tid] = part;
    __syncthreads();
    if (tid == 0) {
        float total = 0.f;
        for (int k = 0; k < kThreads; k++) total += s_part[k];
        const float target = uniform[r] * total;
        // slice that holds the target
        float run = 0.f;
        int k = 0;
        for (; k < kThreads - 1; k++) {
            if (run + s_part[k] > target) break;
            run += s_part[k];
        }
        red[0] = run;
        red[1] = target;
        s_idx[0] = k;
    }
    __syncthreads();
    if (tid == s_idx[0]) {
        float run = red[0];
        const float target = red[1];
        int choice = -1;
        for (int i = lo; i < hi; i++) {
            run += expf((z[i] - zmax) * inv_tau);
            if (run > target) { choice = i; break; }
        }
        if (choice < 0) choice = (hi > lo) ? hi - 1 : s_choice;  // rounding at the very end
        out[r] = choice;
    }
}

}  // namespace

// out [rows] int32; logits [rows, vocab] float32 at row_stride elements;
// temperature, uniform [rows] float32 (temperature may be NULL: all greedy).
extern "C" int kllm_sample(int* out, const float* logits, int64_t row_stride, int rows, int vocab,
                           const float* temperature, const float* uniform, void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) KLLM_FAIL("sample: vocabulary %d", vocab);
    if (temperature && !uniform) KLLM_FAIL("sample: temperature given without uniform numbers");
    kllm_launch((sample_kernel), dim3(rows), dim3(kThreads), 0, (cudaStream_t)stream, out, logits, row_stride, vocab,
                                                             temperature, uniform);
    KLLM_LAUNCH_STATUS();
}
