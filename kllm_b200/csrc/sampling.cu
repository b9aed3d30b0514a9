// Next-token selection on the device, one block per row of float32 logits.
//
// temperature <= 0: greedy, the first index of the maximum with a strict '>'
//   comparison (reference engine/engine.go:216-224).
// temperature  > 0: p = softmax(z / temperature) in float32 and the inverse CDF at
//   a uniform number u in [0, 1) that the caller derives from (seed, request,
//   step), so a draw never depends on what else is in the batch (reference
//   docs/theory/02-autoregressive-decoding.md:122-124 describes the distribution;
//   it ships no sampler).  Thread k owns the contiguous slice k of the row and the
//   slices' sums are combined by a fixed tree, so the order of all additions is fixed
//   by the vocabulary size alone.
#include "common.cuh"

#include <limits.h>

KLLM_EXPORT_LAST_ERROR(sampling)

namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;

// the larger value wins; of two equal values, the one with the smaller index
__device__ __forceinline__ void take_better(float& v, int& i, float v2, int i2) {
    if (v2 > v || (v2 == v && i2 < i)) { v = v2; i = i2; }
}

__global__ void __launch_bounds__(kThreads)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, int64_t row_stride,
              int vocab, const float* __restrict__ temperature, const float* __restrict__ uniform,
              int* __restrict__ last_token, const int* __restrict__ slots, int* __restrict__ host_out) {
    __shared__ float s_val[kWarps];
    __shared__ int s_idx[kWarps];
    __shared__ float s_sum[kWarps];
    __shared__ float s_max, s_total;
    __shared__ int s_choice, s_owner;
    griddep_wait();
    griddep_launch();
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* z = logits + (int64_t)r * row_stride;
    const int seg = ((vocab + kThreads - 1) / kThreads + 3) & ~3;          // a multiple of 4: slices start 16-byte aligned
    const int lo = min(vocab, tid * seg), hi = min(vocab, lo + seg);
    const bool vec = (((uintptr_t)z) & 15) == 0;

    // maximum and its first index: a thread's slice is scanned in index order with a
    // strict '>', and slices are merged with "smaller index wins a tie"
    float best = -INFINITY;
    int best_i = INT_MAX;
    auto see = [&](float v, int i) { if (best_i == INT_MAX || v > best) { best = v; best_i = i; } };
    if (vec) {
#pragma unroll 8
        for (int i = lo; i < hi; i += 4) {
            if (i + 4 <= hi) {
                const float4 v = *reinterpret_cast<const float4*>(z + i);
                see(v.x, i); see(v.y, i + 1); see(v.z, i + 2); see(v.w, i + 3);
            } else {
                for (int k = i; k < hi; k++) see(z[k], k);
            }
        }
    } else {
        for (int i = lo; i < hi; i++) see(z[i], i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        take_better(best, best_i, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, best_i, o));
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        float b = s_val[lane];
        int bi = s_idx[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            take_better(b, bi, __shfl_xor_sync(0xffffffffu, b, o), __shfl_xor_sync(0xffffffffu, bi, o));
        if (lane == 0) { s_max = b; s_choice = bi; }
    }
    __syncthreads();
    const float tau = temperature ? temperature[r] : 0.f;
    if (!(tau > 0.f)) {
        if (tid == 0) {
            out[r] = s_choice;
            if (last_token) last_token[slots[r]] = s_choice;
            if (host_out) { host_out[r] = s_choice; __threadfence_system(); }
        }
        return;
    }
    // weights e^((z - max) / tau): a thread's part, then the parts' running sum over the
    // block (scan inside each warp, then over the warps' totals: a fixed tree)
    const float zmax = s_max;
    const float inv_tau = 1.f / tau;
    float part = 0.f;
    if (vec) {
#pragma unroll 8
        for (int i = lo; i < hi; i += 4) {
            if (i + 4 <= hi) {
                const float4 v = *reinterpret_cast<const float4*>(z + i);
                part += expf((v.x - zmax) * inv_tau);
                part += expf((v.y - zmax) * inv_tau);
                part += expf((v.z - zmax) * inv_tau);
                part += expf((v.w - zmax) * inv_tau);
            } else {
                for (int k = i; k < hi; k++) part += expf((z[k] - zmax) * inv_tau);
            }
        }
    } else {
        for (int i = lo; i < hi; i++) part += expf((z[i] - zmax) * inv_tau);
    }
    float incl = part;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) s_sum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        float w = s_sum[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += up;
        }
        s_sum[lane] = w;                       // inclusive over the warps
        if (lane == 31) s_total = w;
    }
    __syncthreads();
    incl += warp ? s_sum[warp - 1] : 0.f;
    const float target = uniform[r] * s_total;
    // the first thread whose running sum passes the target owns the draw
    const unsigned passed = __ballot_sync(0xffffffffu, incl > target && hi > lo);
    if (lane == 0) s_idx[warp] = passed ? warp * 32 + __ffs(passed) - 1 : kThreads;
    __syncthreads();
    if (warp == 0) {
        int c = s_idx[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c = min(c, __shfl_xor_sync(0xffffffffu, c, o));
        if (lane == 0) s_owner = c;
    }
    __syncthreads();
    int owner = s_owner;
    if (owner == kThreads) owner = min(kThreads - 1, (vocab - 1) / seg);     // rounding at the very end: the last slice
    if (tid == owner) {
        float run = incl - part;
        int choice = -1;
        for (int i = lo; i < hi; i++) {
            run += expf((z[i] - zmax) * inv_tau);
            if (run > target) { choice = i; break; }
        }
        if (choice < 0) choice = (hi > lo) ? hi - 1 : s_choice;
        out[r] = choice;
        if (last_token) last_token[slots[r]] = choice;
        if (host_out) { host_out[r] = choice; __threadfence_system(); }
    }
}

}  // namespace

// out [rows] int32; logits [rows, vocab] float32 at row_stride elements;
// temperature, uniform [rows] float32 (temperature may be NULL: all greedy).
// last_token, slots: optional; row r's choice is also stored at last_token[slots[r]], where
// the embedding kernel of the next step finds it (see embedding.cu).
// host_out: optional, pinned host memory that the device can address [rows]: the choices are
// also written there by the kernel itself, which saves the copy that would follow it; the host
// may read them once an event recorded after this launch has completed.
extern "C" int kllm_sample(int* out, const float* logits, int64_t row_stride, int rows, int vocab,
                           const float* temperature, const float* uniform, int* last_token, const int* slots,
                           int* host_out, void* stream) {
    if (rows <= 0) return 0;
    if (vocab <= 0) KLLM_FAIL("sample: vocabulary %d", vocab);
    if (temperature && !uniform) KLLM_FAIL("sample: temperature given without uniform numbers");
    if (last_token && !slots) KLLM_FAIL("sample: a token table without the rows' slots");
    if (host_out) {                      // the address under which the device sees that host memory
        void* mapped = nullptr;
        const cudaError_t e = cudaHostGetDevicePointer(&mapped, host_out, 0);
        if (e != cudaSuccess || !mapped) {
            (void)cudaGetLastError();
            KLLM_FAIL("sample: the host buffer for the choices is not pinned memory that the device can address (%s)",
                      cudaGetErrorString(e));
        }
        host_out = (int*)mapped;
    }
    kllm_launch((sample_kernel), dim3(rows), dim3(kThreads), 0, (cudaStream_t)stream, out, logits, row_stride, vocab,
                                                             temperature, uniform, last_token, slots, host_out);
    KLLM_LAUNCH_STATUS();
}
