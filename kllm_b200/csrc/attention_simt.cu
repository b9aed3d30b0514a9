// Causal grouped-query attention over the paged cache on the CUDA cores, float32
// arithmetic throughout: the attention of the true 32-bit path (prefill and decode), and
// of bfloat16 models whose head size the tensor-core kernels do not take.
//
// A CTA of 256 threads works on a tile of up to 64 rows, a row being one (query token,
// head): `qt` consecutive tokens of one request times the heads that share kv head g.
// It walks the keys the tile can see in tiles of 64 keys: K and V of the tile go to
// shared memory as float32, the 64 x 64 scores are computed as a register-tiled product
// (thread (ty, tx) owns rows ty + 16 i and keys tx + 16 j: the 16 threads of a row sit in
// one half-warp, shared-memory reads are conflict-free), the online-softmax recurrence
// runs per row with half-warp shuffles, the probabilities go through shared memory, and
// the second product accumulates rows ty + 16 i at dims 4 tx + 64 c in registers.
//
// Formulas as the reference computes them (backend/model.cu:343-408): a query at
// absolute position p sees keys [max(0, p + 1 - window), p], the keys of its own step
// having been written before; score = (q . k) * scale, scale applied after the dot
// (:376); max-subtracted expf; one division by the sum at the end (:395-406).  Optionally a
// bias that is linear in the distance is added to every score, slope[head] * (key position -
// query position): position encodings that act on the scores instead of on q and k.
//
// Steps of single tokens (decode) have few rows per kv head and long contexts; there the
// keys of a token are cut into chunks of `chunk` keys, one CTA each (grid.z), which store
// unnormalised partial results that a second kernel merges in chunk order.  The chunk
// boundaries depend on the token's own position and window alone, so every sum of a row
// is formed in an order that does not depend on the batch.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(attention_simt)

namespace {

constexpr int ROWS = 64, KEYS = 64, THREADS = 256, PLD = KEYS + 4;

__device__ __forceinline__ float4 load4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&lo);
    raw.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}
__device__ __forceinline__ float half_warp_max(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// NC: float4 groups of output dims per thread and row, ceil(hd / 64) rounded up to 1, 2 or 4.
template <typename T, int NC>
__global__ void __launch_bounds__(THREADS)
attn_simt_kernel(T* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                 const T* __restrict__ q, int64_t q_stride, const T* __restrict__ kcache,
                 const T* __restrict__ vcache, const int* __restrict__ q_start, const int* __restrict__ start_pos,
                 const int* __restrict__ block_table, int max_blocks, int n_requests, int n_heads, int n_kv, int hd,
                 int page_size, int window, float scale, int qt, int chunk, int max_splits,
                 const float* __restrict__ slopes) {
    extern __shared__ __align__(16) float sm[];
    const int ld = hd + 4;
    float* Qs = sm;
    float* Ks = Qs + ROWS * ld;
    float* Vs = Ks + KEYS * ld;
    float* Ps = Vs + KEYS * ld;
    griddep_wait();
    griddep_launch();

    // which request and which of its tiles this CTA has
    // CTAs start in the order of blockIdx.x: portions hand out their tiles back to front, every
    // kv head's share of a tile next to each other, so that the longest key ranges start first
    const int g = blockIdx.x % n_kv;
    int tile = chunk > 0 ? blockIdx.x / n_kv : (gridDim.x - 1 - blockIdx.x) / n_kv, s = 0, n_new = 0;
    if (chunk > 0) {
        // keys in chunks: the launcher vouches that every request brings one token, tile = request
        s = tile;
        tile = 0;
        n_new = 1;
        if (s >= n_requests) return;
    } else {
        bool found = false;
        for (s = 0; s < n_requests; s++) {
            n_new = q_start[s + 1] - q_start[s];
            const int nt = (n_new + qt - 1) / qt;
            if (tile < nt) { found = true; break; }
            tile -= nt;
        }
        if (!found) return;
    }
    const int q0 = tile * qt;
    const int nq = min(qt, n_new - q0);
    const int gs = n_heads / n_kv, split = blockIdx.z;
    const int R = nq * gs;
    const int tok0 = q_start[s] + q0;
    const int p0 = start_pos[s] + q0;                       // position of the tile's first token
    const int lo_all = (window > 0 && p0 + 1 > window) ? p0 + 1 - window : 0;
    const int hi_all = p0 + nq;
    int lo = lo_all, hi = hi_all;
    if (chunk > 0) {
        lo = lo_all + split * chunk;
        hi = min(hi_all, lo + chunk);
        if (lo >= hi_all) return;
    }
    const int* table = block_table + (int64_t)s * max_blocks;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int hd4 = hd >> 2;

    for (int e = tid; e < ROWS * hd4; e += THREADS) {
        const int r = e / hd4, c = e - r * hd4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < R) {
            const int tq = r / gs, h = r - tq * gs;
            v = load4(q + (int64_t)(tok0 + tq) * q_stride + (int64_t)(g * gs + h) * hd + 4 * c);
        }
        *reinterpret_cast<float4*>(Qs + r * ld + 4 * c) = v;
    }

    float m[4], l[4], slope[4];
    int pos[4], wlo[4];
    float4 acc[4][NC];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        m[i] = -INFINITY;
        l[i] = 0.f;
        const int r = ty + 16 * i;
        pos[i] = r < R ? p0 + r / gs : -1;                  // -1: no key is visible to a row that does not exist
        slope[i] = (slopes && r < R) ? slopes[g * gs + r % gs] : 0.f;
        wlo[i] = window > 0 ? pos[i] + 1 - window : 0;
#pragma unroll
        for (int c = 0; c < NC; c++) acc[i][c] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const bool active = ty < R;                             // row ty exists; the thread's other rows may not
    const int ri = (R + 15) >> 4;                           // row slots i < ri hold rows of this tile (the same for all threads)

    for (int key0 = lo; key0 < hi; key0 += KEYS) {
        __syncthreads();                                    // the tile before is no longer read
        {
            // four threads per key: one look-up of the key's page, then independent 16-byte loads
            const int k = tid >> 2, kp = key0 + k;
            const bool ok = kp < hi;
            int64_t off = 0;
            if (ok) {
                const int lp = kp / page_size;
                off = (((int64_t)table[lp] * n_kv + g) * page_size + (kp - lp * page_size)) * hd;
            }
#pragma unroll 4
            for (int c = tid & 3; c < hd4; c += 4) {
                float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
                if (ok) {
                    kv = load4(kcache + off + 4 * c);
                    vv = load4(vcache + off + 4 * c);
                }
                *reinterpret_cast<float4*>(Ks + k * ld + 4 * c) = kv;
                *reinterpret_cast<float4*>(Vs + k * ld + 4 * c) = vv;
            }
        }
        __syncthreads();

        float sc[4][4];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) sc[i][j] = 0.f;
        if (active) {
            for (int d = 0; d < hd; d += 4) {
                float4 qv[4], kv[4];
#pragma unroll
                for (int i = 0; i < 4; i++)
                    if (i < ri) qv[i] = *reinterpret_cast<const float4*>(Qs + (ty + 16 * i) * ld + d);
#pragma unroll
                for (int j = 0; j < 4; j++) kv[j] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * j) * ld + d);
#pragma unroll
                for (int i = 0; i < 4; i++)
                    if (i < ri)
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        sc[i][j] += qv[i].x * kv[j].x;
                        sc[i][j] += qv[i].y * kv[j].y;
                        sc[i][j] += qv[i].z * kv[j].z;
                        sc[i][j] += qv[i].w * kv[j].w;
                    }
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (i >= ri) break;
            bool vis[4];
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int kp = key0 + tx + 16 * j;
                vis[j] = kp < hi && kp <= pos[i] && kp >= wlo[i];
                sc[i][j] = vis[j] ? sc[i][j] * scale + slope[i] * (float)(kp - pos[i]) : -INFINITY;
                mx = fmaxf(mx, sc[i][j]);
            }
            mx = half_warp_max(mx);
            const float m_new = fmaxf(m[i], mx);
            float alpha = 1.f, psum = 0.f, p[4] = {0.f, 0.f, 0.f, 0.f};
            if (m_new != -INFINITY) {
                alpha = expf(m[i] - m_new);                 // 0 while nothing had been seen (m = -inf)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    p[j] = vis[j] ? expf(sc[i][j] - m_new) : 0.f;
                    psum += p[j];
                }
            }
            psum = half_warp_sum(psum);
            l[i] = l[i] * alpha + psum;
            m[i] = m_new;
#pragma unroll
            for (int j = 0; j < 4; j++) Ps[(ty + 16 * i) * PLD + tx + 16 * j] = p[j];
#pragma unroll
            for (int c = 0; c < NC; c++) {
                acc[i][c].x *= alpha; acc[i][c].y *= alpha; acc[i][c].z *= alpha; acc[i][c].w *= alpha;
            }
        }
        __syncthreads();
        if (active) {
            const int nk = min(KEYS, hi - key0);
            for (int k = 0; k < nk; k += 4) {
                float4 p4[4];
#pragma unroll
                for (int i = 0; i < 4; i++)
                    if (i < ri) p4[i] = *reinterpret_cast<const float4*>(Ps + (ty + 16 * i) * PLD + k);
#pragma unroll
                for (int kk = 0; kk < 4; kk++) {
#pragma unroll
                    for (int c = 0; c < NC; c++) {
                        const int d = 4 * tx + 64 * c;
                        if (d < hd) {
                            const float4 v = *reinterpret_cast<const float4*>(Vs + (k + kk) * ld + d);
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                if (i >= ri) break;
                                const float pv = kk == 0 ? p4[i].x : kk == 1 ? p4[i].y : kk == 2 ? p4[i].z : p4[i].w;
                                acc[i][c].x += pv * v.x; acc[i][c].y += pv * v.y;
                                acc[i][c].z += pv * v.z; acc[i][c].w += pv * v.w;
                            }
                        }
                    }
                }
            }
        }
    }

#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = ty + 16 * i;
        if (r >= R) continue;
        const int tq = r / gs, h = r - tq * gs;
        const int64_t row = (int64_t)(tok0 + tq) * n_heads + g * gs + h;
        if (chunk == 0) {
            const float inv = 1.f / l[i];
#pragma unroll
            for (int c = 0; c < NC; c++) {
                const int d = 4 * tx + 64 * c;
                if (d < hd)
                    store4(out + row * hd + d, make_float4(acc[i][c].x * inv, acc[i][c].y * inv,
                                                           acc[i][c].z * inv, acc[i][c].w * inv));
            }
        } else {
            float* po = part_o + (row * max_splits + split) * hd;
#pragma unroll
            for (int c = 0; c < NC; c++) {
                const int d = 4 * tx + 64 * c;
                if (d < hd) *reinterpret_cast<float4*>(po + d) = acc[i][c];
            }
            if (tx == 0) *reinterpret_cast<float2*>(part_ml + (row * max_splits + split) * 2) = make_float2(m[i], l[i]);
        }
    }
}

// One warp per (token, head): the chunks' partial results, weighted by exp(m_chunk - max)
// and added in chunk order.
template <typename T>
__global__ void __launch_bounds__(128)
attn_simt_merge_kernel(T* __restrict__ out, const float* __restrict__ part_o, const float* __restrict__ part_ml,
                       const int* __restrict__ positions, int n_rows, int n_heads, int hd, int window, int chunk,
                       int max_splits) {
    griddep_wait();
    griddep_launch();
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int p = positions[row / n_heads];
    const int lo_all = (window > 0 && p + 1 > window) ? p + 1 - window : 0;
    const int ns = (p + 1 - lo_all + chunk - 1) / chunk;
    // the chunks' maxima first (all loads at once), then their weights, then the sums in chunk order
    float M = -INFINITY;
    for (int j0 = 0; j0 < ns; j0 += 32) {
        const int j = j0 + lane;
        const float mj = j < ns ? __ldcg(part_ml + (row * max_splits + j) * 2) : -INFINITY;
        M = fmaxf(M, warp_max(mj));
    }
    float L = 0.f;
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = 0.f;
    for (int j0 = 0; j0 < ns; j0 += 4) {
        float2 ml[4];
        float po[4][8];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int j = min(j0 + u, ns - 1);
            ml[u] = __ldcg(reinterpret_cast<const float2*>(part_ml + (row * max_splits + j) * 2));
            const float* src = part_o + (row * max_splits + j) * hd;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int d = lane + 32 * i;
                po[u][i] = d < hd ? __ldcg(src + d) : 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            if (j0 + u >= ns) break;
            const float b = expf(ml[u].x - M);
            L += ml[u].y * b;
#pragma unroll
            for (int i = 0; i < 8; i++) o[i] += po[u][i] * b;
        }
    }
    const float inv = 1.f / L;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int d = lane + 32 * i;
        if (d < hd) out[row * hd + d] = from_f32<T>(o[i] * inv);
    }
}

size_t smem_bytes(int hd) { return (size_t)(3 * 64 * (hd + 4) + ROWS * PLD) * sizeof(float); }

template <typename T, int NC>
int launch(void* out, float* part_o, float* part_ml, const void* q, int64_t q_stride, const void* kcache,
           const void* vcache, const int* q_start, const int* start_pos, const int* block_table, int max_blocks,
           int n_requests, int max_tiles, int n_heads, int n_kv, int hd, int page_size, int window, float scale,
           int qt, int chunk, int max_splits, const float* slopes, cudaStream_t s) {
    auto kern = attn_simt_kernel<T, NC>;
    static bool raised = false;
    const size_t smem = smem_bytes(hd);
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes(64 * NC));
        if (e != cudaSuccess) {
            snprintf(g_kllm_err, sizeof(g_kllm_err), "attention (simt): shared memory limit: %s", cudaGetErrorString(e));
            return (int)e;
        }
        raised = true;
    }
    kllm_launch(kern, dim3(max_tiles * n_kv, 1, chunk > 0 ? max_splits : 1), dim3(THREADS), smem, s, (T*)out, part_o,
                part_ml, (const T*)q, q_stride, (const T*)kcache, (const T*)vcache, q_start, start_pos, block_table,
                max_blocks, n_requests, n_heads, n_kv, hd, page_size, window, scale, qt, chunk, max_splits, slopes);
    KLLM_LAUNCH_STATUS();
}

}  // namespace

// out [tokens, n_heads * hd] contiguous; q rows at stride q_stride (elements); caches
// [pages, n_kv, page_size, hd]; request s brings rows q_start[s] .. q_start[s + 1]
// starting at cache position start_pos[s]; block_table [n_requests, max_blocks].
// max_tiles: an upper bound of the sum over requests of ceil(rows of s / qt).
// chunk == 0: every tile walks all of its keys and writes `out`.  chunk > 0 (only with
// qt == 1): the keys of a token are cut into chunks of that many keys, at most
// max_splits of them, whose partial results go to part_o [rows, max_splits, hd] and
// part_ml [rows, max_splits, 2] (row = token * n_heads + head) for kllm_attention_simt_merge.
// slopes: optional float32 [n_heads]; slope[h] * (key position - query position) is added to
// the scaled scores of head h.
extern "C" int kllm_attention_simt(void* out, void* part_o, void* part_ml, const void* q, int64_t q_stride,
                                   const void* kcache, const void* vcache, const int* q_start, const int* start_pos,
                                   const int* block_table, int max_blocks, int n_requests, int max_tiles,
                                   int n_heads, int n_kv, int hd, int page_size, int window, float scale, int qt,
                                   int chunk, int max_splits, const float* slopes, int dtype, void* stream) {
    if (n_requests <= 0 || max_tiles <= 0) return 0;
    if (hd <= 0 || hd > 256 || hd % 4) KLLM_FAIL("attention (simt): head size %d is not a multiple of 4 up to 256", hd);
    if (n_kv <= 0 || n_heads % n_kv) KLLM_FAIL("attention (simt): %d heads over %d kv heads", n_heads, n_kv);
    const int gs = n_heads / n_kv;
    if (qt < 1 || qt * gs > ROWS) KLLM_FAIL("attention (simt): %d tokens x %d heads exceed the %d rows of a tile", qt, gs, ROWS);
    if (page_size <= 0) KLLM_FAIL("attention (simt): page size %d", page_size);
    if (chunk < 0 || (chunk > 0 && (qt != 1 || max_splits < 1 || !part_o || !part_ml || n_kv > 65535 || max_splits > 65535)))
        KLLM_FAIL("attention (simt): chunks of keys need one token per tile, scratch buffers and a split count");
    const int esize = dtype == KLLM_F32 ? 4 : 2;
    if (((uintptr_t)q | (uintptr_t)kcache | (uintptr_t)vcache | (uintptr_t)out) % (4 * esize) || (q_stride % 4))
        KLLM_FAIL("attention (simt): operands must be aligned to four elements");
    cudaStream_t s = (cudaStream_t)stream;
#define KLLM_SIMT(T, NC)                                                                                              \
    return launch<T, NC>(out, (float*)part_o, (float*)part_ml, q, q_stride, kcache, vcache, q_start, start_pos,      \
                         block_table, max_blocks, n_requests, max_tiles, n_heads, n_kv, hd, page_size, window, scale, \
                         qt, chunk, max_splits, slopes, s)
    if (dtype == KLLM_F32) {
        if (hd <= 64) KLLM_SIMT(float, 1);
        if (hd <= 128) KLLM_SIMT(float, 2);
        KLLM_SIMT(float, 4);
    } else if (dtype == KLLM_BF16) {
        if (hd <= 64) KLLM_SIMT(bf16, 1);
        if (hd <= 128) KLLM_SIMT(bf16, 2);
        KLLM_SIMT(bf16, 4);
    }
#undef KLLM_SIMT
    KLLM_FAIL("attention (simt): unknown element type %d", dtype);
}

extern "C" int kllm_attention_simt_merge(void* out, const void* part_o, const void* part_ml, const int* positions,
                                         int n_tokens, int n_heads, int hd, int window, int chunk, int max_splits,
                                         int dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (hd <= 0 || hd > 256 || chunk <= 0 || max_splits < 1) KLLM_FAIL("attention merge (simt): bad sizes");
    cudaStream_t s = (cudaStream_t)stream;
    const int n_rows = n_tokens * n_heads;
    if (dtype == KLLM_F32)
        kllm_launch((attn_simt_merge_kernel<float>), dim3((n_rows + 3) / 4), dim3(128), 0, s, (float*)out,
                    (const float*)part_o, (const float*)part_ml, positions, n_rows, n_heads, hd, window, chunk, max_splits);
    else if (dtype == KLLM_BF16)
        kllm_launch((attn_simt_merge_kernel<bf16>), dim3((n_rows + 3) / 4), dim3(128), 0, s, (bf16*)out,
                    (const float*)part_o, (const float*)part_ml, positions, n_rows, n_heads, hd, window, chunk, max_splits);
    else
        KLLM_FAIL("attention merge (simt): unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}
