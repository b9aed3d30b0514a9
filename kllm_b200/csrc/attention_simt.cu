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

// ---- one chunk of one decoding token, float32 storage, head size 64 or 128 ---------
// The tile kernel above gives a decoding token's 1 to 16 rows (the heads of a kv group)
// an eighth of its threads.  Here every thread works: the chunk is walked in sub-tiles of
// KT keys (K and V by 16-byte asynchronous copies, a key's row contiguous); for the scores
// thread (key, head group) forms the dot products of its key with its heads' queries, which
// it reads as broadcasts; one warp per head runs the online softmax over the sub-tile; for
// the second product thread (dims 4 d4 .. 4 d4 + 3, up to four heads, key group) adds up
// its keys, and the key groups' sums meet in shared memory in group order.  Same partial
// results, in the same layout, as the tile kernel writes for a chunk; every sum's order
// depends on the token's position, the window and the head alone.
__device__ __forceinline__ void cp_async16_zfill(float* smem_dst, const float* src, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;                       // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}

constexpr int DEC_THREADS = 256;
constexpr int dec_keys(int hd) { return 8192 / hd; }                        // keys of a sub-tile: 128 or 64
constexpr size_t dec_smem_floats(int hd, int gs) {
    return (size_t)2 * dec_keys(hd) * (hd + 4) + (size_t)gs * hd + (size_t)dec_keys(hd) * gs + 3 * gs;
}

template <int HD, int GS>
__global__ void __launch_bounds__(DEC_THREADS, 2)
attn_simt_decode_kernel(float* __restrict__ part_o, float* __restrict__ part_ml, const float* __restrict__ q,
                        int64_t q_stride, const float* __restrict__ kcache, const float* __restrict__ vcache,
                        const int* __restrict__ q_start, const int* __restrict__ start_pos,
                        const int* __restrict__ block_table, int max_blocks, int n_requests, int n_heads, int n_kv,
                        int page_size, int window, float scale, int chunk, int max_splits,
                        const float* __restrict__ slopes) {
    constexpr int KT = dec_keys(HD), LD = HD + 4, D4 = HD / 4;
    constexpr int HGRP = DEC_THREADS / KT;                  // head groups of the first product
    constexpr int HPG = (GS + HGRP - 1) / HGRP;             // heads of a group
    constexpr int HPT = GS < 4 ? GS : 4;                    // heads of a thread in the second product
    constexpr int HG3 = GS / HPT, KG = DEC_THREADS / (D4 * HG3), KPG = KT / KG;
    static_assert(KG >= 1 && KPG >= 1 && KG * KPG == KT && HG3 * HPT == GS, "thread layout");
    extern __shared__ __align__(16) float sm[];
    float* Ks = sm;                                         // [KT][LD]; at the end the key groups' sums
    float* Vs = Ks + KT * LD;                               // [KT][LD]
    float* Qs = Vs + KT * LD;                               // [GS][HD]
    float* Ps = Qs + GS * HD;                               // [KT][GS]: scores, then probabilities
    float* m_s = Ps + KT * GS;                              // [GS] running maximum, sum, and this sub-tile's factor
    float* l_s = m_s + GS;
    float* a_s = l_s + GS;
    griddep_wait();
    griddep_launch();
    const int g = blockIdx.x % n_kv, s = blockIdx.x / n_kv, split = blockIdx.z;
    if (s >= n_requests) return;
    const int tok = q_start[s], pos = start_pos[s];
    const int lo_all = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    const int lo = lo_all + split * chunk, hi = min(pos + 1, lo + chunk);
    if (lo >= hi) return;
    const int* table = block_table + (int64_t)s * max_blocks;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    auto load_tile = [&](int key0) {
#pragma unroll
        for (int u = 0; u < KT * D4 / DEC_THREADS; u++) {
            const int e = tid + u * DEC_THREADS, k = e / D4, c = e - k * D4, kp = key0 + k;
            const bool ok = kp < hi;
            int64_t off = 0;
            if (ok) {
                const int lp = kp / page_size;
                off = (((int64_t)table[lp] * n_kv + g) * page_size + (kp - lp * page_size)) * HD + 4 * c;
            }
            cp_async16_zfill(Ks + k * LD + 4 * c, kcache + off, ok);
            cp_async16_zfill(Vs + k * LD + 4 * c, vcache + off, ok);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    load_tile(lo);
    for (int e = tid; e < GS * D4; e += DEC_THREADS) {
        const int h = e / D4, c = e - h * D4;
        *reinterpret_cast<float4*>(Qs + h * HD + 4 * c) =
            __ldg(reinterpret_cast<const float4*>(q + (int64_t)tok * q_stride + (int64_t)(g * GS + h) * HD + 4 * c));
    }
    if (tid < GS) { m_s[tid] = -INFINITY; l_s[tid] = 0.f; }

    const int k1 = tid % KT, hg1 = tid / KT;                // first product: key and head group
    const int d4 = tid % D4, hg3 = (tid / D4) % HG3, kg = tid / (D4 * HG3);   // second product
    float4 acc[HPT];
#pragma unroll
    for (int i = 0; i < HPT; i++) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);

    for (int key0 = lo; key0 < hi; key0 += KT) {
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();
        // ---- scores of key k1 with the heads of group hg1 ----
        {
            float4 sc[HPG];
#pragma unroll
            for (int i = 0; i < HPG; i++) sc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (hg1 * HPG < GS) {
#pragma unroll 4
                for (int c = 0; c < D4; c++) {
                    const float4 kv = *reinterpret_cast<const float4*>(Ks + k1 * LD + 4 * c);
#pragma unroll
                    for (int i = 0; i < HPG; i++) {
                        const int h = hg1 * HPG + i;
                        if (h < GS) {
                            const float4 qv = *reinterpret_cast<const float4*>(Qs + h * HD + 4 * c);
                            sc[i].x += qv.x * kv.x; sc[i].y += qv.y * kv.y; sc[i].z += qv.z * kv.z; sc[i].w += qv.w * kv.w;
                        }
                    }
                }
                const int kp = key0 + k1;
#pragma unroll
                for (int i = 0; i < HPG; i++) {
                    const int h = hg1 * HPG + i;
                    if (h < GS) {
                        float v = ((sc[i].x + sc[i].y) + (sc[i].z + sc[i].w)) * scale;
                        if (slopes) v += slopes[g * GS + h] * (float)(kp - pos);
                        Ps[k1 * GS + h] = kp < hi ? v : -INFINITY;
                    }
                }
            }
        }
        __syncthreads();
        // ---- online softmax: one warp per head over the sub-tile's keys ----
        for (int h = warp; h < GS; h += DEC_THREADS / 32) {
            float v[KT / 32], mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < KT / 32; j++) {
                v[j] = Ps[(lane + 32 * j) * GS + h];
                mx = fmaxf(mx, v[j]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float m_old = m_s[h], m_new = fmaxf(m_old, mx);        // finite: key0 itself is below hi
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < KT / 32; j++) {
                const float pj = expf(v[j] - m_new);                    // 0 for a key past the end
                Ps[(lane + 32 * j) * GS + h] = pj;
                sum += pj;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            if (lane == 0) {
                const float alpha = expf(m_old - m_new);                // 0 while nothing had been seen
                a_s[h] = alpha;
                l_s[h] = l_s[h] * alpha + sum;
                m_s[h] = m_new;
            }
        }
        __syncthreads();
        // ---- probabilities x values: dims 4 d4 .. + 3 of heads hg3 * HPT .. of the keys of group kg ----
        {
#pragma unroll
            for (int i = 0; i < HPT; i++) {
                const float al = a_s[hg3 * HPT + i];
                acc[i].x *= al; acc[i].y *= al; acc[i].z *= al; acc[i].w *= al;
            }
#pragma unroll 4
            for (int kk = 0; kk < KPG; kk++) {
                const int k = kg * KPG + kk;
                const float4 vv = *reinterpret_cast<const float4*>(Vs + k * LD + 4 * d4);
                float pr[HPT];
                if constexpr (HPT == 4) {
                    const float4 p4 = *reinterpret_cast<const float4*>(Ps + k * GS + hg3 * 4);
                    pr[0] = p4.x; pr[1] = p4.y; pr[2] = p4.z; pr[3] = p4.w;
                } else {
#pragma unroll
                    for (int i = 0; i < HPT; i++) pr[i] = Ps[k * GS + hg3 * HPT + i];
                }
#pragma unroll
                for (int i = 0; i < HPT; i++) {
                    acc[i].x += pr[i] * vv.x; acc[i].y += pr[i] * vv.y; acc[i].z += pr[i] * vv.z; acc[i].w += pr[i] * vv.w;
                }
            }
        }
        __syncthreads();                                    // K, V and P of this sub-tile are no longer read
        if (key0 + KT < hi) load_tile(key0 + KT);
    }
    // ---- the key groups' sums, added in group order ----
    float* red = Ks;                                        // [KG][GS][HD]
#pragma unroll
    for (int i = 0; i < HPT; i++)
        *reinterpret_cast<float4*>(red + ((size_t)kg * GS + hg3 * HPT + i) * HD + 4 * d4) = acc[i];
    __syncthreads();
    for (int e = tid; e < GS * D4; e += DEC_THREADS) {
        const int h = e / D4, c = e - h * D4;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < KG; k++) {
            const float4 v = *reinterpret_cast<const float4*>(red + ((size_t)k * GS + h) * HD + 4 * c);
            o.x += v.x; o.y += v.y; o.z += v.z; o.w += v.w;
        }
        const int64_t row = (int64_t)tok * n_heads + g * GS + h;
        *reinterpret_cast<float4*>(part_o + (row * max_splits + split) * HD + 4 * c) = o;
        if (c == 0) *reinterpret_cast<float2*>(part_ml + (row * max_splits + split) * 2) = make_float2(m_s[h], l_s[h]);
    }
}

template <int HD, int GS>
int launch_decode(float* part_o, float* part_ml, const void* q, int64_t q_stride, const void* kcache, const void* vcache,
                  const int* q_start, const int* start_pos, const int* block_table, int max_blocks, int n_requests,
                  int n_heads, int n_kv, int page_size, int window, float scale, int chunk, int max_splits,
                  const float* slopes, cudaStream_t s) {
    auto kern = attn_simt_decode_kernel<HD, GS>;
    static bool raised = false;
    constexpr size_t smem = dec_smem_floats(HD, GS) * sizeof(float);
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            snprintf(g_kllm_err, sizeof(g_kllm_err), "attention (simt, decode): shared memory limit: %s", cudaGetErrorString(e));
            return (int)e;
        }
        raised = true;
    }
    kllm_launch(kern, dim3(n_requests * n_kv, 1, max_splits), dim3(DEC_THREADS), smem, s, part_o, part_ml, (const float*)q,
                q_stride, (const float*)kcache, (const float*)vcache, q_start, start_pos, block_table, max_blocks,
                n_requests, n_heads, n_kv, page_size, window, scale, chunk, max_splits, slopes);
    KLLM_LAUNCH_STATUS();
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
    // decoding tokens in float32 at the common head sizes and group widths: the kernel in which every thread works
    if (chunk > 0 && dtype == KLLM_F32 && (hd == 64 || hd == 128) && n_requests == max_tiles) {
#define KLLM_SIMT_DEC(HD_, GS_)                                                                                        \
    if (hd == HD_ && gs == GS_)                                                                                       \
        return launch_decode<HD_, GS_>((float*)part_o, (float*)part_ml, q, q_stride, kcache, vcache, q_start, start_pos, \
                                       block_table, max_blocks, n_requests, n_heads, n_kv, page_size, window, scale,  \
                                       chunk, max_splits, slopes, s)
        KLLM_SIMT_DEC(64, 1); KLLM_SIMT_DEC(64, 2); KLLM_SIMT_DEC(64, 4); KLLM_SIMT_DEC(64, 8); KLLM_SIMT_DEC(64, 16);
        KLLM_SIMT_DEC(128, 1); KLLM_SIMT_DEC(128, 2); KLLM_SIMT_DEC(128, 4); KLLM_SIMT_DEC(128, 8); KLLM_SIMT_DEC(128, 16);
#undef KLLM_SIMT_DEC
    }
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
