// Causal grouped-query attention over the paged cache on tensor cores, bfloat16
// operands with float32 accumulation, one library per head size (compiled with
// -DKLLM_HD=<head size>, a multiple of 16 up to 128).
//
// Two kernels share the tile loader and the softmax recurrence:
//
//  * decode: one query token per CTA and kv head.  The `group` = heads / kv heads
//    query heads that share a kv head form the rows of one 16-row MMA tile (so
//    group <= 16), every key and value is read once for all of them.  The keys of
//    the token are cut into `num_splits` ranges, one CTA each; inside a CTA the
//    four warps take interleaved 16-key slices of every 64-key tile and keep a
//    running (max, sum, output) of their own, merged once at the end in a fixed
//    order.  With more than one split the CTA writes an unnormalised partial
//    result and `attn_combine_kernel` merges the splits, again in a fixed order.
//    The fused form of this kernel (`kllm_attention_decode_fused`) also does the
//    step's rotary encoding and cache write: every CTA rotates its copy of the
//    query in registers, the CTA whose key range ends at the token itself rotates
//    the new key and stores it and the new value into the page before it loads
//    that tile, and the last CTA of a (token, kv head) to finish merges the splits
//    (it is found with one atomic counter; the merge itself runs in split order,
//    so the result does not depend on who is last).  One launch replaces three.
//
//  * prefill: a CTA takes up to 128 rows (64 for head sizes above 64) = (tokens of
//    one request's portion) x (heads of one group), each warp 32 (16) of them as two
//    (one) MMA tiles that share every key and value fragment, and walks the keys from the first
//    visible one to the last token's own position in 64-key tiles that all warps
//    share.  Portions of prompts and single tokens may be mixed in one launch; a
//    CTA finds its request from the prefix sums of the portions' lengths.
//
// Keys and values reach shared memory through cp.async (16-byte pieces, three
// to five stages), rows padded by 16 bytes so that ldmatrix is free of bank conflicts for
// every head size.  Scores, the running maximum, the sum and the output are
// float32; probabilities are rounded to bfloat16 for the second product only.
// Slots of a page beyond a request's length are never read: rows past the last
// key are zero-filled instead of loaded.  The math is the reference's
// (backend/model.cu:343-408): keys [max(0, p + 1 - window), p], scale after the
// dot product, one division by the sum at the end.
#include <mutex>
#include "common.cuh"
#include "attention_tc_static.h"

#ifndef KLLM_HD
#error "compile with -DKLLM_HD=<head size>"
#endif

KLLM_EXPORT_LAST_ERROR(attention_tc)

namespace {

constexpr int HD = KLLM_HD;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 128, "head size must be a multiple of 16 up to 128");
constexpr int KSTEPS = HD / 16;          // MMA k-steps over the head dims (scores)
constexpr int DTILES = HD / 8;           // 8-wide output tiles over the head dims
constexpr int CHUNKS = HD / 8;           // 16-byte pieces of a key row
constexpr int TILE = 64;                 // keys per shared-memory tile
constexpr int ROW = HD + 8;              // padded row, in elements (16 bytes of padding)
constexpr int THREADS = 128;
constexpr int STAGE_ELEMS = 2 * TILE * ROW;                       // K tile then V tile
// Decode CTAs are few and each walks a short key range: the deeper the pipeline,
// the more of the range is in flight at once (with 5 stages a range of 256 keys is
// requested whole before the first tile is used).  Prefill keeps 3 stages and more
// CTAs per SM.
constexpr int DEC_STAGES_DEEP = HD <= 64 ? 5 : (HD <= 96 ? 4 : 3);   // few CTAs: everything in flight at once
constexpr int DEC_PAGES = 256;                                        // block-table entries of a range kept in shared memory
constexpr int DEC_STAGES_WIDE = 3;                                    // many CTAs: more of them per SM
constexpr int PRE_STAGES = 3;
constexpr int PRE_SMEM_BYTES = PRE_STAGES * STAGE_ELEMS * 2;
constexpr int dec_smem_bytes(int stages) { return stages * STAGE_ELEMS * 2; }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;    // 0: the 16 bytes are filled with zeros, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Keys key0 .. key0+63 of kv head g into one stage (K tile, then V tile).  Rows at
// or past `hi` are zero-filled.
// `table` holds the request's pages from logical page `page_base` on (the block table
// itself with base 0, or a copy of the needed slice in shared memory).
__device__ __forceinline__ void load_tile(bf16* stage, const bf16* __restrict__ kcache,
                                          const bf16* __restrict__ vcache, const int* table,
                                          int key0, int hi, int g, int n_kv, int page_size, int page_base = 0) {
    bf16* sk = stage;
    bf16* sv = stage + TILE * ROW;
    const int lp0 = key0 / page_size, in_page = key0 - lp0 * page_size;
    if (in_page + TILE <= page_size) {
        // the whole tile lies in one page: one look-up, rows one after the other
        const int64_t base = (((int64_t)table[lp0 - page_base] * n_kv + g) * page_size + in_page) * HD;
#pragma unroll
        for (int c = threadIdx.x; c < TILE * CHUNKS; c += THREADS) {
            const int row = c / CHUNKS, ch = c - row * CHUNKS;
            const bool valid = key0 + row < hi;
            const int64_t off = valid ? base + row * HD + ch * 8 : 0;
            cp_async16(sk + row * ROW + ch * 8, kcache + off, valid);
            cp_async16(sv + row * ROW + ch * 8, vcache + off, valid);
        }
        return;
    }
    for (int c = threadIdx.x; c < TILE * CHUNKS; c += THREADS) {
        const int row = c / CHUNKS, ch = c - row * CHUNKS;
        const int key = key0 + row;
        const bool valid = key < hi;
        int64_t off = 0;
        if (valid) {
            const int lp = key / page_size;
            const int page = table[lp - page_base];
            off = (((int64_t)page * n_kv + g) * page_size + (key - lp * page_size)) * HD + ch * 8;
        }
        cp_async16(sk + row * ROW + ch * 8, kcache + off, valid);
        cp_async16(sv + row * ROW + ch * 8, vcache + off, valid);
    }
}

// Scores of 16 rows against keys [16*slice, 16*slice+16) of a K tile.
__device__ __forceinline__ void scores16(float (&s)[2][4], const uint32_t (&qa)[KSTEPS][4], const bf16* sk,
                                         int slice, int lane) {
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) s[i][j] = 0.f;
    const int mi = lane >> 3;
    const bf16* base = sk + (16 * slice + (mi >> 1) * 8 + (lane & 7)) * ROW + (mi & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ks++) {
        uint32_t b[4];
        ldmatrix_x4(b, base + ks * 16);
        mma_bf16(s[0], qa[ks], b[0], b[1]);
        mma_bf16(s[1], qa[ks], b[2], b[3]);
    }
}

// o += P (16 rows x 16 keys, bfloat16 fragments) times the values of keys
// [16*slice, 16*slice+16) of a V tile.
__device__ __forceinline__ void accumulate16(float (&o)[DTILES][4], const uint32_t (&pa)[4], const bf16* sv,
                                             int slice, int lane) {
    const int mi = lane >> 3;
    const bf16* base = sv + (16 * slice + (mi & 1) * 8 + (lane & 7)) * ROW + (mi >> 1) * 8;
#pragma unroll
    for (int dp = 0; dp < HD / 16; dp++) {
        uint32_t v[4];
        ldmatrix_x4_trans(v, base + dp * 16);
        mma_bf16(o[2 * dp], pa, v[0], v[1]);
        mma_bf16(o[2 * dp + 1], pa, v[2], v[3]);
    }
}

// ---- decode -------------------------------------------------------------------

// What the fused form needs beside the plain one: this step's k and v rows, the
// cos/sin table of a full-width rotary encoding [max_position, HD], and one counter
// per (token, kv head), zero before the first launch and zero again after each.
struct DecodeFusion {
    const bf16* k_new;
    int64_t k_stride;
    const bf16* v_new;
    int64_t v_stride;
    const float* cos_sin;
    unsigned int* counters;
    int tl_slot;            // timeline row of this launch (-1: none)
    const void* prefetch;   // optional: weights that a later kernel streams, to be brought into L2
    long long prefetch_bytes;
};

// Merge of the splits of one (token, kv head) by one CTA.  (m, l) of row r and split j
// sit at ml + r * ml_r + j * ml_j, the partial output row at po + r * o_r + j * o_j, in
// global memory (GLOBAL: written by other CTAs, read past L1) or in this CTA's shared
// memory.  Every load of a kind is issued together with the others of its kind, so the
// merge costs two round trips: first all (m, l), then the partial outputs, four dims of
// all splits per thread.  Sums run over the splits in order.
template <bool GLOBAL>
__device__ __forceinline__ void merge_splits(bf16* __restrict__ out, const float* ml, int64_t ml_r, int64_t ml_j,
                                             const float* po, int64_t o_r, int64_t o_j, unsigned char* scratch,
                                             int64_t th0, int gs, int num_splits) {
    float* w_sm = reinterpret_cast<float*>(scratch);        // [gs][num_splits]: m, then the split's weight
    float* l_sm = w_sm + gs * num_splits;                   // [gs][num_splits]: l
    float* inv_sm = l_sm + gs * num_splits;                 // [gs]: 1 / sum
    for (int e = threadIdx.x; e < gs * num_splits; e += THREADS) {
        const int r = e / num_splits, j = e - r * num_splits;
        const float2* p = reinterpret_cast<const float2*>(ml + r * ml_r + j * ml_j);
        const float2 v = GLOBAL ? __ldcg(p) : *p;
        w_sm[e] = v.x;
        l_sm[e] = v.y;
    }
    __syncthreads();
    if (threadIdx.x < gs) {
        float* wr = w_sm + threadIdx.x * num_splits;
        const float* lr = l_sm + threadIdx.x * num_splits;
        float M = -INFINITY;
        for (int j = 0; j < num_splits; j++) M = fmaxf(M, wr[j]);
        float L = 0.f;
        for (int j = 0; j < num_splits; j++) {
            const float f = exp2f(wr[j] - M);
            L += lr[j] * f;
            wr[j] = f;
        }
        inv_sm[threadIdx.x] = 1.f / L;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < gs * (HD / 4); e += THREADS) {
        const int r = e / (HD / 4), d = (e - r * (HD / 4)) * 4;
        const float* pr = po + r * o_r + d;
        const float* wr = w_sm + r * num_splits;
        float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j0 = 0; j0 < num_splits; j0 += 8) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (j0 + u < num_splits) {
                    const float4* p = reinterpret_cast<const float4*>(pr + (j0 + u) * o_j);
                    v[u] = GLOBAL ? __ldcg(p) : *p;
                }
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (j0 + u < num_splits) {
                    const float f = wr[j0 + u];
                    O.x += v[u].x * f; O.y += v[u].y * f; O.z += v[u].z * f; O.w += v[u].w * f;
                }
        }
        const float inv = inv_sm[r];
        uint2 pk;
        pk.x = pack_bf16(O.x * inv, O.y * inv);
        pk.y = pack_bf16(O.z * inv, O.w * inv);
        *reinterpret_cast<uint2*>(out + (th0 + r) * HD + d) = pk;
    }
}

template <bool FUSED, int DEC_STAGES>
__global__ void __launch_bounds__(THREADS)
attn_decode_kernel(bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                   const bf16* __restrict__ q, int64_t q_stride, bf16* __restrict__ kcache,
                   bf16* __restrict__ vcache, const int* __restrict__ positions,
                   const int* __restrict__ token_req, const int* __restrict__ block_table, int max_blocks,
                   int n_heads, int n_kv, int page_size, int window, float scale_log2e, int num_splits,
                   const DecodeFusion fu) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    __shared__ int s_is_last;
    __shared__ int s_pages[DEC_PAGES];
    __shared__ bf16 s_newkv[2 * HD];       // the writer CTA's rotated new key, then the new value
    // Plain form: the kernel before this one wrote this step's keys into the pages.
    // Fused form: nobody but this kernel writes this layer's pages, so their tiles may
    // be requested while the projection kernel before it is still finishing.
    TL_BEGIN();
    if (!FUSED) { griddep_wait(); griddep_launch(); }
    const int split = blockIdx.x, g = blockIdx.y, t = blockIdx.z;
    const int gs = n_heads / n_kv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tq = lane & 3;
    const bool whole_row = !token_req && max_blocks <= DEC_PAGES;
    const int* table = block_table + (int64_t)(token_req ? token_req[t] : t) * max_blocks;
    if (whole_row) {
        for (int i = threadIdx.x; i < max_blocks; i += THREADS) s_pages[i] = table[i];
    }
    const int len = positions[t] + 1;
    if (whole_row) __syncthreads();
    const int start = (window > 0 && len > window) ? len - window : 0;
    const int total = len - start;
    const int chunk = (((total + num_splits - 1) / num_splits) + TILE - 1) / TILE * TILE;
    const int lo = start + split * chunk;
    const int hi = min(len, lo + chunk);
    const int ntiles = lo < hi ? (hi - lo + TILE - 1) / TILE : 0;

    // This range's slice of the block table, read once and together: otherwise every
    // tile's copies would wait for their own look-up, one memory round trip after the
    // other.  Without token_req (token t is request t) and with a narrow table the whole
    // row is read at the same time as the position, before the range is known.
    const int* pages = table;
    int page_base = 0;
    if (whole_row) {
        pages = s_pages;
    } else if (ntiles > 0) {
        const int first = lo / page_size, count = (hi - 1) / page_size - first + 1;
        if (count <= DEC_PAGES) {
            for (int i = threadIdx.x; i < count; i += THREADS) s_pages[i] = table[first + i];
            __syncthreads();
            pages = s_pages;
            page_base = first;
        }
    }
    // the tiles do not depend on the query: start them first
#pragma unroll
    for (int s = 0; s < DEC_STAGES - 1; s++) {
        if (s < ntiles) load_tile(smem + s * STAGE_ELEMS, kcache, vcache, pages, lo + s * TILE, hi, g, n_kv, page_size, page_base);
        cp_async_commit();
    }
    if (FUSED) l2_prefetch_slice(fu.prefetch, fu.prefetch_bytes, THREADS);   // after this kernel's own requests
    // neither do the rotation's angles
    const int p_new = len - 1;
    constexpr int ROT = (FUSED && KSTEPS >= 2) ? KSTEPS / 2 : 1;
    float rc[ROT][4][2], rs[ROT][4][2];
    if (FUSED) {
        const float* cs = fu.cos_sin + (int64_t)p_new * HD;
#pragma unroll
        for (int ks = 0; ks < KSTEPS / 2; ks++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int j = ks * 16 + 2 * tq + (i >= 2 ? 8 : 0);
                const float2 c2 = *reinterpret_cast<const float2*>(cs + j), s2 = *reinterpret_cast<const float2*>(cs + HD / 2 + j);
                rc[ks][i][0] = c2.x; rc[ks][i][1] = c2.y; rs[ks][i][0] = s2.x; rs[ks][i][1] = s2.y;
            }
    }
    TL_MARK(1);
    if (FUSED) { griddep_wait(); griddep_launch(); }
    TL_MARK(2);

    uint32_t qa[KSTEPS][4];
    {
        const bf16* qb = q + (int64_t)t * q_stride + (int64_t)g * gs * HD;
        const bool v0 = gid < gs, v1 = gid + 8 < gs;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            const int c = ks * 16 + 2 * tq;
            qa[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(qb + gid * HD + c) : 0u;
            qa[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(qb + (gid + 8) * HD + c) : 0u;
            qa[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(qb + gid * HD + c + 8) : 0u;
            qa[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(qb + (gid + 8) * HD + c + 8) : 0u;
        }
    }
    // The CTA whose range holds the token's own position owns the new key and value:
    // it stores them into the page for later steps and, instead of reading them back,
    // writes them over their row of the shared-memory tile once that tile has landed.
    const bool writer = FUSED && lo <= p_new && p_new < hi;
    if (FUSED) {
        // rotate_half on the query fragments: dims d and d + HD/2 sit in the same
        // register slot of k-steps ks and ks + KSTEPS/2 (rotation in float32, stored
        // as bfloat16 like the separate kernel does; reference backend/model.cu:170-184)
        const float* cs = fu.cos_sin + (int64_t)p_new * HD;
#pragma unroll
        for (int ks = 0; ks < KSTEPS / 2; ks++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float c0 = rc[ks][i][0], c1 = rc[ks][i][1], s0 = rs[ks][i][0], s1 = rs[ks][i][1];
                const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&qa[ks][i]);
                const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&qa[ks + KSTEPS / 2][i]);
                const float a0 = __low2float(a), a1 = __high2float(a), b0 = __low2float(b), b1 = __high2float(b);
                qa[ks][i] = pack_bf16(a0 * c0 - b0 * s0, a1 * c1 - b1 * s1);
                qa[ks + KSTEPS / 2][i] = pack_bf16(b0 * c0 + a0 * s0, b1 * c1 + a1 * s1);
            }
        if (writer) {
            const int lp = p_new / page_size;
            const int64_t dst = (((int64_t)pages[lp - page_base] * n_kv + g) * page_size + (p_new - lp * page_size)) * HD;
            const bf16* kr = fu.k_new + (int64_t)t * fu.k_stride + (int64_t)g * HD;
            const bf16* vr = fu.v_new + (int64_t)t * fu.v_stride + (int64_t)g * HD;
            for (int j = threadIdx.x; j < HD / 2; j += THREADS) {
                const float c = cs[j], sn = cs[HD / 2 + j];
                const float a = __bfloat162float(kr[j]), b = __bfloat162float(kr[j + HD / 2]);
                const bf16 k0 = __float2bfloat16_rn(a * c - b * sn), k1 = __float2bfloat16_rn(b * c + a * sn);
                kcache[dst + j] = k0; kcache[dst + j + HD / 2] = k1;
                s_newkv[j] = k0; s_newkv[j + HD / 2] = k1;
            }
            for (int j = threadIdx.x; j < HD; j += THREADS) {
                const bf16 vv = vr[j];
                vcache[dst + j] = vv;
                s_newkv[HD + j] = vv;
            }
        }
    }
    float o[DTILES][4];
#pragma unroll
    for (int i = 0; i < DTILES; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) o[i][j] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    TL_MARK(3);

    for (int i = 0; i < ntiles; i++) {
        cp_async_wait<DEC_STAGES - 2>();
        __syncthreads();
        const int nxt = i + DEC_STAGES - 1;
        if (nxt < ntiles)
            load_tile(smem + (nxt % DEC_STAGES) * STAGE_ELEMS, kcache, vcache, pages, lo + nxt * TILE, hi, g, n_kv, page_size, page_base);
        cp_async_commit();
        bf16* sk = smem + (i % DEC_STAGES) * STAGE_ELEMS;
        bf16* sv = sk + TILE * ROW;
        if (writer && i == ntiles - 1) {       // the token's own row: whatever the page held there is replaced
            const int row = p_new - (lo + i * TILE);
            for (int j = threadIdx.x; j < HD; j += THREADS) {
                sk[row * ROW + j] = s_newkv[j];
                sv[row * ROW + j] = s_newkv[HD + j];
            }
            __syncthreads();
        }
        const int key_base = lo + i * TILE + 16 * warp;
        if (key_base < hi) {
            float s[2][4];
            scores16(s, qa, sk, warp, lane);
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (key_base + nt * 8 + 2 * tq + (j & 1) >= hi) s[nt][j] = -INFINITY;
            float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
            float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);   // finite: key_base itself is visible
            const float c0 = exp2f((m0 - n0) * scale_log2e), c1 = exp2f((m1 - n1) * scale_log2e);
            m0 = n0; m1 = n1;
            float p[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                p[nt][0] = exp2f((s[nt][0] - n0) * scale_log2e);
                p[nt][1] = exp2f((s[nt][1] - n0) * scale_log2e);
                p[nt][2] = exp2f((s[nt][2] - n1) * scale_log2e);
                p[nt][3] = exp2f((s[nt][3] - n1) * scale_log2e);
            }
            l0 = l0 * c0 + (p[0][0] + p[0][1] + p[1][0] + p[1][1]);
            l1 = l1 * c1 + (p[0][2] + p[0][3] + p[1][2] + p[1][3]);
#pragma unroll
            for (int i2 = 0; i2 < DTILES; i2++) { o[i2][0] *= c0; o[i2][1] *= c0; o[i2][2] *= c1; o[i2][3] *= c1; }
            uint32_t pa[4] = {pack_bf16(p[0][0], p[0][1]), pack_bf16(p[0][2], p[0][3]),
                              pack_bf16(p[1][0], p[1][1]), pack_bf16(p[1][2], p[1][3])};
            accumulate16(o, pa, sv, warp, lane);
        }
    }
    cp_async_wait<0>();
    __syncthreads();
    TL_MARK(4);
    // merge the four warps, in warp order
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    float* sm_m = reinterpret_cast<float*>(smem_raw);       // [4][16]
    float* sm_l = sm_m + 64;                                // [4][16]
    float* sm_o = sm_l + 64;                                // [4][16][HD]
    if (tq == 0) {
        sm_m[warp * 16 + gid] = m0; sm_m[warp * 16 + gid + 8] = m1;
        sm_l[warp * 16 + gid] = l0; sm_l[warp * 16 + gid + 8] = l1;
    }
#pragma unroll
    for (int dt = 0; dt < DTILES; dt++) {
        float* r0 = sm_o + (warp * 16 + gid) * HD + dt * 8 + 2 * tq;
        float* r1 = sm_o + (warp * 16 + gid + 8) * HD + dt * 8 + 2 * tq;
        r0[0] = o[dt][0]; r0[1] = o[dt][1]; r1[0] = o[dt][2]; r1[1] = o[dt][3];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < gs * HD; e += THREADS) {
        const int r = e / HD, d = e - r * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; w++) M = fmaxf(M, sm_m[w * 16 + r]);
        float L = 0.f, O = 0.f;
        if (M > -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const float f = exp2f((sm_m[w * 16 + r] - M) * scale_log2e);   // 0 for a warp without keys
                L += sm_l[w * 16 + r] * f;
                O += sm_o[(w * 16 + r) * HD + d] * f;
            }
        }
        const int h = g * gs + r;
        if (num_splits == 1) {
            out[(int64_t)t * n_heads * HD + (int64_t)h * HD + d] = __float2bfloat16_rn(O / L);
        } else {
            const int64_t slot = ((int64_t)t * n_heads + h) * num_splits + split;
            part_o[slot * HD + d] = O;
            if (d == 0) { part_ml[slot * 2] = M * scale_log2e; part_ml[slot * 2 + 1] = L; }
        }
    }
    TL_MARK(5);
    if (FUSED && num_splits > 1) {
        // the last CTA of this (token, kv head) to get here merges all splits
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned int prev = atomicAdd(fu.counters + (int64_t)t * n_kv + g, 1u);
            s_is_last = (prev == (unsigned int)num_splits - 1u);
            if (s_is_last) fu.counters[(int64_t)t * n_kv + g] = 0u;      // ready for the next launch
        }
        __syncthreads();
        TL_MARK(6);
        // marks: start, copies issued, dependency wait over, query ready, tiles done,
        // partial written, counted (, merged: only the CTA that merges)
        if (!s_is_last) { TL_END(fu.tl_slot, 200); return; }
        __threadfence();
        const int64_t th0 = (int64_t)t * n_heads + (int64_t)g * gs;
        merge_splits<true>(out, part_ml + th0 * num_splits * 2, num_splits * 2, 2, part_o + th0 * num_splits * HD,
                           (int64_t)num_splits * HD, HD, smem_raw, th0, gs, num_splits);
        TL_MARK(7);
        TL_END(fu.tl_slot, 201);
    }
}

// Merge the splits of the decode kernel, in split order: one block per (token, head).
__global__ void attn_combine_kernel(bf16* __restrict__ out, const float* __restrict__ part_o,
                                    const float* __restrict__ part_ml, int num_splits) {
    griddep_wait();
    griddep_launch();
    const int64_t th = blockIdx.x;
    const float* ml = part_ml + th * num_splits * 2;
    float M = -INFINITY;
    for (int j = 0; j < num_splits; j++) M = fmaxf(M, ml[2 * j]);
    float L = 0.f;
    for (int j = 0; j < num_splits; j++) L += ml[2 * j + 1] * exp2f(ml[2 * j] - M);
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float O = 0.f;
        for (int j = 0; j < num_splits; j++)
            O += part_o[(th * num_splits + j) * HD + d] * exp2f(ml[2 * j] - M);
        out[th * HD + d] = __float2bfloat16_rn(O / L);
    }
}

// ---- prefill ------------------------------------------------------------------

// Rows per warp in the prefill kernel: two 16-row MMA tiles share every key and value
// fragment (half the shared-memory reads per flop) where the registers allow it.
constexpr int MT = HD <= 64 ? 2 : 1;
constexpr int PRE_ROWS = 4 * 16 * MT;          // rows (token x head of the group) per CTA

__global__ void __launch_bounds__(THREADS)
attn_prefill_kernel(bf16* __restrict__ out, const bf16* __restrict__ q, int64_t q_stride,
                    const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                    const int* __restrict__ q_start, const int* __restrict__ start_pos,
                    const int* __restrict__ block_table, int max_blocks, int n_requests, int n_heads,
                    int n_kv, int page_size, int window, float scale_log2e, int tokens_per_tile) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* smem = reinterpret_cast<bf16*>(smem_raw);
    __shared__ int s_req, s_tok0;
    griddep_wait();
    griddep_launch();
    const int g = blockIdx.x % n_kv;
    const int gs = n_heads / n_kv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tq = lane & 3;
    if (threadIdx.x == 0) {
        // CTAs start in the order of blockIdx.x: hand out the tiles back to front, every
        // kv head's share of a tile next to each other, so that those with the longest key
        // ranges (the ends of the portions) start first and the short ones fill the tail
        int tile = (gridDim.x - 1 - blockIdx.x) / n_kv, req = -1, tok0 = 0;
        for (int s = 0; s < n_requests; s++) {
            const int n = q_start[s + 1] - q_start[s];
            const int nt = (n + tokens_per_tile - 1) / tokens_per_tile;
            if (tile < nt) { req = s; tok0 = q_start[s] + tile * tokens_per_tile; break; }
            tile -= nt;
        }
        s_req = req; s_tok0 = tok0;
    }
    __syncthreads();
    const int req = s_req;
    if (req < 0) return;                       // the grid is an upper bound on the tiles
    const int tok0 = s_tok0;
    const int q_end = q_start[req + 1];
    const int n_tok = min(tokens_per_tile, q_end - tok0);
    const int pos0 = start_pos[req] + (tok0 - q_start[req]);      // position of the tile's first token
    const int lo = (window > 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0;
    const int hi = pos0 + n_tok;                                   // last token's position + 1
    const int* table = block_table + (int64_t)req * max_blocks;
    const int ntiles = (hi - lo + TILE - 1) / TILE;

    // this thread's rows, two per MMA tile: (token, head of the group)
    int pr[MT][2], wr[MT][2];            // position of the row's token (-1: row unused), first visible key
    bool vr[MT][2];
    uint32_t qa[MT][KSTEPS][4];
    int64_t orow[MT][2];
#pragma unroll
    for (int m = 0; m < MT; m++) {
        const bf16* qp[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int r = (16 * MT) * warp + 16 * m + gid + 8 * h;
            const int tt = r / gs, hh = r - tt * gs;
            vr[m][h] = tt < n_tok;
            pr[m][h] = vr[m][h] ? pos0 + tt : -1;
            wr[m][h] = (window > 0) ? pr[m][h] + 1 - window : 0;
            qp[h] = q + (int64_t)(tok0 + tt) * q_stride + (int64_t)(g * gs + hh) * HD;
            orow[m][h] = (int64_t)(tok0 + tt) * n_heads * HD + (int64_t)(g * gs + hh) * HD;
        }
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            const int c = ks * 16 + 2 * tq;
            qa[m][ks][0] = vr[m][0] ? *reinterpret_cast<const uint32_t*>(qp[0] + c) : 0u;
            qa[m][ks][1] = vr[m][1] ? *reinterpret_cast<const uint32_t*>(qp[1] + c) : 0u;
            qa[m][ks][2] = vr[m][0] ? *reinterpret_cast<const uint32_t*>(qp[0] + c + 8) : 0u;
            qa[m][ks][3] = vr[m][1] ? *reinterpret_cast<const uint32_t*>(qp[1] + c + 8) : 0u;
        }
    }
    // key range that this warp's rows can see at all
    const int wrow0 = 16 * MT * warp;
    const int wt_first = wrow0 / gs, wt_last = min(n_tok - 1, (wrow0 + 16 * MT - 1) / gs);
    const bool warp_active = wt_first < n_tok;
    const int warp_hi = pos0 + wt_last + 1;
    const int warp_full_below = pos0 + wt_first;                    // keys <= this are causal for every row

    float o[MT][DTILES][4];
    float mx[MT][2], l[MT][2];
#pragma unroll
    for (int m = 0; m < MT; m++) {
#pragma unroll
        for (int i = 0; i < DTILES; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) o[m][i][j] = 0.f;
        mx[m][0] = mx[m][1] = -INFINITY;
        l[m][0] = l[m][1] = 0.f;
    }

#pragma unroll
    for (int s = 0; s < PRE_STAGES - 1; s++) {
        if (s < ntiles) load_tile(smem + s * STAGE_ELEMS, kcache, vcache, table, lo + s * TILE, hi, g, n_kv, page_size);
        cp_async_commit();
    }
    const int mi = lane >> 3;
    for (int i = 0; i < ntiles; i++) {
        cp_async_wait<PRE_STAGES - 2>();
        __syncthreads();
        const int nxt = i + PRE_STAGES - 1;
        if (nxt < ntiles)
            load_tile(smem + (nxt % PRE_STAGES) * STAGE_ELEMS, kcache, vcache, table, lo + nxt * TILE, hi, g, n_kv, page_size);
        cp_async_commit();
        const bf16* sk = smem + (i % PRE_STAGES) * STAGE_ELEMS;
        const bf16* sv = sk + TILE * ROW;
        const int key0 = lo + i * TILE;
        if (!warp_active || key0 >= warp_hi) continue;             // nothing of this tile is visible to the warp
        const bool need_mask = window > 0 || key0 + TILE - 1 > warp_full_below;
        // scores of the warp's rows against the 64 keys: every key fragment serves all MT tiles
        float s[MT][8][4];
#pragma unroll
        for (int m = 0; m < MT; m++)
#pragma unroll
            for (int nt = 0; nt < 8; nt++)
#pragma unroll
                for (int j = 0; j < 4; j++) s[m][nt][j] = 0.f;
#pragma unroll
        for (int sl = 0; sl < 4; sl++) {
            const bf16* base = sk + (16 * sl + (mi >> 1) * 8 + (lane & 7)) * ROW + (mi & 1) * 8;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++) {
                uint32_t b[4];
                ldmatrix_x4(b, base + ks * 16);
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    mma_bf16(s[m][2 * sl], qa[m][ks], b[0], b[1]);
                    mma_bf16(s[m][2 * sl + 1], qa[m][ks], b[2], b[3]);
                }
            }
        }
        uint32_t pa[MT][4][4];           // probabilities as bfloat16 A fragments, per 16-key slice
#pragma unroll
        for (int m = 0; m < MT; m++) {
            if (need_mask) {
#pragma unroll
                for (int nt = 0; nt < 8; nt++)
#pragma unroll
                    for (int j = 0; j < 2; j++) {
                        const int key = key0 + nt * 8 + 2 * tq + j;
                        if (key > pr[m][0] || key < wr[m][0]) s[m][nt][j] = -INFINITY;
                        if (key > pr[m][1] || key < wr[m][1]) s[m][nt][2 + j] = -INFINITY;
                    }
            }
            float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                t0 = fmaxf(t0, fmaxf(s[m][nt][0], s[m][nt][1]));
                t1 = fmaxf(t1, fmaxf(s[m][nt][2], s[m][nt][3]));
            }
            t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1));
            t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
            t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1));
            t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
            const float n0 = fmaxf(mx[m][0], t0), n1 = fmaxf(mx[m][1], t1);
            // a row that has seen no key yet keeps max -inf: subtract 0 instead, all its p are exp2(-inf) = 0
            const float b0 = (n0 == -INFINITY) ? 0.f : n0, b1 = (n1 == -INFINITY) ? 0.f : n1;
            const float c0 = exp2f((mx[m][0] - b0) * scale_log2e), c1 = exp2f((mx[m][1] - b1) * scale_log2e);
            mx[m][0] = n0; mx[m][1] = n1;
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int nt = 0; nt < 8; nt++) {
                s[m][nt][0] = exp2f((s[m][nt][0] - b0) * scale_log2e);
                s[m][nt][1] = exp2f((s[m][nt][1] - b0) * scale_log2e);
                s[m][nt][2] = exp2f((s[m][nt][2] - b1) * scale_log2e);
                s[m][nt][3] = exp2f((s[m][nt][3] - b1) * scale_log2e);
                sum0 += s[m][nt][0] + s[m][nt][1];
                sum1 += s[m][nt][2] + s[m][nt][3];
            }
            l[m][0] = l[m][0] * c0 + sum0;
            l[m][1] = l[m][1] * c1 + sum1;
#pragma unroll
            for (int i2 = 0; i2 < DTILES; i2++) {
                o[m][i2][0] *= c0; o[m][i2][1] *= c0; o[m][i2][2] *= c1; o[m][i2][3] *= c1;
            }
#pragma unroll
            for (int sl = 0; sl < 4; sl++) {
                pa[m][sl][0] = pack_bf16(s[m][2 * sl][0], s[m][2 * sl][1]);
                pa[m][sl][1] = pack_bf16(s[m][2 * sl][2], s[m][2 * sl][3]);
                pa[m][sl][2] = pack_bf16(s[m][2 * sl + 1][0], s[m][2 * sl + 1][1]);
                pa[m][sl][3] = pack_bf16(s[m][2 * sl + 1][2], s[m][2 * sl + 1][3]);
            }
        }
        // output += P . V: every value fragment serves all MT tiles
#pragma unroll
        for (int sl = 0; sl < 4; sl++) {
            const bf16* base = sv + (16 * sl + (mi & 1) * 8 + (lane & 7)) * ROW + (mi >> 1) * 8;
#pragma unroll
            for (int dp = 0; dp < HD / 16; dp++) {
                uint32_t v[4];
                ldmatrix_x4_trans(v, base + dp * 16);
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    mma_bf16(o[m][2 * dp], pa[m][sl], v[0], v[1]);
                    mma_bf16(o[m][2 * dp + 1], pa[m][sl], v[2], v[3]);
                }
            }
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int m = 0; m < MT; m++) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            float lv = l[m][h];
            lv += __shfl_xor_sync(0xffffffffu, lv, 1);
            lv += __shfl_xor_sync(0xffffffffu, lv, 2);
            if (!vr[m][h]) continue;
            const float inv = 1.f / lv;
            bf16* op = out + orow[m][h];
#pragma unroll
            for (int dt = 0; dt < DTILES; dt++)
                *reinterpret_cast<uint32_t*>(op + dt * 8 + 2 * tq) =
                    pack_bf16(o[m][dt][2 * h] * inv, o[m][dt][2 * h + 1] * inv);
        }
    }
}

bool g_attr_set = false;

int set_attributes() {
    if (g_attr_set) return 0;
    cudaError_t e = cudaSuccess;
    auto raise = [&](auto kernel, int bytes) {
        if (e == cudaSuccess) e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    };
    raise(attn_decode_kernel<false, DEC_STAGES_DEEP>, dec_smem_bytes(DEC_STAGES_DEEP));
    raise(attn_decode_kernel<true, DEC_STAGES_DEEP>, dec_smem_bytes(DEC_STAGES_DEEP));
    raise(attn_decode_kernel<false, DEC_STAGES_WIDE>, dec_smem_bytes(DEC_STAGES_WIDE));
    raise(attn_decode_kernel<true, DEC_STAGES_WIDE>, dec_smem_bytes(DEC_STAGES_WIDE));
    raise(attn_prefill_kernel, PRE_SMEM_BYTES);
    if (e != cudaSuccess) {
        snprintf(g_kllm_err, sizeof(g_kllm_err), "attention: cannot get %d bytes of shared memory: %s", dec_smem_bytes(DEC_STAGES_DEEP),
                 cudaGetErrorString(e));
        return (int)e;
    }
    g_attr_set = true;
    return 0;
}

int check_common(int n_heads, int n_kv, int hd, int page_size, const void* q, int64_t q_stride) {
    if (hd != HD) KLLM_FAIL("attention: this library was built for head size %d, not %d", HD, hd);
    if (n_kv <= 0 || n_heads % n_kv) KLLM_FAIL("attention: %d heads over %d kv heads", n_heads, n_kv);
    if (page_size <= 0) KLLM_FAIL("attention: page size %d", page_size);
    if (((uintptr_t)q & 3) || (q_stride & 1)) KLLM_FAIL("attention: q must be 4-byte aligned with an even row stride");
    return 0;
}

}  // namespace

extern "C" int kllm_attention_tc_head_dim() { return HD; }

// Decode form: every token on its own (any batch is valid, one token per request
// is what it is made for).  part_o [n_tokens, n_heads, num_splits, HD] float32 and
// part_ml [n_tokens, n_heads, num_splits, 2] float32 are scratch for num_splits > 1.
extern "C" int kllm_attention_decode(void* out, void* part_o, void* part_ml, const void* q, int64_t q_stride,
                                     const void* kcache, const void* vcache, const int* positions,
                                     const int* token_req, const int* block_table, int max_blocks,
                                     int n_tokens, int n_heads, int n_kv, int hd, int page_size, int window,
                                     float scale, int num_splits, void* stream) {
    if (n_tokens <= 0) return 0;
    int rc = check_common(n_heads, n_kv, hd, page_size, q, q_stride);
    if (rc) return rc;
    if (n_heads / n_kv > 16) KLLM_FAIL("attention decode: %d heads per kv head, at most 16", n_heads / n_kv);
    if (num_splits < 1 || (num_splits > 1 && (!part_o || !part_ml))) KLLM_FAIL("attention decode: bad split arguments");
    if (n_tokens > 65535 || n_kv > 65535) KLLM_FAIL("attention decode: grid too large");
    if ((rc = set_attributes())) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    const float sl2e = scale * 1.4426950408889634f;
    dim3 grid(num_splits, n_kv, n_tokens);
    // few CTAs (they fit the GPU two per SM): the deep pipeline; many: the wide one
    const bool deep = (int64_t)num_splits * n_kv * n_tokens <= 2 * 148;
    if (deep)
        kllm_launch((attn_decode_kernel<false, DEC_STAGES_DEEP>), dim3(grid), dim3(THREADS),
                    dec_smem_bytes(DEC_STAGES_DEEP), s, 
        (bf16*)out, (float*)part_o, (float*)part_ml, (const bf16*)q, q_stride, (bf16*)kcache,
        (bf16*)vcache, positions, token_req, block_table, max_blocks, n_heads, n_kv, page_size, window, sl2e,
        num_splits, DecodeFusion{});
    else
        kllm_launch((attn_decode_kernel<false, DEC_STAGES_WIDE>), dim3(grid), dim3(THREADS),
                    dec_smem_bytes(DEC_STAGES_WIDE), s, 
        (bf16*)out, (float*)part_o, (float*)part_ml, (const bf16*)q, q_stride, (bf16*)kcache,
        (bf16*)vcache, positions, token_req, block_table, max_blocks, n_heads, n_kv, page_size, window, sl2e,
        num_splits, DecodeFusion{});
    if (num_splits > 1)
        kllm_launch((attn_combine_kernel), dim3(n_tokens * n_heads), dim3(HD < 64 ? 32 : 64), 0, s, (bf16*)out, (const float*)part_o,
                                                                          (const float*)part_ml, num_splits);
    KLLM_LAUNCH_STATUS();
}

// Decode form with the step's rotary encoding, cache write and split merge inside
// (one token per request).  q [n, n_heads*HD], k_new and v_new [n, n_kv*HD] are this
// step's projections, unrotated; cos_sin [max_position, HD] (cos | sin); counters
// [n_tokens * n_kv] unsigned, all zero (the kernel leaves them zero).
extern "C" int kllm_attention_decode_fused(void* out, void* part_o, void* part_ml, void* counters, const void* q,
                                           int64_t q_stride, const void* k_new, int64_t k_stride,
                                           const void* v_new, int64_t v_stride, const float* cos_sin,
                                           void* kcache, void* vcache, const int* positions,
                                           const int* token_req, const int* block_table, int max_blocks,
                                           int n_tokens, int n_heads, int n_kv, int hd, int page_size, int window,
                                           float scale, int num_splits, const void* prefetch,
                                           int64_t prefetch_bytes, void* stream) {
    if (n_tokens <= 0) return 0;
    int rc = check_common(n_heads, n_kv, hd, page_size, q, q_stride);
    if (rc) return rc;
    if (prefetch && ((uintptr_t)prefetch & 15)) KLLM_FAIL("attention decode (fused): the matrix to prefetch must be 16-byte aligned");
    if (KSTEPS % 2) KLLM_FAIL("attention decode (fused): head size %d is not a multiple of 32", HD);
    if (n_heads / n_kv > 16) KLLM_FAIL("attention decode: %d heads per kv head, at most 16", n_heads / n_kv);
    if (num_splits < 1 || (num_splits > 1 && (!part_o || !part_ml || !counters)))
        KLLM_FAIL("attention decode (fused): bad split arguments");
    if (num_splits > 256) KLLM_FAIL("attention decode (fused): %d splits, at most 256", num_splits);
    if (((uintptr_t)part_o & 15) || ((uintptr_t)part_ml & 7) || ((uintptr_t)cos_sin & 7) || ((uintptr_t)out & 7))
        KLLM_FAIL("attention decode (fused): scratch, cos/sin table and out must be 16-byte aligned");
    if (!k_new || !v_new || !cos_sin) KLLM_FAIL("attention decode (fused): k, v and the cos/sin table are needed");
    if (n_tokens > 65535 || n_kv > 65535) KLLM_FAIL("attention decode: grid too large");
    if ((rc = set_attributes())) return rc;
    const float sl2e = scale * 1.4426950408889634f;
    DecodeFusion fu{(const bf16*)k_new, k_stride, (const bf16*)v_new, v_stride, cos_sin, (unsigned int*)counters, TL_SLOT(),
                    prefetch, prefetch ? (long long)prefetch_bytes : 0LL};
    dim3 grid(num_splits, n_kv, n_tokens);
    const bool deep = (int64_t)num_splits * n_kv * n_tokens <= 2 * 148;
    auto go = [&](auto kernel, size_t smem) {
        return kllm_launch(kernel, grid, dim3(THREADS), smem, (cudaStream_t)stream, (bf16*)out, (float*)part_o,
                           (float*)part_ml, (const bf16*)q, q_stride, (bf16*)kcache, (bf16*)vcache, positions, token_req,
                           block_table, max_blocks, n_heads, n_kv, page_size, window, sl2e, num_splits, fu);
    };
    if (deep) go(attn_decode_kernel<true, DEC_STAGES_DEEP>, dec_smem_bytes(DEC_STAGES_DEEP));
    else go(attn_decode_kernel<true, DEC_STAGES_WIDE>, dec_smem_bytes(DEC_STAGES_WIDE));
    KLLM_LAUNCH_STATUS();
}

// ---- the entry point that allocates nothing (see attention_tc_static.h) ----------
//
// In host code the name of a __device__ array is only a handle for the runtime, not
// an address a kernel could use; the device address is asked for once per device.
static __device__ __align__(256) float g_static_scratch[KLLM_ATTN_STATIC_SCRATCH_FLOATS];
static constexpr int kMaxDevices = 64;
static float* g_static_scratch_addr[kMaxDevices] = {};
static std::mutex g_static_scratch_lock;     // threads may make their first call on a device together

extern "C" int kllm_attention_decode_static(void* out, const void* q, int64_t q_stride, const void* kcache,
                                            const void* vcache, const int* positions, const int* token_req,
                                            const int* block_table, int max_blocks, int n_tokens, int n_heads,
                                            int n_kv, int hd, int page_size, int window, float scale,
                                            int num_splits, void* stream) {
    if (n_tokens <= 0) return 0;
    if (num_splits < 1) KLLM_FAIL("attention decode (static scratch): num_splits %d", num_splits);
    float* part_o = nullptr;
    float* part_ml = nullptr;
    if (num_splits > 1) {
        const int64_t slots = (int64_t)n_tokens * n_heads * num_splits;
        const int64_t need = slots * (HD + 2);
        if (need > (int64_t)KLLM_ATTN_STATIC_SCRATCH_FLOATS)
            KLLM_FAIL("attention decode (static scratch): %d tokens x %d heads x %d splits need %lld floats of "
                      "scratch, the built-in array holds %d; use fewer splits or the entry point that takes "
                      "scratch buffers", n_tokens, n_heads, num_splits, (long long)need,
                      KLLM_ATTN_STATIC_SCRATCH_FLOATS);
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) {
            snprintf(g_kllm_err, sizeof(g_kllm_err), "attention decode (static scratch): cudaGetDevice: %s",
                     cudaGetErrorString(e));
            return (int)e;
        }
        if (dev < 0 || dev >= kMaxDevices) KLLM_FAIL("attention: device ordinal %d not supported", dev);
        {
            std::lock_guard<std::mutex> hold(g_static_scratch_lock);
            if (g_static_scratch_addr[dev] == nullptr) {
                float* p = nullptr;
                e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
                if (e != cudaSuccess || p == nullptr) {
                    snprintf(g_kllm_err, sizeof(g_kllm_err),
                             "attention decode (static scratch): cudaGetSymbolAddress on device %d: %s", dev,
                             cudaGetErrorString(e));
                    return e != cudaSuccess ? (int)e : KLLM_ERR_ARG;
                }
                g_static_scratch_addr[dev] = p;
            }
            part_o = g_static_scratch_addr[dev];
        }
        part_ml = part_o + slots * HD;
    }
    return kllm_attention_decode(out, part_o, part_ml, q, q_stride, kcache, vcache, positions, token_req,
                                 block_table, max_blocks, n_tokens, n_heads, n_kv, hd, page_size, window, scale,
                                 num_splits, stream);
}

// Prefill form: requests' portions q_start[s]..q_start[s+1] (prefix sums, [n_requests+1])
// starting at cache position start_pos[s].
extern "C" int kllm_attention_prefill(void* out, const void* q, int64_t q_stride, const void* kcache,
                                      const void* vcache, const int* q_start, const int* start_pos,
                                      const int* block_table, int max_blocks, int n_tokens, int n_requests,
                                      int n_heads, int n_kv, int hd, int page_size, int window, float scale,
                                      void* stream) {
    if (n_tokens <= 0) return 0;
    int rc = check_common(n_heads, n_kv, hd, page_size, q, q_stride);
    if (rc) return rc;
    const int gs = n_heads / n_kv;
    if (gs > 64) KLLM_FAIL("attention prefill: %d heads per kv head, at most 64", gs);
    if ((rc = set_attributes())) return rc;
    const int tpt = PRE_ROWS / gs;
    const int max_tiles = n_tokens / tpt + n_requests;          // >= sum of ceil(n_s / tpt)
    const float sl2e = scale * 1.4426950408889634f;
    dim3 grid(max_tiles * n_kv);
    kllm_launch((attn_prefill_kernel), dim3(grid), dim3(THREADS), PRE_SMEM_BYTES, (cudaStream_t)stream, 
        (bf16*)out, (const bf16*)q, q_stride, (const bf16*)kcache, (const bf16*)vcache, q_start, start_pos,
        block_table, max_blocks, n_requests, n_heads, n_kv, page_size, window, sl2e, tpt);
    KLLM_LAUNCH_STATUS();
}
