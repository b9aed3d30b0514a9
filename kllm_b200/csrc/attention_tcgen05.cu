// Causal grouped-query attention of prompt portions over the paged cache on the
// fifth-generation tensor cores: both products (scores = Q.K^T and output = P.V) are
// tcgen05.mma instructions, with the operands in shared memory and the accumulators in
// tensor memory (TMEM).  One library per head size (-DKLLM_HD=64 or 128), bfloat16
// operands, float32 accumulation.
//
// A CTA takes 128 rows = (tokens of one request's portion) x (heads of one kv group) and
// walks that portion's keys in tiles of 64.  Its warps have four roles that meet only at
// mbarriers, so loading, the tensor core and the softmax of neighbouring tiles run at the
// same time (issuing one tcgen05.mma keeps a thread busy for a hundred cycles and more,
// so each of the two products has an issuing warp of its own):
//
//   warp 6   loader: K and V tiles by cp.async into a ring of stages, written directly in
//            the 128-byte-swizzled layout that the MMA's shared-memory descriptors name
//            (rows of 64 elements, 8-row groups of 1024 bytes, the 16-byte piece index
//            XORed with the row index modulo 8; head sizes above 64 as panels of 64
//            dims); the copies' completion arrives on the stage's mbarrier;
//   warp 4   one lane issues Q.K^T of a tile (M=128, N=64, K=16 per instruction) into one
//            of two score buffers in TMEM as soon as that buffer has been read out and
//            the tile has landed, that is up to two tiles ahead of the softmax;
//   warp 5   one lane issues P.V of a tile (V as the MN-major operand), accumulating into
//            the output in TMEM, once the tile's probabilities are in shared memory, and
//            hands the stage back to the loader;
//   warps 0-3  softmax: every thread owns one row, reads its 64 scores from TMEM
//            (tcgen05.ld 32x32b), applies the mask and the online-softmax recurrence
//            without any cross-thread traffic, and writes its probabilities as bfloat16
//            into a swizzled shared-memory tile.
// The softmax warps are one warp group, the others (with an idle warp) a second one that
// hands most of its registers to the first (setmaxnreg), so that two CTAs fit an SM.
//
// The output accumulates in TMEM over all tiles (P.V with accumulation); a row's
// probabilities are taken relative to a reference maximum that is only moved when the
// running maximum has grown by more than a factor 2^8 since (then the row of the
// accumulator is read, rescaled and written back, tcgen05.ld / tcgen05.st, between two
// P.V products).  Sum and output share the reference, so the quotient at the end is the
// softmax-weighted mean exactly as with a reference moved at every tile; what a row does
// depends on its own scores only.
//
// Every wait on an mbarrier is bounded by a cycle count: a wait that runs out raises a
// flag in shared memory and sets the status word, every role leaves its loop, and the
// CTA frees its TMEM and returns.  Math as in the reference (backend/model.cu:343-408):
// keys [max(0, p + 1 - window), p], scale after the dot product, one division by the sum
// at the end; probabilities are rounded to bfloat16 for the second product only.
#include "common.cuh"

#ifndef KLLM_HD
#error "compile with -DKLLM_HD=64 or 128"
#endif

KLLM_EXPORT_LAST_ERROR(attention_tcgen05)

#include "tc5_common.cuh"

namespace {

constexpr int HD = KLLM_HD;
static_assert(HD == 64 || HD == 128, "head size 64 or 128");
constexpr int PANELS = HD / 64;            // 64-dim panels of a row
constexpr int ROWS = 128;                  // query rows per CTA = TMEM lanes
constexpr int TILE = 64;                   // keys per tile
constexpr int THREADS = 256;                          // 4 softmax warps; the two MMA-issuing warps, the loader warp, an idle one
constexpr int SOFTMAX_THREADS = 128;
constexpr int Q_BYTES = PANELS * ROWS * 128;          // [panel][128 rows][64 dims]
constexpr int KV_BYTES = PANELS * TILE * 128;         // [panel][64 keys][64 dims]
constexpr int P_BYTES = ROWS * 128;                   // [128 rows][64 keys]
constexpr int STAGES = HD == 64 ? 4 : 2;
constexpr int SMEM_BYTES = 1024 + Q_BYTES + P_BYTES + STAGES * 2 * KV_BYTES;
constexpr float kRescaleAt = 8.f;                     // move a row's reference when its maximum grew by 2^8
constexpr int TMEM_COLS = 256;                        // two score buffers (2 x 64) + output tile (HD): a power of two

__device__ __forceinline__ void cp_async16(unsigned dst, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes));
}
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group %0;\n" ::"n"(N));
}
// shared-memory writes of this thread become visible to the tensor core's (async proxy) reads
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor
// version 1.  K-major operands: 8-row groups 1024 bytes apart (stride offset), leading
// offset 1.  MN-major operands: 8-k groups 1024 bytes apart (stride offset), 64-element
// panels `lbo_bytes` apart (leading offset).
__device__ __forceinline__ uint64_t make_desc(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;       // descriptor version for this architecture
    d |= (uint64_t)2 << 61;       // SWIZZLE_128B
    return d;
}

// Instruction descriptor: float32 accumulator, bfloat16 A and B, M x N, B optionally MN-major.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void tmem_st32(unsigned taddr, const float (&v)[32]) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
// byte offset of 16-byte piece `ch` (0..7) of row `r` inside a swizzled panel of 128-byte rows
__device__ __forceinline__ unsigned swz(int r, int ch) {
    return (unsigned)((r >> 3) * 1024 + (r & 7) * 128 + ((ch ^ (r & 7)) << 4));
}
// 2^x for x <= 0 (and -inf -> 0): the hardware approximation, one instruction
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// the barrier gets one arrival when all cp.async copies that this thread has issued so far have landed
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// keys key0 .. key0+63 of kv head g into a stage (K panels, then V panels), by the 32
// lanes of the loader warp.  A lane keeps its 16-byte piece of the row and walks the rows.
__device__ __forceinline__ void load_kv(unsigned stage, const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                                        const int* __restrict__ table, int key0, int hi, int g, int n_kv, int page_size,
                                        int lane) {
    constexpr int PIECES = HD / 8;                        // 16-byte pieces of a row
    constexpr int ROWS_PER_PASS = 32 / PIECES;            // 4 (HD 64) or 2 (HD 128)
    const int piece = lane % PIECES, r0 = lane / PIECES;
    const unsigned col = (unsigned)((piece >> 3) * (TILE * 128));
    const int64_t head_off = (int64_t)g * page_size * HD + piece * 8;
    const int64_t page_elems = (int64_t)n_kv * page_size * HD;
    const int lp0 = key0 / page_size, in_page = key0 - lp0 * page_size;
    if (in_page + TILE <= page_size) {
        // the whole tile lies in one page: one look-up, the rows follow one another
        const int64_t base = (int64_t)table[lp0] * page_elems + head_off + (int64_t)in_page * HD;
#pragma unroll 8
        for (int j = 0; j < TILE / ROWS_PER_PASS; j++) {
            const int row = r0 + j * ROWS_PER_PASS;
            const bool valid = key0 + row < hi;
            const int64_t off = valid ? base + row * HD : 0;
            const unsigned dst = col + swz(row, piece & 7);
            cp_async16(stage + dst, kcache + off, valid);
            cp_async16(stage + KV_BYTES + dst, vcache + off, valid);
        }
        return;
    }
#pragma unroll 4
    for (int j = 0; j < TILE / ROWS_PER_PASS; j++) {
        const int row = r0 + j * ROWS_PER_PASS;
        const int key = key0 + row;
        const bool valid = key < hi;
        int64_t off = 0;
        if (valid) {
            const int lp = key / page_size;
            off = (int64_t)table[lp] * page_elems + head_off + (int64_t)(key - lp * page_size) * HD;
        }
        const unsigned dst = col + swz(row, piece & 7);
        cp_async16(stage + dst, kcache + off, valid);
        cp_async16(stage + KV_BYTES + dst, vcache + off, valid);
    }
}

__global__ void __launch_bounds__(THREADS, HD == 64 ? 2 : 1)
attn_prefill_tc5_kernel(bf16* __restrict__ out, const bf16* __restrict__ q, int64_t q_stride,
                        const bf16* __restrict__ kcache, const bf16* __restrict__ vcache,
                        const int* __restrict__ q_start, const int* __restrict__ start_pos,
                        const int* __restrict__ block_table, int max_blocks, int n_requests, int n_heads,
                        int n_kv, int page_size, int window, float scale_log2e, int tokens_per_tile, int* status) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_kv_full[STAGES], bar_kv_empty[STAGES], bar_q_full, bar_s_full[2], bar_s_free[2],
        bar_p_full, bar_o_full;
    __shared__ unsigned s_tmem;
    __shared__ int s_req, s_tok0, s_abort;
    const int g = blockIdx.x % n_kv;          // CTAs start in the order of blockIdx.x: all kv heads' longest tiles first
    const int gs = n_heads / n_kv;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        int tile = (gridDim.x - 1 - blockIdx.x) / n_kv, req = -1, tok0 = 0;       // longest key ranges first
        for (int s = 0; s < n_requests; s++) {
            const int n = q_start[s + 1] - q_start[s];
            const int nt = (n + tokens_per_tile - 1) / tokens_per_tile;
            if (tile < nt) { req = s; tok0 = q_start[s] + tile * tokens_per_tile; break; }
            tile -= nt;
        }
        s_req = req; s_tok0 = tok0; s_abort = 0;
        for (int s = 0; s < STAGES; s++) { mbar_init(&bar_kv_full[s], 32); mbar_init(&bar_kv_empty[s], 1); }
        mbar_init(&bar_q_full, 32);
        for (int b = 0; b < 2; b++) { mbar_init(&bar_s_full[b], 1); mbar_init(&bar_s_free[b], SOFTMAX_THREADS); }
        mbar_init(&bar_p_full, SOFTMAX_THREADS);
        mbar_init(&bar_o_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    const int req = s_req;
    if (req < 0) return;                       // the grid is an upper bound on the tiles
    if (warp == 4) {                           // TMEM: one warp allocates, everybody learns the address
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    griddep_wait();
    griddep_launch();
    const unsigned tmem = s_tmem;
    const int tok0 = s_tok0;
    const int n_tok = min(tokens_per_tile, q_start[req + 1] - tok0);
    const int pos0 = start_pos[req] + (tok0 - q_start[req]);
    const int lo = (window > 0 && pos0 + 1 > window) ? pos0 + 1 - window : 0;
    const int hi = pos0 + n_tok;
    const int* table = block_table + (int64_t)req * max_blocks;
    const int ntiles = (hi - lo + TILE - 1) / TILE;      // at least 1: a row sees its own key
    volatile int* abort_flag = &s_abort;

    // The softmax warps keep 64 scores and more in registers; the other warp group needs
    // almost none and hands its share over (the kernel is compiled for two CTAs of 256
    // threads per SM, 128 registers each).

    const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;       // swizzled tiles want 1024-byte alignment
    const unsigned sQ = base, sP = base + Q_BYTES, sKV = sP + P_BYTES;

    if (warp >= 4) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 64;\n" ::);
      if (warp == 6) {
        // ---- loader ----------------------------------------------------------------
        for (int c = lane; c < ROWS * (HD / 8); c += 32) {     // Q tile: each row's HD dims, zero for unused rows
            const int r = c / (HD / 8), piece = c - r * (HD / 8);
            const int t2 = r / gs, h2 = r - t2 * gs;
            const bool ok = t2 < n_tok;
            const bf16* src = ok ? q + (int64_t)(tok0 + t2) * q_stride + (int64_t)(g * gs + h2) * HD + piece * 8 : q;
            cp_async16(sQ + (unsigned)((piece >> 3) * (ROWS * 128)) + swz(r, piece & 7), src, ok);
        }
        cp_async_arrive(&bar_q_full);
        for (int j = 0; j < ntiles; j++) {
            const int s = j % STAGES;
            if (!mbar_wait(&bar_kv_empty[s], (((unsigned)(j / STAGES)) & 1u) ^ 1u, abort_flag, status, 1)) break;
            load_kv(sKV + (unsigned)s * 2u * KV_BYTES, kcache, vcache, table, lo + j * TILE, hi, g, n_kv, page_size, lane);
            cp_async_arrive(&bar_kv_full[s]);
        }
        cp_async_wait<0>();                    // nothing of this warp is in flight when the CTA ends
      } else if (warp == 4) {
        // ---- issuer of the scores ---------------------------------------------------
        constexpr uint32_t IDESC_S = make_idesc(ROWS, TILE, false);
        bool ok = mbar_wait(&bar_q_full, 0, abort_flag, status, 2);
        for (int j = 0; ok && j < ntiles; j++) {            // scores of tile j into buffer j & 1, up to two tiles ahead
            const int s = j % STAGES, b = j & 1;
            ok = mbar_wait(&bar_kv_full[s], ((unsigned)(j / STAGES)) & 1u, abort_flag, status, 3) &&
                 mbar_wait(&bar_s_free[b], (((unsigned)(j >> 1)) & 1u) ^ 1u, abort_flag, status, 4);
            if (!ok) break;
            fence_async_smem();                // the copies landed through the generic proxy
            tc_fence_after();
            if (lane == 0) {
                const unsigned st = sKV + (unsigned)s * 2u * KV_BYTES;
#pragma unroll
                for (int kk = 0; kk < HD / 16; kk++) {
                    const unsigned a = sQ + (unsigned)((kk >> 2) * (ROWS * 128) + (kk & 3) * 32);
                    const unsigned bb = st + (unsigned)((kk >> 2) * (TILE * 128) + (kk & 3) * 32);
                    umma(tmem + (unsigned)(b * 64), make_desc(a, 16, 1024), make_desc(bb, 16, 1024), IDESC_S, kk > 0);
                }
                umma_commit(&bar_s_full[b]);
            }
            __syncwarp();
        }
      } else if (warp == 5) {
        // ---- issuer of the output products --------------------------------------------
        constexpr uint32_t IDESC_O = make_idesc(ROWS, HD, true);
        bool ok = true;
        for (int j = 0; ok && j < ntiles; j++) {
            const int s = j % STAGES;
            // the stage's arrival was seen by the other issuer; this warp has to see it too
            ok = mbar_wait(&bar_kv_full[s], ((unsigned)(j / STAGES)) & 1u, abort_flag, status, 5) &&
                 mbar_wait(&bar_p_full, (unsigned)j & 1u, abort_flag, status, 5);
            if (!ok) break;
            fence_async_smem();
            tc_fence_after();
            if (lane == 0) {                   // output += P . V
                const unsigned st = sKV + (unsigned)s * 2u * KV_BYTES;
#pragma unroll
                for (int kk = 0; kk < TILE / 16; kk++) {
                    const unsigned a = sP + (unsigned)(kk * 32);
                    const unsigned bb = st + KV_BYTES + (unsigned)(kk * 2048);
                    umma(tmem + 128, make_desc(a, 16, 1024), make_desc(bb, TILE * 128, 1024), IDESC_O, j > 0 || kk > 0);
                }
                umma_commit(&bar_o_full);
                umma_commit(&bar_kv_empty[s]);
            }
            __syncwarp();
        }
      }                                        // warp 7 only fills the warp group
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 184;\n" ::);
        // ---- softmax: this thread's row is (token, head of the group) ---------------
        const int row = threadIdx.x;
        const int tt = row / gs, hh = row - tt * gs;
        const bool valid_row = tt < n_tok;
        const int p_row = valid_row ? pos0 + tt : -1;                       // -1: sees no key
        const int w_row = (window > 0) ? p_row + 1 - window : 0;
        const unsigned lane_base = (unsigned)(warp * 32) << 16;
        const unsigned t_o = tmem + lane_base + 128;
        float m_ref = -INFINITY, l_run = 0.f;          // the row's reference maximum; its sum relative to it
        bool ok = true;
        for (int j = 0; j < ntiles; j++) {
            const int b = j & 1;
            ok = mbar_wait(&bar_s_full[b], ((unsigned)(j >> 1)) & 1u, abort_flag, status, 6);
            if (!ok) break;
            tc_fence_after();
            float s[TILE];
            {
                float (*s2)[32] = reinterpret_cast<float (*)[32]>(s);
                const unsigned t_s = tmem + lane_base + (unsigned)(b * 64);
                tmem_ld32(t_s, s2[0]);
                tmem_ld32(t_s + 32, s2[1]);
                tmem_ld_wait();
            }
            tc_fence_before();
            mbar_arrive(&bar_s_free[b]);       // the buffer may take the scores of tile j + 2
            const int key0 = lo + j * TILE;
            // the mask matters only where the tile crosses this row's diagonal or window edge
            if (key0 + TILE - 1 > p_row || key0 < w_row) {
#pragma unroll
                for (int jj = 0; jj < TILE; jj++) {
                    const int key = key0 + jj;
                    if (key > p_row || key < w_row) s[jj] = -INFINITY;
                }
            }
            float mx4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
            for (int jj = 4; jj < TILE; jj++) mx4[jj & 3] = fmaxf(mx4[jj & 3], s[jj]);
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // move the reference only for a first key or a maximum that outgrew it by 2^8
            const bool move = mx > m_ref && (mx - m_ref) * scale_log2e > kRescaleAt;
            float corr = 1.f;
            if (move) {
                corr = (m_ref == -INFINITY) ? 0.f : exp2f((m_ref - mx) * scale_log2e);
                m_ref = mx;
            }
            const float neg = (m_ref == -INFINITY) ? 0.f : -m_ref * scale_log2e;   // p = 2^(s * scale - m * scale): one FMA each
            float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int jj = 0; jj < TILE; jj++) {
                s[jj] = fast_exp2(fmaf(s[jj], scale_log2e, neg));
                sum4[jj & 3] += s[jj];
            }
            l_run = l_run * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
            if (j > 0) {
                // the product of tile j - 1 read the P tile that is written below, and must be
                // over before the accumulator is rescaled; it has had this long to finish
                ok = mbar_wait(&bar_o_full, (unsigned)(j - 1) & 1u, abort_flag, status, 7);
                if (!ok) break;
            }
            if (j > 0 && __any_sync(0xffffffffu, move)) {
                // rows of this warp rescale what the products so far have added up (rows that
                // did not move multiply by one); the product of tile j - 1 is over (see above),
                // the one of tile j waits for this thread's probabilities
                tc_fence_after();
#pragma unroll
                for (int cb = 0; cb < HD / 32; cb++) {
                    float t[32];
                    tmem_ld32(t_o + cb * 32, t);
                    tmem_ld_wait();
#pragma unroll
                    for (int jj = 0; jj < 32; jj++) t[jj] *= corr;
                    tmem_st32(t_o + cb * 32, t);
                }
                tmem_st_wait();
            }
            const unsigned sPb = sP;
#pragma unroll
            for (int c = 0; c < 8; c++) {      // 8 keys = 16 bytes per piece, swizzled like an operand row
                uint4 pk;
                pk.x = pack_bf16(s[8 * c], s[8 * c + 1]);
                pk.y = pack_bf16(s[8 * c + 2], s[8 * c + 3]);
                pk.z = pack_bf16(s[8 * c + 4], s[8 * c + 5]);
                pk.w = pack_bf16(s[8 * c + 6], s[8 * c + 7]);
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(sPb + swz(row, c)), "r"(pk.x), "r"(pk.y), "r"(pk.z), "r"(pk.w) : "memory");
            }
            fence_async_smem();
            tc_fence_before();
            mbar_arrive(&bar_p_full);          // P of tile j is in shared memory, the accumulator is rescaled
        }
        if (ok) ok = mbar_wait(&bar_o_full, (unsigned)(ntiles - 1) & 1u, abort_flag, status, 9);
        if (ok) {
            tc_fence_after();
            const float inv = 1.f / l_run;
            bf16* orow = out + (int64_t)(tok0 + tt) * n_heads * HD + (int64_t)(g * gs + hh) * HD;
#pragma unroll
            for (int cb = 0; cb < HD / 32; cb++) {
                float t[32];
                tmem_ld32(t_o + cb * 32, t);
                tmem_ld_wait();
                if (valid_row) {
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        uint4 pk;
                        pk.x = pack_bf16(t[8 * c] * inv, t[8 * c + 1] * inv);
                        pk.y = pack_bf16(t[8 * c + 2] * inv, t[8 * c + 3] * inv);
                        pk.z = pack_bf16(t[8 * c + 4] * inv, t[8 * c + 5] * inv);
                        pk.w = pack_bf16(t[8 * c + 6] * inv, t[8 * c + 7] * inv);
                        *reinterpret_cast<uint4*>(orow + cb * 32 + 8 * c) = pk;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 4)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS));
}

bool g_attr_set = false;

}  // namespace

extern "C" int kllm_attention_tcgen05_head_dim() { return HD; }

// Same contract as the mma.sync prefill kernel: requests' portions
// q_start[s]..q_start[s+1] start at cache position start_pos[s]; out [n, n_heads*HD].
// status: device int that a bounded wait which ran out sets (1: loader, 2-5: tensor-core
// issuer, 6-9: softmax).
extern "C" int kllm_attention_prefill_tcgen05(void* out, const void* q, int64_t q_stride, const void* kcache,
                                              const void* vcache, const int* q_start, const int* start_pos,
                                              const int* block_table, int max_blocks, int n_tokens,
                                              int n_requests, int n_heads, int n_kv, int hd, int page_size,
                                              int window, float scale, int* status, void* stream) {
    if (n_tokens <= 0) return 0;
    if (hd != HD) KLLM_FAIL("attention (tcgen05): this library was built for head size %d, not %d", HD, hd);
    if (n_kv <= 0 || n_heads % n_kv) KLLM_FAIL("attention: %d heads over %d kv heads", n_heads, n_kv);
    const int gs = n_heads / n_kv;
    if (gs > ROWS) KLLM_FAIL("attention (tcgen05): %d heads per kv head, at most %d", gs, ROWS);
    if (page_size <= 0) KLLM_FAIL("attention: page size %d", page_size);
    if (((uintptr_t)q & 15) || (q_stride & 7) || ((uintptr_t)out & 15) || ((uintptr_t)kcache & 15) || ((uintptr_t)vcache & 15))
        KLLM_FAIL("attention (tcgen05): q, out and the caches must be 16-byte aligned, q's row stride a multiple of 8");
    if (!g_attr_set) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) {
            snprintf(g_kllm_err, sizeof(g_kllm_err), "attention (tcgen05): %d bytes of shared memory refused: %s",
                     SMEM_BYTES, cudaGetErrorString(e));
            return (int)e;
        }
        g_attr_set = true;
    }
    const int tpt = ROWS / gs;
    const int max_tiles = n_tokens / tpt + n_requests;
    const float sl2e = scale * 1.4426950408889634f;
    kllm_launch((attn_prefill_tc5_kernel), dim3(max_tiles * n_kv), dim3(THREADS), SMEM_BYTES, (cudaStream_t)stream,
                (bf16*)out, (const bf16*)q, q_stride, (const bf16*)kcache, (const bf16*)vcache, q_start, start_pos,
                block_table, max_blocks, n_requests, n_heads, n_kv, page_size, window, sl2e, tpt, status);
    KLLM_LAUNCH_STATUS();
}
