// Y[n, N] = X[n, K] . W[N, K]^T for a handful of rows n (decode steps): the
// weights are streamed from HBM exactly once, straight into registers, and meet the
// activations on the tensor cores (mma.sync m16n8k16, bfloat16 operands, float32
// accumulation) with the WEIGHTS as the 16-row operand and the tokens as the
// 8-column one.  The reference runs these products through cublasSgemm
// (backend/model.cu:496-503, :1090-1115); at a few rows they are pure weight
// streaming and the work around them (norm before, activation or residual sum
// after) costs more launches than the product itself, so it is folded in:
//
//   prologue  X_BF16      X is a bfloat16 matrix [n, K]
//             X_F32_NORM  X = rmsnorm(x) * gain of float32 rows x (optionally
//                         gathered by `rows`), computed by every CTA for itself in
//                         float32 and kept in shared memory as bfloat16
//                         (formula: backend/model.cu:101-122)
//   epilogue  STORE_BF16  Y as bfloat16
//             STORE_F32   Y as float32 (logits)
//             ADD_F32     Y is added into a float32 matrix (the residual stream)
//             SWIGLU      W holds a gate and an up matrix [F, K] each; the output is
//                         silu(gate row) * (up row) as bfloat16 [n, F]
//                         (backend/model.cu:477-483, :1112-1114)
//
// Layout of the work: a tile is 16 weight rows (for SWIGLU 8 gate rows and the 8 up
// rows that go with them).  A CTA of 16 warps, one per SM, walks tiles tile = blockIdx.x,
// += gridDim.x; inside a tile the warps take the K dimension in interleaved steps
// of 32 elements, each lane loading 16 contiguous bytes of two weight rows per
// step.  A lane's 8 consecutive k-values feed two MMAs; the same permutation of k
// is applied to the activations, so the sum is unchanged.  The sixteen partial
// tiles are added in warp order through shared memory: no atomics, and every output
// element belongs to one CTA, so ADD_F32 is race-free and the order of all sums
// depends on K alone.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(skinny_gemm)

namespace {

constexpr int THREADS = 512;       // one CTA per SM: X is prepared once per SM, all 16 warps stream weights
constexpr int WARPS = 16;
constexpr int UNROLL = 4;          // k-steps of 32 in flight per lane and buffer
constexpr int NORM_F4 = 16;        // float4 a lane may hold in the one-pass norm prologue
constexpr int EARLY_START_TILES = 3;   // most tiles per CTA of a kernel that starts early

enum { X_BF16 = 0, X_F32_NORM = 1 };
enum { STORE_BF16 = 0, STORE_F32 = 1, ADD_F32 = 2, SWIGLU = 3 };

struct Args {
    const bf16* w;        // [N, K] at w_stride; SWIGLU: the gate matrix [F, K]
    const bf16* w_up;     // SWIGLU: the up matrix [F, K] at w_stride
    int w_stride;         // elements between weight rows (K, or more for a slice of columns)
    int N;                // output columns (SWIGLU: F)
    int K;
    int n;                // rows of X (tokens)
    const bf16* x_bf16;   // X_BF16: [n, K] at x_stride
    int64_t x_stride;
    const float* x_f32;   // X_F32_NORM: rows of width K
    const float* gain;    // [K]
    const int* rows;      // optional gather of x_f32 rows
    float eps;
    bf16* y_bf16;         // STORE_BF16, SWIGLU
    float* y_f32;         // STORE_F32, ADD_F32
    int64_t y_stride;
    int tl_slot;            // timeline row of this launch (-1: none)
    const void* prefetch;   // optional: weights of a later kernel, to be brought into L2
    int64_t prefetch_bytes;
};

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// the same load at a compile-time offset from p: the address needs no arithmetic of its own
template <int BYTES>
__device__ __forceinline__ uint4 ldg_stream_at(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4+%5];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "n"(BYTES));
    return v;
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;                     // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
// wait until at most `pending` of this thread's latest copy groups are still in flight
__device__ __forceinline__ void cp_async_wait_pending(int pending) {
    if (pending >= 3) asm volatile("cp.async.wait_group 3;\n" ::: "memory");
    else if (pending == 2) asm volatile("cp.async.wait_group 2;\n" ::: "memory");
    else if (pending == 1) asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    else asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}

__host__ __device__ inline int x_row_elems(int K) {      // row stride of X in shared memory, elements
    return K + (((K * 2) % 128 == 0) ? 32 : 0);           // bytes = 64 (mod 128): 16-byte reads of 8 rows x 4
}                                                         // quarter-row offsets hit 8 different bank groups

// EXACT: K is a multiple of 2048, so every warp has whole batches of k-steps only.
template <int NT, int PRO, int EPI, bool EXACT>
__global__ void __launch_bounds__(THREADS)
skinny_gemm_kernel(const Args a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    TL_BEGIN();
    const int K = a.K, N = a.N, n = a.n, WS = a.w_stride;
    const int XS = x_row_elems(K);
    bf16* xs = reinterpret_cast<bf16*>(smem_raw);                         // [8*NT][XS]
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)8 * NT * XS * 2);   // [WARPS][16][8*NT]
    float* gain_s = red + WARPS * 16 * 8 * NT;                                   // [K], norm prologue only
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    constexpr int ROWS_PER_TILE = (EPI == SWIGLU) ? 8 : 16;
    const int n_tiles = (N + ROWS_PER_TILE - 1) / ROWS_PER_TILE;
    const int steps = K / 32;
    const int my_steps = (steps > warp) ? (steps - warp + WARPS - 1) / WARPS : 0;
    const int nb = max(1, ((steps + WARPS - 1) / WARPS + UNROLL - 1) / UNROLL);   // batches per tile, same for all warps

    // this lane's two weight rows of a tile (rows past the end repeat the last one)
    auto row_ptrs = [&](int tile, const bf16*& pa, const bf16*& pb) {
        if (EPI == SWIGLU) {
            const int r = min(tile * 8 + g, N - 1);
            pa = a.w + (int64_t)r * WS + 8 * t;
            pb = a.w_up + (int64_t)r * WS + 8 * t;
        } else {
            pa = a.w + (int64_t)min(tile * 16 + g, N - 1) * WS + 8 * t;
            pb = a.w + (int64_t)min(tile * 16 + g + 8, N - 1) * WS + 8 * t;
        }
    };
    // Two register buffers of UNROLL k-steps each take turns: while one is being
    // multiplied the other is in flight.  No buffer is ever copied, so nothing waits
    // for a load before its data is needed.
    uint4 buf0a[UNROLL], buf0b[UNROLL], buf1a[UNROLL], buf1b[UNROLL];
    // With two token tiles per weight tile the kernel is bound by its instruction count, not
    // by memory: there a batch whose k-steps all exist is loaded and multiplied without a test
    // per step, its addresses fixed offsets from one pointer (EXACT: K is a multiple of 2048
    // and no batch needs the tests at all); 1.3 to 1.9 times faster than the loop with a test
    // per step.  With one token tile the loads keep their tests: without them a decode step
    // of batch 8 was measured slower (0.822 ms against 0.802, alternating runs of the two
    // builds), while its MMAs without the tests, where K is a multiple of 2048, make it a
    // little faster (0.797).
    constexpr bool WHOLE_BATCHES = NT == 2;              // loads without a test per step
    constexpr bool WHOLE_MMA = NT == 2 || EXACT;         // MMAs without a test per step
    auto load_batch = [&](uint4 (&ra)[UNROLL], uint4 (&rb)[UNROLL], int tile, int b) {
        const bf16 *pa, *pb;
        row_ptrs(tile, pa, pb);
        const int s0 = b * UNROLL;
        pa += (warp + s0 * WARPS) * 32;
        pb += (warp + s0 * WARPS) * 32;
        if (WHOLE_BATCHES && (EXACT || s0 + UNROLL <= my_steps)) {
            static_assert(UNROLL == 4, "the offsets below are written out for four k-steps");
            constexpr int STEP = WARPS * 32 * 2;        // bytes from a warp's k-step to its next
            ra[0] = ldg_stream_at<0>(pa); rb[0] = ldg_stream_at<0>(pb);
            ra[1] = ldg_stream_at<STEP>(pa); rb[1] = ldg_stream_at<STEP>(pb);
            ra[2] = ldg_stream_at<2 * STEP>(pa); rb[2] = ldg_stream_at<2 * STEP>(pb);
            ra[3] = ldg_stream_at<3 * STEP>(pa); rb[3] = ldg_stream_at<3 * STEP>(pb);
        } else {
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                if (s0 + u < my_steps) {
                    ra[u] = ldg_stream(pa + u * WARPS * 32);
                    rb[u] = ldg_stream(pb + u * WARPS * 32);
                }
            }
        }
    };

    int cur_tile = blockIdx.x, cur_b = 0;     // the batch that sits in the buffer used next
    if (cur_tile < n_tiles) load_batch(buf0a, buf0b, cur_tile, 0);   // weights do not depend on X: start them first
    if (PRO == X_F32_NORM)                                 // the gain is a weight too: on its way before X exists
        for (int c = threadIdx.x; c < K / 4; c += THREADS) cp_async16(gain_s + 4 * c, a.gain + 4 * c, true);
    l2_prefetch_slice(a.prefetch, a.prefetch_bytes, THREADS);
    griddep_wait();        // X (and, for ADD_F32, the matrix added into) come from the kernels before
    griddep_launch();
    TL_MARK(1);

    // ---- prologue: X into shared memory as bfloat16, rows past n are zero ----
    int x_groups = 0;            // X_BF16: copy groups of X, one per batch of k-steps (the last takes the rest)
    if (PRO == X_BF16) {
        // All copies in flight at once, in groups by the k range that a batch of the main
        // loop needs: the first tile's batch b waits for groups 0..b only, so a long X is
        // still arriving while its first part is already being multiplied.
        constexpr int KB = UNROLL * WARPS * 32;
        x_groups = min(nb, 4);
        for (int gi = 0; gi < x_groups; gi++) {
            const int k_lo = gi * KB, k_hi = (gi == x_groups - 1) ? K : min(K, (gi + 1) * KB);
            const int pieces = (k_hi - k_lo) / 8;
            for (int c = threadIdx.x; c < 8 * NT * pieces; c += THREADS) {
                const int r = c / pieces, ch = c - r * pieces;
                cp_async16(xs + r * XS + k_lo + ch * 8, a.x_bf16 + (int64_t)(r < n ? r : 0) * a.x_stride + k_lo + ch * 8, r < n);
            }
            cp_async_commit();
        }
    } else {
        // WARPS / (8*NT) warps share a row: each takes a contiguous part of it, the
        // parts' sums of squares are added in part order
        constexpr int PARTS = WARPS / (8 * NT);
        const int r = warp / PARTS, part = warp - r * PARTS;
        const int span = K / PARTS;                      // K % 32 == 0 and PARTS <= 2: a multiple of 16
        const int lo_k = part * span;
        bf16* dst = xs + r * XS;
        float* ss_part = red;                            // [8*NT][PARTS], free until the first tile ends
        const bool live = r < n;
        const float* src = live ? a.x_f32 + (int64_t)(a.rows ? a.rows[r] : r) * K : nullptr;
        const bool one_pass = span <= NORM_F4 * 128;
        float4 v[NORM_F4];
        float ss = 0.f;
        if (live) {
            if (one_pass) {
#pragma unroll
                for (int i = 0; i < NORM_F4; i++) {
                    const int k = lo_k + (i * 32 + lane) * 4;
                    v[i] = (k < lo_k + span) ? *reinterpret_cast<const float4*>(src + k) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
                for (int i = 0; i < NORM_F4; i++) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
            } else {
                for (int k = lo_k + lane * 4; k < lo_k + span; k += 128) {
                    const float4 w4 = *reinterpret_cast<const float4*>(src + k);
                    ss += w4.x * w4.x + w4.y * w4.y + w4.z * w4.z + w4.w * w4.w;
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) ss_part[r * PARTS + part] = ss;
        }
        cp_async_wait_all();       // the gain
        __syncthreads();
        if (live) {
            float tot = 0.f;
#pragma unroll
            for (int q = 0; q < PARTS; q++) tot += ss_part[r * PARTS + q];
            const float scale = rsqrtf(tot / (float)K + a.eps);
            auto put = [&](int k, const float4& w4) {
                const float4 gn = *reinterpret_cast<const float4*>(gain_s + k);
                __nv_bfloat162 lo2 = __floats2bfloat162_rn(w4.x * scale * gn.x, w4.y * scale * gn.y);
                __nv_bfloat162 hi2 = __floats2bfloat162_rn(w4.z * scale * gn.z, w4.w * scale * gn.w);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo2);
                pk.y = *reinterpret_cast<uint32_t*>(&hi2);
                *reinterpret_cast<uint2*>(dst + k) = pk;
            };
            if (one_pass) {
#pragma unroll
                for (int i = 0; i < NORM_F4; i++) {
                    const int k = lo_k + (i * 32 + lane) * 4;
                    if (k < lo_k + span) put(k, v[i]);
                }
            } else {
                for (int k = lo_k + lane * 4; k < lo_k + span; k += 128) put(k, *reinterpret_cast<const float4*>(src + k));
            }
        } else {
            for (int k = lo_k + lane * 8; k < lo_k + span; k += 256) *reinterpret_cast<uint4*>(dst + k) = make_uint4(0, 0, 0, 0);
        }
    }
    if (PRO != X_BF16) __syncthreads();
    TL_MARK(2);

    // ---- tiles ----
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

    // multiply the batch (cur_tile, cur_b) held in x while the following batch loads into y
    auto phase = [&](uint4 (&xa)[UNROLL], uint4 (&xb)[UNROLL], uint4 (&ya)[UNROLL], uint4 (&yb)[UNROLL]) {
        int nxt_tile = cur_tile, nxt_b = cur_b + 1;
        if (nxt_b == nb) { nxt_b = 0; nxt_tile += gridDim.x; }
        if (nxt_tile < n_tiles) load_batch(ya, yb, nxt_tile, nxt_b);
        if (PRO == X_BF16 && x_groups > 0) {                 // the first tile: the part of X that this batch reads
            const int have = min(cur_b, x_groups - 1) + 1;
            cp_async_wait_pending(x_groups - have);
            __syncthreads();
            if (have == x_groups) x_groups = 0;
        }
        {
            const int s0 = cur_b * UNROLL;
            const bf16* xk = xs + g * XS + (warp + s0 * WARPS) * 32 + 8 * t;       // this lane's X row 0 at the batch's first k-step
            if (WHOLE_MMA && (EXACT || s0 + UNROLL <= my_steps)) {
#pragma unroll
                for (int u = 0; u < UNROLL; u++) {
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        const uint4 xv = *reinterpret_cast<const uint4*>(xk + nt * 8 * XS + u * WARPS * 32);
                        mma_bf16(acc[nt], xa[u].x, xb[u].x, xa[u].y, xb[u].y, xv.x, xv.y);
                        mma_bf16(acc[nt], xa[u].z, xb[u].z, xa[u].w, xb[u].w, xv.z, xv.w);
                    }
                }
            } else {
#pragma unroll
                for (int u = 0; u < UNROLL; u++) {
                    if (s0 + u < my_steps) {
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) {
                            const uint4 xv = *reinterpret_cast<const uint4*>(xk + nt * 8 * XS + u * WARPS * 32);
                            mma_bf16(acc[nt], xa[u].x, xb[u].x, xa[u].y, xb[u].y, xv.x, xv.y);
                            mma_bf16(acc[nt], xa[u].z, xb[u].z, xa[u].w, xb[u].w, xv.z, xv.w);
                        }
                    }
                }
            }
        }
        if (cur_b == nb - 1) {
            // the warps' partial tiles, added in warp order
            const int tile = cur_tile;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                float* r0 = red + ((warp * 16 + g) * 8 * NT) + nt * 8 + 2 * t;
                float* r1 = red + ((warp * 16 + g + 8) * 8 * NT) + nt * 8 + 2 * t;
                r0[0] = acc[nt][0]; r0[1] = acc[nt][1]; r1[0] = acc[nt][2]; r1[1] = acc[nt][3];
                acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
            }
            __syncthreads();
            constexpr int OUT_ROWS = (EPI == SWIGLU) ? 8 : 16;
            for (int e = threadIdx.x; e < OUT_ROWS * 8 * NT; e += THREADS) {
                const int r = e / (8 * NT), c = e - r * (8 * NT);      // weight row in the tile, token
                const int col = tile * OUT_ROWS + r;
                if (c >= n || col >= N) continue;
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < WARPS; w++) v += red[(w * 16 + r) * 8 * NT + c];
                if (EPI == SWIGLU) {
                    float u = 0.f;
#pragma unroll
                    for (int w = 0; w < WARPS; w++) u += red[(w * 16 + r + 8) * 8 * NT + c];
                    a.y_bf16[(int64_t)c * a.y_stride + col] = __float2bfloat16_rn((v / (1.f + expf(-v))) * u);
                } else if (EPI == STORE_BF16) {
                    a.y_bf16[(int64_t)c * a.y_stride + col] = __float2bfloat16_rn(v);
                } else if (EPI == STORE_F32) {
                    a.y_f32[(int64_t)c * a.y_stride + col] = v;
                } else {
                    a.y_f32[(int64_t)c * a.y_stride + col] += v;
                }
            }
            __syncthreads();
        }
        cur_tile = nxt_tile;
        cur_b = nxt_b;
    };
    while (cur_tile < n_tiles) {
        phase(buf0a, buf0b, buf1a, buf1b);
        if (cur_tile >= n_tiles) break;
        phase(buf1a, buf1b, buf0a, buf0b);
    }
    if (PRO == X_BF16) cp_async_wait_pending(0);            // a CTA without a tile: nothing in flight at its end
    TL_MARK(3);
    TL_END(a.tl_slot, 100 + PRO * 10 + EPI);        // marks: start, dependency wait over, X ready, tiles done
}

size_t smem_bytes(int nt, int K) {        // X, the warps' partial tiles, the norm's gain
    return (size_t)8 * nt * x_row_elems(K) * 2 + (size_t)WARPS * 16 * 8 * nt * 4 + (size_t)K * 4;
}

template <int NT, int PRO, int EPI, bool EXACT>
int launch_exact(const Args& a, cudaStream_t s) {
    static int max_grid = 0;            // per instantiation: CTAs that fit the GPU at this kernel's register use
    static size_t attr_smem = 0;
    const size_t smem = smem_bytes(NT, a.K);
    auto kern = skinny_gemm_kernel<NT, PRO, EPI, EXACT>;
    if (smem > attr_smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            snprintf(g_kllm_err, sizeof(g_kllm_err), "skinny_gemm: %zu bytes of shared memory refused: %s", smem,
                     cudaGetErrorString(e));
            return (int)e;
        }
        attr_smem = smem;
    }
    int per_sm = 0, dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THREADS, smem);
    max_grid = max(1, per_sm) * max(1, sms);
    const int rows_per_tile = (EPI == SWIGLU) ? 8 : 16;
    const int n_tiles = (a.N + rows_per_tile - 1) / rows_per_tile;
    const int grid = min(n_tiles, max_grid);
    // A kernel of a few tiles per CTA starts early, beside the tail of the kernel before it,
    // so that its first weights and the next kernel's share of L2 are on their way while it
    // waits.  One with many tiles gains nothing from that and was measured to stream
    // slower when it got an early start (at 12 tiles per CTA and K = 4096 at half speed:
    // 235 MB in 72 us instead of 45), so it starts when the kernel before it has ended.
    const bool early = n_tiles <= EARLY_START_TILES * grid;
    kllm_launch_dep(early, (kern), dim3(grid), dim3(THREADS), smem, s, a);
    KLLM_LAUNCH_STATUS();
}

template <int NT, int PRO, int EPI>
int launch(const Args& a, cudaStream_t s) {
    return a.K % (WARPS * UNROLL * 32) == 0 ? launch_exact<NT, PRO, EPI, true>(a, s) : launch_exact<NT, PRO, EPI, false>(a, s);
}

template <int NT, int PRO>
int launch_epi(const Args& a, int epi, cudaStream_t s) {
    switch (epi) {
        case STORE_BF16: return launch<NT, PRO, STORE_BF16>(a, s);
        case STORE_F32: return launch<NT, PRO, STORE_F32>(a, s);
        case ADD_F32: return launch<NT, PRO, ADD_F32>(a, s);
        case SWIGLU: return launch<NT, PRO, SWIGLU>(a, s);
    }
    KLLM_FAIL("skinny_gemm: unknown epilogue %d", epi);
}

}  // namespace

// Largest number of rows of X this kernel takes.
extern "C" int kllm_skinny_gemm_max_rows() { return 16; }

// 1 if (n, K) can run here (shared memory holds X), else 0.
extern "C" int kllm_skinny_gemm_fits(int n, int K) {
    if (n < 1 || n > 16 || K < 32 || K % 32) return 0;
    return smem_bytes(n <= 8 ? 1 : 2, K) <= 227 * 1024 ? 1 : 0;
}

// prologue 0: x_bf16 [n, K] at x_stride.  prologue 1: x_f32 rows of width K (row r is
// rows[r] when rows is given), normalised with gain [K] and eps.
// epilogue 0/3: y_bf16 [n, N] at y_stride (3: w = gate [N, K], w_up = up [N, K]);
// epilogue 1: y_f32 written; epilogue 2: y_f32 += result.
// w_stride: elements from one weight row to the next (>= K; more than K when the call
// multiplies a slice of the columns of a wider matrix, which is how a K too long for
// shared memory is taken: one call per slice, each adding into y_f32).
// prefetch: optional, `prefetch_bytes` bytes that a later kernel will stream; they are
// requested into L2 before this kernel's own work.
extern "C" int kllm_skinny_gemm(const void* w, const void* w_up, int64_t w_stride, int N, int K, int n, const void* x_bf16,
                                int64_t x_stride, const float* x_f32, const float* gain, const int* rows,
                                float eps, void* y_bf16, float* y_f32, int64_t y_stride, int prologue,
                                int epilogue, const void* prefetch, int64_t prefetch_bytes, void* stream) {
    if (n <= 0 || N <= 0) return 0;
    if (!kllm_skinny_gemm_fits(n, K))
        KLLM_FAIL("skinny_gemm: %d rows of width %d not supported (1..16 rows, width a multiple of 32 that fits "
                  "shared memory)", n, K);
    if (prologue == X_BF16 && (!x_bf16 || (x_stride % 8) || ((uintptr_t)x_bf16 & 15)))
        KLLM_FAIL("skinny_gemm: bfloat16 X must be 16-byte aligned with a row stride that is a multiple of 8");
    if (prologue == X_F32_NORM && (!x_f32 || !gain || ((uintptr_t)x_f32 & 15) || ((uintptr_t)gain & 15)))
        KLLM_FAIL("skinny_gemm: float32 X and gain must be 16-byte aligned");
    if (((uintptr_t)w & 15) || w_stride < K || (w_stride % 8) || w_stride > INT32_MAX)
        KLLM_FAIL("skinny_gemm: weights must be 16-byte aligned, their row stride a multiple of 8 and at least K");
    if (epilogue == SWIGLU && (!w_up || ((uintptr_t)w_up & 15))) KLLM_FAIL("skinny_gemm: SWIGLU needs the up matrix");
    if ((epilogue == STORE_BF16 || epilogue == SWIGLU) ? !y_bf16 : !y_f32) KLLM_FAIL("skinny_gemm: no output buffer");
    Args a;
    a.w = (const bf16*)w; a.w_up = (const bf16*)w_up; a.w_stride = (int)w_stride; a.N = N; a.K = K; a.n = n;
    a.x_bf16 = (const bf16*)x_bf16; a.x_stride = x_stride; a.x_f32 = x_f32; a.gain = gain; a.rows = rows; a.eps = eps;
    a.y_bf16 = (bf16*)y_bf16; a.y_f32 = y_f32; a.y_stride = y_stride;
    if (prefetch && ((uintptr_t)prefetch & 15)) KLLM_FAIL("skinny_gemm: the matrix to prefetch must be 16-byte aligned");
    a.prefetch = prefetch; a.prefetch_bytes = prefetch ? prefetch_bytes : 0;
    a.tl_slot = TL_SLOT();
    cudaStream_t s = (cudaStream_t)stream;
    if (n <= 8) {
        if (prologue == X_BF16) return launch_epi<1, X_BF16>(a, epilogue, s);
        if (prologue == X_F32_NORM) return launch_epi<1, X_F32_NORM>(a, epilogue, s);
    } else {
        if (prologue == X_BF16) return launch_epi<2, X_BF16>(a, epilogue, s);
        if (prologue == X_F32_NORM) return launch_epi<2, X_F32_NORM>(a, epilogue, s);
    }
    KLLM_FAIL("skinny_gemm: unknown prologue %d", prologue);
}
