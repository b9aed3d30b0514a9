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
// rows that go with them).  A CTA of 8 warps walks tiles tile = blockIdx.x,
// += gridDim.x; inside a tile the warps take the K dimension in interleaved steps
// of 32 elements, each lane loading 16 contiguous bytes of two weight rows per
// step.  A lane's 8 consecutive k-values feed two MMAs; the same permutation of k
// is applied to the activations, so the sum is unchanged.  The eight partial
// tiles are added in warp order through shared memory: no atomics, and every output
// element belongs to one CTA, so ADD_F32 is race-free and the order of all sums
// depends on K alone.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(skinny_gemm)

namespace {

constexpr int THREADS = 256;
constexpr int WARPS = 8;
constexpr int UNROLL = 4;          // k-steps of 32 in flight per lane and buffer

enum { X_BF16 = 0, X_F32_NORM = 1 };
enum { STORE_BF16 = 0, STORE_F32 = 1, ADD_F32 = 2, SWIGLU = 3 };

struct Args {
    const bf16* w;        // [N, K]; SWIGLU: the gate matrix [F, K]
    const bf16* w_up;     // SWIGLU: the up matrix [F, K]
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

__host__ __device__ inline int x_row_elems(int K) {      // row stride of X in shared memory, elements
    return K + (((K * 2) % 128 == 0) ? 32 : 0);           // bytes = 64 (mod 128): 16-byte reads of 8 rows x 4
}                                                         // quarter-row offsets hit 8 different bank groups

template <int NT, int PRO, int EPI>
__global__ void __launch_bounds__(THREADS)
skinny_gemm_kernel(const Args a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int K = a.K, N = a.N, n = a.n;
    const int XS = x_row_elems(K);
    bf16* xs = reinterpret_cast<bf16*>(smem_raw);                         // [8*NT][XS]
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)8 * NT * XS * 2);   // [WARPS][16][8*NT]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    constexpr int ROWS_PER_TILE = (EPI == SWIGLU) ? 8 : 16;
    const int n_tiles = (N + ROWS_PER_TILE - 1) / ROWS_PER_TILE;
    const int steps = K / 32;
    const int my_steps = (steps > warp) ? (steps - warp + WARPS - 1) / WARPS : 0;
    const int nb = (my_steps + UNROLL - 1) / UNROLL;

    // pointers of this lane's two weight rows for a tile (rows past the end repeat the last one)
    auto row_ptrs = [&](int tile, const bf16*& pa, const bf16*& pb) {
        if (EPI == SWIGLU) {
            const int r = min(tile * 8 + g, N - 1);
            pa = a.w + (int64_t)r * K + 8 * t;
            pb = a.w_up + (int64_t)r * K + 8 * t;
        } else {
            pa = a.w + (int64_t)min(tile * 16 + g, N - 1) * K + 8 * t;
            pb = a.w + (int64_t)min(tile * 16 + g + 8, N - 1) * K + 8 * t;
        }
    };
    uint4 ca[UNROLL], cb[UNROLL];      // current batch
    uint4 na[UNROLL], nbuf[UNROLL];    // next batch
    auto load_batch = [&](uint4 (&ra)[UNROLL], uint4 (&rb)[UNROLL], const bf16* pa, const bf16* pb, int b) {
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int s = b * UNROLL + u;
            if (s < my_steps) {
                const int off = (warp + s * WARPS) * 32;
                ra[u] = ldg_stream(pa + off);
                rb[u] = ldg_stream(pb + off);
            } else {
                ra[u] = make_uint4(0, 0, 0, 0);
                rb[u] = make_uint4(0, 0, 0, 0);
            }
        }
    };

    int tile = blockIdx.x;
    const bf16 *pa = nullptr, *pb = nullptr;
    if (tile < n_tiles && nb > 0) {          // weights do not depend on X: start them first
        row_ptrs(tile, pa, pb);
        load_batch(ca, cb, pa, pb, 0);
    }

    // ---- prologue: X into shared memory as bfloat16, rows past n are zero ----
    if (PRO == X_BF16) {
        const int chunks = K / 8;
        for (int c = threadIdx.x; c < 8 * NT * chunks; c += THREADS) {
            const int r = c / chunks, ch = c - r * chunks;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < n) v = *reinterpret_cast<const uint4*>(a.x_bf16 + (int64_t)r * a.x_stride + ch * 8);
            *reinterpret_cast<uint4*>(xs + r * XS + ch * 8) = v;
        }
    } else {
        for (int r = warp; r < 8 * NT; r += WARPS) {
            bf16* dst = xs + r * XS;
            if (r >= n) {
                for (int i = lane * 8; i < K; i += 32 * 8) *reinterpret_cast<uint4*>(dst + i) = make_uint4(0, 0, 0, 0);
                continue;
            }
            const float* src = a.x_f32 + (int64_t)(a.rows ? a.rows[r] : r) * K;
            float ss = 0.f;
            for (int i = lane * 4; i < K; i += 32 * 4) {
                const float4 v = *reinterpret_cast<const float4*>(src + i);
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
            ss = warp_sum(ss);
            const float scale = rsqrtf(ss / (float)K + a.eps);
            for (int i = lane * 4; i < K; i += 32 * 4) {
                const float4 v = *reinterpret_cast<const float4*>(src + i);
                const float4 gn = *reinterpret_cast<const float4*>(a.gain + i);
                __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * scale * gn.x, v.y * scale * gn.y);
                __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * scale * gn.z, v.w * scale * gn.w);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo);
                pk.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(dst + i) = pk;
            }
        }
    }
    __syncthreads();

    // ---- tiles ----
    for (; tile < n_tiles; tile += gridDim.x) {
        float acc[NT][4];
#pragma unroll
        for (int i = 0; i < NT; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
        const int next_tile = tile + gridDim.x;
        for (int b = 0; b < nb; b++) {
            if (b + 1 < nb) {
                load_batch(na, nbuf, pa, pb, b + 1);
            } else if (next_tile < n_tiles) {
                row_ptrs(next_tile, pa, pb);
                load_batch(na, nbuf, pa, pb, 0);
            }
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                const int s = b * UNROLL + u;
                if (s < my_steps) {
                    const int k0 = (warp + s * WARPS) * 32 + 8 * t;
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        const uint4 xb = *reinterpret_cast<const uint4*>(xs + (nt * 8 + g) * XS + k0);
                        mma_bf16(acc[nt], ca[u].x, cb[u].x, ca[u].y, cb[u].y, xb.x, xb.y);
                        mma_bf16(acc[nt], ca[u].z, cb[u].z, ca[u].w, cb[u].w, xb.z, xb.w);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; u++) { ca[u] = na[u]; cb[u] = nbuf[u]; }
        }
        // the eight warps' partial tiles, added in warp order
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            float* r0 = red + ((warp * 16 + g) * 8 * NT) + nt * 8 + 2 * t;
            float* r1 = red + ((warp * 16 + g + 8) * 8 * NT) + nt * 8 + 2 * t;
            r0[0] = acc[nt][0]; r0[1] = acc[nt][1]; r1[0] = acc[nt][2]; r1[1] = acc[nt][3];
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
}

size_t smem_bytes(int nt, int K) { return (size_t)8 * nt * x_row_elems(K) * 2 + (size_t)WARPS * 16 * 8 * nt * 4; }

template <int NT, int PRO, int EPI>
int launch(const Args& a, cudaStream_t s) {
    static int max_grid = 0;            // per instantiation: CTAs that fit the GPU at this kernel's register use
    static size_t attr_smem = 0;
    const size_t smem = smem_bytes(NT, a.K);
    auto kern = skinny_gemm_kernel<NT, PRO, EPI>;
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
    kern<<<grid, THREADS, smem, s>>>(a);
    KLLM_LAUNCH_STATUS();
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
extern "C" int kllm_skinny_gemm(const void* w, const void* w_up, int N, int K, int n, const void* x_bf16,
                                int64_t x_stride, const float* x_f32, const float* gain, const int* rows,
                                float eps, void* y_bf16, float* y_f32, int64_t y_stride, int prologue,
                                int epilogue, void* stream) {
    if (n <= 0 || N <= 0) return 0;
    if (!kllm_skinny_gemm_fits(n, K))
        KLLM_FAIL("skinny_gemm: %d rows of width %d not supported (1..16 rows, width a multiple of 32 that fits "
                  "shared memory)", n, K);
    if (prologue == X_BF16 && (!x_bf16 || (x_stride % 8) || ((uintptr_t)x_bf16 & 15)))
        KLLM_FAIL("skinny_gemm: bfloat16 X must be 16-byte aligned with a row stride that is a multiple of 8");
    if (prologue == X_F32_NORM && (!x_f32 || !gain || ((uintptr_t)x_f32 & 15) || ((uintptr_t)gain & 15)))
        KLLM_FAIL("skinny_gemm: float32 X and gain must be 16-byte aligned");
    if ((uintptr_t)w & 15) KLLM_FAIL("skinny_gemm: weights must be 16-byte aligned");
    if (epilogue == SWIGLU && (!w_up || ((uintptr_t)w_up & 15))) KLLM_FAIL("skinny_gemm: SWIGLU needs the up matrix");
    if ((epilogue == STORE_BF16 || epilogue == SWIGLU) ? !y_bf16 : !y_f32) KLLM_FAIL("skinny_gemm: no output buffer");
    Args a;
    a.w = (const bf16*)w; a.w_up = (const bf16*)w_up; a.N = N; a.K = K; a.n = n;
    a.x_bf16 = (const bf16*)x_bf16; a.x_stride = x_stride; a.x_f32 = x_f32; a.gain = gain; a.rows = rows; a.eps = eps;
    a.y_bf16 = (bf16*)y_bf16; a.y_f32 = y_f32; a.y_stride = y_stride;
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
