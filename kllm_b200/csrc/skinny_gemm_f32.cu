// Y[n, N] = X[n, K] . W[N, K]^T in true float32 for up to 8 rows n (decode steps of the
// 32-bit path): the weights are streamed from HBM exactly once and meet the activations
// in FMA instructions on the CUDA cores; no tensor cores, no reduced-precision mode.
// The reference runs these products through cublasSgemm (backend/model.cu:496-503,
// :1090-1115); at a few rows the library picks matrix-vector kernels by the row count,
// which stream at a fraction of the memory's speed and sum in an order that depends on
// the batch.  Here every output element is one warp's sum in an order that depends on K
// alone.  Prologues and epilogues as in skinny_gemm.cu:
//
//   prologue  X_PLAIN     X is a float32 matrix [n, K]
//             X_NORM      X = rmsnorm(x) * gain of float32 rows x (optionally gathered by
//                         `rows`), computed by every CTA for itself (backend/model.cu:101-122)
//   epilogue  STORE       Y as float32
//             ADD         Y is added into a float32 matrix (the residual stream)
//             SWIGLU      W holds a gate and an up matrix [F, K] each; the output is
//                         silu(gate row) * (up row) as float32 [n, F]
//                         (backend/model.cu:477-483, :1112-1114)
//
// Layout of the work: a CTA of 16 warps, one per SM, keeps X in shared memory.  A warp
// takes four weight rows at a time (SWIGLU: two gate rows and their two up rows); its
// lanes split K in interleaved float4 pieces, so a lane's X values (8 rows x float4, read
// once per k step) serve all four weight rows from registers.  The lanes' partial sums
// meet in a butterfly of shuffles whose order is fixed.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(skinny_gemm_f32)

namespace {

constexpr int THREADS = 512, WARPS = 16, ROWS = 8, WR = 4;      // X rows; weight rows per warp and pass
constexpr int UNROLL = 2;                                       // k steps of 128 in flight per lane
enum { X_PLAIN = 0, X_NORM = 1 };
enum { STORE = 0, ADD = 1, SWIGLU = 2 };

struct Args {
    const float* w;       // [N, K] at w_stride; SWIGLU: the gate matrix [F, K]
    const float* w_up;    // SWIGLU: the up matrix
    int64_t w_stride;
    int N, K, n;
    const float* x;       // rows of width K at x_stride
    int64_t x_stride;
    const float* gain;    // X_NORM: [K]
    const int* rows;      // X_NORM: optional gather of rows
    float eps;
    float* y;             // [n, N] at y_stride
    int64_t y_stride;
};

__device__ __forceinline__ float4 ldg_stream(const float* p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];\n"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

template <int PRO, int EPI>
__global__ void __launch_bounds__(THREADS, 1)
skinny_f32_kernel(const Args a) {
    extern __shared__ __align__(16) float xs[];            // [ROWS][K]
    __shared__ float ss_part[ROWS][2];
    const int K = a.K, N = a.N, n = a.n;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int OUT_PER_TILE = EPI == SWIGLU ? 2 : WR;   // output columns of a warp's pass
    const int n_tiles = (N + OUT_PER_TILE - 1) / OUT_PER_TILE;
    const int steps = K / 128;

    // the four weight rows of a tile (rows past the end repeat the last one; their sums are not stored)
    auto row_ptr = [&](int tile, int r) -> const float* {
        if (EPI == SWIGLU) {
            const int col = min(tile * 2 + (r & 1), N - 1);
            return (r < 2 ? a.w : a.w_up) + (int64_t)col * a.w_stride + 4 * lane;
        }
        return a.w + (int64_t)min(tile * WR + r, N - 1) * a.w_stride + 4 * lane;
    };
    int tile = blockIdx.x * WARPS + warp;
    const int tile_step = gridDim.x * WARPS;
    float4 wbuf[UNROLL][WR];
    auto load_w = [&](int t, int s0) {
#pragma unroll
        for (int u = 0; u < UNROLL; u++)
            if (s0 + u < steps) {
#pragma unroll
                for (int r = 0; r < WR; r++) wbuf[u][r] = ldg_stream(row_ptr(t, r) + (s0 + u) * 128);
            }
    };
    if (tile < n_tiles) load_w(tile, 0);           // weights do not depend on X: on their way first
    griddep_wait();
    griddep_launch();

    // ---- X into shared memory as float32, rows past n are zero ----
    {
        const int r = warp >> 1, half = warp & 1;                  // two warps share a row
        const int span = K / 2, lo_k = half * span;                // K % 128 == 0: a multiple of 4
        const bool live = r < n;
        const float* src = live ? a.x + (int64_t)((PRO == X_NORM && a.rows) ? a.rows[r] : r) * a.x_stride : nullptr;
        float* dst = xs + (size_t)r * K;
        if (PRO == X_NORM) {
            float ss = 0.f;
            if (live)
                for (int k = lo_k + lane * 4; k < lo_k + span; k += 128) {
                    const float4 v = __ldcg(reinterpret_cast<const float4*>(src + k));
                    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                }
            ss = warp_sum(ss);
            if (lane == 0) ss_part[r][half] = ss;
            __syncthreads();
            const float scale = rsqrtf((ss_part[r][0] + ss_part[r][1]) / (float)K + a.eps);
            for (int k = lo_k + lane * 4; k < lo_k + span; k += 128) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (live) {
                    v = __ldcg(reinterpret_cast<const float4*>(src + k));
                    const float4 g4 = __ldg(reinterpret_cast<const float4*>(a.gain + k));
                    v.x = v.x * scale * g4.x; v.y = v.y * scale * g4.y; v.z = v.z * scale * g4.z; v.w = v.w * scale * g4.w;
                }
                *reinterpret_cast<float4*>(dst + k) = v;
            }
        } else {
            for (int k = lo_k + lane * 4; k < lo_k + span; k += 128)
                *reinterpret_cast<float4*>(dst + k) =
                    live ? __ldcg(reinterpret_cast<const float4*>(src + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    __syncthreads();

    // ---- tiles ----
    for (; tile < n_tiles; tile += tile_step) {
        float acc[WR][ROWS];
#pragma unroll
        for (int r = 0; r < WR; r++)
#pragma unroll
            for (int c = 0; c < ROWS; c++) acc[r][c] = 0.f;
        for (int s0 = 0; s0 < steps; s0 += UNROLL) {
            float4 wcur[UNROLL][WR];
#pragma unroll
            for (int u = 0; u < UNROLL; u++)
#pragma unroll
                for (int r = 0; r < WR; r++) wcur[u][r] = wbuf[u][r];
            // the next k steps of this tile, or the first of the warp's next tile
            if (s0 + UNROLL < steps) load_w(tile, s0 + UNROLL);
            else if (tile + tile_step < n_tiles) load_w(tile + tile_step, 0);
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                if (s0 + u >= steps) break;
                const int k = (s0 + u) * 128 + 4 * lane;
#pragma unroll
                for (int c = 0; c < ROWS; c++) {
                    const float4 xv = *reinterpret_cast<const float4*>(xs + (size_t)c * K + k);
#pragma unroll
                    for (int r = 0; r < WR; r++) {
                        acc[r][c] = fmaf(wcur[u][r].x, xv.x, acc[r][c]);
                        acc[r][c] = fmaf(wcur[u][r].y, xv.y, acc[r][c]);
                        acc[r][c] = fmaf(wcur[u][r].z, xv.z, acc[r][c]);
                        acc[r][c] = fmaf(wcur[u][r].w, xv.w, acc[r][c]);
                    }
                }
            }
        }
        // the lanes' partial sums, in a fixed butterfly; lane r * 8 + c keeps output (r, c)
        float mine = 0.f, partner = 0.f;
#pragma unroll
        for (int r = 0; r < WR; r++)
#pragma unroll
            for (int c = 0; c < ROWS; c++) {
                const float v = warp_sum(acc[r][c]);
                if (lane == r * ROWS + c) mine = v;
                if (EPI == SWIGLU && lane + 2 * ROWS == r * ROWS + c) partner = v;     // the up row of this gate row
            }
        const int r = lane / ROWS, c = lane % ROWS;
        if (c < n) {
            if (EPI == SWIGLU) {
                const int col = tile * 2 + r;
                if (r < 2 && col < N) a.y[(int64_t)c * a.y_stride + col] = (mine / (1.f + expf(-mine))) * partner;
            } else {
                const int col = tile * WR + r;
                if (col < N) {
                    float* dst = a.y + (int64_t)c * a.y_stride + col;
                    if (EPI == ADD) *dst += mine; else *dst = mine;
                }
            }
        }
    }
}

template <int PRO, int EPI>
int launch(const Args& a, cudaStream_t s) {
    static size_t attr_smem = 0;
    const size_t smem = (size_t)ROWS * a.K * sizeof(float);
    auto kern = skinny_f32_kernel<PRO, EPI>;
    if (smem > attr_smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            snprintf(g_kllm_err, sizeof(g_kllm_err), "skinny_gemm_f32: %zu bytes of shared memory refused: %s", smem,
                     cudaGetErrorString(e));
            return (int)e;
        }
        attr_smem = smem;
    }
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int out_per_tile = EPI == SWIGLU ? 2 : WR;
    const int n_tiles = (a.N + out_per_tile - 1) / out_per_tile;
    const int grid = max(1, min((n_tiles + WARPS - 1) / WARPS, max(1, sms)));
    kllm_launch_dep(n_tiles <= 3 * grid * WARPS, (kern), dim3(grid), dim3(THREADS), smem, s, a);
    KLLM_LAUNCH_STATUS();
}

}  // namespace

// 1 if (n, K) can run here: up to 8 rows, K a multiple of 128 whose 8 rows fit shared memory.
extern "C" int kllm_skinny_gemm_f32_fits(int n, int K) {
    return (n >= 1 && n <= ROWS && K >= 128 && K % 128 == 0 && (size_t)ROWS * K * 4 <= 220 * 1024) ? 1 : 0;
}

// prologue 0: x float32 [n, K] at x_stride.  prologue 1: rows of x (row r is rows[r] when rows is
// given) normalised with gain [K] and eps.  epilogue 0: y written; 1: y += result; 2: w = gate
// [N, K], w_up = up [N, K], y = silu(gate) * up.  w_stride: elements from one weight row to the
// next (more than K when the call multiplies a slice of the columns of a wider matrix).
extern "C" int kllm_skinny_gemm_f32(const float* w, const float* w_up, int64_t w_stride, int N, int K, int n,
                                    const float* x, int64_t x_stride, const float* gain, const int* rows, float eps,
                                    float* y, int64_t y_stride, int prologue, int epilogue, void* stream) {
    if (n <= 0 || N <= 0) return 0;
    if (!kllm_skinny_gemm_f32_fits(n, K))
        KLLM_FAIL("skinny_gemm_f32: %d rows of width %d not supported (1..8 rows, width a multiple of 128 that fits "
                  "shared memory)", n, K);
    if (!w || !x || !y || ((uintptr_t)w & 15) || ((uintptr_t)x & 15) || (w_stride % 4) || (x_stride % 4) || w_stride < K)
        KLLM_FAIL("skinny_gemm_f32: operands must be 16-byte aligned with row strides that are multiples of 4");
    if (prologue == X_NORM && (!gain || ((uintptr_t)gain & 15))) KLLM_FAIL("skinny_gemm_f32: the norm needs a 16-byte aligned gain");
    if (epilogue == SWIGLU && (!w_up || ((uintptr_t)w_up & 15))) KLLM_FAIL("skinny_gemm_f32: SWIGLU needs the up matrix");
    Args a;
    a.w = w; a.w_up = w_up; a.w_stride = w_stride; a.N = N; a.K = K; a.n = n; a.x = x; a.x_stride = x_stride;
    a.gain = gain; a.rows = rows; a.eps = eps; a.y = y; a.y_stride = y_stride;
    cudaStream_t s = (cudaStream_t)stream;
#define KLLM_F32_CASE(P, E) if (prologue == P && epilogue == E) return launch<P, E>(a, s)
    KLLM_F32_CASE(X_PLAIN, STORE); KLLM_F32_CASE(X_PLAIN, ADD); KLLM_F32_CASE(X_PLAIN, SWIGLU);
    KLLM_F32_CASE(X_NORM, STORE); KLLM_F32_CASE(X_NORM, ADD); KLLM_F32_CASE(X_NORM, SWIGLU);
#undef KLLM_F32_CASE
    KLLM_FAIL("skinny_gemm_f32: unknown prologue %d or epilogue %d", prologue, epilogue);
}
