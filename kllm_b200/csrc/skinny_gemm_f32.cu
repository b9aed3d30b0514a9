// Y[n, N] = X[n, K] . W[N, K]^T in true float32 for up to 8 rows n (decode steps of the
// 32-bit path): the weights are streamed from HBM exactly once and meet the activations
// in FMA instructions on the CUDA cores; no tensor cores, no reduced-precision mode.
// The reference runs these products through cublasSgemm (backend/model.cu:496-503,
// :1090-1115); at a few rows the library picks matrix-vector kernels by the row count,
// which stream at a fraction of the memory's speed and sum in an order that depends on
// the batch.  Here every output element is summed in an order that depends on K alone.
// Prologues and epilogues as in skinny_gemm.cu:
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
// Layout of the work: a CTA of 16 warps, one per SM, keeps X in shared memory.  A tile is
// eight weight rows (SWIGLU: four gate rows and their four up rows).  The warps of a CTA
// are two row groups (four rows each) times eight k slices: a warp takes the k steps of
// 128 elements of its slice, its lanes split a step in float4 pieces, so a lane's X values
// (8 rows x float4, read once per k step) serve its four weight rows from registers.  Two
// register buffers take turns, so the next step's (or the next tile's) weights are in
// flight while this one's are multiplied.  The lanes' partial sums meet in a butterfly of
// shuffles, the eight slices' sums in shared memory, added in slice order: every order is
// fixed by K alone.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(skinny_gemm_f32)

namespace {

constexpr int THREADS = 512, WARPS = 16, ROWS = 8, WR = 4;      // X rows; weight rows per warp
constexpr int KSLICES = 8, GROUPS = 2;                          // the 16 warps: k slices x row groups
constexpr int UNROLL = 2;                                       // k steps of 128 per register buffer
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
    __shared__ float red[KSLICES * GROUPS * 32];           // per warp: its 4 rows x 8 tokens
    const int K = a.K, N = a.N, n = a.n;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grp = warp & 1, ks = warp >> 1;
    constexpr int OUT_PER_TILE = EPI == SWIGLU ? WR : GROUPS * WR;   // output columns of a tile
    const int n_tiles = (N + OUT_PER_TILE - 1) / OUT_PER_TILE;
    const int steps = K / 128;
    const int my_steps = steps > ks ? (steps - ks + KSLICES - 1) / KSLICES : 0;
    const int nb = max(1, ((steps + KSLICES - 1) / KSLICES + UNROLL - 1) / UNROLL);   // batches per tile, same for all warps

    // this warp's four weight rows of a tile (rows past the end repeat the last one; their sums are not stored)
    auto row_ptr = [&](int tile, int r) -> const float* {
        if (EPI == SWIGLU) return (grp == 0 ? a.w : a.w_up) + (int64_t)min(tile * WR + r, N - 1) * a.w_stride + 4 * lane;
        return a.w + (int64_t)min(tile * GROUPS * WR + grp * WR + r, N - 1) * a.w_stride + 4 * lane;
    };
    float4 buf0[UNROLL][WR], buf1[UNROLL][WR];
    auto load_batch = [&](float4 (&buf)[UNROLL][WR], int tile, int b) {
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int i = b * UNROLL + u;
            if (i < my_steps) {
                const int off = (ks + i * KSLICES) * 128;
#pragma unroll
                for (int r = 0; r < WR; r++) buf[u][r] = ldg_stream(row_ptr(tile, r) + off);
            }
        }
    };
    int cur_tile = blockIdx.x, cur_b = 0;          // the batch that sits in the buffer used next
    if (cur_tile < n_tiles) load_batch(buf0, cur_tile, 0);     // weights do not depend on X: on their way first
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
    float acc[WR][ROWS];
#pragma unroll
    for (int r = 0; r < WR; r++)
#pragma unroll
        for (int c = 0; c < ROWS; c++) acc[r][c] = 0.f;

    // multiply the batch (cur_tile, cur_b) held in `cur` while the following batch loads into `nxt`
    auto phase = [&](float4 (&cur)[UNROLL][WR], float4 (&nxt)[UNROLL][WR]) {
        int nxt_tile = cur_tile, nxt_b = cur_b + 1;
        if (nxt_b == nb) { nxt_b = 0; nxt_tile += gridDim.x; }
        if (nxt_tile < n_tiles) load_batch(nxt, nxt_tile, nxt_b);
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            const int i = cur_b * UNROLL + u;
            if (i < my_steps) {
                const int k = (ks + i * KSLICES) * 128 + 4 * lane;
#pragma unroll
                for (int c = 0; c < ROWS; c++) {
                    const float4 xv = *reinterpret_cast<const float4*>(xs + (size_t)c * K + k);
#pragma unroll
                    for (int r = 0; r < WR; r++) {
                        acc[r][c] = fmaf(cur[u][r].x, xv.x, acc[r][c]);
                        acc[r][c] = fmaf(cur[u][r].y, xv.y, acc[r][c]);
                        acc[r][c] = fmaf(cur[u][r].z, xv.z, acc[r][c]);
                        acc[r][c] = fmaf(cur[u][r].w, xv.w, acc[r][c]);
                    }
                }
            }
        }
        if (cur_b == nb - 1) {
            // The lanes' partial sums: 32 values on 32 lanes are summed by halving (each step a
            // lane hands half of its values to the partner lane and adds what it is handed), so
            // that lane r * 8 + c ends with the warp's sum of (row r, token c): 31 shuffles instead
            // of 160, in a fixed order.
            float v[WR * ROWS];
#pragma unroll
            for (int r = 0; r < WR; r++)
#pragma unroll
                for (int c = 0; c < ROWS; c++) { v[r * ROWS + c] = acc[r][c]; acc[r][c] = 0.f; }
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) {
                const bool upper = (lane & o) != 0;
#pragma unroll
                for (int j = 0; j < o; j++) {
                    const float send = upper ? v[j] : v[j + o];
                    const float keep = upper ? v[j + o] : v[j];
                    v[j] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                }
            }
            const float mine = v[0];
            red[warp * 32 + lane] = mine;              // warp = ks * GROUPS + grp
            __syncthreads();
            const int tile = cur_tile;
            if (threadIdx.x < (EPI == SWIGLU ? 32 : 64)) {
                const int e = threadIdx.x, g2 = e >> 5, rc = e & 31, r = rc / ROWS, c = rc % ROWS;
                float v = 0.f, up = 0.f;
#pragma unroll
                for (int q = 0; q < KSLICES; q++) v += red[(q * GROUPS + g2) * 32 + rc];      // the slices, in order
                if (EPI == SWIGLU) {
#pragma unroll
                    for (int q = 0; q < KSLICES; q++) up += red[(q * GROUPS + 1) * 32 + rc];
                }
                const int col = EPI == SWIGLU ? tile * WR + r : tile * GROUPS * WR + g2 * WR + r;
                if (c < n && col < N) {
                    float* dst = a.y + (int64_t)c * a.y_stride + col;
                    if (EPI == SWIGLU) *dst = (v / (1.f + expf(-v))) * up;
                    else if (EPI == ADD) *dst += v;
                    else *dst = v;
                }
            }
            __syncthreads();
        }
        cur_tile = nxt_tile;
        cur_b = nxt_b;
    };
    while (cur_tile < n_tiles) {
        phase(buf0, buf1);
        if (cur_tile >= n_tiles) break;
        phase(buf1, buf0);
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
    const int out_per_tile = EPI == SWIGLU ? WR : GROUPS * WR;
    const int n_tiles = (a.N + out_per_tile - 1) / out_per_tile;
    const int grid = max(1, min(n_tiles, max(1, sms)));
    kllm_launch_dep(n_tiles <= 3 * grid, (kern), dim3(grid), dim3(THREADS), smem, s, a);
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
