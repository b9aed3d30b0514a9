// y = x . W^T for prompt portions on the fifth-generation tensor cores, with the work
// that follows a projection folded into its epilogue.
//
//   x [M, K] bfloat16 (activations, K contiguous), W [N, K] bfloat16 (a projection's
//   weight as the checkpoint stores it, K contiguous), float32 accumulation.
//
// Epilogues (what the reference does in separate kernels after cublasSgemm,
// backend/model.cu:496-503 for the products, :477-483 for the gated activation,
// :97-110 for the residual sum):
//   0  y[M, N] bfloat16 = acc
//   1  y[M, N] float32  = acc
//   2  y[M, N] float32 += acc                        (residual stream)
//   3  y[M, N] bfloat16 = silu(acc_gate) * acc_up    (W = gate rows, W_up = up rows)
//
// A persistent CTA per SM walks output tiles of 128 x BN.  BN, the accumulator's width,
// is a multiple of 16 up to 256 (the gated epilogue spends half of the columns on
// `up`).  Measured on this GPU, an M = 128 instruction takes the same time whatever its
// N, so anything narrower than 256 leaves the tensor core partly idle: 256 is the
// default and narrower tiles are for matrices with fewer columns.  Ten warps, three roles:
//   warp 0   producer: one lane issues TMA loads (cp.async.bulk.tensor, 128-byte
//            swizzle) of the x and W tiles of a 64-wide k block into a ring of
//            shared-memory stages, each guarded by a full/empty pair of mbarriers;
//   warp 1   one lane issues tcgen05.mma (M = 128, N = BN, K = 16; four per k block)
//            from the stage into one of two accumulators in tensor memory and commits
//            the stage back to the producer; after the last k block it commits the
//            accumulator to the epilogue;
//   warps 2-9  epilogue: a thread owns one row of one half of the tile's columns, reads
//            it from tensor memory 32 columns at a time (tcgen05.ld), applies the
//            epilogue and stores.  With two accumulators the epilogue of a tile overlaps
//            the products of the next.
// A row of the result is a sum over k in one fixed order, whatever else is in the batch.
//
// Every wait on an mbarrier is bounded by a cycle count; a wait that runs out raises a
// flag in shared memory and sets *status, all roles leave their loops, the producer
// waits (bounded) for copies it still has in flight, and the CTA frees its tensor
// memory and returns.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(gemm_tcgen05)

#include "tc5_common.cuh"

namespace {

constexpr int BM = 128;                    // rows of a tile = lanes of tensor memory
constexpr int BK = TC5_BK;                 // k block: 64 bfloat16 = one 128-byte swizzled row
constexpr int THREADS = 320;
constexpr int EPI_THREADS = 256;
constexpr int A_BYTES = BM * 128;
constexpr int MAX_BN = 256;                // accumulators sit 256 columns apart in tensor memory
constexpr int TMEM_COLS = 2 * MAX_BN;
constexpr int MAX_STAGES = 8;
constexpr int SMEM_BYTES = 1024 + 4 * (A_BYTES + MAX_BN * 128);    // four stages of the widest tile

enum Epilogue { EPI_BF16 = 0, EPI_F32 = 1, EPI_ADD_F32 = 2, EPI_SWIGLU = 3 };

// 32 consecutive results of one row, columns col..col+31 of the output, those below
// `limit` (the end of the tile or of the matrix); res: what the float32 destination held
template <int EPI>
__device__ __forceinline__ void store_chunk(void* y, int64_t ldy, int row, int col, int limit, const float (&v)[32],
                                            const float4 (&res)[8]) {
    if (EPI == EPI_BF16 || EPI == EPI_SWIGLU) {
        bf16* p = (bf16*)y + (int64_t)row * ldy + col;
        if (col + 32 <= limit) {
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint4 pk;
                pk.x = pack_bf16(v[8 * c], v[8 * c + 1]);
                pk.y = pack_bf16(v[8 * c + 2], v[8 * c + 3]);
                pk.z = pack_bf16(v[8 * c + 4], v[8 * c + 5]);
                pk.w = pack_bf16(v[8 * c + 6], v[8 * c + 7]);
                *reinterpret_cast<uint4*>(p + 8 * c) = pk;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (col + j < limit) p[j] = __float2bfloat16_rn(v[j]);
        }
    } else {
        float* p = (float*)y + (int64_t)row * ldy + col;
        if (col + 32 <= limit) {
#pragma unroll
            for (int c = 0; c < 8; c++) {
                float4 o = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
                if (EPI == EPI_ADD_F32) { o.x += res[c].x; o.y += res[c].y; o.z += res[c].z; o.w += res[c].w; }
                *reinterpret_cast<float4*>(p + 4 * c) = o;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (col + j < limit) p[j] = (EPI == EPI_ADD_F32 ? p[j] : 0.f) + v[j];
        }
    }
}

// what the destination holds at columns col..col+31 of a row (whole chunks only; a
// ragged chunk is read where it is added)
__device__ __forceinline__ void load_residual(const void* y, int64_t ldy, int row, int col, int limit, bool row_ok,
                                              float4 (&res)[8]) {
    if (row_ok && col + 32 <= limit) {
        const float* p = (const float*)y + (int64_t)row * ldy + col;
#pragma unroll
        for (int c = 0; c < 8; c++) res[c] = *reinterpret_cast<const float4*>(p + 4 * c);
    }
}

template <int EPI>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_b2, void* __restrict__ y, int64_t ldy, int M, int N, int K,
                int bn, int stages, int* status) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[MAX_STAGES], bar_empty[MAX_STAGES], bar_acc_full[2], bar_acc_empty[2];
    __shared__ unsigned s_tmem;
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int nout = (EPI == EPI_SWIGLU) ? bn / 2 : bn;            // output columns of a tile
    const int b_bytes = bn * 128, stage_bytes = A_BYTES + b_bytes;
    const int m_tiles = (M + BM - 1) / BM;
    const int n_tiles = (N + nout - 1) / nout;
    const int tiles = m_tiles * n_tiles;
    const int kblocks = (K + BK - 1) / BK;
    volatile int* abort_flag = &s_abort;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) { mbar_init(&bar_full[s], 1); mbar_init(&bar_empty[s], 1); }
        for (int a = 0; a < 2; a++) { mbar_init(&bar_acc_full[a], 1); mbar_init(&bar_acc_empty[a], EPI_THREADS); }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = s_tmem;
    griddep_launch();

    if (warp == 0) {
        // ---- producer ----------------------------------------------------------
        if (lane == 0) {
            prefetch_map(&map_a);
            prefetch_map(&map_b);
            if (EPI == EPI_SWIGLU) prefetch_map(&map_b2);
        }
        griddep_wait();
        int s = 0;
        unsigned ph = 0;
        int issued = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < tiles; tile += gridDim.x) {
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * nout;
            for (int kb = 0; kb < kblocks; kb++) {
                ok = mbar_wait(&bar_empty[s], ph ^ 1u, abort_flag, status, 1);
                if (!ok) break;
                if (lane == 0) {
                    const unsigned a = base + (unsigned)(s * stage_bytes), b = a + A_BYTES;
                    mbar_expect_tx(&bar_full[s], (unsigned)stage_bytes);
                    tma_load_2d(a, &map_a, kb * BK, m0, &bar_full[s]);
                    tma_load_2d(b, &map_b, kb * BK, n0, &bar_full[s]);
                    if (EPI == EPI_SWIGLU) tma_load_2d(b + (unsigned)(b_bytes / 2), &map_b2, kb * BK, n0, &bar_full[s]);
                }
                __syncwarp();
                issued++;
                if (++s == stages) { s = 0; ph ^= 1u; }
            }
        }
        if (!ok || *abort_flag) {
            // copies still in flight must land before the shared memory goes away: wait,
            // with the same bound, for the stages armed last
            const int back = issued < stages ? issued : stages;
            for (int j = 0; j < back; j++) {
                int sj = s - 1 - j;
                unsigned pj = ph;
                if (sj < 0) { sj += stages; pj ^= 1u; }
                const long long t0 = clock64();
                while (!mbar_try_wait(&bar_full[sj], pj) && clock64() - t0 < kCycleLimit) {}
            }
        }
    } else if (warp == 1) {
        // ---- tensor-core issuer ------------------------------------------------
        const uint32_t idesc = make_idesc(BM, bn);
        griddep_wait();
        int s = 0, acc = 0;
        unsigned ph = 0, acc_ph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < tiles; tile += gridDim.x) {
            ok = mbar_wait(&bar_acc_empty[acc], acc_ph ^ 1u, abort_flag, status, 2);
            if (!ok) break;
            tc_fence_after();
            const unsigned d = tmem + (unsigned)(acc * MAX_BN);
            for (int kb = 0; kb < kblocks; kb++) {
                ok = mbar_wait(&bar_full[s], ph, abort_flag, status, 3);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const unsigned a = base + (unsigned)(s * stage_bytes), b = a + A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BK / 16; kk++)
                        umma(d, make_desc(a + kk * 32), make_desc(b + kk * 32), idesc, kb > 0 || kk > 0);
                    umma_commit(&bar_empty[s]);
                }
                __syncwarp();
                if (++s == stages) { s = 0; ph ^= 1u; }
            }
            if (!ok) break;
            if (lane == 0) umma_commit(&bar_acc_full[acc]);
            __syncwarp();
            acc ^= 1;
            if (acc == 0) acc_ph ^= 1u;
        }
    } else {
        // ---- epilogue ----------------------------------------------------------
        griddep_wait();
        const int quarter = warp & 3;                      // the 32 lanes of tensor memory this warp may read
        const int half = (warp - 2) >> 2;                  // which half of the tile's 32-column chunks
        const unsigned lane_base = (unsigned)(quarter * 32) << 16;
        const int chunks = (nout + 31) / 32;
        const int c_lo = half == 0 ? 0 : (chunks + 1) / 2, c_hi = half == 0 ? (chunks + 1) / 2 : chunks;
        int acc = 0;
        unsigned acc_ph = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * nout;
            const int row = m0 + quarter * 32 + lane;
            const bool row_ok = row < M;
            const int limit = min(N, n0 + nout);
            float4 res[8];
            if (EPI == EPI_ADD_F32) load_residual(y, ldy, row, n0 + c_lo * 32, limit, row_ok, res);   // under the products
            if (!mbar_wait(&bar_acc_full[acc], acc_ph, abort_flag, status, 4)) break;
            tc_fence_after();
            const unsigned t = tmem + lane_base + (unsigned)(acc * MAX_BN);
#pragma unroll 1
            for (int c = c_lo; c < c_hi; c++) {
                float v[32];
                float4 res_next[8];
                tmem_ld32(t + c * 32, v);
                if (EPI == EPI_SWIGLU) {
                    float u[32];
                    tmem_ld32(t + bn / 2 + c * 32, u);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 32; j++) v[j] = silu_mul(v[j], u[j]);
                } else {
                    if (EPI == EPI_ADD_F32 && c + 1 < c_hi) load_residual(y, ldy, row, n0 + (c + 1) * 32, limit, row_ok, res_next);
                    tmem_ld_wait();
                }
                const int col = n0 + c * 32;
                if (row_ok && col < limit) store_chunk<EPI>(y, ldy, row, col, limit, v, res);
                if (EPI == EPI_ADD_F32) {
#pragma unroll
                    for (int j = 0; j < 8; j++) res[j] = res_next[j];
                }
            }
            tc_fence_before();
            mbar_arrive(&bar_acc_empty[acc]);
            acc ^= 1;
            if (acc == 0) acc_ph ^= 1u;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS));
}

// ---- host side -----------------------------------------------------------------

// Accumulator width: a tile's time does not shrink with its width (see the top of the
// file), so the widest one with the fewest waves of tiles wins.
int pick_bn(int M, int N, int epilogue) {
    const int sms = sm_count();
    const int m_tiles = (M + BM - 1) / BM;
    const int step = epilogue == EPI_SWIGLU ? 64 : 16;       // the up half starts on a 32-column chunk
    long long best = -1;
    int best_bn = MAX_BN;
    for (int bn = MAX_BN; bn >= 64; bn -= step) {
        const int nout = epilogue == EPI_SWIGLU ? bn / 2 : bn;
        const long long tiles = (long long)m_tiles * ((N + nout - 1) / nout);
        const long long waves = (tiles + sms - 1) / sms;
        if (best < 0 || waves < best) { best = waves; best_bn = bn; }
    }
    return best_bn;
}

template <int EPI>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2, void* y, int64_t ldy, int M, int N, int K,
           int bn, int* status, cudaStream_t stream) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc5_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) {
            snprintf(g_kllm_err, sizeof(g_kllm_err), "gemm (tcgen05): %d bytes of shared memory refused: %s", SMEM_BYTES,
                     cudaGetErrorString(e));
            return (int)e;
        }
        attr_set = true;
    }
    const int nout = (EPI == EPI_SWIGLU) ? bn / 2 : bn;
    const long long tiles = (long long)((M + BM - 1) / BM) * ((N + nout - 1) / nout);
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    int stages = (SMEM_BYTES - 1024) / (A_BYTES + bn * 128);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    kllm_launch((gemm_tc5_kernel<EPI>), dim3(grid), dim3(THREADS), SMEM_BYTES, stream, ma, mb, mb2, y, ldy, M, N, K, bn, stages,
                status);
    KLLM_LAUNCH_STATUS();
}

}  // namespace

// Share of the tensor-core time that tiles of the widest accumulator would use for an
// M x N product, in percent: full tiles / (waves x CTAs).  Callers use it to choose
// between this kernel and the library product.
extern "C" int kllm_gemm_tcgen05_efficiency(int M, int N, int epilogue) {
    if (M <= 0 || N <= 0) return 0;
    const int nout = epilogue == EPI_SWIGLU ? MAX_BN / 2 : MAX_BN;
    const double full = ((double)M / BM) * ((double)N / nout);
    const long long tiles = (long long)((M + BM - 1) / BM) * ((N + nout - 1) / nout);
    const long long waves = (tiles + sm_count() - 1) / sm_count();
    return (int)(100.0 * full / (double)(waves * sm_count()));
}

// 1 if the kernel takes these sizes and addresses, else 0 (the caller then uses the
// library product and separate elementwise kernels).
extern "C" int kllm_gemm_tcgen05_fits(const void* x, int64_t ldx, const void* w, int64_t ldw, const void* w_up, int M,
                                      int N, int K, const void* y, int64_t ldy, int epilogue) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (epilogue < 0 || epilogue > 3) return 0;
    if ((K & 7) || (ldx & 7) || (ldw & 7)) return 0;                      // TMA: 16-byte rows
    if (((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ((uintptr_t)w_up & 15) || ((uintptr_t)y & 15)) return 0;
    const bool bf16_out = epilogue == EPI_BF16 || epilogue == EPI_SWIGLU;
    if (bf16_out ? (ldy & 7) : (ldy & 3)) return 0;                        // 16-byte vector stores
    if (epilogue == EPI_SWIGLU && !w_up) return 0;
    return 1;
}

// bn: accumulator width of a tile, 0 = chosen here, else a multiple of 16 (64 for the
// gated epilogue) from 64 to 256.  status: device int that a wait which ran out sets
// (1: producer, 2: accumulator, 3: stage, 4: epilogue).
extern "C" int kllm_gemm_tcgen05(const void* x, int64_t ldx, const void* w, int64_t ldw, const void* w_up, int M, int N,
                                 int K, void* y, int64_t ldy, int epilogue, int bn, int* status, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!kllm_gemm_tcgen05_fits(x, ldx, w, ldw, w_up, M, N, K, y, ldy, epilogue))
        KLLM_FAIL("gemm (tcgen05): sizes %d x %d x %d, strides %lld/%lld/%lld or an address not taken (k and strides "
                  "multiples of 8, 16-byte aligned addresses)", M, N, K, (long long)ldx, (long long)ldw, (long long)ldy);
    if (bn == 0) bn = pick_bn(M, N, epilogue);
    if (bn < 64 || bn > MAX_BN || bn % (epilogue == EPI_SWIGLU ? 64 : 16))
        KLLM_FAIL("gemm (tcgen05): accumulator width %d, a multiple of %d from 64 to %d", bn, epilogue == EPI_SWIGLU ? 64 : 16, MAX_BN);
    CUtensorMap ma, mb, mb2;
    const int b_rows = epilogue == EPI_SWIGLU ? bn / 2 : bn;
    int r = tensor_map(&ma, x, ldx, M, K, BM);
    if (r) return r;
    r = tensor_map(&mb, w, ldw, N, K, b_rows);
    if (r) return r;
    if (epilogue == EPI_SWIGLU) {
        r = tensor_map(&mb2, w_up, ldw, N, K, b_rows);
        if (r) return r;
    } else {
        mb2 = mb;
    }
    cudaStream_t s = (cudaStream_t)stream;
    switch (epilogue) {
        case EPI_BF16: return launch<EPI_BF16>(ma, mb, mb2, y, ldy, M, N, K, bn, status, s);
        case EPI_F32: return launch<EPI_F32>(ma, mb, mb2, y, ldy, M, N, K, bn, status, s);
        case EPI_ADD_F32: return launch<EPI_ADD_F32>(ma, mb, mb2, y, ldy, M, N, K, bn, status, s);
        default: return launch<EPI_SWIGLU>(ma, mb, mb2, y, ldy, M, N, K, bn, status, s);
    }
}
