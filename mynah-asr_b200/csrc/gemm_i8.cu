// Integer contraction C[M,N] = A[M,K] * B[N,K]^T on the 5th-generation tensor cores (tcgen05.mma kind::i8).
//
// This is the int8-activation mode of the quantised matmul for any number of rows: the arithmetic the
// reference runs below 17 rows by default and for every row count with MYNAH_ASR_QGEMM=1
// (src/qmat.c:508-551, 598-643: activation rows quantised once by quantize_act_int8, then
// out[t,i] = (float)(sum_k qx[t,k] * qw[i,k]) * ws[i] * sx[t], qgemm_block :464-500). The int32 sums are
// exact and order-independent, so a row's result does not depend on M, on the tile it falls in or on what
// else is in the batch, and it is bit-identical to the reference's.
//
//   * operands are the stored bytes: activations [M,K] int8 written by the producing kernel, weights [N,K]
//     int8 exactly as the reference-native format holds them; TMA (cp.async.bulk.tensor.2d, 128-byte
//     swizzle, every CTA loads its own tiles) stages 128 x 128-byte A tiles and BN x 128-byte B tiles into a
//     shared-memory ring guarded by mbarriers;
//   * one elected thread issues tcgen05.mma kind::i8 (M = 128, N = BN, K = 32: four per staged tile) into an
//     int32 accumulator in tensor memory, double-buffered so the epilogue of one tile overlaps the MMAs of
//     the next;
//   * eight epilogue warps read the accumulator (tcgen05.ld), convert, apply the weight-row and the
//     activation-row scale in the reference's order, then the same fused tail as the fp16 contraction
//     (bias, SiLU / ReLU, f32 store, residual accumulate or fp16 operand planes).
//
// One MMA per product at the int8 rate: this is the mode whose ceiling is the tensor-core peak, where the
// three-product fp16 split of the f32-grade mode stops at a third of it.
#include "gemm.h"

namespace mb {

static constexpr int I8_BK = 128;           // bytes (= int8 elements) of K per staged tile row: one swizzle span
static constexpr int I8_EPI_WARPS = 8;
static constexpr int I8_THREADS = (2 + I8_EPI_WARPS) * 32;   // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue
static constexpr int I8_SMEM_LIMIT = 232448;

template <int BN>
struct I8Cfg {
    static constexpr int A_BYTES = GEMM_BM * I8_BK;
    static constexpr int B_BYTES = BN * I8_BK;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // the epilogue warps' turning buffers: only the wide tiles have them (the narrow ones serve few-row contractions)
    static constexpr bool BLOCK_EPILOGUE = BN >= 128;
    static constexpr int EPI_BYTES = BLOCK_EPILOGUE ? I8_EPI_WARPS * GEMM_BLOCK_STAGE_FLOATS * 4 : 0;
    static constexpr int STAGES_RAW = (I8_SMEM_LIMIT - 2048 - EPI_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 2048;
    static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    static_assert(TMEM_COLS <= 512, "TMEM has 512 columns");
};

// D[tmem] (+)= A[smem] * B[smem]; int8 inputs, int32 accumulators.
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// instruction descriptor: D s32, A s8, B s8, both K-major, M x N
__host__ __device__ constexpr uint32_t umma_idesc_i8(int M, int N) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

template <int BN>
__global__ void __launch_bounds__(I8_THREADS, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmEpilogue ep,
               const float *__restrict__ row_scale, const float *__restrict__ col_scale, const int M, const int N, const int K,
               int *status) {
    using Cfg = I8Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *tiles = smem;
    float *epi_stage = reinterpret_cast<float *>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
    uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + Cfg::STAGES * Cfg::STAGE_BYTES + Cfg::EPI_BYTES);
    uint64_t *empty_bar = full_bar + Cfg::STAGES;
    uint64_t *acc_full = empty_bar + Cfg::STAGES;      // [2] MMA -> epilogue
    uint64_t *acc_empty = acc_full + 2;                // [2] epilogue -> MMA
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_k = K / I8_BK;
    const GemmUnits units(M, N, BN, gridDim.x);
    const int total = units.total;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        for (int s = 0; s < Cfg::STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], I8_EPI_WARPS); }
        mbar_fence_init();
    }
    if (warp == 1) { tc_alloc(tmem_slot, Cfg::TMEM_COLS); tc_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------- TMA producer
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x) {
            int m0, n0, width;
            units.at(tile, BN, m0, n0, width);               // a strip still loads BN rows of B: the MMAs read the first `width`
            for (int kb = 0; kb < num_k; kb++, it++) {
                const int s = it % Cfg::STAGES;
                const uint32_t ph = (it / Cfg::STAGES) & 1;
                if (!mbar_wait(&empty_bar[s], ph ^ 1)) { ok = false; break; }
                uint8_t *st = tiles + s * Cfg::STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
                tma_load_2d(st, &tmA, kb * I8_BK, m0, &full_bar[s]);
                tma_load_2d(st + Cfg::A_BYTES, &tmB, kb * I8_BK, n0, &full_bar[s]);
            }
        }
        if (!ok) {
            atomicExch(status, ST_TIMEOUT_PRODUCER);
            // let copies already in flight land before the CTA's shared memory goes away
            for (int j = it > Cfg::STAGES ? it - Cfg::STAGES : 0; j < it; j++)
                mbar_wait(&full_bar[j % Cfg::STAGES], (j / Cfg::STAGES) & 1);
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------ MMA issuer
        int it = 0, lt = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total && ok; tile += gridDim.x, lt++) {
            int m0, n0, width;
            units.at(tile, BN, m0, n0, width);
            const uint32_t idesc = umma_idesc_i8(GEMM_BM, width);
            const int buf = lt & 1;
            const uint32_t acc = tmem_base + buf * BN;
            if (!mbar_wait(&acc_empty[buf], ((lt >> 1) & 1) ^ 1)) { ok = false; break; }
            tc_fence_after();
            for (int kb = 0; kb < num_k; kb++, it++) {
                const int s = it % Cfg::STAGES;
                const uint32_t ph = (it / Cfg::STAGES) & 1;
                if (!mbar_wait(&full_bar[s], ph)) { ok = false; break; }
                tc_fence_after();
                const uint32_t a = smem_u32(tiles + s * Cfg::STAGE_BYTES);
                const uint32_t b = a + Cfg::A_BYTES;
#pragma unroll
                for (int kk = 0; kk < I8_BK / 32; kk++) {
                    const uint32_t off = kk * 32;   // 32 int8 = 32 bytes inside the swizzle atom
                    tc_mma_i8(acc, umma_desc_sw128(a + off), umma_desc_sw128(b + off), idesc, (kb | kk) != 0);
                }
                tc_commit(&empty_bar[s]);           // frees the stage once these MMAs have read it
            }
            tc_commit(&acc_full[buf]);              // accumulator complete (or abandoned)
        }
        if (!ok) atomicExch(status, ST_TIMEOUT_MMA);
    } else if (warp >= 2) {
        // -------------------------------------------------------------- epilogue
        const int lg = warp & 3;                       // TMEM lane group this warp may read
        const int half = (warp - 2) >> 2;              // even or odd 32-column chunks of the tile
        const int row = lg * 32 + lane;
        int lt = 0;
        bool fits = true;
        // the block form pays when a CTA walks several tiles (stores set the pace); with one tile per CTA the run is
        // latency-bound and the shorter row form is used. Both produce the same bits.
        const bool blk_ok = Cfg::BLOCK_EPILOGUE && gemm_block_ok(ep) && total > (int)gridDim.x;
        float *stage = epi_stage + (warp - 2) * GEMM_BLOCK_STAGE_FLOATS;
        for (int tile = blockIdx.x; tile < total; tile += gridDim.x, lt++) {
            int m0, n0, width;
            units.at(tile, BN, m0, n0, width);
            const int buf = lt & 1;
            const uint32_t acc = tmem_base + buf * BN + ((uint32_t)(lg * 32) << 16);
            if (!mbar_wait(&acc_full[buf], (lt >> 1) & 1)) {
                if (lane == 0) atomicExch(status, ST_TIMEOUT_EPILOGUE);
                break;
            }
            tc_fence_after();
            const int m = m0 + row;
            const float sx = m < M ? row_scale[m] : 0.0f;
            if (num_k > 0) {
#pragma unroll 1
                for (int c = half; c < width / 32; c += 2) {
                    const int nb = n0 + c * 32;
                    const bool blk = blk_ok && nb + 32 <= N;            // warp-uniform
                    if (blk && m0 + lg * 32 >= M) continue;             // none of this warp's 32 rows exists
                    float4 res[8];
                    if (blk) gemm_block_prefetch(ep, m0 + lg * 32, M, nb, lane, res);
                    if (blk) {
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            float v[16];
                            tc_ld16(acc + (uint32_t)(c * 32 + h * 16), v);
                            tc_wait_ld();
#pragma unroll
                            for (int j = 0; j < 16; j++)     // (float)int32 * ws * sx, left to right (src/qmat.c:299)
                                v[j] = __fmul_rn(__fmul_rn(__int2float_rn(__float_as_int(v[j])), col_scale[nb + h * 16 + j]), sx);
                            gemm_block_stage(v, h, stage, lane);
                        }
                        fits &= gemm_block_store(ep, res, m0 + lg * 32, M, nb, stage, lane);
                        continue;
                    }
                    float v[32];
                    tc_ld32(acc + (uint32_t)(c * 32), v);
                    tc_wait_ld();
                    if (m < M && nb < N) {
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            // (float)int32 * ws * sx, left to right (src/qmat.c:299)
                            const float ws = nb + j < N ? col_scale[nb + j] : 0.0f;
                            v[j] = __fmul_rn(__fmul_rn(__int2float_rn(__float_as_int(v[j])), ws), sx);
                        }
                        fits &= gemm_epilogue_row(ep, v, m, nb, N);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
        if (!fits) atomicCAS(status, ST_OK, ST_RANGE);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tc_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn i8_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// int8 [rows, K] row-major with row stride ld bytes: box = 128 bytes (K) x box_rows, 128B swizzle.
static int i8_make_map(CUtensorMap *m, const int8_t *base, int rows, int K, int ld, int box_rows) {
    EncodeTiledFn fn = i8_encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled entry point unavailable"); return -1; }
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld % 16) != 0) {
        set_error("gemm_i8: operand base/stride not 16-byte aligned");
        return -1;
    }
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld};
    cuuint32_t box[2] = {(cuuint32_t)I8_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d)", (int)r); return -1; }
    return 0;
}

template <int BN>
static int i8_launch(const int8_t *a, int lda, const float *row_scale, const int8_t *b, int ldb, const float *col_scale,
                     const GemmEpilogue &ep, int M, int N, int K, int *status, cudaStream_t stream) {
    using Cfg = I8Cfg<BN>;
    CUtensorMap ta, tb;
    if (i8_make_map(&ta, a, M, K, lda, GEMM_BM)) return -1;
    if (i8_make_map(&tb, b, N, K, ldb, BN)) return -1;
    static PerDevice configured = {};
    int dev = 0;
    if (configured.below(Cfg::SMEM_BYTES, &dev)) {
        MB_CUDA(cudaFuncSetAttribute(gemm_i8_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        configured.record(dev, Cfg::SMEM_BYTES);
    }
    const int sms = device_sm_count();
    // fewer tiles than SMs: the kernel cuts them into column strips (GemmUnits) when the grid leaves room
    const int total = cdiv(N, BN) * cdiv(M, GEMM_BM), strips = BN % 128 == 0 ? 4 : BN % 64 == 0 ? 2 : 1;
    dim3 grid(total >= sms ? sms : total * strips <= sms ? total * strips : total * 2 <= sms && strips >= 2 ? total * 2 : total);
    gemm_i8_kernel<BN><<<grid, I8_THREADS, Cfg::SMEM_BYTES, stream>>>(ta, tb, ep, row_scale, col_scale, M, N, K, status);
    MB_CUDA(cudaGetLastError());
    return 0;
}

int gemm_i8(const int8_t *a, int lda, const float *row_scale, const int8_t *b, int ldb, const float *col_scale,
            const GemmEpilogue &ep, int M, int N, int K, int *status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % I8_BK != 0) { set_error("gemm_i8: K=%d must be a positive multiple of %d", K, I8_BK); return -1; }
    if (!row_scale || !col_scale) { set_error("gemm_i8: scales missing"); return -1; }
    const int sms = device_sm_count();
    // tile width by waves x time of one tile, as for the fp16 contraction (an output element sees the same
    // integers whatever the width)
    const int tm = cdiv(M, GEMM_BM);
    int bn = 256;
    long best = -1;
    for (int cand = 256; cand >= 32; cand >>= 1) {
        const long cost = (long)cdiv(tm * cdiv(N, cand), sms) * (cand + 48);
        if (best < 0 || cost < best) { best = cost; bn = cand; }
    }
    if (bn == 256) return i8_launch<256>(a, lda, row_scale, b, ldb, col_scale, ep, M, N, K, status, stream);
    if (bn == 128) return i8_launch<128>(a, lda, row_scale, b, ldb, col_scale, ep, M, N, K, status, stream);
    if (bn == 64) return i8_launch<64>(a, lda, row_scale, b, ldb, col_scale, ep, M, N, K, status, stream);
    return i8_launch<32>(a, lda, row_scale, b, ldb, col_scale, ep, M, N, K, status, stream);
}

}  // namespace mb
