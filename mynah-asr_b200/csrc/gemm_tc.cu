// Dense contraction C[M,N] = A[M,K] * B[N,K]^T on the 5th-generation tensor cores.
//
// This is the large-M half of the quantised matmul (the reference's
// mynah_asr_qmat_mul, src/qmat.c:503-651, and mynah_asr_gemm_wt, src/backend.c:68-81):
// weights arrive already decoded to fp16 (hi, lo) planes resident in HBM, activations
// as fp16 (hi, lo) planes written by the producing kernel's epilogue.
//
//   * TMA (cp.async.bulk.tensor.2d, 128-byte swizzle, every CTA loads its own tiles) stages 128 x 64
//     A tiles and BN x 64 B tiles into a shared-memory ring guarded by mbarriers;
//   * one elected thread issues tcgen05.mma (kind::f16, M=128, N=BN, K=16) into TMEM
//     accumulators; with NTERMS=3 every k-step issues hi*hi into one accumulator and
//     lo*hi + hi*lo into a second one (the lo planes are pre-scaled by 2^11, the
//     epilogue adds the second accumulator back times 2^-11), so the product carries
//     ~22 significant bits per operand (f32-grade parity with the reference's sgemm);
//     with NTERMS=1 only hi*hi (fast mode);
//   * the kernel is persistent (one CTA per SM walks the output tiles) and the
//     accumulators are double-buffered in TMEM, so the epilogue of one tile overlaps
//     the MMAs of the next; eight epilogue warps read the accumulator with tcgen05.ld
//     and apply the fused tail: + bias, SiLU / ReLU, then either store f32, accumulate into the residual
//     stream (x += alpha * y), or store the result as fp16 (hi, lo) planes for the
//     next contraction.
//
// Row stability: an output row depends only on its own A row and on B; the k order
// and the instruction sequence are the same for every tile position and every M, so
// a row's bits do not depend on what else is in the batch.
#include "gemm.h"

namespace mb {

static constexpr int BM = GEMM_BM;
static constexpr int BK = 64;
static constexpr int EPI_WARPS = 8;
static constexpr int GEMM_THREADS = (2 + EPI_WARPS) * 32;   // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue
static constexpr int SMEM_LIMIT = 232448;  // 227 KB

template <int BN, int NTERMS>
struct GemmCfg {
    static constexpr int NPLANES = NTERMS == 1 ? 1 : 2;
    static constexpr int A_BYTES = BM * BK * 2;
    static constexpr int B_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = NPLANES * (A_BYTES + B_BYTES);
    // the epilogue warps' turning buffers: only the wide tiles have them — the narrow ones serve contractions with few
    // rows, which are latency-bound and want every stage of the operand ring instead
    static constexpr bool BLOCK_EPILOGUE = BN >= 128;
    static constexpr int EPI_BYTES = BLOCK_EPILOGUE ? EPI_WARPS * GEMM_BLOCK_STAGE_FLOATS * 4 : 0;
    static constexpr int STAGES_RAW = (SMEM_LIMIT - 2048 - EPI_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 6 ? 6 : STAGES_RAW;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 2048;
    // NTERMS == 3 keeps a second accumulator for the cross terms (lo*hi + hi*lo);
    // everything is double-buffered so the epilogue of tile i overlaps the MMAs of tile i+1
    static constexpr int ACC_COLS = NTERMS == 1 ? BN : 2 * BN;
    static constexpr int TMEM_COLS = 2 * ACC_COLS < 32 ? 32 : 2 * ACC_COLS;
    static_assert(TMEM_COLS <= 512, "TMEM has 512 columns");
};

// Persistent kernel: one CTA per SM walks the output tiles (n fastest, so the CTAs in
// flight share a few A row-blocks while B stays L2-resident).
template <int BN, int NTERMS>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA_hi, const __grid_constant__ CUtensorMap tmA_lo,
               const __grid_constant__ CUtensorMap tmB_hi, const __grid_constant__ CUtensorMap tmB_lo,
               const GemmEpilogue ep, const int M, const int N, const int K, int *status) {
    using Cfg = GemmCfg<BN, NTERMS>;
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
    const int num_k = K / BK;
    const GemmUnits units(M, N, BN, gridDim.x);
    const int total = units.total;

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA_hi);
        tma_prefetch_desc(&tmB_hi);
        if (NTERMS > 1) { tma_prefetch_desc(&tmA_lo); tma_prefetch_desc(&tmB_lo); }
        for (int s = 0; s < Cfg::STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; b++) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], EPI_WARPS); }
        mbar_fence_init();
    }
    if (warp == 1) { tc_alloc(tmem_slot, Cfg::TMEM_COLS); tc_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------- TMA producer
        int it = 0;                                    // k-blocks issued so far (ring position)
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
                tma_load_2d(st, &tmA_hi, kb * BK, m0, &full_bar[s]);
                if (NTERMS > 1) tma_load_2d(st + Cfg::A_BYTES, &tmA_lo, kb * BK, m0, &full_bar[s]);
                uint8_t *bt = st + Cfg::NPLANES * Cfg::A_BYTES;
                tma_load_2d(bt, &tmB_hi, kb * BK, n0, &full_bar[s]);
                if (NTERMS > 1) tma_load_2d(bt + Cfg::B_BYTES, &tmB_lo, kb * BK, n0, &full_bar[s]);
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
            const uint32_t idesc = umma_idesc_f16(BM, width);
            const int buf = lt & 1;
            const uint32_t acc = tmem_base + buf * Cfg::ACC_COLS;
            // the epilogue must have drained this accumulator (two tiles ago)
            if (!mbar_wait(&acc_empty[buf], ((lt >> 1) & 1) ^ 1)) { ok = false; break; }
            tc_fence_after();
            for (int kb = 0; kb < num_k; kb++, it++) {
                const int s = it % Cfg::STAGES;
                const uint32_t ph = (it / Cfg::STAGES) & 1;
                if (!mbar_wait(&full_bar[s], ph)) { ok = false; break; }
                tc_fence_after();
                const uint32_t a_hi = smem_u32(tiles + s * Cfg::STAGE_BYTES);
                const uint32_t a_lo = a_hi + Cfg::A_BYTES;
                const uint32_t b_hi = a_hi + Cfg::NPLANES * Cfg::A_BYTES;
                const uint32_t b_lo = b_hi + Cfg::B_BYTES;
#pragma unroll
                for (int kk = 0; kk < BK / 16; kk++) {
                    const uint32_t off = kk * 32;   // 16 fp16 = 32 bytes inside the swizzle atom
                    tc_mma_f16(acc, umma_desc_sw128(a_hi + off), umma_desc_sw128(b_hi + off), idesc, (kb | kk) != 0);
                    if (NTERMS > 1) {
                        tc_mma_f16(acc + BN, umma_desc_sw128(a_lo + off), umma_desc_sw128(b_hi + off), idesc,
                                   (kb | kk) != 0);
                        tc_mma_f16(acc + BN, umma_desc_sw128(a_hi + off), umma_desc_sw128(b_lo + off), idesc, 1);
                    }
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
            const uint32_t acc = tmem_base + buf * Cfg::ACC_COLS + ((uint32_t)(lg * 32) << 16);
            if (!mbar_wait(&acc_full[buf], (lt >> 1) & 1)) {
                if (lane == 0) atomicExch(status, ST_TIMEOUT_EPILOGUE);
                break;
            }
            tc_fence_after();
            const int m = m0 + row;
            if (num_k > 0) {
#pragma unroll 1
                for (int c = half; c < width / 32; c += 2) {
                    const int nb = n0 + c * 32;
                    const bool blk = blk_ok && nb + 32 <= N;            // warp-uniform
                    if (blk && m0 + lg * 32 >= M) continue;             // none of this warp's 32 rows exists
                    float4 res[8];
                    if (blk) gemm_block_prefetch(ep, m0 + lg * 32, M, nb, lane, res);
                    if (blk) {
                        // two halves of 16 columns: fewer live registers than the whole 32 x (hi*hi, cross) at once
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            float v[16];
                            tc_ld16(acc + (uint32_t)(c * 32 + h * 16), v);
                            if (NTERMS > 1) {
                                float x[16];
                                tc_ld16(acc + (uint32_t)(BN + c * 32 + h * 16), x);
                                tc_wait_ld();
#pragma unroll
                                for (int j = 0; j < 16; j++) v[j] = fmaf(x[j], H16_LO_INV, v[j]);
                            } else {
                                tc_wait_ld();
                            }
                            gemm_block_stage(v, h, stage, lane);
                        }
                        fits &= gemm_block_store(ep, res, m0 + lg * 32, M, nb, stage, lane);
                        continue;
                    }
                    float v[32];
                    tc_ld32(acc + (uint32_t)(c * 32), v);
                    if (NTERMS > 1) {
                        float x[32];
                        tc_ld32(acc + (uint32_t)(BN + c * 32), x);
                        tc_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; j++) v[j] = fmaf(x[j], H16_LO_INV, v[j]);
                    } else {
                        tc_wait_ld();
                    }
                    if (m < M && nb < N) {
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

static EncodeTiledFn encode_fn() {
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

// fp16 [rows, K] row-major with row stride ld (halves): box = 64 (K) x box_rows, 128B swizzle.
static int make_map(CUtensorMap *m, const __half *base, int rows, int K, int ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled entry point unavailable"); return -1; }
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld % 8) != 0) {
        set_error("gemm_tc: operand base/stride not 16-byte aligned");
        return -1;
    }
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d)", (int)r); return -1; }
    return 0;
}

template <int BN, int NTERMS>
static int launch(const GemmOperand &A, const GemmOperand &B, const GemmEpilogue &ep, int M, int N, int K,
                  int *status, cudaStream_t stream) {
    using Cfg = GemmCfg<BN, NTERMS>;
    CUtensorMap ta_hi, ta_lo, tb_hi, tb_lo;
    if (make_map(&ta_hi, A.hi, M, K, A.ld, BM)) return -1;
    if (make_map(&tb_hi, B.hi, N, K, B.ld, BN)) return -1;
    if (NTERMS > 1) {
        if (make_map(&ta_lo, A.lo, M, K, A.ld, BM)) return -1;
        if (make_map(&tb_lo, B.lo, N, K, B.ld, BN)) return -1;
    } else {
        ta_lo = ta_hi; tb_lo = tb_hi;
    }
    static PerDevice configured = {};
    int dev = 0;
    if (configured.below(Cfg::SMEM_BYTES, &dev)) {
        MB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN, NTERMS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Cfg::SMEM_BYTES));
        configured.record(dev, Cfg::SMEM_BYTES);
    }
    const int sms = device_sm_count();
    // fewer tiles than SMs: the kernel cuts them into column strips (GemmUnits) when the grid leaves room
    const int total = cdiv(N, BN) * cdiv(M, BM), strips = BN % 128 == 0 ? 4 : BN % 64 == 0 ? 2 : 1;
    dim3 grid(total >= sms ? sms : total * strips <= sms ? total * strips : total * 2 <= sms && strips >= 2 ? total * 2 : total);
    gemm_tc_kernel<BN, NTERMS><<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(ta_hi, ta_lo, tb_hi, tb_lo, ep, M,
                                                                               N, K, status);
    MB_CUDA(cudaGetLastError());
    return 0;
}

int gemm_tc(const GemmOperand &A, const GemmOperand &B, const GemmEpilogue &ep, int M, int N, int K, int nterms,
            int *status, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % BK != 0) { set_error("gemm_tc: K=%d must be a positive multiple of %d", K, BK); return -1; }
    if (nterms != 1 && (!A.lo || !B.lo)) { set_error("gemm_tc: 3-term mode needs lo planes"); return -1; }
    // Narrower N tiles when the output has too few 128-wide tiles to occupy the SMs (small M: decoder
    // positions, streaming chunks): more CTAs pull the operands. An output element sees the same k order
    // and the same instruction sequence whatever the tile width, so its bits do not change with it.
    const int sms = device_sm_count();
    // waves of CTAs x time of one tile (the MMAs scale with the tile width, prologue and epilogue do not)
    const int tm = cdiv(M, BM);
    int bn = 128;
    long best = -1;
    for (int cand = 128; cand >= 32; cand >>= 1) {
        const long cost = (long)cdiv(tm * cdiv(N, cand), sms) * (cand + 48);
        if (best < 0 || cost < best) { best = cost; bn = cand; }
    }
    if (nterms == 1) {
        if (bn == 128 && N >= 256) return launch<256, 1>(A, B, ep, M, N, K, status, stream);
        if (bn == 128) return launch<128, 1>(A, B, ep, M, N, K, status, stream);
        if (bn == 64) return launch<64, 1>(A, B, ep, M, N, K, status, stream);
        return launch<32, 1>(A, B, ep, M, N, K, status, stream);
    }
    if (!A.lo || !B.lo) { set_error("gemm_tc: 3-term mode needs lo planes"); return -1; }
    if (bn == 128) return launch<128, 3>(A, B, ep, M, N, K, status, stream);
    if (bn == 64) return launch<64, 3>(A, B, ep, M, N, K, status, stream);
    return launch<32, 3>(A, B, ep, M, N, K, status, stream);
}

}  // namespace mb
