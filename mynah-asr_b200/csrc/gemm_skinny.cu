// Contraction for a handful of rows: out[m, n] = sum_k X[m, k] W[n, k], 128 rows per launch at most — the linears of one
// decoder position (mynah_asr_aed_decode, src/decoder_aed.c:183-228, calls mynah_asr_qmat_mul with one row per
// utterance) and of a streaming step of a small stream group (mynah_asr_enc_stream_step, src/encoder.c:826-866).
//
// With so few rows the work is streaming W once; the output has too few 128-wide tiles to occupy the device, and a
// tile of the large-M kernel would spend most of its TMA traffic on zero-filled activation rows. So the roles are
// swapped: 128 rows of W are the M side of tcgen05.mma (kind::f16, M = 128, N = NB = the rows of X rounded up to 32),
// the accumulator holds out^T (lane = n, column = m), and stores run along n (one 128-byte line per warp store).
// K is cut into S slices handled by the S CTAs of a thread-block cluster, so that tiles x S CTAs pull the weights;
// each CTA leaves its slice's sums in its own shared memory, and after a cluster barrier CTA r adds the S slices
// of rows m = r, r + S, ... in slice order through distributed shared memory and applies the fused tail. The order of
// the additions is fixed by the slice index and S depends only on the weight's shape, so an output row's bits do not
// depend on how many rows share the launch. Operands are the same fp16 (hi, lo) planes and the same three products
// per term (one in fast mode) as in gemm_tc.cu. No multicast; every CTA loads its own tiles.
// The kernel is launched chained (common.cuh): its first ring of weight tiles is requested before it waits for the
// kernel in front of it. Optionally the rows it completes are layer-normalised on the spot (GemmEpilogue::ln_*): per-row
// counters tell the warp that stores a row's last tile, and that warp normalises the row.
#include "gemm.h"
#include "ln_row.cuh"

namespace mb {

static constexpr int SK_BK = 64;
static constexpr int SK_ROWS = 128;                       // rows of W per tile (MMA M)
static constexpr int SK_THREADS = 6 * 32;                 // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
static constexpr int SK_SMEM_LIMIT = 232448;

template <int NB, int NTERMS>
struct SkinnyCfg {
    static constexpr int NPLANES = NTERMS == 1 ? 1 : 2;
    static constexpr int W_BYTES = SK_ROWS * SK_BK * 2;
    static constexpr int X_BYTES = NB * SK_BK * 2;
    static constexpr int STAGE_BYTES = NPLANES * (W_BYTES + X_BYTES);
    static constexpr int PART_BYTES = NB * SK_ROWS * 4;       // this CTA's slice sums, [m][n]
    static constexpr int STAGES_RAW = (SK_SMEM_LIMIT - 2048 - PART_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + PART_BYTES + 2048;
    static constexpr int ACC_COLS = NTERMS == 1 ? NB : 2 * NB;
    static constexpr int TMEM_COLS = ACC_COLS < 32 ? 32 : ACC_COLS;
    static_assert(STAGES >= 2, "at least two stages");
};

// hardware barrier over every thread of the cluster (no spinning in software; every thread of every CTA reaches it on
// every path through the kernel)
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of CTA `rank`'s copy of a shared-memory location of this CTA, and a load through such an address
__device__ __forceinline__ uint32_t cluster_addr(const float *own, uint32_t rank) {
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(own)), "r"(rank));
    return ra;
}
__device__ __forceinline__ float ld_cluster_at(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));      // volatile: stays behind the cluster barrier
    return v;
}

// fused tail for one element (the per-element operations and their order are those of gemm_epilogue_row)
__device__ __forceinline__ bool skinny_store(const GemmEpilogue &ep, float x, float bias, int m, int n) {
    x += bias;
    x = gemm_act(ep, x);
    bool fits = true;
    if (ep.mode != OUT_H16) {
        float *o = ep.out + (size_t)m * ep.ldo + n;
        if (ep.mode == OUT_RESID) *o += ep.alpha * x;
        else *o = x;
    }
    if (ep.mode == OUT_H16 || ep.mode == OUT_F32_H16) {
        __half h, l;
        fits = split_h16(x, h, l);
        ep.out_hi[(size_t)m * ep.ldh + n] = h;
        if (ep.out_lo) ep.out_lo[(size_t)m * ep.ldh + n] = l;
    }
    return fits;
}

// LayerNorm(s) of row m of ep.out (width N = NV * 128) by one warp, as GemmEpilogue describes them
template <int NV>
__device__ __forceinline__ void ln_tail_nv(const GemmEpilogue &ep, int m, int lane) {
    if (ep.ln2_w) {
        ln_row<NV, true>(ep.out, ep.ln_w, ep.ln_b, ep.out, nullptr, nullptr, nullptr, nullptr, m, ACT_NONE, lane);
        __syncwarp();                                             // every lane reads back what it wrote itself
        ln_row<NV, true>(ep.out, ep.ln2_w, ep.ln2_b, nullptr, ep.ln_hi, ep.ln_lo, nullptr, nullptr, m, ACT_NONE, lane);
    } else {
        ln_row<NV, true>(ep.out, ep.ln_w, ep.ln_b, ep.ln_hi ? nullptr : ep.out, ep.ln_hi, ep.ln_lo, nullptr, nullptr, m, ACT_NONE, lane);
    }
}
__device__ __forceinline__ void ln_tail(const GemmEpilogue &ep, int N, int m, int lane) {
    switch (N) {
        case 128: ln_tail_nv<1>(ep, m, lane); break;
        case 256: ln_tail_nv<2>(ep, m, lane); break;
        case 512: ln_tail_nv<4>(ep, m, lane); break;
        case 640: ln_tail_nv<5>(ep, m, lane); break;
        case 1024: ln_tail_nv<8>(ep, m, lane); break;
        case 2048: ln_tail_nv<16>(ep, m, lane); break;
        default: break;                                           // the host does not ask for the tail at other widths
    }
}
// widths ln_tail serves
bool gemm_skinny_ln_width(int d) { return d == 128 || d == 256 || d == 512 || d == 640 || d == 1024 || d == 2048; }

// LayerNorm of the rows this launch completes. Called by the four epilogue warps of a CTA after they have stored their
// 128 columns of rows first, first + step, ...: every CTA counts in on each of its rows; the warp that brings a row's
// count to the number of tiles normalises it (its reads go to the L2, where the other CTAs' stores are).
__device__ __forceinline__ void ln_finished_rows(const GemmEpilogue &ep, int N, int Mb, int first, int step, int tiles, int w, int lane) {
    __threadfence();
    asm volatile("bar.sync 1, 128;" ::: "memory");                // the four epilogue warps: all columns of this CTA's rows are out
    for (int m = first + w * step; m < Mb; m += 4 * step) {
        int last = 0;
        if (lane == 0) last = atomicAdd(ep.ln_count + m, 1) == tiles - 1;
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
            __threadfence();
            if (lane == 0) ep.ln_count[m] = 0;                    // ready for the next launch
            ln_tail(ep, N, m, lane);
        }
    }
}

// grid = tiles * S CTAs in clusters of S; CTA = (tile of 128 W rows, K slice)
template <int NB, int NTERMS>
__global__ void __launch_bounds__(SK_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmW_hi, const __grid_constant__ CUtensorMap tmW_lo,
                   const __grid_constant__ CUtensorMap tmX_hi, const __grid_constant__ CUtensorMap tmX_lo,
                   const GemmEpilogue ep, const int Mb, const int N, const int K, const int S, int *status) {
    using Cfg = SkinnyCfg<NB, NTERMS>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *tiles = smem;
    float *part = reinterpret_cast<float *>(smem + Cfg::STAGES * Cfg::STAGE_BYTES);
    uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + Cfg::STAGES * Cfg::STAGE_BYTES + Cfg::PART_BYTES);
    uint64_t *empty_bar = full_bar + Cfg::STAGES;
    uint64_t *acc_full = empty_bar + Cfg::STAGES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x / S, slice = blockIdx.x % S;      // slice == rank in the cluster (clusters of S along x)
    const int n0 = tile * SK_ROWS;
    const int num_k = K / SK_BK / S, kb0 = slice * num_k;

    chain_trigger();
    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmW_hi);
        tma_prefetch_desc(&tmX_hi);
        if (NTERMS > 1) { tma_prefetch_desc(&tmW_lo); tma_prefetch_desc(&tmX_lo); }
        for (int s = 0; s < Cfg::STAGES; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(acc_full, 1);
        mbar_fence_init();
    }
    if (warp == 1) { tc_alloc(tmem_slot, Cfg::TMEM_COLS); tc_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------- TMA producer
        bool ok = true;
        // the weights do not depend on the kernels before this one: the first ring of W tiles is under way before
        // chain_wait() lets the activation rows be read
        const int pre = num_k < Cfg::STAGES ? num_k : Cfg::STAGES;
        for (int it = 0; it < pre; it++) {
            uint8_t *st = tiles + it * Cfg::STAGE_BYTES;
            const int k = (kb0 + it) * SK_BK;
            mbar_expect_tx(&full_bar[it], Cfg::STAGE_BYTES);
            tma_load_2d(st, &tmW_hi, k, n0, &full_bar[it]);
            if (NTERMS > 1) tma_load_2d(st + Cfg::W_BYTES, &tmW_lo, k, n0, &full_bar[it]);
        }
        chain_wait();
        for (int it = 0; it < pre; it++) {
            uint8_t *xt = tiles + it * Cfg::STAGE_BYTES + Cfg::NPLANES * Cfg::W_BYTES;
            const int k = (kb0 + it) * SK_BK;
            tma_load_2d(xt, &tmX_hi, k, 0, &full_bar[it]);
            if (NTERMS > 1) tma_load_2d(xt + Cfg::X_BYTES, &tmX_lo, k, 0, &full_bar[it]);
        }
        int it = pre;
        for (; it < num_k; it++) {
            const int s = it % Cfg::STAGES;
            const uint32_t ph = (it / Cfg::STAGES) & 1;
            if (!mbar_wait(&empty_bar[s], ph ^ 1)) { ok = false; break; }
            uint8_t *st = tiles + s * Cfg::STAGE_BYTES;
            const int k = (kb0 + it) * SK_BK;
            mbar_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
            tma_load_2d(st, &tmW_hi, k, n0, &full_bar[s]);
            if (NTERMS > 1) tma_load_2d(st + Cfg::W_BYTES, &tmW_lo, k, n0, &full_bar[s]);
            uint8_t *xt = st + Cfg::NPLANES * Cfg::W_BYTES;
            tma_load_2d(xt, &tmX_hi, k, 0, &full_bar[s]);
            if (NTERMS > 1) tma_load_2d(xt + Cfg::X_BYTES, &tmX_lo, k, 0, &full_bar[s]);
        }
        if (!ok) {
            atomicExch(status, ST_TIMEOUT_PRODUCER);
            for (int j = it > Cfg::STAGES ? it - Cfg::STAGES : 0; j < it; j++)     // copies in flight land first
                mbar_wait(&full_bar[j % Cfg::STAGES], (j / Cfg::STAGES) & 1);
        }
    } else if (warp == 1 && lane == 0) {
        // ------------------------------------------------------------ MMA issuer
        const uint32_t idesc = umma_idesc_f16(SK_ROWS, NB);
        bool ok = true;
        for (int it = 0; it < num_k; it++) {
            const int s = it % Cfg::STAGES;
            const uint32_t ph = (it / Cfg::STAGES) & 1;
            if (!mbar_wait(&full_bar[s], ph)) { ok = false; break; }
            tc_fence_after();
            const uint32_t w_hi = smem_u32(tiles + s * Cfg::STAGE_BYTES);
            const uint32_t w_lo = w_hi + Cfg::W_BYTES;
            const uint32_t x_hi = w_hi + Cfg::NPLANES * Cfg::W_BYTES;
            const uint32_t x_lo = x_hi + Cfg::X_BYTES;
#pragma unroll
            for (int kk = 0; kk < SK_BK / 16; kk++) {
                const uint32_t off = kk * 32;
                // the same three products as the large-M kernel, with the operand roles swapped: x * w
                tc_mma_f16(tmem_base, umma_desc_sw128(w_hi + off), umma_desc_sw128(x_hi + off), idesc, (it | kk) != 0);
                if (NTERMS > 1) {
                    tc_mma_f16(tmem_base + NB, umma_desc_sw128(w_hi + off), umma_desc_sw128(x_lo + off), idesc, (it | kk) != 0);
                    tc_mma_f16(tmem_base + NB, umma_desc_sw128(w_lo + off), umma_desc_sw128(x_hi + off), idesc, 1);
                }
            }
            tc_commit(&empty_bar[s]);
        }
        tc_commit(acc_full);
        if (!ok) atomicExch(status, ST_TIMEOUT_MMA);
    } else if (warp >= 2) {
        // ------------------------------------------------- epilogue, first half: this slice's sums
        const int lg = warp & 3;                                  // TMEM lane group of this warp
        const int nl = lg * 32 + lane;
        const uint32_t acc = tmem_base + ((uint32_t)(lg * 32) << 16);
        const bool have = mbar_wait(acc_full, 0);
        if (!have && lane == 0) atomicExch(status, ST_TIMEOUT_EPILOGUE);
        tc_fence_after();
        chain_wait();                                             // before the residual is read or anything is written
#pragma unroll 1
        for (int c = 0; c < NB / 32; c++) {
            float v[32];
            if (have && num_k > 0) {
                tc_ld32(acc + (uint32_t)(c * 32), v);
                if (NTERMS > 1) {
                    float x[32];
                    tc_ld32(acc + (uint32_t)(NB + c * 32), x);
                    tc_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; j++) v[j] = fmaf(x[j], H16_LO_INV, v[j]);
                } else {
                    tc_wait_ld();
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++) v[j] = 0.0f;
            }
#pragma unroll
            for (int j = 0; j < 32; j++) part[(c * 32 + j) * SK_ROWS + nl] = v[j];
        }
    }
    tc_fence_before();
    __syncthreads();
    if (S == 1) {
        if (warp >= 2) {                                          // a single slice: the fused tail straight from this CTA's sums
            const int nl = (warp - 2) * 32 + lane, n = n0 + nl;
            const float bias = ep.bias && n < N ? ep.bias[n] : 0.0f;
            bool fits = true;
            if (n < N)
                for (int m = 0; m < Mb; m++) fits &= skinny_store(ep, part[m * SK_ROWS + nl], bias, m, n);
            if (!fits) atomicCAS(status, ST_OK, ST_RANGE);
            if (ep.ln_w) ln_finished_rows(ep, N, Mb, 0, 1, (int)gridDim.x, warp - 2, lane);
        }
    } else {
        cluster_barrier();                                        // every slice's sums are in place
        if (warp >= 2) {
            // -------------------------------------------- second half: rows m = slice, slice + S, ... of this tile
            const int nl = (warp - 2) * 32 + lane, n = n0 + nl;
            const float bias = ep.bias && n < N ? ep.bias[n] : 0.0f;
            bool fits = true;
            // the S remote reads of a row are all issued before the first addition (S <= 8), two rows at a time
            uint32_t base[8];
#pragma unroll
            for (int s = 0; s < 8; s++) base[s] = cluster_addr(part + nl, (uint32_t)(s < S ? s : 0));
            for (int m = slice; m < Mb; m += 2 * S) {
                const int m2 = m + S;
                float t[8], u[8];
#pragma unroll
                for (int s = 0; s < 8; s++) {
                    if (s < S) {
                        t[s] = ld_cluster_at(base[s] + (uint32_t)(m * SK_ROWS * 4));
                        u[s] = m2 < Mb ? ld_cluster_at(base[s] + (uint32_t)(m2 * SK_ROWS * 4)) : 0.0f;
                    }
                }
                float x = t[0], y = u[0];
#pragma unroll
                for (int s = 1; s < 8; s++) if (s < S) { x += t[s]; y += u[s]; }
                if (n < N) {
                    fits &= skinny_store(ep, x, bias, m, n);
                    if (m2 < Mb) fits &= skinny_store(ep, y, bias, m2, n);
                }
            }
            if (!fits) atomicCAS(status, ST_OK, ST_RANGE);
            if (ep.ln_w) ln_finished_rows(ep, N, Mb, slice, S, (int)gridDim.x / S, warp - 2, lane);
        }
        cluster_barrier();                                        // nobody's shared memory goes away while it is read
    }
    if (warp == 1) tc_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn sk_encode_fn() {
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

static int sk_map(CUtensorMap *m, const __half *base, int rows, int K, int ld, int box_rows) {
    EncodeTiledFn fn = sk_encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled entry point unavailable"); return -1; }
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld % 8) != 0) { set_error("gemm_skinny: operand base/stride not 16-byte aligned"); return -1; }
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)SK_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed (%d)", (int)r); return -1; }
    return 0;
}

static int gemm_skinny_slices(int N, int K, int sms) {
    const int tiles = cdiv(N, SK_ROWS), num_k = K / SK_BK;
    int s = 1;
    while (s * 2 <= 8 && tiles * s * 2 <= sms && num_k % (s * 2) == 0) s *= 2;
    return s;
}

template <int NB, int NTERMS>
static int sk_launch(const GemmOperand &X, const GemmOperand &W, const GemmEpilogue &ep, int Mb, int N, int K, int *status,
                     cudaStream_t stream, bool chain) {
    using Cfg = SkinnyCfg<NB, NTERMS>;
    CUtensorMap tw_hi, tw_lo, tx_hi, tx_lo;
    if (sk_map(&tw_hi, W.hi, N, K, W.ld, SK_ROWS)) return -1;
    if (sk_map(&tx_hi, X.hi, Mb, K, X.ld, NB)) return -1;
    if (NTERMS > 1) {
        if (sk_map(&tw_lo, W.lo, N, K, W.ld, SK_ROWS)) return -1;
        if (sk_map(&tx_lo, X.lo, Mb, K, X.ld, NB)) return -1;
    } else {
        tw_lo = tw_hi; tx_lo = tx_hi;
    }
    static PerDevice configured = {};
    int dev = 0;
    if (configured.below(Cfg::SMEM_BYTES, &dev)) {
        MB_CUDA(cudaFuncSetAttribute(gemm_skinny_kernel<NB, NTERMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        configured.record(dev, Cfg::SMEM_BYTES);
    }
    const int S = gemm_skinny_slices(N, K, device_sm_count());
    MB_CUDA(launch_kernel(gemm_skinny_kernel<NB, NTERMS>, dim3((unsigned)(cdiv(N, SK_ROWS) * S)), dim3(SK_THREADS), Cfg::SMEM_BYTES, stream, chain, S,
                          tw_hi, tw_lo, tx_hi, tx_lo, ep, Mb, N, K, S, status));
    return 0;
}

int gemm_skinny(const GemmOperand &X, const GemmOperand &W, const GemmEpilogue &ep, int M, int N, int K, int nterms, int *status,
                cudaStream_t stream, bool chain) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % SK_BK != 0) { set_error("gemm_skinny: K=%d must be a positive multiple of %d", K, SK_BK); return -1; }
    if (nterms != 1 && (!X.lo || !W.lo)) { set_error("gemm_skinny: 3-term mode needs lo planes"); return -1; }
    if (ep.ln_w && (!ep.ln_b || !ep.ln_count || !ep.out || ep.mode == OUT_H16 || ep.ldo != N || !gemm_skinny_ln_width(N) ||
                    (ep.ln2_w && (!ep.ln2_b || !ep.ln_hi)))) {
        set_error("gemm_skinny: the LayerNorm tail needs an f32 output of row stride N = %d (a register-LayerNorm width), planes and counters", N);
        return -1;
    }
    // more than 128 rows: groups of 128 (a row's bits do not depend on the group it is in)
    for (int r = 0; r < M; r += 128) {
        const int mb = M - r < 128 ? M - r : 128;
        GemmOperand x{X.hi + (size_t)r * X.ld, X.lo ? X.lo + (size_t)r * X.ld : nullptr, X.ld};
        GemmEpilogue e = ep;
        if (e.out) e.out += (size_t)r * e.ldo;
        if (e.out_hi) e.out_hi += (size_t)r * e.ldh;
        if (e.out_lo) e.out_lo += (size_t)r * e.ldh;
        if (e.ln_w) { if (e.ln_hi) e.ln_hi += (size_t)r * N; if (e.ln_lo) e.ln_lo += (size_t)r * N; e.ln_count += r; }
        int rc;
        if (nterms == 1) rc = mb <= 32 ? sk_launch<32, 1>(x, W, e, mb, N, K, status, stream, chain) : mb <= 64 ? sk_launch<64, 1>(x, W, e, mb, N, K, status, stream, chain) : sk_launch<128, 1>(x, W, e, mb, N, K, status, stream, chain);
        else rc = mb <= 32 ? sk_launch<32, 3>(x, W, e, mb, N, K, status, stream, chain) : mb <= 64 ? sk_launch<64, 3>(x, W, e, mb, N, K, status, stream, chain) : sk_launch<128, 3>(x, W, e, mb, N, K, status, stream, chain);
        if (rc) return rc;
    }
    return 0;
}

}  // namespace mb
