// Relative-position self-attention on the 5th-generation tensor cores: the full-context case
// (left < 0) with 128-wide heads of the reference's attention (src/encoder.c:315-410),
//
//   s[t,j] = ((q_t + bias_u) . k_j + (q_t + bias_v) . rk[T-1+j-t]) / sqrt(dk),  ctx_t = softmax_j(s[t,:]) v
//
// One CTA owns 128 queries of one (segment, head) and walks the keys in tiles of 64.
//   * Tensor memory (all 512 columns): the two query operands Qu = q + bias_u and Qv = q + bias_v as
//     fp16 (the A operand is read from tensor memory, 64 columns each), the content scores S (64), the
//     position band BD (192) and the context accumulator O (128).
//   * Shared memory: K and V tiles (two stages each), a ring of four 64-row chunks of rk, all placed by
//     TMA with the 128-byte swizzle; the probabilities P as fp16 in the same swizzled layout (the A operand
//     of P.V); and a 48 KB buffer in which the band's skew is undone.
//   * Position term: the tile needs bd[t, T-1+j-t], i.e. for query row r and key column c of the tile
//     the band column c - r + 127. The band of 128 rows x 64 keys spans 191 positions = three rk chunks;
//     it is one or two tcgen05.mma per k-step (the ring wraps), 128 x 192. A softmax warp copies the 96
//     columns its 32 rows touch into shared memory as [column][lane] and reads them back at
//     (c + 31 - lane): both sides conflict-free.
//   * Softmax: thread = query row, exp2 with the scale folded in, running maximum kept per row; the
//     accumulator is rescaled only when the maximum has grown by more than 2^8 (the stale reference
//     cancels in the final division), P rounded to fp16 as in the warp-level kernel.
//   * V is the B operand of P.V in its natural [key, dk] layout (MN-major descriptor).
//   * Pipeline: as soon as the softmax warps hold S(i) and BD(i) in registers / shared memory the issuers
//     score tile i+1 under the exponentials of tile i; P.V(i) follows when P(i) is in shared memory.
// Warps 0-3: softmax / epilogue; warp 4 (one thread): TMA producer; warps 5 and 6 (one thread each): MMA issuers
// (content scores and P.V; position band) — one thread gets a tcgen05.mma out only every 45-90 cycles.
// Every mbarrier wait is bounded; a wait that runs out sets the status word and the CTA unwinds.
#include "kernels.h"

namespace mb {

static constexpr int TA_Q = 128, TA_K = 64, TA_DK = 128;
// softmax warps per quadrant of 32 query rows: with 2, each takes half of a tile's keys and the pair agrees on
// the row maximum through shared memory (measured slower on the 16 x 60 s workload: 5.2 against 4.8 ms per step)
static constexpr int TA_HALVES = 1;
static constexpr int TA_SM_WARPS = 4 * TA_HALVES;            // softmax warps: quadrant = warp % 4, key half = warp / 4
static constexpr int TA_W_TMA = TA_SM_WARPS, TA_W_MMA = TA_SM_WARPS + 1, TA_W_BD = TA_SM_WARPS + 2;
static constexpr int TA_THREADS = (TA_SM_WARPS + 3) * 32;
static constexpr int TA_COL_QU = 0, TA_COL_QV = 64, TA_COL_S = 128, TA_COL_BD = 192, TA_COL_O = 384, TA_TMEM = 512;
static constexpr int TA_HALF = TA_K * 128;                 // one 64-row x 64-column fp16 box: 8 KB
static constexpr int TA_KV_STAGE = 2 * TA_HALF;            // one K (or V) tile: dk halves 0, 1
static constexpr int TA_RK_SLOTS = 4;
static constexpr int TA_RK_PLANE = TA_RK_SLOTS * TA_HALF;  // one dk half of the ring: 32 KB
static constexpr int TA_SKEW_COLS = TA_K / TA_HALVES + 32;  // band columns one softmax warp needs: its keys + 31 rows of skew
static constexpr int TA_P_BYTES = TA_Q * TA_K * 2;         // 16 KB
static constexpr int TA_SMEM = 4 * TA_KV_STAGE + 2 * TA_RK_PLANE + TA_P_BYTES + TA_SM_WARPS * TA_SKEW_COLS * 32 * 4 + 3 * TA_Q * 4 + 256 + 1024;

struct AttnTcDev {
    const float *q;
    int ldq;
    const float *bias_u, *bias_v;
    float *ctx_f32;
    __half *ctx_hi, *ctx_lo;
    const int *seg_off, *seg_len, *rk_off;
    int d;
    float scale2;                  // log2(e) / sqrt(dk)
    int *status;
};

__device__ __forceinline__ void ta_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void ta_st16(uint32_t taddr, const uint32_t *r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void ta_st32(uint32_t taddr, const uint32_t *r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void ta_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ta_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t ta_pack(float x, float y) {
    __half2 h = __floats2half2_rn(x, y);
    return *reinterpret_cast<uint32_t *>(&h);
}
// B operand in its [k rows][64 n] layout (n contiguous, 128-byte swizzle): eight-row k groups 1024 bytes
// apart (stride byte offset), 64-wide n blocks `lbo` bytes apart (leading byte offset)
__device__ __forceinline__ uint64_t ta_desc_mn(uint32_t smem_addr, uint32_t lbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(lbo >> 4) << 16;
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__global__ void __launch_bounds__(TA_THREADS, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
               const __grid_constant__ CUtensorMap tmR, const AttnTcDev a) {
    const int b = blockIdx.z, h = blockIdx.y, t0 = blockIdx.x * TA_Q;
    const int len = a.seg_len[b];
    if (t0 >= len) return;                                   // the whole CTA leaves before any barrier exists
    extern __shared__ uint8_t ta_smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(ta_smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *kst = smem;                                     // K: 2 stages x (2 dk halves x 8 KB)
    uint8_t *vst = kst + 2 * TA_KV_STAGE;                    // V: the same
    uint8_t *rkr = vst + 2 * TA_KV_STAGE;                    // [dk half][slot][64 rows][128 B]
    uint8_t *pst = rkr + 2 * TA_RK_PLANE;                    // P: 128 rows x 64 keys fp16, 128-byte swizzle
    float *skew = reinterpret_cast<float *>(pst + TA_P_BYTES);               // [warp][64][32]
    float *xmax = skew + TA_SM_WARPS * TA_SKEW_COLS * 32;                    // [tile parity][row]: tile maximum of key half 1
    float *xsum = xmax + 2 * TA_Q;                                           // [row]: row sum of key half 1
    uint64_t *k_full = reinterpret_cast<uint64_t *>(xsum + TA_Q);
    uint64_t *k_empty = k_full + 2;
    uint64_t *v_full = k_empty + 2;
    uint64_t *v_empty = v_full + 2;
    uint64_t *rk_full = v_empty + 2;
    uint64_t *rk_empty = rk_full + TA_RK_SLOTS;
    uint64_t *q_full = rk_empty + TA_RK_SLOTS;
    uint64_t *s_full = q_full + 1;
    uint64_t *sbd_free = s_full + 1;
    uint64_t *p_full = sbd_free + 1;
    uint64_t *pv_done = p_full + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(pv_done + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int off = a.seg_off[b], ho = h * TA_DK;
    const int nkt = (len + TA_K - 1) / TA_K;                 // key tiles
    const int pbase = len - 1 - t0 - (TA_Q - 1);             // rk position of band column 0 of key tile 0 (may be negative)
    const int rk0 = a.rk_off[b];

    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmR);
        for (int i = 0; i < 2; i++) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
        for (int i = 0; i < TA_RK_SLOTS; i++) { mbar_init(&rk_full[i], 1); mbar_init(&rk_empty[i], 1); }
        mbar_init(q_full, TA_SM_WARPS); mbar_init(s_full, 2); mbar_init(sbd_free, TA_SM_WARPS); mbar_init(p_full, TA_SM_WARPS); mbar_init(pv_done, 1);
        mbar_fence_init();
    }
    if (warp == TA_W_MMA) { tc_alloc(tmem_slot, TA_TMEM); tc_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == TA_W_TMA) {
        if (lane == 0) {
            // ------------------------------------------------------------------ TMA producer
            bool ok = true;
            int loaded = 0;                                  // rk chunks requested so far
            for (int i = 0; i < nkt && ok; i++) {
                const int s = i & 1;
                const uint32_t eph = (uint32_t)(((i >> 1) & 1) ^ 1);
                if (i >= 2 && !mbar_wait(&k_empty[s], eph)) { ok = false; break; }
                mbar_expect_tx(&k_full[s], TA_KV_STAGE);
                tma_load_2d(kst + s * TA_KV_STAGE, &tmK, ho, off + i * TA_K, &k_full[s]);
                tma_load_2d(kst + s * TA_KV_STAGE + TA_HALF, &tmK, ho + 64, off + i * TA_K, &k_full[s]);
                // rk chunks i, i+1, i+2 cover the band of key tile i; chunk c lives in slot c % 4
                for (; loaded <= i + 2 && ok; loaded++) {
                    const int c = loaded, sl = c & (TA_RK_SLOTS - 1);
                    if (c >= TA_RK_SLOTS && !mbar_wait(&rk_empty[sl], (uint32_t)((((c >> 2) & 1) ^ 1)))) { ok = false; break; }
                    mbar_expect_tx(&rk_full[sl], 2 * TA_HALF);
                    tma_load_2d(rkr + sl * TA_HALF, &tmR, ho, rk0 + pbase + c * TA_K, &rk_full[sl]);
                    tma_load_2d(rkr + TA_RK_PLANE + sl * TA_HALF, &tmR, ho + 64, rk0 + pbase + c * TA_K, &rk_full[sl]);
                }
                if (!ok) break;
                if (i >= 2 && !mbar_wait(&v_empty[s], eph)) { ok = false; break; }
                mbar_expect_tx(&v_full[s], TA_KV_STAGE);
                tma_load_2d(vst + s * TA_KV_STAGE, &tmV, ho, off + i * TA_K, &v_full[s]);
                tma_load_2d(vst + s * TA_KV_STAGE + TA_HALF, &tmV, ho + 64, off + i * TA_K, &v_full[s]);
            }
            if (!ok) atomicExch(a.status, ST_TIMEOUT_PRODUCER);
        }
    } else if (warp == TA_W_MMA) {
        if (lane == 0) {
            // ------------------------------------------------------------------ MMA issuer: content scores and P.V
            constexpr uint32_t idesc_s = umma_idesc_f16(TA_Q, TA_K);
            constexpr uint32_t idesc_pv = umma_idesc_f16(TA_Q, TA_DK) | (1u << 16);      // B operand MN-major
            const uint64_t kdesc0 = umma_desc_sw128(smem_u32(kst));
            const uint64_t pdesc0 = umma_desc_sw128(smem_u32(pst)), vdesc0 = ta_desc_mn(smem_u32(vst), TA_HALF);
            bool ok = mbar_wait(q_full, 0);
            // S(i) = Qu K^T
            auto issue_s = [&](int i) -> bool {
                const int s = i & 1;
                if (!mbar_wait(&k_full[s], (uint32_t)((i >> 1) & 1))) return false;
                tc_fence_after();
                const uint64_t kd = kdesc0 + (uint64_t)((s * TA_KV_STAGE) >> 4);
#pragma unroll
                for (int kk = 0; kk < TA_DK / 16; kk++)
                    ta_mma_ts(tmem_base + TA_COL_S, tmem_base + TA_COL_QU + 8 * kk, kd + (uint64_t)(((kk >> 2) * TA_HALF + (kk & 3) * 32) >> 4),
                              idesc_s, kk != 0);
                tc_commit(s_full);
                tc_commit(&k_empty[s]);
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int i = 0; i < nkt && ok; i++) {
                const int s = i & 1;
                if (i + 1 < nkt) {
                    // the softmax warps hold S(i) and BD(i) in registers / shared memory: score the next tile under them
                    if (!mbar_wait(sbd_free, (uint32_t)(i & 1))) { ok = false; break; }
                    tc_fence_after();
                    if (!issue_s(i + 1)) { ok = false; break; }
                }
                // O += P V
                if (!mbar_wait(p_full, (uint32_t)(i & 1)) || !mbar_wait(&v_full[s], (uint32_t)((i >> 1) & 1))) { ok = false; break; }
                tc_fence_after();
                const uint64_t vd = vdesc0 + (uint64_t)((s * TA_KV_STAGE) >> 4);
#pragma unroll
                for (int kk = 0; kk < TA_K / 16; kk++)
                    tc_mma_f16(tmem_base + TA_COL_O, pdesc0 + (uint64_t)((kk * 32) >> 4), vd + (uint64_t)((kk * 2048) >> 4), idesc_pv, (i | kk) != 0);
                tc_commit(pv_done);
                tc_commit(&v_empty[s]);
            }
            if (!ok) atomicExch(a.status, ST_TIMEOUT_MMA);
        }
    } else if (warp == TA_W_BD) {
        if (lane == 0) {
            // ------------------------------------------------------------------ MMA issuer: position band
            // BD(i) = Qv RK^T over the chunks i, i+1, i+2 (ring slots s0, s0+1, .., wrapping after slot 3). A second
            // issuing thread, because one thread gets a tcgen05.mma out only every 45-90 cycles
            const uint64_t rdesc0 = umma_desc_sw128(smem_u32(rkr));
            bool ok = mbar_wait(q_full, 0);
            for (int i = 0; i < nkt && ok; i++) {
                if (i > 0 && !mbar_wait(sbd_free, (uint32_t)((i - 1) & 1))) { ok = false; break; }
                for (int c = (i == 0 ? 0 : i + 2); c <= i + 2 && ok; c++)
                    ok = mbar_wait(&rk_full[c & (TA_RK_SLOTS - 1)], (uint32_t)((c >> 2) & 1));
                if (!ok) break;
                tc_fence_after();
                const int s0 = i & (TA_RK_SLOTS - 1);
                const int n1 = TA_RK_SLOTS - s0 < 3 ? TA_RK_SLOTS - s0 : 3, n2 = 3 - n1;
                const uint32_t id1 = umma_idesc_f16(TA_Q, 64 * n1), id2 = umma_idesc_f16(TA_Q, n2 > 0 ? 64 * n2 : 64);
                const uint64_t rd1 = rdesc0 + (uint64_t)((s0 * TA_HALF) >> 4);
#pragma unroll
                for (int kk = 0; kk < TA_DK / 16; kk++) {
                    const uint64_t ko = (uint64_t)(((kk >> 2) * TA_RK_PLANE + (kk & 3) * 32) >> 4);
                    ta_mma_ts(tmem_base + TA_COL_BD, tmem_base + TA_COL_QV + 8 * kk, rd1 + ko, id1, kk != 0);
                    if (n2 > 0) ta_mma_ts(tmem_base + TA_COL_BD + 64 * n1, tmem_base + TA_COL_QV + 8 * kk, rdesc0 + ko, id2, kk != 0);
                }
                tc_commit(s_full);
                tc_commit(&rk_empty[s0]);                    // chunk i is not used after key tile i
            }
            if (!ok) atomicExch(a.status, ST_TIMEOUT_MMA);
        }
    } else {
        // ---------------------------------------------------------------------- softmax warps
        // Two warps share a quadrant of 32 query rows (tensor-memory lanes): warp qd handles keys 0-31 of
        // every tile, warp qd + 4 keys 32-63. They agree on the tile maximum through shared memory.
        const int qd = warp & 3, hf = warp >> 2;
        const int r = qd * 32 + lane, t = t0 + r;
        const bool valid = t < len;
        const uint32_t trow = tmem_base + ((uint32_t)(qd * 32) << 16);
        const int pair_bar = 1 + qd;                         // named barrier of the two warps of a quadrant
        // ---- Qu (key half 0) / Qv (key half 1) into tensor memory: column c holds elements 2c, 2c+1 as fp16
        {
            const float *qrow = a.q + (size_t)(off + (valid ? t : 0)) * a.ldq + ho;
#pragma unroll 1
            for (int w2 = hf; w2 < 2; w2 += TA_HALVES) {     // operand 0: Qu, 1: Qv
                const float *bias = (w2 ? a.bias_v : a.bias_u) + ho;
#pragma unroll 1
                for (int c4 = 0; c4 < TA_DK / 32; c4++) {
                    uint32_t ru[16];
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (valid) x = *reinterpret_cast<const float4 *>(qrow + c4 * 32 + 4 * j);
                        const float4 u = *reinterpret_cast<const float4 *>(bias + c4 * 32 + 4 * j);
                        ru[2 * j] = ta_pack(x.x + u.x, x.y + u.y); ru[2 * j + 1] = ta_pack(x.z + u.z, x.w + u.w);
                    }
                    ta_st16(trow + (w2 ? TA_COL_QV : TA_COL_QU) + 16 * c4, ru);
                }
            }
            ta_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_full);
        }
        float *skw = skew + warp * TA_SKEW_COLS * 32;
        uint8_t *prow = pst + r * 128;                       // this row of P: eight 16-byte pieces at (piece ^ (r & 7))
        constexpr int NC = TA_K / TA_HALVES;                 // keys per warp and tile
        constexpr int OC = TA_DK / TA_HALVES;                // context columns per warp
        const int cbase = 96 - 32 * qd + NC * hf;            // first band column this warp's rows and keys touch
        float m_ref = -3.0e38f, l = 0.f;
        bool ok = true;
        // A wait that runs out clears `ok`: the warp then skips the work but still meets its partner at the
        // pair barriers, so neither of the two can be left waiting at one.
        for (int i = 0; i < nkt; i++) {
            if (ok && !__all_sync(0xffffffffu, mbar_wait(s_full, (uint32_t)(i & 1)))) {
                ok = false;
                if (lane == 0) atomicExch(a.status, ST_TIMEOUT_EPILOGUE);
            }
            tc_fence_after();
            // ---- band -> shared memory as [column][lane]; the content scores are fetched under the copy
            float x[NC];
            float mt = -3.0e38f;
            if (ok) {
            {
                float v[TA_SKEW_COLS];
#pragma unroll
                for (int q3 = 0; q3 < TA_SKEW_COLS / 32; q3++) tc_ld32(trow + TA_COL_BD + cbase + 32 * q3, v + 32 * q3);
#pragma unroll
                for (int q3 = 0; q3 < NC / 32; q3++) tc_ld32(trow + TA_COL_S + NC * hf + 32 * q3, x + 32 * q3);
                tc_wait_ld();
#pragma unroll
                for (int e = 0; e < TA_SKEW_COLS; e++) skw[e * 32 + lane] = v[e];
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(sbd_free);            // S and BD may be overwritten by the next tile's MMAs
            const int j0 = i * TA_K + NC * hf;
            const float *sk = skw + (31 - lane) * 32 + lane;
#pragma unroll
            for (int c = 0; c < NC; c++) x[c] += sk[c * 32];          // unscaled; the scale is folded into the exponent below
            if (j0 + NC > len) {                             // ragged last tile: keys past the segment
#pragma unroll
                for (int c = 0; c < NC; c++)
                    if (j0 + c >= len) x[c] = -3.0e38f;
            }
#pragma unroll
            for (int c = 0; c < NC; c += 4) mt = fmaxf(fmaxf(mt, fmaxf(x[c], x[c + 1])), fmaxf(x[c + 2], x[c + 3]));
            }
            // the two key halves agree on the tile maximum of the row (buffers alternate by tile parity)
            if (TA_HALVES == 2) {
                float *xm = xmax + (i & 1) * TA_Q;
                if (hf) xm[r] = mt;
                asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
                if (!hf) { const float o = xm[r]; xm[r] = mt; mt = fmaxf(mt, o); }
                asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
                if (hf) mt = fmaxf(mt, xm[r]);
            }
            // P(i-1) has to be consumed, and O at rest, before either is touched
            if (ok && i > 0 && !__all_sync(0xffffffffu, mbar_wait(pv_done, (uint32_t)((i - 1) & 1)))) {
                ok = false;
                if (lane == 0) atomicExch(a.status, ST_TIMEOUT_EPILOGUE);
            }
            if (!ok) continue;
            tc_fence_after();
            // ---- running maximum: move the reference only when it lags by more than 8 (in log2 units)
            mt *= a.scale2;
            const bool grow = mt > m_ref + 8.f;
            if (__any_sync(0xffffffffu, grow)) {
                const float alpha = grow ? ta_ex2(m_ref - mt) : 1.f;
                if (grow) m_ref = mt;
                l *= alpha;
                if (i > 0) {                                 // this warp's half of the accumulator columns
#pragma unroll 1
                    for (int c4 = 0; c4 < OC / 32; c4++) {
                        float o[32];
                        tc_ld32(trow + TA_COL_O + OC * hf + 32 * c4, o);
                        tc_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; e++) o[e] *= alpha;
                        ta_st32(trow + TA_COL_O + OC * hf + 32 * c4, reinterpret_cast<const uint32_t *>(o));
                    }
                    ta_wait_st();
                }
            }
#pragma unroll
            for (int c8 = 0; c8 < NC / 8; c8++) {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float p0 = ta_ex2(fmaf(x[c8 * 8 + 2 * e], a.scale2, -m_ref)), p1 = ta_ex2(fmaf(x[c8 * 8 + 2 * e + 1], a.scale2, -m_ref));
                    l += p0 + p1;
                    w[e] = ta_pack(p0, p1);
                }
                *reinterpret_cast<uint4 *>(prow + (((c8 + (NC / 8) * hf) ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy stores -> visible to the tensor core
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        // ---- normalise and store: each warp its half of the context columns
        if (TA_HALVES == 2) {
            if (hf) xsum[r] = l;
            asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
            if (!hf) { const float o = xsum[r]; xsum[r] = l; l += o; }
            asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
            if (hf) l += xsum[r];
        }
        if (ok && !__all_sync(0xffffffffu, mbar_wait(pv_done, (uint32_t)((nkt - 1) & 1)))) { ok = false; if (lane == 0) atomicExch(a.status, ST_TIMEOUT_EPILOGUE); }
        if (ok) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            const size_t idx0 = (size_t)(off + t) * a.d + ho + OC * hf;
#pragma unroll 1
            for (int c4 = 0; c4 < OC / 32; c4++) {
                float o[32];
                tc_ld32(trow + TA_COL_O + OC * hf + 32 * c4, o);
                tc_wait_ld();
                if (!valid) continue;
#pragma unroll
                for (int e = 0; e < 32; e++) o[e] *= inv;
                if (a.ctx_f32) {
#pragma unroll
                    for (int e = 0; e < 32; e += 4)
                        *reinterpret_cast<float4 *>(a.ctx_f32 + idx0 + c4 * 32 + e) = make_float4(o[e], o[e + 1], o[e + 2], o[e + 3]);
                }
                if (a.ctx_hi) {
                    __align__(16) __half hh[32], ll[32];
#pragma unroll
                    for (int e = 0; e < 32; e++) split_h16(o[e], hh[e], ll[e]);
#pragma unroll
                    for (int e = 0; e < 32; e += 8) {
                        *reinterpret_cast<uint4 *>(a.ctx_hi + idx0 + c4 * 32 + e) = *reinterpret_cast<const uint4 *>(hh + e);
                        if (a.ctx_lo) *reinterpret_cast<uint4 *>(a.ctx_lo + idx0 + c4 * 32 + e) = *reinterpret_cast<const uint4 *>(ll + e);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == TA_W_MMA) tc_dealloc(tmem_base, TA_TMEM);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*TaEncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                               const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// fp16 [rows, d] row-major: boxes of 64 rows x 64 columns, 128-byte swizzle, zeros outside the tensor
static int ta_make_map(CUtensorMap *m, const __half *base, long long rows, int d) {
    static TaEncodeFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<TaEncodeFn>(p);
    }
    if (!fn) { set_error("cuTensorMapEncodeTiled entry point unavailable"); return -1; }
    cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)d * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)TA_K};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("attention: cuTensorMapEncodeTiled failed (%d)", (int)r); return -1; }
    return 0;
}

bool attention_tc_eligible(const AttnArgs &a) {
    return a.left < 0 && a.H > 0 && a.d / a.H == TA_DK && a.d % 8 == 0 && a.ldq % 4 == 0 && a.rows > 0 && a.rk_rows > 0 &&
           a.status != nullptr && (reinterpret_cast<uintptr_t>(a.k) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.v) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(a.rk) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.q) & 15) == 0;
}

int attention_tc(const AttnArgs &a, cudaStream_t st) {
    CUtensorMap tk, tv, tr;
    if (ta_make_map(&tk, a.k, a.rows, a.d) || ta_make_map(&tv, a.v, a.rows, a.d) || ta_make_map(&tr, a.rk, a.rk_rows, a.d)) return -1;
    static PerDevice configured = {};
    int dev = 0;
    if (configured.below((size_t)TA_SMEM, &dev)) {
        MB_CUDA(cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TA_SMEM));
        configured.record(dev, (size_t)TA_SMEM);
    }
    AttnTcDev dv;
    dv.q = a.q; dv.ldq = a.ldq; dv.bias_u = a.bias_u; dv.bias_v = a.bias_v; dv.ctx_f32 = a.ctx_f32;
    dv.ctx_hi = a.ctx_h.hi; dv.ctx_lo = a.ctx_h.lo;
    dv.seg_off = a.seg_off; dv.seg_len = a.seg_len; dv.rk_off = a.rk_off;
    dv.d = a.d; dv.scale2 = 1.4426950408889634f / sqrtf((float)TA_DK); dv.status = a.status;
    dim3 grid(cdiv(a.max_len, TA_Q), a.H, a.batch);
    attn_tc_kernel<<<grid, TA_THREADS, TA_SMEM, st>>>(tk, tv, tr, dv);
    MB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace mb
