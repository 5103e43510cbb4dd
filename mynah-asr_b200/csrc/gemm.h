// Operand/epilogue descriptions shared by the contraction kernels.
#pragma once
#include "common.cuh"

namespace mb {

// A K-major fp16 operand: rows x K, row stride ld (in halves), as (hi, lo) planes.
struct GemmOperand {
    const __half *hi;
    const __half *lo;   // may be null for single-term (fast) mode
    int ld;
};

enum { ACT_NONE = 0, ACT_SILU = 1, ACT_RELU = 2 };
enum {
    OUT_F32 = 0,     // out[m,n]  = act(acc + bias[n])
    OUT_RESID = 1,   // out[m,n] += alpha * act(acc + bias[n])       (residual stream, in place)
    OUT_H16 = 2,     // (hi,lo)[m,n] = split(act(acc + bias[n]))      (operand of the next contraction)
    OUT_F32_H16 = 3  // both
};

struct GemmEpilogue {
    int mode;
    int act;
    float alpha;
    const float *bias;   // [N] or null
    float *out;          // f32 destination (OUT_F32 / OUT_RESID / OUT_F32_H16)
    int ldo;
    __half *out_hi;      // fp16 planes (OUT_H16 / OUT_F32_H16)
    __half *out_lo;
    int ldh;
};

static constexpr int GEMM_BM = 128;      // rows of an output tile (one tcgen05.mma M)

#ifdef __CUDACC__
// Work units of the persistent loop. Whole waves of gridDim.x tiles come first; the tiles of the last, partial
// wave are cut into 2 or 4 column strips when that still fits one wave, so that the tail costs a half or a
// quarter of a tile time instead of a whole one (752 tiles on 148 CTAs: 5.25 instead of 6 tile times). A strip
// runs the same instruction sequence over its columns as the whole tile would, so no output bit depends on it.
struct GemmUnits {
    int tiles_n, full, split, total;          // full: tiles in whole waves; split: strips per tail tile
    __device__ GemmUnits(int M, int N, int BN_, int ctas) {
        tiles_n = (N + BN_ - 1) / BN_;
        const int tiles = tiles_n * ((M + GEMM_BM - 1) / GEMM_BM);
        full = tiles / ctas * ctas;
        const int rem = tiles - full;
        split = 1;
        if (rem > 0) {
            if (rem * 4 <= ctas && BN_ % 128 == 0) split = 4;
            else if (rem * 2 <= ctas && BN_ % 64 == 0) split = 2;
        }
        total = full + rem * split;
    }
    __device__ void at(int u, int BN_, int &m0, int &n0, int &width) const {
        int tile = u, sub = 0;
        if (u >= full) { tile = full + (u - full) / split; sub = (u - full) % split; }
        width = u >= full ? BN_ / split : BN_;
        m0 = (tile / tiles_n) * GEMM_BM;
        n0 = (tile % tiles_n) * BN_ + sub * width;
    }
};

// Fused tail for a 32 x 32 block of the output handled by one warp: on entry lane r holds the 32 consecutive columns
// [nb, nb + 32) of row m_base + r (the layout tcgen05.ld delivers: lane = row). A thread writing its own row would
// make every store instruction of the warp touch 32 different rows; instead the block goes through `stage` (32 x 32
// floats of shared memory owned by the warp, XOR-swizzled so that both the row-wise writes and the column-wise reads
// are free of bank conflicts) and leaves row by row, lane = column: every store (and the read of a residual
// accumulate) is one contiguous 128-byte line. Returns false if a value written as fp16 planes was out of range.
static constexpr int GEMM_EPI_STAGE_FLOATS = 32 * 32;
__device__ __forceinline__ bool gemm_epilogue_warp(const GemmEpilogue &ep, float (&v)[32], int m_base, int M, int nb, int N,
                                                   float *stage, int lane) {
    bool fits = true;
    const int nvalid = N - nb < 32 ? N - nb : 32;
#pragma unroll
    for (int j = 0; j < 32; j++) {
        float x = v[j];
        if (ep.bias && j < nvalid) x += ep.bias[nb + j];
        if (ep.act == ACT_SILU) x = x * __frcp_rn(1.0f + __expf(-x));   // exp(-x) -> inf gives x * 0
        else if (ep.act == ACT_RELU) x = fmaxf(x, 0.0f);
        stage[lane * 32 + (j ^ lane)] = x;
    }
    __syncwarp();
    const int rows = M - m_base < 32 ? M - m_base : 32;
    if (ep.mode != OUT_H16) {
        const bool in_n = lane < nvalid;
        float *o = ep.out + (size_t)m_base * ep.ldo + nb + lane;
        if (ep.mode == OUT_RESID) {
#pragma unroll 4
            for (int r = 0; r < rows; r++) if (in_n) o[(size_t)r * ep.ldo] += ep.alpha * stage[r * 32 + (lane ^ r)];
        } else {
#pragma unroll 4
            for (int r = 0; r < rows; r++) if (in_n) o[(size_t)r * ep.ldo] = stage[r * 32 + (lane ^ r)];
        }
    }
    if (ep.mode == OUT_H16 || ep.mode == OUT_F32_H16) {
        // two rows per pass: lanes 0..15 take columns 2l, 2l + 1 of row r, lanes 16..31 those of row r + 1
        const int half = lane >> 4, c = 2 * (lane & 15);
        const bool pair_ok = c + 1 < nvalid && (ep.ldh & 1) == 0 && (nb & 1) == 0;
        for (int r0 = 0; r0 < rows; r0 += 2) {
            const int r = r0 + half;
            if (r >= rows) continue;
            const float a = stage[r * 32 + (c ^ r)], b = stage[r * 32 + ((c + 1) ^ r)];
            __half ah, al, bh, bl;
            const size_t off = (size_t)(m_base + r) * ep.ldh + nb + c;
            if (pair_ok) {
                fits &= split_h16(a, ah, al);
                fits &= split_h16(b, bh, bl);
                *reinterpret_cast<__half2 *>(ep.out_hi + off) = __halves2half2(ah, bh);
                if (ep.out_lo) *reinterpret_cast<__half2 *>(ep.out_lo + off) = __halves2half2(al, bl);
            } else {
                if (c < nvalid) { fits &= split_h16(a, ah, al); ep.out_hi[off] = ah; if (ep.out_lo) ep.out_lo[off] = al; }
                if (c + 1 < nvalid) { fits &= split_h16(b, bh, bl); ep.out_hi[off + 1] = bh; if (ep.out_lo) ep.out_lo[off + 1] = bl; }
            }
        }
    }
    __syncwarp();
    return fits;
}

#endif

// C = A * B^T on tcgen05 tensor cores; nterms 1 (hi*hi) or 3 (hi*hi + lo*hi + hi*lo).
// K must be a multiple of 64. status: device int receiving a non-zero code if a
// bounded wait inside the kernel ran out.
int gemm_tc(const GemmOperand &A, const GemmOperand &B, const GemmEpilogue &ep, int M, int N, int K, int nterms,
            int *status, cudaStream_t stream);

// Integer contraction on the tensor cores (gemm_i8.cu): acc[m,n] = sum_k a[m,k] * b[n,k] in int32 (exact), then
// v = (float)acc * col_scale[n] * row_scale[m] — the arithmetic of the reference's int8-activation dots
// (dot_q8_*, src/qmat.c:285-364: (float)int32 * ws * sx) — followed by the same fused tail as gemm_tc.
// a: [M, K] int8 row-major (activation rows quantised by quantize_act_int8's rule), b: [N, K] int8 row-major
// (reference-native per-row int8 weights). K must be a multiple of 128; lda / ldb in bytes, multiples of 16.
int gemm_i8(const int8_t *a, int lda, const float *row_scale, const int8_t *b, int ldb, const float *col_scale,
            const GemmEpilogue &ep, int M, int N, int K, int *status, cudaStream_t stream);

}  // namespace mb
