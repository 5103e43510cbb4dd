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

// Split-K for contractions with few rows and few output tiles (one decoder position): `splits` CTAs share an output
// tile, each sums a K slice into `part` (f32, [unit][128][tile width]); the last to arrive (counted in `counters`, one int
// per tile, zero between launches) adds the slices in slice order and applies the fused tail, so the result does not
// depend on which CTA came last. splits <= 1: off.
struct GemmSplit {
    int splits;
    float *part;
    int *counters;
};
static constexpr int GEMM_SPLIT_BN = 64;                 // tile width of the split-K path
// K slices for an [*, N] x [N, K] contraction on `sms` SMs: a function of the weight's shape alone (never of the row
// count), so a row's bits do not depend on how many rows share the launch.
inline int gemm_split_slices(int N, int K, int sms) {
    const int tiles = (N + GEMM_SPLIT_BN - 1) / GEMM_SPLIT_BN, num_k = K / 64;
    int s = 1;
    while (tiles * s * 2 <= sms && s * 2 <= 16 && num_k % (s * 2) == 0 && num_k / (s * 2) >= 2) s *= 2;
    return s;
}
// floats of `part` / ints of `counters` that M rows of such a contraction need
inline size_t gemm_split_part_floats(int M, int N, int K, int sms) {
    const size_t tiles = (size_t)((N + GEMM_SPLIT_BN - 1) / GEMM_SPLIT_BN) * ((M + GEMM_BM - 1) / GEMM_BM);
    const int s = gemm_split_slices(N, K, sms);
    return s > 1 ? tiles * s * GEMM_BM * GEMM_SPLIT_BN : 0;       // at most ceil(M / 128) * sms * 128 * 64
}
inline size_t gemm_split_counters(int M, int N) {
    return (size_t)((N + GEMM_SPLIT_BN - 1) / GEMM_SPLIT_BN) * ((M + GEMM_BM - 1) / GEMM_BM);
}

#ifdef __CUDACC__
// Work units of the persistent loop. Whole waves of gridDim.x tiles come first; the tiles of the last, partial
// wave are cut into 2 or 4 column strips when that still fits one wave, so that the tail costs a half or a
// quarter of a tile time instead of a whole one (752 tiles on 148 CTAs: 5.25 instead of 6 tile times). A strip
// runs the same instruction sequence over its columns as the whole tile would, so no output bit depends on it.
struct GemmUnits {
    int tiles_n, full, split, total, slices;  // full: tiles in whole waves; split: strips per tail tile; slices: K slices per tile
    __device__ GemmUnits(int M, int N, int BN_, int ctas, int slices_ = 1) {
        tiles_n = (N + BN_ - 1) / BN_;
        slices = slices_;
        const int tiles = tiles_n * ((M + GEMM_BM - 1) / GEMM_BM);
        if (slices > 1) { full = tiles * slices; split = 1; total = full; return; }   // split-K: no column strips
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
    // split-K form: unit u = tile * slices + slice (for slices == 1 the same as above with slice = 0)
    __device__ void at(int u, int BN_, int &m0, int &n0, int &width, int &slice) const {
        if (slices <= 1) { slice = 0; at(u, BN_, m0, n0, width); return; }
        const int tile = u / slices;
        slice = u % slices;
        width = BN_;
        m0 = (tile / tiles_n) * GEMM_BM;
        n0 = (tile % tiles_n) * BN_;
    }
};

// Fused tail for 32 consecutive columns [nb, nb+32) of output row m.
// Returns false if a value written as fp16 planes was out of their range (see split_h16).
__device__ __forceinline__ bool gemm_epilogue_row(const GemmEpilogue &ep, float (&v)[32], int m, int nb, int N) {
    bool fits = true;
    const int nvalid = N - nb < 32 ? N - nb : 32;
#pragma unroll
    for (int j = 0; j < 32; j++) {
        float x = v[j];
        if (ep.bias && j < nvalid) x += ep.bias[nb + j];
        if (ep.act == ACT_SILU) x = x * __frcp_rn(1.0f + __expf(-x));   // exp(-x) -> inf gives x * 0
        else if (ep.act == ACT_RELU) x = fmaxf(x, 0.0f);
        v[j] = x;
    }
    if (ep.mode != OUT_H16) {
        float *o = ep.out + (size_t)m * ep.ldo + nb;
        const bool vec = nvalid == 32 && ((reinterpret_cast<uintptr_t>(o) & 15) == 0);
        if (ep.mode == OUT_RESID) {
            if (vec) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    float4 r = *reinterpret_cast<float4 *>(o + j);
                    r.x += ep.alpha * v[j]; r.y += ep.alpha * v[j + 1];
                    r.z += ep.alpha * v[j + 2]; r.w += ep.alpha * v[j + 3];
                    *reinterpret_cast<float4 *>(o + j) = r;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++) if (j < nvalid) o[j] += ep.alpha * v[j];
            }
        } else {
            if (vec) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    *reinterpret_cast<float4 *>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++) if (j < nvalid) o[j] = v[j];
            }
        }
    }
    if (ep.mode == OUT_H16 || ep.mode == OUT_F32_H16) {
        __half *ph = ep.out_hi + (size_t)m * ep.ldh + nb;
        __half *pl = ep.out_lo ? ep.out_lo + (size_t)m * ep.ldh + nb : nullptr;
        const bool vec = nvalid == 32 && ((reinterpret_cast<uintptr_t>(ph) & 15) == 0);
        if (vec) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
                __align__(16) __half h[8], l[8];
#pragma unroll
                for (int i = 0; i < 8; i++) fits &= split_h16(v[j + i], h[i], l[i]);
                *reinterpret_cast<uint4 *>(ph + j) = *reinterpret_cast<uint4 *>(h);
                if (pl) *reinterpret_cast<uint4 *>(pl + j) = *reinterpret_cast<uint4 *>(l);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++) {
                if (j < nvalid) {
                    __half h, l;
                    fits &= split_h16(v[j], h, l);
                    ph[j] = h;
                    if (pl) pl[j] = l;
                }
            }
        }
    }
    return fits;
}
#endif

// C = A * B^T on tcgen05 tensor cores; nterms 1 (hi*hi) or 3 (hi*hi + lo*hi + hi*lo).
// K must be a multiple of 64. status: device int receiving a non-zero code if a
// bounded wait inside the kernel ran out.
// split: optional split-K workspace (see GemmSplit; the slice count is gemm_split_slices(N, K, SMs), `splits` of the
// argument is ignored); null = every tile sums its whole K.
int gemm_tc(const GemmOperand &A, const GemmOperand &B, const GemmEpilogue &ep, int M, int N, int K, int nterms,
            int *status, cudaStream_t stream, const GemmSplit *split = nullptr);

// Integer contraction on the tensor cores (gemm_i8.cu): acc[m,n] = sum_k a[m,k] * b[n,k] in int32 (exact), then
// v = (float)acc * col_scale[n] * row_scale[m] — the arithmetic of the reference's int8-activation dots
// (dot_q8_*, src/qmat.c:285-364: (float)int32 * ws * sx) — followed by the same fused tail as gemm_tc.
// a: [M, K] int8 row-major (activation rows quantised by quantize_act_int8's rule), b: [N, K] int8 row-major
// (reference-native per-row int8 weights). K must be a multiple of 128; lda / ldb in bytes, multiples of 16.
int gemm_i8(const int8_t *a, int lda, const float *row_scale, const int8_t *b, int ldb, const float *col_scale,
            const GemmEpilogue &ep, int M, int N, int K, int *status, cudaStream_t stream);

}  // namespace mb
