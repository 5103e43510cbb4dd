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
    // Optional LayerNorm of the finished rows (few-row kernel only; the other kernels ignore it): when the last tile of
    // row m has been written to `out`, that row (ldo == N, one of ln_row's widths) is normalised by the CTA that
    // completed it — the LayerNorm that follows a residual update, without a launch of its own.
    //   ln_w, ln_b alone: into the planes (ln_hi, ln_lo), or, without planes, into `out` in place;
    //   with ln2_w, ln2_b: (ln_w, ln_b) into `out` in place, then (ln2_w, ln2_b) of that result into the planes
    //   (a block's closing LayerNorm followed by the next block's opening one).
    // ln_count: one int per row, zero between launches.
    const float *ln_w = nullptr;
    const float *ln_b = nullptr;
    const float *ln2_w = nullptr;
    const float *ln2_b = nullptr;
    __half *ln_hi = nullptr;
    __half *ln_lo = nullptr;
    int *ln_count = nullptr;
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

// ---- the same fused tail for a 32 x 32 block (32 rows from m_base, columns [nb, nb + 32)) held one row per lane.
// Stored row by row, every store instruction of a warp touches 32 different 128-byte lines with 16 bytes each, and the
// load/store unit spends one cycle per line. Here the block is turned through 4 KB of shared memory (float4 columns
// XOR-swizzled by the row: no bank conflicts either way) so that an instruction covers four whole lines: eight lanes
// take the eight float4 of one row. Values and operation order per element are those of gemm_epilogue_row.
static constexpr int GEMM_BLOCK_STAGE_FLOATS = 32 * 32;           // shared memory per epilogue warp

// true if the block form can be used for every full-width chunk of this contraction (pointer and stride alignment)
__device__ __forceinline__ bool gemm_block_ok(const GemmEpilogue &ep) {
    bool ok = !ep.bias || (reinterpret_cast<uintptr_t>(ep.bias) & 15) == 0;
    if (ep.mode != OUT_H16) ok = ok && (reinterpret_cast<uintptr_t>(ep.out) & 15) == 0 && (ep.ldo & 3) == 0;
    if (ep.mode == OUT_H16 || ep.mode == OUT_F32_H16)
        ok = ok && (reinterpret_cast<uintptr_t>(ep.out_hi) & 7) == 0 && (reinterpret_cast<uintptr_t>(ep.out_lo) & 7) == 0 && (ep.ldh & 3) == 0;
    return ok;
}

// residual values of this lane's eight float4 positions (rows i * 4 + lane / 8, columns 4 (lane % 8) ..), asked for
// before the accumulator is read so that the loads are in flight meanwhile
__device__ __forceinline__ void gemm_block_prefetch(const GemmEpilogue &ep, int m_base, int M, int nb, int lane, float4 (&res)[8]) {
    if (ep.mode != OUT_RESID) return;
    const float *o = ep.out + (size_t)(m_base + (lane >> 3)) * ep.ldo + nb + (lane & 7) * 4;
#pragma unroll
    for (int i = 0; i < 8; i++)
        res[i] = m_base + i * 4 + (lane >> 3) < M ? *reinterpret_cast<const float4 *>(o + (size_t)i * 4 * ep.ldo) : make_float4(0.f, 0.f, 0.f, 0.f);
}

__device__ __forceinline__ float gemm_act(const GemmEpilogue &ep, float x) {
    if (ep.act == ACT_SILU) return x * __frcp_rn(1.0f + __expf(-x));
    if (ep.act == ACT_RELU) return fmaxf(x, 0.0f);
    return x;
}

// this lane's row, columns [16 h, 16 h + 16) of the block, into the turning buffer
__device__ __forceinline__ void gemm_block_stage(const float (&v)[16], int h, float *stage, int lane) {
    float4 *s4 = reinterpret_cast<float4 *>(stage);
#pragma unroll
    for (int j = 0; j < 4; j++) s4[lane * 8 + ((4 * h + j) ^ (lane & 7))] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
}

// after both halves were staged: the fused tail and the stores
__device__ __forceinline__ bool gemm_block_store(const GemmEpilogue &ep, const float4 (&res)[8], int m_base, int M,
                                                 int nb, float *stage, int lane) {
    float4 *s4 = reinterpret_cast<float4 *>(stage);
    __syncwarp();
    const int q = lane & 7, r0 = lane >> 3, col = nb + q * 4;
    const float4 b = ep.bias ? *reinterpret_cast<const float4 *>(ep.bias + col) : make_float4(0.f, 0.f, 0.f, 0.f);
    bool fits = true;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int r = i * 4 + r0, m = m_base + r;
        float4 t = s4[r * 8 + (q ^ (r & 7))];
        if (ep.bias) { t.x += b.x; t.y += b.y; t.z += b.z; t.w += b.w; }
        t.x = gemm_act(ep, t.x); t.y = gemm_act(ep, t.y); t.z = gemm_act(ep, t.z); t.w = gemm_act(ep, t.w);
        if (m >= M) continue;
        if (ep.mode != OUT_H16) {
            float4 *o = reinterpret_cast<float4 *>(ep.out + (size_t)m * ep.ldo + col);
            if (ep.mode == OUT_RESID) {
                float4 a = res[i];
                a.x += ep.alpha * t.x; a.y += ep.alpha * t.y; a.z += ep.alpha * t.z; a.w += ep.alpha * t.w;
                *o = a;
            } else {
                *o = t;
            }
        }
        if (ep.mode == OUT_H16 || ep.mode == OUT_F32_H16) {
            __half h0, h1, h2, h3, l0, l1, l2, l3;
            fits &= split_h16(t.x, h0, l0);
            fits &= split_h16(t.y, h1, l1);
            fits &= split_h16(t.z, h2, l2);
            fits &= split_h16(t.w, h3, l3);
            const size_t off = (size_t)m * ep.ldh + col;
            const __half2 ha = __halves2half2(h0, h1), hb = __halves2half2(h2, h3), la = __halves2half2(l0, l1), lb = __halves2half2(l2, l3);
            *reinterpret_cast<uint2 *>(ep.out_hi + off) = make_uint2(*reinterpret_cast<const uint32_t *>(&ha), *reinterpret_cast<const uint32_t *>(&hb));
            if (ep.out_lo) *reinterpret_cast<uint2 *>(ep.out_lo + off) = make_uint2(*reinterpret_cast<const uint32_t *>(&la), *reinterpret_cast<const uint32_t *>(&lb));
        }
    }
    __syncwarp();                                                   // the stage is free for the next block
    return fits;
}
#endif

// C = A * B^T on tcgen05 tensor cores; nterms 1 (hi*hi) or 3 (hi*hi + lo*hi + hi*lo).
// K must be a multiple of 64. status: device int receiving a non-zero code if a
// bounded wait inside the kernel ran out.
int gemm_tc(const GemmOperand &A, const GemmOperand &B, const GemmEpilogue &ep, int M, int N, int K, int nterms,
            int *status, cudaStream_t stream);

// The same contraction for a handful of rows (a decoder position): gemm_skinny.cu. X: [M, K] activation planes, W: [N, K]
// weight planes; K slices over the CTAs of a cluster, added in slice order (the count depends on N and K alone).
// GemmEpilogue's ln_* fields are honoured for the widths gemm_skinny_ln_width accepts (and ldo == N).
bool gemm_skinny_ln_width(int d);
// chain: launched as a chained kernel (common.cuh): its weight tiles are requested while the kernel before it still runs.
int gemm_skinny(const GemmOperand &X, const GemmOperand &W, const GemmEpilogue &ep, int M, int N, int K, int nterms, int *status,
                cudaStream_t stream, bool chain = false);

// Integer contraction on the tensor cores (gemm_i8.cu): acc[m,n] = sum_k a[m,k] * b[n,k] in int32 (exact), then
// v = (float)acc * col_scale[n] * row_scale[m] — the arithmetic of the reference's int8-activation dots
// (dot_q8_*, src/qmat.c:285-364: (float)int32 * ws * sx) — followed by the same fused tail as gemm_tc.
// a: [M, K] int8 row-major (activation rows quantised by quantize_act_int8's rule), b: [N, K] int8 row-major
// (reference-native per-row int8 weights). K must be a multiple of 128; lda / ldb in bytes, multiples of 16.
int gemm_i8(const int8_t *a, int lda, const float *row_scale, const int8_t *b, int ldb, const float *col_scale,
            const GemmEpilogue &ep, int M, int N, int K, int *status, cudaStream_t stream);

}  // namespace mb
