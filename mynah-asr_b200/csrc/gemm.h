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

#ifdef __CUDACC__
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
int gemm_tc(const GemmOperand &A, const GemmOperand &B, const GemmEpilogue &ep, int M, int N, int K, int nterms,
            int *status, cudaStream_t stream);

}  // namespace mb
