// One LayerNorm row by one warp with the row held in registers (d = NV * 128): the body of ln_reg_kernel
// (elementwise.cu), shared with the kernels that normalise rows they have just completed (gemm_skinny.cu).
// Mean and variance are accumulated in double like the reference's layer_norm_f (src/encoder.c:25-37):
// y = ((x - mu) * inv) * w + b. L2: read the row past the L1 (it was written by other CTAs of the same launch).
#pragma once
#include "common.cuh"
#include "gemm.h"

namespace mb {

// int8 row by the reference's activation rule (quantize_act_int8, src/qmat.c:186-202)
__device__ __forceinline__ int8_t act_q8(float y, float inv) {
    const float v = __fmul_rn(y, inv);
    int q = (int)(v >= 0.0f ? __fadd_rn(v, 0.5f) : __fsub_rn(v, 0.5f));
    q = q > 127 ? 127 : (q < -127 ? -127 : q);
    return (int8_t)q;
}

template <int NV, bool L2>
__device__ __forceinline__ void ln_row(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ b,
                                       float *__restrict__ out, __half *__restrict__ hi, __half *__restrict__ lo, int8_t *__restrict__ q8,
                                       float *__restrict__ sx8, int row, int act, int lane) {
    constexpr int d = NV * 128;
    const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)row * d);
    float4 v[NV];
#pragma unroll
    for (int j = 0; j < NV; j++) v[j] = L2 ? __ldcg(xr + lane + 32 * j) : xr[lane + 32 * j];
    double s = 0.0;
#pragma unroll
    for (int j = 0; j < NV; j++) s += (double)v[j].x + (double)v[j].y + (double)v[j].z + (double)v[j].w;
    const double mu = warp_sum_d(s) / d;
    double q = 0.0;
#pragma unroll
    for (int j = 0; j < NV; j++) {
        const double a = v[j].x - mu, c = v[j].y - mu, e = v[j].z - mu, f = v[j].w - mu;
        q += a * a + c * c + e * e + f * f;
    }
    const double var = warp_sum_d(q) / d;
    const float inv = (float)(1.0 / sqrt(var + 1e-5));
    const float muf = (float)mu;
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; j++) {          // the finished values replace the inputs in the registers
        const int i = lane + 32 * j;
        const float4 ww = reinterpret_cast<const float4 *>(w)[i];
        const float4 bb = reinterpret_cast<const float4 *>(b)[i];
        float y[4] = {((v[j].x - muf) * inv) * ww.x + bb.x, ((v[j].y - muf) * inv) * ww.y + bb.y,
                      ((v[j].z - muf) * inv) * ww.z + bb.z, ((v[j].w - muf) * inv) * ww.w + bb.w};
        if (act == ACT_SILU) {
#pragma unroll
            for (int e = 0; e < 4; e++) y[e] = silu_f(y[e]);
        }
        v[j] = make_float4(y[0], y[1], y[2], y[3]);
        amax = fmaxf(fmaxf(amax, fmaxf(fabsf(y[0]), fabsf(y[1]))), fmaxf(fabsf(y[2]), fabsf(y[3])));
    }
    float qinv = 0.0f;
    if (q8) {
        amax = warp_max(amax);
        qinv = amax > 0.0f ? 127.0f / amax : 0.0f;
        if (lane == 0) sx8[row] = amax > 0.0f ? amax / 127.0f : 0.0f;
    }
#pragma unroll
    for (int j = 0; j < NV; j++) {
        const int i = lane + 32 * j;
        const float y[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
        if (q8) reinterpret_cast<char4 *>(q8 + (size_t)row * d)[i] = make_char4(act_q8(y[0], qinv), act_q8(y[1], qinv), act_q8(y[2], qinv), act_q8(y[3], qinv));
        if (out) reinterpret_cast<float4 *>(out + (size_t)row * d)[i] = make_float4(y[0], y[1], y[2], y[3]);
        if (hi) {
            __align__(8) __half h[4], l[4];
#pragma unroll
            for (int e = 0; e < 4; e++) split_h16(y[e], h[e], l[e]);
            reinterpret_cast<uint2 *>(hi + (size_t)row * d)[i] = *reinterpret_cast<uint2 *>(h);
            if (lo) reinterpret_cast<uint2 *>(lo + (size_t)row * d)[i] = *reinterpret_cast<uint2 *>(l);
        }
    }
}

}  // namespace mb
