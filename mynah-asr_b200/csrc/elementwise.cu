// Row-wise and channel-wise pieces of the FastConformer block that are bound by
// HBM bandwidth: LayerNorm, the conv-module middle (GLU -> depthwise conv ->
// folded BatchNorm -> SiLU), positional embedding. Each one reads its input once,
// coalesced and vectorised, and writes the operand form the next contraction wants.
#include "kernels.h"
#include "ln_row.cuh"

namespace mb {

// ---------------------------------------------------------------- LayerNorm
// One warp per row. Mean and variance are accumulated in double like the
// reference's layer_norm_f (src/encoder.c:25-37): y = ((x - mu) * inv) * w + b.
__global__ void __launch_bounds__(256)
ln_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ b,
          float *__restrict__ out, __half *__restrict__ hi, __half *__restrict__ lo, int8_t *__restrict__ q8,
          float *__restrict__ sx8, int T, int d, int act) {
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= T) return;
    const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)row * d);
    const int n4 = d >> 2;
    double s = 0.0;
    for (int i = lane; i < n4; i += 32) { const float4 v = xr[i]; s += (double)v.x + (double)v.y + (double)v.z + (double)v.w; }
    const double mu = warp_sum_d(s) / d;
    double q = 0.0;
    for (int i = lane; i < n4; i += 32) {
        const float4 v = xr[i];
        const double a = v.x - mu, c = v.y - mu, e = v.z - mu, f = v.w - mu;
        q += a * a + c * c + e * e + f * f;
    }
    const double var = warp_sum_d(q) / d;
    const float inv = (float)(1.0 / sqrt(var + 1e-5));
    const float muf = (float)mu;
    float qinv = 0.0f;
    if (q8) {               // one more pass for the row's absolute maximum
        float amax = 0.0f;
        for (int i = lane; i < n4; i += 32) {
            const float4 v = xr[i];
            const float4 ww = reinterpret_cast<const float4 *>(w)[i];
            const float4 bb = reinterpret_cast<const float4 *>(b)[i];
            float y[4] = {((v.x - muf) * inv) * ww.x + bb.x, ((v.y - muf) * inv) * ww.y + bb.y,
                          ((v.z - muf) * inv) * ww.z + bb.z, ((v.w - muf) * inv) * ww.w + bb.w};
#pragma unroll
            for (int j = 0; j < 4; j++) amax = fmaxf(amax, fabsf(act == ACT_SILU ? silu_f(y[j]) : y[j]));
        }
        amax = warp_max(amax);
        qinv = amax > 0.0f ? 127.0f / amax : 0.0f;
        if (lane == 0) sx8[row] = amax > 0.0f ? amax / 127.0f : 0.0f;
    }
    for (int i = lane; i < n4; i += 32) {
        const float4 v = xr[i];
        const float4 ww = reinterpret_cast<const float4 *>(w)[i];
        const float4 bb = reinterpret_cast<const float4 *>(b)[i];
        float y[4] = {((v.x - muf) * inv) * ww.x + bb.x, ((v.y - muf) * inv) * ww.y + bb.y,
                      ((v.z - muf) * inv) * ww.z + bb.z, ((v.w - muf) * inv) * ww.w + bb.w};
        if (act == ACT_SILU) {
#pragma unroll
            for (int j = 0; j < 4; j++) y[j] = silu_f(y[j]);
        }
        if (q8) reinterpret_cast<char4 *>(q8 + (size_t)row * d)[i] = make_char4(act_q8(y[0], qinv), act_q8(y[1], qinv), act_q8(y[2], qinv), act_q8(y[3], qinv));
        if (out) reinterpret_cast<float4 *>(out + (size_t)row * d)[i] = make_float4(y[0], y[1], y[2], y[3]);
        if (hi) {
            __align__(8) __half h[4], l[4];
#pragma unroll
            for (int j = 0; j < 4; j++) split_h16(y[j], h[j], l[j]);
            reinterpret_cast<uint2 *>(hi + (size_t)row * d)[i] = *reinterpret_cast<uint2 *>(h);
            if (lo) reinterpret_cast<uint2 *>(lo + (size_t)row * d)[i] = *reinterpret_cast<uint2 *>(l);
        }
    }
}

// The same arithmetic with the row held in registers (d = NV * 128): one read of x instead of three.
template <int NV>
__global__ void __launch_bounds__(256)
ln_reg_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ b,
              float *__restrict__ out, __half *__restrict__ hi, __half *__restrict__ lo, int8_t *__restrict__ q8,
              float *__restrict__ sx8, int T, int act) {
    chain_trigger();
    chain_wait();
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= T) return;
    ln_row<NV, false>(x, w, b, out, hi, lo, q8, sx8, row, act, lane);
}

int layer_norm(const float *x, const float *w, const float *b, float *out_f32, H16 out_h, int T, int d, int act,
               cudaStream_t st, bool chain) {
    return layer_norm_q8(x, w, b, out_f32, out_h, nullptr, nullptr, T, d, act, st, chain);
}

int layer_norm_q8(const float *x, const float *w, const float *b, float *out_f32, H16 out_h, int8_t *q8, float *sx8, int T, int d,
                  int act, cudaStream_t st, bool chain) {
    if (T <= 0) return 0;
    if (d % 4) { set_error("layer_norm: d=%d must be a multiple of 4", d); return -1; }
    const dim3 grid(cdiv(T, 8));
#define LN_REG(NV) MB_CUDA(launch_kernel(ln_reg_kernel<NV>, grid, dim3(256), 0, st, chain, 1, x, w, b, out_f32, out_h.hi, out_h.lo, q8, sx8, T, act))
    if (d == 128) LN_REG(1);
    else if (d == 256) LN_REG(2);
    else if (d == 512) LN_REG(4);
    else if (d == 640) LN_REG(5);
    else if (d == 1024) LN_REG(8);
    else if (d == 2048) LN_REG(16);
    else
#undef LN_REG
    ln_kernel<<<cdiv(T, 8), 256, 0, st>>>(x, w, b, out_f32, out_h.hi, out_h.lo, q8, sx8, T, d, act);
    MB_CUDA(cudaGetLastError());
    return 0;
}

// -------------------------------------------------- GLU + depthwise conv (+BN+SiLU)
// h2 [rows, 2d]: a = h2[:, :d], b = h2[:, d:], g = a * sigmoid(b). Depthwise conv of
// width k along time with zero padding at the segment edges (causal: k-1 on the
// left; symmetric: (k-1)/2 each side) — src/encoder.c:421-444. A block covers 128 channels
// x a time tile of TT rows; the tile plus its k-1 halo is staged in shared memory so every GLU
// value is computed once. A thread owns four adjacent channels (16-byte loads, 8-byte plane
// stores) and four consecutive output rows, whose windows it slides through registers.
static constexpr int DW_TT = 64;
static constexpr int DW_CH = 128;
static constexpr int DW_TY = 16;                  // thread rows per block: DW_TT / DW_TY outputs each
static constexpr int DW_RPT = DW_TT / DW_TY;      // 4
static constexpr int DW_KMAX = 32;

template <int KW>      // KW > 0: compile-time kernel width; 0: runtime width up to DW_KMAX
__global__ void __launch_bounds__(32 * DW_TY)
glu_dw_kernel(const float *__restrict__ h2, const float *__restrict__ dw_w, const float *__restrict__ dw_b,
              const float *__restrict__ scale, const float *__restrict__ shift, float *__restrict__ out,
              __half *__restrict__ hi, __half *__restrict__ lo, const int *__restrict__ seg_off,
              const int *__restrict__ seg_len, int d, int k, int pad_left) {
    __shared__ float4 g[(DW_TT + DW_KMAX - 1) * (DW_CH / 4)];
    const int b = blockIdx.z;
    const int len = seg_len[b], off = seg_off[b];
    const int t0 = blockIdx.y * DW_TT;
    if (t0 >= len) return;
    const int c = blockIdx.x * DW_CH + 4 * threadIdx.x;           // d is a multiple of 4
    const bool cok = c < d;
    const int rows = DW_TT + k - 1;
    for (int r = threadIdx.y; r < rows; r += DW_TY) {
        const int t = t0 - pad_left + r;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (cok && t >= 0 && t < len) {
            const float *p = h2 + (size_t)(off + t) * (2 * d);
            const float4 x = *reinterpret_cast<const float4 *>(p + c), y = *reinterpret_cast<const float4 *>(p + d + c);
            v = make_float4(x.x * sigmoid_fast(y.x), x.y * sigmoid_fast(y.y), x.z * sigmoid_fast(y.z), x.w * sigmoid_fast(y.w));
        }
        g[r * (DW_CH / 4) + threadIdx.x] = v;
    }
    __syncthreads();
    if (!cok) return;
    const int tend = len - t0 < DW_TT ? len - t0 : DW_TT;
    const int tt0 = threadIdx.y * DW_RPT;
    if (tt0 >= tend) return;
    float4 acc[DW_RPT];
    const float4 bias = dw_b ? *reinterpret_cast<const float4 *>(dw_b + c) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < DW_RPT; i++) acc[i] = bias;
    // row tt0 + i uses staged rows tt0 + i + j, j < k: walk the staged rows once, each feeds up to DW_RPT outputs
    constexpr int KU = KW > 0 ? KW : DW_KMAX;
    const float *w0 = dw_w + (size_t)c * k, *w1 = w0 + k, *w2 = w1 + k, *w3 = w2 + k;
#pragma unroll
    for (int rr = 0; rr < KU + DW_RPT - 1; rr++) {
        if (KW == 0 && rr >= k + DW_RPT - 1) break;
        const float4 v = g[(tt0 + rr) * (DW_CH / 4) + threadIdx.x];
#pragma unroll
        for (int i = 0; i < DW_RPT; i++) {
            const int j = rr - i;                                 // tap of output i fed by this row
            if (j >= 0 && j < KU && (KW > 0 || j < k)) {
                acc[i].x = fmaf(w0[j], v.x, acc[i].x); acc[i].y = fmaf(w1[j], v.y, acc[i].y);
                acc[i].z = fmaf(w2[j], v.z, acc[i].z); acc[i].w = fmaf(w3[j], v.w, acc[i].w);
            }
        }
    }
    float4 sc = make_float4(1.f, 1.f, 1.f, 1.f), sh = make_float4(0.f, 0.f, 0.f, 0.f);
    if (scale) { sc = *reinterpret_cast<const float4 *>(scale + c); sh = *reinterpret_cast<const float4 *>(shift + c); }
#pragma unroll
    for (int i = 0; i < DW_RPT; i++) {
        if (tt0 + i >= tend) break;
        const size_t o = (size_t)(off + t0 + tt0 + i) * d + c;
        if (scale) {
            const float y[4] = {silu_f(acc[i].x * sc.x + sh.x), silu_f(acc[i].y * sc.y + sh.y), silu_f(acc[i].z * sc.z + sh.z),
                                silu_f(acc[i].w * sc.w + sh.w)};
            if (hi) {
                __align__(8) __half h[4], l[4];
#pragma unroll
                for (int e = 0; e < 4; e++) split_h16(y[e], h[e], l[e]);
                *reinterpret_cast<uint2 *>(hi + o) = *reinterpret_cast<const uint2 *>(h);
                if (lo) *reinterpret_cast<uint2 *>(lo + o) = *reinterpret_cast<const uint2 *>(l);
            }
            if (out) *reinterpret_cast<float4 *>(out + o) = make_float4(y[0], y[1], y[2], y[3]);
        } else {
            *reinterpret_cast<float4 *>(out + o) = acc[i];
        }
    }
}

int glu_dwconv(const float *h2, const float *dw_w, const float *dw_b, const float *scale, const float *shift,
               float *out_f32, H16 out_h, const int *seg_off, const int *seg_len, int batch, int max_len, int d,
               int k, int pad_left, cudaStream_t st) {
    if (batch <= 0 || max_len <= 0) return 0;
    if (k > DW_KMAX) { set_error("glu_dwconv: kernel width %d > %d", k, DW_KMAX); return -1; }
    if (d % 4) { set_error("glu_dwconv: d=%d must be a multiple of 4", d); return -1; }
    dim3 grid(cdiv(d, DW_CH), cdiv(max_len, DW_TT), batch);
    if (k == 9)
        glu_dw_kernel<9><<<grid, dim3(32, DW_TY), 0, st>>>(h2, dw_w, dw_b, scale, shift, out_f32, out_h.hi, out_h.lo, seg_off,
                                                 seg_len, d, k, pad_left);
    else
        glu_dw_kernel<0><<<grid, dim3(32, DW_TY), 0, st>>>(h2, dw_w, dw_b, scale, shift, out_f32, out_h.hi, out_h.lo, seg_off,
                                                 seg_len, d, k, pad_left);
    MB_CUDA(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------- misc
__global__ void scale_kernel(float *x, size_t n, float s) {
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i < n) x[i] *= s;
}
int scale_inplace(float *x, size_t n, float s, cudaStream_t st) {
    if (n == 0 || s == 1.0f) return 0;
    scale_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(x, n, s);
    MB_CUDA(cudaGetLastError());
    return 0;
}

// Relative positional embedding [2T-1, d]: row p is position T-1-p, interleaved
// sin/cos of pos * 10000^(-2j/d), evaluated in double (src/encoder.c:201-211).
__global__ void pos_emb_kernel(__half *hi, __half *lo, int T, int d) {
    const int p = blockIdx.x;
    const double pos = (double)(T - 1 - p);
    for (int j = threadIdx.x; j < d / 2; j += blockDim.x) {
        const double f = pos * pow(10000.0, -2.0 * j / (double)d);
        const float s = (float)sin(f), c = (float)cos(f);
        __half h, l;
        split_h16(s, h, l);
        hi[(size_t)p * d + 2 * j] = h; lo[(size_t)p * d + 2 * j] = l;
        split_h16(c, h, l);
        hi[(size_t)p * d + 2 * j + 1] = h; lo[(size_t)p * d + 2 * j + 1] = l;
    }
}
int pos_emb(H16 pe, int T, int d, cudaStream_t st) {
    if (T <= 0) return 0;
    pos_emb_kernel<<<2 * T - 1, 128, 0, st>>>(pe.hi, pe.lo, T, d);
    MB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace mb
