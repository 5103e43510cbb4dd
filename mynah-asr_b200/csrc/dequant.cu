// Block-format decode on device: ggml Q8_0 / Q4_0 / Q4_K / Q6_K and the reference's
// own per-row int8 / per-32 int4 -> f32, and f32 -> fp16 (hi, lo) operand planes.
// Layouts and arithmetic follow third_party/ingot/src/dequant.c:55-83,131-156,
// 222-273,352-445 (ggml) and src/qmat.c:152-169 (native). Every product below is
// exact in f32 (an f16 scale has 11 significant bits, the integer factor at most
// 8), so the decoded values are bit-identical to the reference's eager decode.
#include "kernels.h"

namespace mb {

__device__ __forceinline__ float f16_at(const uint8_t *p) {
    return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8))));
}

// One thread per 32-element block (Q8_0, Q4_0) ----------------------------------
__global__ void dq_q8_0_kernel(const uint8_t *src, float *dst, size_t nblk) {
    size_t b = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (b >= nblk) return;
    const uint8_t *blk = src + b * 34;
    const float d = f16_at(blk);
    float *o = dst + b * 32;
#pragma unroll
    for (int i = 0; i < 32; i++) o[i] = d * (float)(int8_t)blk[2 + i];
}

__global__ void dq_q4_0_kernel(const uint8_t *src, float *dst, size_t nblk) {
    size_t b = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (b >= nblk) return;
    const uint8_t *blk = src + b * 18;
    const float d = f16_at(blk);
    float *o = dst + b * 32;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const uint8_t q = blk[2 + i];
        o[i] = d * (float)((int)(q & 0x0F) - 8);
        o[i + 16] = d * (float)((int)(q >> 4) - 8);
    }
}

// One thread per 32-element sub-block of a 256-element super-block -----------------
__device__ __forceinline__ void k4_scale_min(const uint8_t *s, int j, int &sc, int &mn) {
    if (j < 4) { sc = s[j] & 63; mn = s[j + 4] & 63; }
    else { sc = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4); mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4); }
}

__global__ void dq_q4_k_kernel(const uint8_t *src, float *dst, size_t nsub) {
    size_t s = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (s >= nsub) return;
    const size_t b = s >> 3;
    const int j = (int)(s & 7);
    const uint8_t *blk = src + b * 144;
    const float d = f16_at(blk), dmin = f16_at(blk + 2);
    int sc, mn;
    k4_scale_min(blk + 4, j, sc, mn);
    const float dd = d * (float)sc, mm = dmin * (float)mn;
    const uint8_t *q = blk + 16 + (j >> 1) * 32;
    float *o = dst + b * 256 + j * 32;
    const int sh = (j & 1) * 4;
#pragma unroll
    for (int i = 0; i < 32; i++) o[i] = dd * (float)((q[i] >> sh) & 0x0F) - mm;
}

__global__ void dq_q6_k_kernel(const uint8_t *src, float *dst, size_t nsub) {
    size_t s = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (s >= nsub) return;
    const size_t b = s >> 3;
    const int sub = (int)(s & 7), half = sub >> 2, j = sub & 3;
    const uint8_t *blk = src + b * 210;
    const uint8_t *ql = blk + half * 64 + (j & 1) * 32;
    const uint8_t *qh = blk + 128 + half * 32;
    const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192) + half * 8;
    const float d = f16_at(blk + 208);
    float *o = dst + b * 256 + half * 128 + j * 32;
#pragma unroll
    for (int i = 0; i < 32; i++) {
        const int lo = (j < 2) ? (ql[i] & 0x0F) : (ql[i] >> 4);
        const int q = (lo | (((qh[i] >> (2 * j)) & 3) << 4)) - 32;
        o[i] = d * (float)sc[(i >> 4) + 2 * j] * (float)q;
    }
}

// Reference-native formats (src/qmat.c:152-169) ------------------------------------
__global__ void dq_mq8_kernel(const int8_t *q, const float *scales, float *dst, int n, int k) {
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i >= (size_t)n * k) return;
    dst[i] = (float)q[i] * scales[i / k];
}
__global__ void dq_mq4_kernel(const uint8_t *q, const float *scales, float *dst, int n, int k) {
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;   // one byte = two elements
    if (i >= (size_t)n * k / 2) return;
    const size_t e = i * 2;
    const float s = scales[e / 32];
    const uint8_t b = q[i];
    dst[e] = (float)((int)(b & 0x0F) - 8) * s;
    dst[e + 1] = (float)((int)(b >> 4) - 8) * s;
}

int dequant_to_f32(int fmt, const void *src, const float *scales, float *dst, int n, int k, cudaStream_t st) {
    const size_t ne = (size_t)n * k;
    const int TPB = 256;
    switch (fmt) {
    case FMT_F32:
        MB_CUDA(cudaMemcpyAsync(dst, src, ne * 4, cudaMemcpyDeviceToDevice, st));
        return 0;
    case FMT_GGML_Q8_0:
        dq_q8_0_kernel<<<(unsigned)((ne / 32 + TPB - 1) / TPB), TPB, 0, st>>>((const uint8_t *)src, dst, ne / 32);
        break;
    case FMT_GGML_Q4_0:
        dq_q4_0_kernel<<<(unsigned)((ne / 32 + TPB - 1) / TPB), TPB, 0, st>>>((const uint8_t *)src, dst, ne / 32);
        break;
    case FMT_GGML_Q4_K:
        dq_q4_k_kernel<<<(unsigned)((ne / 32 + TPB - 1) / TPB), TPB, 0, st>>>((const uint8_t *)src, dst, ne / 32);
        break;
    case FMT_GGML_Q6_K:
        dq_q6_k_kernel<<<(unsigned)((ne / 32 + TPB - 1) / TPB), TPB, 0, st>>>((const uint8_t *)src, dst, ne / 32);
        break;
    case FMT_MYNAH_Q8:
        dq_mq8_kernel<<<(unsigned)((ne + TPB - 1) / TPB), TPB, 0, st>>>((const int8_t *)src, scales, dst, n, k);
        break;
    case FMT_MYNAH_Q4:
        dq_mq4_kernel<<<(unsigned)((ne / 2 + TPB - 1) / TPB), TPB, 0, st>>>((const uint8_t *)src, scales, dst, n, k);
        break;
    default:
        set_error("dequant: unknown format %d", fmt);
        return -1;
    }
    MB_CUDA(cudaGetLastError());
    return 0;
}

size_t format_bytes(int fmt, int n, int k) {
    const size_t ne = (size_t)n * k;
    switch (fmt) {
    case FMT_F32: return ne * 4;
    case FMT_GGML_Q8_0: return ne / 32 * 34;
    case FMT_GGML_Q4_0: return ne / 32 * 18;
    case FMT_GGML_Q4_K: return ne / 256 * 144;
    case FMT_GGML_Q6_K: return ne / 256 * 210;
    case FMT_MYNAH_Q8: return ne;
    case FMT_MYNAH_Q4: return ne / 2;
    default: return 0;
    }
}

int format_block(int fmt) {
    switch (fmt) {
    case FMT_GGML_Q4_K: case FMT_GGML_Q6_K: return 256;
    case FMT_F32: case FMT_MYNAH_Q8: return 1;
    default: return 32;
    }
}

// f32 -> (hi, lo) fp16 planes -------------------------------------------------------
__global__ void split_kernel(const float *__restrict__ x, __half *__restrict__ hi, __half *__restrict__ lo,
                             size_t n4, float scale, int *status) {
    size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const float4 v = reinterpret_cast<const float4 *>(x)[i];
    __align__(8) __half h[4], l[4];
    bool fits = split_h16(v.x * scale, h[0], l[0]);
    fits &= split_h16(v.y * scale, h[1], l[1]);
    fits &= split_h16(v.z * scale, h[2], l[2]);
    fits &= split_h16(v.w * scale, h[3], l[3]);
    reinterpret_cast<uint2 *>(hi)[i] = *reinterpret_cast<uint2 *>(h);
    if (lo) reinterpret_cast<uint2 *>(lo)[i] = *reinterpret_cast<uint2 *>(l);
    if (!fits && status) atomicCAS(status, ST_OK, ST_RANGE);
}

int split_to_h16(const float *x, __half *hi, __half *lo, size_t n, cudaStream_t st, int *status) {
    if (n == 0) return 0;
    if (n % 4) { set_error("split_to_h16: element count %zu not a multiple of 4", n); return -1; }
    const size_t n4 = n / 4;
    split_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(x, hi, lo, n4, 1.0f, status);
    MB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace mb
