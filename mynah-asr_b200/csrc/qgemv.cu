// Small-M quantised matmul: out[T,n] = x[T,k] W^T for a handful of rows (decoder
// steps, streaming chunks), streaming the STORED blocks from HBM exactly once — the
// device counterpart of the reference's T <= 16 branch of mynah_asr_qmat_mul
// (src/qmat.c:508-597). This path is bound by HBM bandwidth: per weight row the
// kernel moves n*k*bytes_per_param and does 2*T flops per weight.
//
// Work split: lanes own fixed positions of a 1024-wide slice of K (one 32-element
// block each), so a lane's activations live in registers for the whole kernel;
// warps of a CTA split K into 1024-slices (k <= 8192, the reference's QMAT_K_MAX)
// and rows into groups; every warp streams RPI rows per step. Block formats whose
// rows are not 16-byte aligned (18/34/210-byte blocks) are staged through shared
// memory with cp.async on aligned 16-byte chunks and decoded from there.
//
// Two arithmetic modes, as in the reference:
//   A16  f32 activations x exactly decoded weights, f32 FMA    (default)
//   A8   activations quantised per row to int8 (quantize_act_int8, src/qmat.c:186-202)
//        and integer block dots (dp4a); the int32 dot of every 32-block is exact
#include <mutex>

#include "../../include/mynah_b200.h"
#include "kernels.h"
#include "qweight.h"

namespace mb {

static constexpr int QV_WARPS = 8;
static constexpr int QV_RPI = 4;          // rows in flight per warp
static constexpr int QV_STAGE = 1152;     // bytes per staged row slice (34*32 + alignment slack)

__device__ __forceinline__ void cp_async16(void *dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ float h16_at(const uint8_t *p) {
    return __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(p)));
}

template <int FMT> struct Fmt;
template <> struct Fmt<FMT_F32>       { static constexpr bool staged = false; };
template <> struct Fmt<FMT_MYNAH_Q8>  { static constexpr bool staged = false; };
template <> struct Fmt<FMT_MYNAH_Q4>  { static constexpr bool staged = false; };
template <> struct Fmt<FMT_GGML_Q8_0> { static constexpr bool staged = true; };
template <> struct Fmt<FMT_GGML_Q4_0> { static constexpr bool staged = true; };
template <> struct Fmt<FMT_GGML_Q4_K> { static constexpr bool staged = true; };
template <> struct Fmt<FMT_GGML_Q6_K> { static constexpr bool staged = true; };

// bytes of one 1024-element K slice of a row
__host__ __device__ inline int slice_bytes(int fmt) {
    switch (fmt) {
    case FMT_GGML_Q8_0: return 32 * 34;
    case FMT_GGML_Q4_0: return 32 * 18;
    case FMT_GGML_Q4_K: return 4 * 144;
    case FMT_GGML_Q6_K: return 4 * 210;
    default: return 0;
    }
}

// Decode the 32 weights owned by `lane` from a staged row slice (block formats).
// Layouts: third_party/ingot/src/dequant.c:72-83 (Q4_0), 131-156 (Q8_0),
// 55-68 + 222-273 (Q4_K), 352-445 (Q6_K).
template <int FMT>
__device__ __forceinline__ void decode32(const uint8_t *s, int lane, float (&w)[32]) {
    if (FMT == FMT_GGML_Q8_0) {
        const uint8_t *p = s + lane * 34;
        const float d = h16_at(p);
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const unsigned short u = *reinterpret_cast<const unsigned short *>(p + 2 + 2 * i);
            w[2 * i] = d * (float)(int8_t)(u & 0xFF);
            w[2 * i + 1] = d * (float)(int8_t)(u >> 8);
        }
    } else if (FMT == FMT_GGML_Q4_0) {
        const uint8_t *p = s + lane * 18;
        const float d = h16_at(p);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const unsigned short u = *reinterpret_cast<const unsigned short *>(p + 2 + 2 * i);
            w[2 * i] = d * (float)((int)(u & 0xF) - 8);
            w[2 * i + 16] = d * (float)((int)((u >> 4) & 0xF) - 8);
            w[2 * i + 1] = d * (float)((int)((u >> 8) & 0xF) - 8);
            w[2 * i + 17] = d * (float)((int)(u >> 12) - 8);
        }
    } else if (FMT == FMT_GGML_Q4_K) {
        const uint8_t *p = s + (lane >> 3) * 144;
        const int j = lane & 7;
        const float d = h16_at(p), dmin = h16_at(p + 2);
        const uint8_t *sc = p + 4;
        int scv, mnv;
        if (j < 4) { scv = sc[j] & 63; mnv = sc[j + 4] & 63; }
        else { scv = (sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4); mnv = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
        const float dd = d * (float)scv, mm = dmin * (float)mnv;
        const uint8_t *q = p + 16 + (j >> 1) * 32;
        const int sh = (j & 1) * 4;
#pragma unroll
        for (int i = 0; i < 32; i++) w[i] = dd * (float)((q[i] >> sh) & 0x0F) - mm;
    } else if (FMT == FMT_GGML_Q6_K) {
        const uint8_t *p = s + (lane >> 3) * 210;
        const int sub = lane & 7, half = sub >> 2, j = sub & 3;
        const uint8_t *ql = p + half * 64 + (j & 1) * 32;
        const uint8_t *qh = p + 128 + half * 32;
        const int8_t *sc = reinterpret_cast<const int8_t *>(p + 192) + half * 8 + 2 * j;
        const float d = h16_at(p + 208);
        const float d0 = d * (float)sc[0], d1 = d * (float)sc[1];
#pragma unroll
        for (int i = 0; i < 32; i++) {
            const int lo4 = (j < 2) ? (ql[i] & 0x0F) : (ql[i] >> 4);
            const int q = (lo4 | (((qh[i] >> (2 * j)) & 3) << 4)) - 32;
            w[i] = (i < 16 ? d0 : d1) * (float)q;
        }
    }
}

struct QvArgs {
    const uint8_t *raw;
    const float *scales;
    int n, k;
    size_t row_bytes;
    const float *x;
    int ldx;
    float *out;
    int ldo;
    const float *bias;
    int T;
};

template <int FMT, int TB>
__global__ void __launch_bounds__(QV_WARPS * 32)
qgemv_kernel(const QvArgs a, const int kch, const int rg_count) {
    __shared__ __align__(16) uint8_t stage[Fmt<FMT>::staged ? QV_WARPS * QV_RPI * QV_STAGE : 16];
    __shared__ float red[QV_WARPS][QV_RPI][TB];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ch = warp % kch, rg = warp / kch;
    const bool warp_on = rg < rg_count;
    const int kbase = ch * 1024;
    // which 32 elements this lane owns, and whether they exist
    constexpr bool interleaved = FMT == FMT_F32;      // element j*32+lane instead of lane*32+j
    const bool lane_on = interleaved ? true : (kbase + lane * 32 < a.k);

    float xr[TB][32];
#pragma unroll
    for (int t = 0; t < TB; t++)
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const int e = kbase + (interleaved ? j * 32 + lane : lane * 32 + j);
            xr[t][j] = (t < a.T && e < a.k) ? a.x[(size_t)t * a.ldx + e] : 0.0f;
        }

    const int tile_rows = rg_count * QV_RPI;
    for (int tile = blockIdx.x * tile_rows; tile < a.n; tile += gridDim.x * tile_rows) {
        const int row0 = tile + rg * QV_RPI;
        float acc[QV_RPI][TB];
#pragma unroll
        for (int r = 0; r < QV_RPI; r++)
#pragma unroll
            for (int t = 0; t < TB; t++) acc[r][t] = 0.0f;

        if (warp_on) {
            if (Fmt<FMT>::staged) {
                const int sb = slice_bytes(FMT);
                uint8_t *ws = stage + warp * QV_RPI * QV_STAGE;
#pragma unroll
                for (int r = 0; r < QV_RPI; r++) {
                    if (row0 + r >= a.n) continue;
                    const uint8_t *src = a.raw + (size_t)(row0 + r) * a.row_bytes + (size_t)ch * sb;
                    const size_t left = a.row_bytes - (size_t)ch * sb;
                    const int nb = left < (size_t)sb ? (int)left : sb;
                    const uintptr_t s0 = reinterpret_cast<uintptr_t>(src) & ~uintptr_t(15);
                    const int span = (int)(((reinterpret_cast<uintptr_t>(src) + nb + 15) & ~uintptr_t(15)) - s0);
                    for (int o = lane * 16; o < span; o += 512)
                        cp_async16(ws + r * QV_STAGE + o, reinterpret_cast<const void *>(s0 + o));
                }
                cp_async_wait_all();
                __syncwarp();
#pragma unroll
                for (int r = 0; r < QV_RPI; r++) {
                    if (row0 + r >= a.n || !lane_on) continue;
                    const uint8_t *src = a.raw + (size_t)(row0 + r) * a.row_bytes + (size_t)ch * sb;
                    float w[32];
                    decode32<FMT>(ws + r * QV_STAGE + (reinterpret_cast<uintptr_t>(src) & 15), lane, w);
#pragma unroll
                    for (int j = 0; j < 32; j++)
#pragma unroll
                        for (int t = 0; t < TB; t++) acc[r][t] += w[j] * xr[t][j];
                }
                __syncwarp();
            } else if (FMT == FMT_F32) {
#pragma unroll
                for (int r = 0; r < QV_RPI; r++) {
                    if (row0 + r >= a.n) continue;
                    const float *wr = reinterpret_cast<const float *>(a.raw) + (size_t)(row0 + r) * a.k + kbase;
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int e = j * 32 + lane;
                        const float wv = (kbase + e < a.k) ? __ldg(wr + e) : 0.0f;
#pragma unroll
                        for (int t = 0; t < TB; t++) acc[r][t] += wv * xr[t][j];
                    }
                }
            } else if (FMT == FMT_MYNAH_Q8) {
#pragma unroll
                for (int r = 0; r < QV_RPI; r++) {
                    if (row0 + r >= a.n || !lane_on) continue;
                    const int8_t *wr = reinterpret_cast<const int8_t *>(a.raw) + (size_t)(row0 + r) * a.k + kbase + lane * 32;
                    const float s = a.scales[row0 + r];
                    __align__(16) int8_t q[32];
                    *reinterpret_cast<uint4 *>(q) = __ldg(reinterpret_cast<const uint4 *>(wr));
                    *reinterpret_cast<uint4 *>(q + 16) = __ldg(reinterpret_cast<const uint4 *>(wr) + 1);
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const float wv = (float)q[j] * s;          // dequant_row, src/qmat.c:153-156
#pragma unroll
                        for (int t = 0; t < TB; t++) acc[r][t] += wv * xr[t][j];
                    }
                }
            } else if (FMT == FMT_MYNAH_Q4) {
#pragma unroll
                for (int r = 0; r < QV_RPI; r++) {
                    if (row0 + r >= a.n || !lane_on) continue;
                    const size_t e0 = (size_t)(row0 + r) * a.k + kbase + lane * 32;
                    const float s = a.scales[e0 / 32];
                    __align__(16) uint8_t q[16];
                    *reinterpret_cast<uint4 *>(q) = __ldg(reinterpret_cast<const uint4 *>(a.raw + e0 / 2));
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const float w0 = (float)((int)(q[j] & 0x0F) - 8) * s, w1 = (float)((int)(q[j] >> 4) - 8) * s;
#pragma unroll
                        for (int t = 0; t < TB; t++) acc[r][t] += w0 * xr[t][2 * j] + w1 * xr[t][2 * j + 1];
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < QV_RPI; r++)
#pragma unroll
                for (int t = 0; t < TB; t++) {
                    const float v = warp_sum(acc[r][t]);
                    if (lane == 0) red[warp][r][t] = v;
                }
        }
        __syncthreads();
        // K slices are combined in a fixed order so a row's bits never depend on scheduling
        if (warp_on && ch == 0 && lane < QV_RPI * TB) {
            const int r = lane / TB, t = lane % TB;
            if (row0 + r < a.n && t < a.T) {
                float v = 0.0f;
                for (int c = 0; c < kch; c++) v += red[rg * kch + c][r][t];
                if (a.bias) v += a.bias[row0 + r];
                a.out[(size_t)t * a.ldo + row0 + r] = v;
            }
        }
        __syncthreads();
    }
}

template <int FMT>
static int launch_fmt(const QvArgs &a0, cudaStream_t st) {
    int kch = 1;
    while (kch * 1024 < a0.k) kch *= 2;
    if (kch > QV_WARPS) { set_error("qgemv: k=%d exceeds %d", a0.k, QV_WARPS * 1024); return -1; }
    const int rg = QV_WARPS / kch;
    const int tile_rows = rg * QV_RPI;
    int blocks = cdiv(a0.n, tile_rows);
    if (blocks > 148 * 4) blocks = 148 * 4;
    for (int t0 = 0; t0 < a0.T; t0 += 4) {
        QvArgs a = a0;
        a.T = a0.T - t0 < 4 ? a0.T - t0 : 4;
        a.x = a0.x + (size_t)t0 * a0.ldx;
        a.out = a0.out + (size_t)t0 * a0.ldo;
        if (a.T == 1) qgemv_kernel<FMT, 1><<<blocks, QV_WARPS * 32, 0, st>>>(a, kch, rg);
        else if (a.T == 2) qgemv_kernel<FMT, 2><<<blocks, QV_WARPS * 32, 0, st>>>(a, kch, rg);
        else qgemv_kernel<FMT, 4><<<blocks, QV_WARPS * 32, 0, st>>>(a, kch, rg);
        MB_CUDA(cudaGetLastError());
    }
    return 0;
}

int qgemv(const QWeight &w, const float *x, int ldx, float *out, int ldo, const float *bias, int T, cudaStream_t st) {
    if (T <= 0 || w.n <= 0) return 0;
    if (w.fmt != FMT_F32 && w.k % 32) { set_error("qgemv: k=%d not a multiple of 32", w.k); return -1; }
    QvArgs a;
    a.raw = w.raw; a.scales = w.scales; a.n = w.n; a.k = w.k;
    a.row_bytes = format_bytes(w.fmt, 1, w.k);
    a.x = x; a.ldx = ldx; a.out = out; a.ldo = ldo; a.bias = bias; a.T = T;
    switch (w.fmt) {
    case FMT_F32: return launch_fmt<FMT_F32>(a, st);
    case FMT_MYNAH_Q8: return launch_fmt<FMT_MYNAH_Q8>(a, st);
    case FMT_MYNAH_Q4: return launch_fmt<FMT_MYNAH_Q4>(a, st);
    case FMT_GGML_Q8_0: return launch_fmt<FMT_GGML_Q8_0>(a, st);
    case FMT_GGML_Q4_0: return launch_fmt<FMT_GGML_Q4_0>(a, st);
    case FMT_GGML_Q4_K: return launch_fmt<FMT_GGML_Q4_K>(a, st);
    case FMT_GGML_Q6_K: return launch_fmt<FMT_GGML_Q6_K>(a, st);
    default: set_error("qgemv: unknown format %d", w.fmt); return -1;
    }
}

// ------------------------------------------------------------------- A8 mode
// One warp per (row t, weight row): lanes own one 32-block each per 1024 slice.
// Activation rows are quantised once by act_quant_kernel.
__global__ void __launch_bounds__(256)
act_quant_kernel(const float *__restrict__ x, int8_t *__restrict__ qx, float *__restrict__ sx, int T, int k) {
    const int t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    const float *xr = x + (size_t)t * k;
    float amax = 0.0f;
    for (int i = lane; i < k; i += 32) amax = fmaxf(amax, fabsf(xr[i]));
    amax = warp_max(amax);
    if (amax == 0.0f) {
        for (int i = lane; i < k; i += 32) qx[(size_t)t * k + i] = 0;
        if (lane == 0) sx[t] = 0.0f;
        return;
    }
    const float inv = 127.0f / amax;
    for (int i = lane; i < k; i += 32) {
        const float v = __fmul_rn(xr[i], inv);
        int q = (int)(v >= 0.0f ? __fadd_rn(v, 0.5f) : __fsub_rn(v, 0.5f));
        q = q > 127 ? 127 : (q < -127 ? -127 : q);
        qx[(size_t)t * k + i] = (int8_t)q;
    }
    if (lane == 0) sx[t] = amax / 127.0f;
}

template <int FMT>
__global__ void __launch_bounds__(256)
qgemv_a8_kernel(const uint8_t *__restrict__ raw, const float *__restrict__ scales, int n, int k, size_t row_bytes,
                const int8_t *__restrict__ qx, const float *__restrict__ sx, float *__restrict__ out,
                int32_t *__restrict__ dots, int T) {
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int t = blockIdx.y;
    if (row >= n) return;
    const int nblk = k / 32;
    float facc = 0.0f;
    int iacc = 0;
    for (int blk = lane; blk < nblk; blk += 32) {
        const int8_t *xa = qx + (size_t)t * k + blk * 32;
        int wq[8];
        float d = 1.0f;
        if (FMT == FMT_GGML_Q8_0) {
            const uint8_t *p = raw + (size_t)row * row_bytes + (size_t)blk * 34;
            d = h16_at(p);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const unsigned lo = *reinterpret_cast<const unsigned short *>(p + 2 + 4 * i);
                const unsigned hi = *reinterpret_cast<const unsigned short *>(p + 4 + 4 * i);
                wq[i] = (int)(lo | (hi << 16));
            }
        } else if (FMT == FMT_GGML_Q4_0) {
            const uint8_t *p = raw + (size_t)row * row_bytes + (size_t)blk * 18;
            d = h16_at(p);
            // element i = low nibble of byte i, element i+16 = high nibble
#pragma unroll
            for (int i = 0; i < 4; i++) {
                unsigned lo = 0, hi = 0;
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    const unsigned q = p[2 + 4 * i + b];
                    lo |= (((q & 0x0F) - 8) & 0xFF) << (8 * b);
                    hi |= (((q >> 4) - 8) & 0xFF) << (8 * b);
                }
                wq[i] = (int)lo;
                wq[4 + i] = (int)hi;
            }
        } else if (FMT == FMT_MYNAH_Q8) {
            const int8_t *p = reinterpret_cast<const int8_t *>(raw) + (size_t)row * k + blk * 32;
#pragma unroll
            for (int i = 0; i < 8; i++) wq[i] = *reinterpret_cast<const int *>(p + 4 * i);
        } else {   // FMT_MYNAH_Q4: byte j = element 2j | (2j+1) << 4
            const uint8_t *p = raw + ((size_t)row * k + blk * 32) / 2;
            d = scales[((size_t)row * k) / 32 + blk];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const unsigned q0 = p[2 * i], q1 = p[2 * i + 1];
                wq[i] = (int)((((q0 & 0x0F) - 8) & 0xFF) | ((((q0 >> 4) - 8) & 0xFF) << 8) |
                              ((((q1 & 0x0F) - 8) & 0xFF) << 16) | ((((q1 >> 4) - 8) & 0xFF) << 24));
            }
        }
        int dot = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) dot = __dp4a(wq[i], *reinterpret_cast<const int *>(xa + 4 * i), dot);
        if (dots) dots[((size_t)t * n + row) * nblk + blk] = dot;
        if (FMT == FMT_MYNAH_Q8) iacc += dot;
        else facc += (float)dot * d;
    }
    if (FMT == FMT_MYNAH_Q8) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) iacc += __shfl_xor_sync(0xffffffffu, iacc, o);
        // (float)int32 * ws * sx, left to right (src/qmat.c:299)
        if (lane == 0) out[(size_t)t * n + row] = __fmul_rn(__fmul_rn((float)iacc, scales[row]), sx[t]);
    } else {
        facc = warp_sum(facc);
        if (lane == 0) out[(size_t)t * n + row] = facc * sx[t];
    }
}

int act_quant_rows(const float *x, int8_t *qx, float *sx, int T, int k, cudaStream_t st) {
    if (T <= 0) return 0;
    act_quant_kernel<<<cdiv(T, 8), 256, 0, st>>>(x, qx, sx, T, k);
    MB_CUDA(cudaGetLastError());
    return 0;
}

int qgemv_a8(const QWeight &w, const float *x, float *out, int T, int32_t *block_dots, float *sx_out, cudaStream_t st) {
    if (T <= 0) return 0;
    if (w.k % 32) { set_error("qgemv_a8: k=%d not a multiple of 32", w.k); return -1; }
    int8_t *qx = nullptr;
    float *sx = sx_out;
    MB_CUDA(cudaMallocAsync(&qx, (size_t)T * w.k, st));
    if (!sx) MB_CUDA(cudaMallocAsync(&sx, (size_t)T * sizeof(float), st));
    act_quant_kernel<<<cdiv(T, 8), 256, 0, st>>>(x, qx, sx, T, w.k);
    dim3 grid(cdiv(w.n, 8), T);
    const size_t rb = format_bytes(w.fmt, 1, w.k);
    int rc = 0;
    switch (w.fmt) {
    case FMT_GGML_Q8_0: qgemv_a8_kernel<FMT_GGML_Q8_0><<<grid, 256, 0, st>>>(w.raw, w.scales, w.n, w.k, rb, qx, sx, out, block_dots, T); break;
    case FMT_GGML_Q4_0: qgemv_a8_kernel<FMT_GGML_Q4_0><<<grid, 256, 0, st>>>(w.raw, w.scales, w.n, w.k, rb, qx, sx, out, block_dots, T); break;
    case FMT_MYNAH_Q8: qgemv_a8_kernel<FMT_MYNAH_Q8><<<grid, 256, 0, st>>>(w.raw, w.scales, w.n, w.k, rb, qx, sx, out, block_dots, T); break;
    case FMT_MYNAH_Q4: qgemv_a8_kernel<FMT_MYNAH_Q4><<<grid, 256, 0, st>>>(w.raw, w.scales, w.n, w.k, rb, qx, sx, out, block_dots, T); break;
    default: set_error("qgemv_a8: format %d has no int8-activation mode", w.fmt); rc = -1;
    }
    if (rc == 0 && cudaGetLastError() != cudaSuccess) { set_error("qgemv_a8 launch failed"); rc = -1; }
    cudaFreeAsync(qx, st);
    if (!sx_out) cudaFreeAsync(sx, st);
    return rc;
}

// ------------------------------------------------- allocation-free A8 entry point
// Some hosts of this library must not allocate device memory once they are running:
// a streaming server that feeds chunks from a real-time audio thread cannot afford
// cudaMalloc / cudaFree (they serialise against every other stream of the process and
// take an unbounded time), and a deployment that sizes its GPU memory up front wants
// no pool growing behind its back. For them the int8-activation product is offered in
// a form whose only scratch — the quantised activation rows and their scales — lives
// in a fixed array inside the library image. Every GPU that loads the library carries
// these ~128 KB until the process exits.
static constexpr int NOALLOC_MAX_T = 16;        // rows of activations per call
static constexpr int NOALLOC_MAX_K = 8192;      // the reference's QMAT_K_MAX (src/qmat.c:181)
static constexpr size_t NOALLOC_SX_OFF = (size_t)NOALLOC_MAX_T * NOALLOC_MAX_K;
static __device__ __align__(256) unsigned char g_a8_scratch[NOALLOC_SX_OFF + 256];

// In host code `g_a8_scratch` is only a stand-in for the symbol, not a device address; the
// address has to be asked for once per device, with that device current.
static unsigned char *a8_scratch_for_current_device() {
    static std::mutex mu;
    static unsigned char *ptr[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { set_error("noalloc: cannot identify the current device"); return nullptr; }
    std::lock_guard<std::mutex> lk(mu);
    if (!ptr[dev]) {
        void *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_a8_scratch);
        if (e != cudaSuccess) { set_error("noalloc: cudaGetSymbolAddress -> %s", cudaGetErrorString(e)); return nullptr; }
        ptr[dev] = static_cast<unsigned char *>(p);
    }
    return ptr[dev];
}

}  // namespace mb

extern "C" int mynah_b200_qmat_mul_a8_static(const mynah_b200_qmat *m, const float *x_dev, float *out_dev, int T) {
    using namespace mb;
    if (!m || !x_dev || !out_dev || T < 0) { set_error("qmat_mul_a8_static: bad argument"); return -1; }
    if (T == 0) return 0;
    const QmatView v = qmat_view(m);
    const QWeight &w = *v.w;
    if (T > NOALLOC_MAX_T || w.k > NOALLOC_MAX_K) {
        set_error("qmat_mul_a8_static: T=%d, k=%d exceed the built-in scratch (T <= %d, k <= %d)", T, w.k, NOALLOC_MAX_T,
                  NOALLOC_MAX_K);
        return -1;
    }
    if (w.k % 32) { set_error("qmat_mul_a8_static: k=%d not a multiple of 32", w.k); return -1; }
    // every refusal happens before the first launch, so a refused call never touches the shared array
    if (w.fmt != FMT_GGML_Q8_0 && w.fmt != FMT_GGML_Q4_0 && w.fmt != FMT_MYNAH_Q8 && w.fmt != FMT_MYNAH_Q4) {
        set_error("qmat_mul_a8_static: format %d has no int8-activation mode (Q8_0, Q4_0 and the two native formats have)", w.fmt);
        return -1;
    }
    unsigned char *scratch = a8_scratch_for_current_device();      // first call on a device resolves the symbol
    if (!scratch) return -1;
    int8_t *qx = reinterpret_cast<int8_t *>(scratch);
    float *sx = reinterpret_cast<float *>(scratch + NOALLOC_SX_OFF);
    // nothing in the scratch has to start at zero: rows [0, T) of qx and sx are fully rewritten here
    act_quant_kernel<<<cdiv(T, 8), 256, 0, v.stream>>>(x_dev, qx, sx, T, w.k);
    dim3 grid(cdiv(w.n, 8), T);
    const size_t rb = format_bytes(w.fmt, 1, w.k);
    switch (w.fmt) {
    case FMT_GGML_Q8_0: qgemv_a8_kernel<FMT_GGML_Q8_0><<<grid, 256, 0, v.stream>>>(w.raw, w.scales, w.n, w.k, rb, qx, sx, out_dev, nullptr, T); break;
    case FMT_GGML_Q4_0: qgemv_a8_kernel<FMT_GGML_Q4_0><<<grid, 256, 0, v.stream>>>(w.raw, w.scales, w.n, w.k, rb, qx, sx, out_dev, nullptr, T); break;
    case FMT_MYNAH_Q8: qgemv_a8_kernel<FMT_MYNAH_Q8><<<grid, 256, 0, v.stream>>>(w.raw, w.scales, w.n, w.k, rb, qx, sx, out_dev, nullptr, T); break;
    case FMT_MYNAH_Q4: qgemv_a8_kernel<FMT_MYNAH_Q4><<<grid, 256, 0, v.stream>>>(w.raw, w.scales, w.n, w.k, rb, qx, sx, out_dev, nullptr, T); break;
    default: break;      // refused above
    }
    const cudaError_t le = cudaGetLastError();
    note_launch(2);
    const cudaError_t e = le != cudaSuccess ? le : cudaStreamSynchronize(v.stream);
    if (le != cudaSuccess) cudaStreamSynchronize(v.stream);    // the first kernel may be running: do not return over it
    if (e != cudaSuccess) { set_error("qmat_mul_a8_static: %s", cudaGetErrorString(e)); return -1; }
    return 0;
}
