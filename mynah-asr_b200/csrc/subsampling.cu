// dw-striding 8x subsampling front-end (the reference's conv2d_s2 /
// mynah_asr_subsampling_forward, src/subsampling.c:107-269), channel-last on device.
//
// The reference keeps activations channel-major [C, T, F] and runs the pointwise
// 1x1 convs as [C,C] x [C,S] GEMMs. Here activations are [T, F, C] so that
//   * the 3x3 stride-2 convs read and write 256 consecutive channels per (t, f)
//     (coalesced), and
//   * each pointwise conv is a plain row-major contraction [S, C] x [C, C]^T on the
//     tensor cores, its epilogue applying bias + ReLU, and the last one emits the
//     [T', F'*C] operand of the output linear directly (the linear's columns are
//     permuted once at load time from the reference's channel-major flatten
//     c*F'+f to f*C+c).
// Zero padding: causal (2 left, 1 right) or symmetric (1, 1) on both axes.
#include "kernels.h"

namespace mb {

// stage 0: full conv 1 -> C, 3x3, stride 2, + bias + ReLU.   feats [T,F] -> out [To,Fo,C]
__global__ void __launch_bounds__(256)
conv_in_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ b,
               float *__restrict__ out, int T, int F, int C, int To, int Fo, int pl) {
    const size_t total = (size_t)To * Fo * C;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        const int fo = (int)((i / C) % Fo);
        const int to = (int)(i / ((size_t)C * Fo));
        float acc = 0.0f;
#pragma unroll
        for (int dt = 0; dt < 3; dt++) {
            const int t = to * 2 - pl + dt;
            if (t < 0 || t >= T) continue;
#pragma unroll
            for (int df = 0; df < 3; df++) {
                const int f = fo * 2 - pl + df;
                if (f < 0 || f >= F) continue;
                acc += w[c * 9 + dt * 3 + df] * x[(size_t)t * F + f];
            }
        }
        out[i] = fmaxf(acc + b[c], 0.0f);
    }
}

int conv_in_relu(const float *feats, const float *w, const float *b, float *out, int T, int F, int C, int To, int Fo,
                 int pl, cudaStream_t st) {
    const size_t total = (size_t)To * Fo * C;
    if (total == 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    conv_in_kernel<<<blocks, 256, 0, st>>>(feats, w, b, out, T, F, C, To, Fo, pl);
    MB_CUDA(cudaGetLastError());
    return 0;
}

// stage 0 fused into the first depthwise conv: the [T1, F1, C] activation of stage 0 (the
// largest tensor of the whole model: 196 MB for 60 s of audio) is never materialised.
// Every stage-1 output needs a 3x3 patch of stage-0 outputs, i.e. a 7x7 patch of the
// input; a CTA stages the input rows it needs in shared memory (read by all channels as
// broadcasts, fetched as 16-byte pieces into registers) and one thread per channel recomputes the
// nine stage-0 values in registers.
// Stage-0 positions outside [0,T1) x [0,F1) are the depthwise conv's own zero padding.
static constexpr int FUSE_F2 = 8;      // stage-1 frequency positions per CTA

__global__ void __launch_bounds__(256)
conv_in_dw_kernel(const float *__restrict__ x, const float *__restrict__ w0, const float *__restrict__ b0,
                  const float *__restrict__ w1, const float *__restrict__ b1, __half *__restrict__ hi,
                  __half *__restrict__ lo, int T, int F, int C, int T1, int F1, int T2, int F2, int pl) {
    __shared__ __align__(16) float patch[7][4 * FUSE_F2 + 4];
    const int t2 = blockIdx.y, f2base = blockIdx.x * FUSE_F2;
    // stage-0 rows 2*t2 - pl + {0,1,2} need input rows 2*(that) - pl + {0,1,2}
    const int trow0 = 2 * (2 * t2 - pl) - pl;           // first input row of the patch
    const int fcol0 = 2 * (2 * f2base - pl) - pl;       // first input column of the patch
    const int pw = 4 * FUSE_F2 + 3;
    for (int i = threadIdx.x; i < 7 * pw; i += blockDim.x) {
        const int r = i / pw, c = i % pw, t = trow0 + r, f = fcol0 + c;
        patch[r][c] = (t >= 0 && t < T && f >= 0 && f < F) ? x[(size_t)t * F + f] : 0.0f;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float k0[9], k1[9];
#pragma unroll
        for (int i = 0; i < 9; i++) { k0[i] = w0[c * 9 + i]; k1[i] = w1[c * 9 + i]; }
        const float bias0 = b0[c], bias1 = b1[c];
        for (int j = 0; j < FUSE_F2; j++) {
            const int f2 = f2base + j;
            if (f2 >= F2) break;
            // the 7 x 7 input window of this output, as 16-byte broadcast loads (one shared-memory
            // instruction per four values instead of one per multiply-add)
            float in[7][8];
#pragma unroll
            for (int r = 0; r < 7; r++) {
                const float4 lo4 = *reinterpret_cast<const float4 *>(&patch[r][4 * j]);
                const float4 hi4 = *reinterpret_cast<const float4 *>(&patch[r][4 * j + 4]);
                in[r][0] = lo4.x; in[r][1] = lo4.y; in[r][2] = lo4.z; in[r][3] = lo4.w;
                in[r][4] = hi4.x; in[r][5] = hi4.y; in[r][6] = hi4.z; in[r][7] = hi4.w;
            }
            float acc = 0.0f;
#pragma unroll
            for (int dt = 0; dt < 3; dt++) {
                const int t1 = 2 * t2 - pl + dt;
                if (t1 < 0 || t1 >= T1) continue;
#pragma unroll
                for (int df = 0; df < 3; df++) {
                    const int f1 = 2 * f2 - pl + df;
                    if (f1 < 0 || f1 >= F1) continue;
                    // stage-0 output (t1, f1): input window starts at patch row 2*dt, column 4*j + 2*df
                    float v = 0.0f;
#pragma unroll
                    for (int a = 0; a < 3; a++)
#pragma unroll
                        for (int b = 0; b < 3; b++) v += k0[a * 3 + b] * in[2 * dt + a][2 * df + b];
                    acc += k1[dt * 3 + df] * fmaxf(v + bias0, 0.0f);
                }
            }
            __half h, l;
            split_h16(bias1 + acc, h, l);
            const size_t o = ((size_t)t2 * F2 + f2) * C + c;
            hi[o] = h;
            lo[o] = l;
        }
    }
}

int conv_in_dw_fused(const float *feats, const float *w0, const float *b0, const float *w1, const float *b1, H16 out,
                     int T, int F, int C, int T1, int F1, int T2, int F2, int pl, cudaStream_t st) {
    if (T2 <= 0 || F2 <= 0) return 0;
    dim3 grid(cdiv(F2, FUSE_F2), T2);
    conv_in_dw_kernel<<<grid, 256, 0, st>>>(feats, w0, b0, w1, b1, out.hi, out.lo, T, F, C, T1, F1, T2, F2, pl);
    MB_CUDA(cudaGetLastError());
    return 0;
}

// stages 1-2: depthwise 3x3 stride 2 + bias.   x [T,F,C] f32 -> (hi,lo) [To*Fo, C]
__global__ void __launch_bounds__(256)
dw3x3_kernel(const float *__restrict__ x, const float *__restrict__ w, const float *__restrict__ b,
             __half *__restrict__ hi, __half *__restrict__ lo, int T, int F, int C, int To, int Fo, int pl) {
    const size_t total = (size_t)To * Fo * C;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        const int fo = (int)((i / C) % Fo);
        const int to = (int)(i / ((size_t)C * Fo));
        float acc = 0.0f;
#pragma unroll
        for (int dt = 0; dt < 3; dt++) {
            const int t = to * 2 - pl + dt;
            if (t < 0 || t >= T) continue;
#pragma unroll
            for (int df = 0; df < 3; df++) {
                const int f = fo * 2 - pl + df;
                if (f < 0 || f >= F) continue;
                acc += w[c * 9 + dt * 3 + df] * x[((size_t)t * F + f) * C + c];
            }
        }
        __half h, l;
        split_h16(b[c] + acc, h, l);
        hi[i] = h;
        lo[i] = l;
    }
}

int dwconv3x3_s2(const float *x, const float *w, const float *b, H16 out, int T, int F, int C, int To, int Fo, int pl,
                 cudaStream_t st) {
    const size_t total = (size_t)To * Fo * C;
    if (total == 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    dw3x3_kernel<<<blocks, 256, 0, st>>>(x, w, b, out.hi, out.lo, T, F, C, To, Fo, pl);
    MB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace mb
