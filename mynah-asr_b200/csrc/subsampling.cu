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
