// Log-mel front end (the reference's mynah_asr_log_mel, src/features.c:106-167):
// pre-emphasis -> zero centre pad n_fft/2 -> Hann window centred in n_fft ->
// radix-2 FFT in double -> |X|^2 -> sparse triangular mel projection in double ->
// log(x + guard) -> float; optional per-feature normalisation over the valid
// frames (mean, std with ddof=1, (x-mu)/(std+1e-5)).
//
// One CTA per frame: the frame is gathered straight from the f32 audio with the
// pre-emphasis applied on the fly, the FFT runs in shared memory in double (the
// reference keeps double for parity with its numpy oracle, src/features.c:13-15;
// at ~0.14 GFLOP per minute of audio it costs nothing), twiddles come from an exact
// host table. Frames >= valid stay zero, as in the reference.
#include "kernels.h"

namespace mb {

static constexpr int MEL_MAX_FFT = 1024;

// blockIdx.y selects one of several signals (streams of a lock-step group): signal y starts at
// audio + y * sig_stride and its frames go to feats + y * feat_stride. `base` is the absolute sample index
// of audio[0] (streaming keeps only the tail of the signal; 0 offline), t0 the first frame of this launch.
__global__ void __launch_bounds__(128)
mel_frame_kernel(const float *__restrict__ audio_all, long long S, const double *__restrict__ win,
                 const double *__restrict__ tw, const float *__restrict__ fb, const int *__restrict__ mlo,
                 const int *__restrict__ mhi, float *__restrict__ feats_all, int n_fft, int log2n, int hop, int n_mels,
                 double preemph, double guard, long long base, int t0, long long sig_stride, long long feat_stride) {
    // one double of padding after every 16: the bit-reversed stores and the small-stride stages would
    // otherwise pile a warp's accesses onto one bank pair
#define PD(i) ((i) + ((i) >> 4))
    __shared__ double re[MEL_MAX_FFT + MEL_MAX_FFT / 16], im[MEL_MAX_FFT + MEL_MAX_FFT / 16];
    const float *audio = audio_all + blockIdx.y * sig_stride - base;      // audio[s] is sample s of the signal
    float *feats = feats_all + blockIdx.y * feat_stride - (long long)t0 * n_mels;
    const int t = t0 + blockIdx.x;
    const long long start = (long long)t * hop - n_fft / 2;      // index into the unpadded signal
    for (int i = threadIdx.x; i < n_fft; i += blockDim.x) {
        const long long s = start + i;
        double y = 0.0;
        if (s >= 0 && s < S) y = s == 0 ? (double)audio[0] : (double)audio[s] - preemph * (double)audio[s - 1];
        const int r = (int)(__brev((unsigned)i) >> (32 - log2n));
        re[PD(r)] = y * win[i];
        im[PD(r)] = 0.0;
    }
    __syncthreads();
    for (int len = 2, sh = log2n - 1; len <= n_fft; len <<= 1, sh--) {
        const int half = len >> 1;
        for (int i = threadIdx.x; i < n_fft / 2; i += blockDim.x) {
            const int grp = i / half, k = i % half;
            const int a0 = grp * len + k, a = PD(a0), bq = PD(a0 + half);
            const double wr = tw[2 * (k << sh)], wi = tw[2 * (k << sh) + 1];
            const double xr = re[bq] * wr - im[bq] * wi, xi = re[bq] * wi + im[bq] * wr;
            re[bq] = re[a] - xr; im[bq] = im[a] - xi;
            re[a] += xr;         im[a] += xi;
        }
        __syncthreads();
    }
    const int nb = n_fft / 2 + 1;
    for (int i = threadIdx.x; i < nb; i += blockDim.x) re[PD(i)] = re[PD(i)] * re[PD(i)] + im[PD(i)] * im[PD(i)];   // power, in place
    __syncthreads();
    for (int m = threadIdx.x; m < n_mels; m += blockDim.x) {
        double acc = 0.0;
        for (int b = mlo[m]; b < mhi[m]; b++) acc += re[PD(b)] * (double)fb[(size_t)b * n_mels + m];
        feats[(size_t)t * n_mels + m] = (float)log(acc + guard);
    }
#undef PD
}

// per-feature normalisation: a CTA owns eight adjacent mel bins, thread (x, y) walks the frames y, y + 128, ..
// of bin x (a warp reads four 32-byte runs); mean, then the centred sum of squares, in double as the reference
static constexpr int MN_BX = 8, MN_BY = 128;

__device__ __forceinline__ double mel_norm_reduce(double v, double (*red)[MN_BX], int x, int y) {
    red[y][x] = v;
    __syncthreads();
    for (int o = MN_BY / 2; o > 0; o >>= 1) { if (y < o) red[y][x] += red[y + o][x]; __syncthreads(); }
    const double r = red[0][x];
    __syncthreads();
    return r;
}

__global__ void __launch_bounds__(MN_BX * MN_BY)
mel_norm_kernel(float *feats, int valid, int n_mels) {
    __shared__ double red[MN_BY][MN_BX];
    const int x = threadIdx.x, y = threadIdx.y, m = blockIdx.x * MN_BX + x;
    const bool on = m < n_mels;
    double s = 0.0;
    if (on) for (int t = y; t < valid; t += MN_BY) s += (double)feats[(size_t)t * n_mels + m];
    const double mu = mel_norm_reduce(s, red, x, y) / valid;
    double q = 0.0;
    if (on) for (int t = y; t < valid; t += MN_BY) { const double c = (double)feats[(size_t)t * n_mels + m] - mu; q += c * c; }
    const double inv = 1.0 / (sqrt(mel_norm_reduce(q, red, x, y) / (valid - 1)) + 1e-5);
    if (on) for (int t = y; t < valid; t += MN_BY) {
        float *v = feats + (size_t)t * n_mels + m;
        *v = (float)(((double)*v - mu) * inv);
    }
}

int log_mel_device(const MelCfg &c, const float *audio, size_t n_samples, const float *mel_fb, const int *mel_lo,
                   const int *mel_hi, const double *win, const double *twiddle, float *feats, int T, int valid,
                   cudaStream_t st) {
    if (c.n_fft > MEL_MAX_FFT || (c.n_fft & (c.n_fft - 1))) { set_error("log_mel: n_fft %d unsupported", c.n_fft); return -1; }
    MB_CUDA(cudaMemsetAsync(feats, 0, (size_t)T * c.n_mels * sizeof(float), st));
    if (valid <= 0) return 0;
    int log2n = 0;
    while ((1 << log2n) < c.n_fft) log2n++;
    mel_frame_kernel<<<valid, 128, 0, st>>>(audio, (long long)n_samples, win, twiddle, mel_fb, mel_lo, mel_hi, feats,
                                            c.n_fft, log2n, c.hop, c.n_mels, c.preemph, c.guard, 0, 0, 0, 0);
    MB_CUDA(cudaGetLastError());
    if (c.normalize && valid > 1) {
        mel_norm_kernel<<<cdiv(c.n_mels, MN_BX), dim3(MN_BX, MN_BY), 0, st>>>(feats, valid, c.n_mels);
        MB_CUDA(cudaGetLastError());
    }
    return 0;
}

// Frames [t0, t0 + n_frames) of `n_sig` signals whose samples [base, total) sit at tail + y * sig_stride
// (the streaming counterpart: mel_one_frame of src/features.c:170-189, no normalisation). The caller
// keeps sample base - 1 .. in the buffer when base > 0 (the pre-emphasis reads one sample back).
int log_mel_stream_device(const MelCfg &c, const float *tail, long long base, long long total, long long sig_stride, int n_sig,
                          const float *mel_fb, const int *mel_lo, const int *mel_hi, const double *win, const double *twiddle,
                          float *feats, long long feat_stride, int t0, int n_frames, cudaStream_t st) {
    if (c.n_fft > MEL_MAX_FFT || (c.n_fft & (c.n_fft - 1))) { set_error("log_mel: n_fft %d unsupported", c.n_fft); return -1; }
    if (n_frames <= 0 || n_sig <= 0) return 0;
    int log2n = 0;
    while ((1 << log2n) < c.n_fft) log2n++;
    mel_frame_kernel<<<dim3(n_frames, n_sig), 128, 0, st>>>(tail, total, win, twiddle, mel_fb, mel_lo, mel_hi, feats, c.n_fft, log2n,
                                                            c.hop, c.n_mels, c.preemph, c.guard, base, t0, sig_stride, feat_stride);
    MB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace mb
