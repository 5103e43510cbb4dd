// Voice activity and offline segment planning with the audio resident on the device.
//
// The reference plans the segments of a long file on the host before anything reaches the encoder: a Silero-style
// network gives one speech probability per 32 ms frame (mynah_asr_vad_feed, src/vad.c:316-385), a hysteresis turns
// the probabilities into padded speech spans (mynah_asr_vad_speech_spans, src/vad.c:417-492), the spans — widened
// and merged — become segments, and anything longer than the model's limit is cut at the 20 ms window of least
// energy (plan_segments_vad, plan_segments, find_split_point, src/mynah_asr.c:1177-1323). Frame by frame on one
// core this serialises in front of the path; here the audio is uploaded once and
//
//   * vad_encode_kernel runs everything of the network that does not depend on the recurrent state for ALL frames
//     at once (one CTA per frame): lookbehind | frame | reflect pad -> STFT as a product with the basis -> magnitude
//     -> the conv + ReLU blocks -> the LSTM's input contribution b_ih + b_hh + W_ih x;
//   * vad_lstm_kernel walks the frames in order with one CTA: thread r keeps row r of W_hh in registers, the state
//     lives in shared memory, and the head (ReLU -> 1x1 conv -> sigmoid) gives the frame's probability;
//   * window_energy_kernel forms the double-precision sum of squares of every candidate 20 ms window of a search
//     range, one thread per window, in the reference's summation order (so the minimum falls on the same window);
//   * the decisions that are integer / double logic over those numbers — hysteresis, padding, widening, merging,
//     cutting — run on the host exactly as the reference states them.
#include <math.h>
#include <string.h>

#include <vector>

#include "../../include/mynah_b200.h"
#include "kernels.h"

using namespace mb;

namespace {

constexpr int VAD_MAX_ENC = 8;

struct VadDev {
    int frame, context, pad, n_fft, hop, n_bins, stft_frames, hidden, n_enc;
    int cin[VAD_MAX_ENC], cout[VAD_MAX_ENC], k[VAD_MAX_ENC], stride[VAD_MAX_ENC], pl[VAD_MAX_ENC], pr[VAD_MAX_ENC];
    const float *basis, *enc_w[VAD_MAX_ENC], *enc_b[VAD_MAX_ENC], *w_ih, *w_hh, *b_ih, *b_hh, *head_w;
    float head_b;
    int act_max;                       // floats of the larger activation buffer
};

__device__ __forceinline__ int conv_len(int t_in, int k, int stride, int pl, int pr) { return (t_in + pl + pr - k) / stride + 1; }

// One CTA per frame. Shared memory: buf [context + frame + pad] | spec [2 n_bins stft_frames] | act0 | act1.
__global__ void __launch_bounds__(256)
vad_encode_kernel(const VadDev v, const float *__restrict__ audio, long long n_samples, float *__restrict__ xz) {
    extern __shared__ float sm[];
    const int C = v.context, F = v.frame, P = v.pad, N = C + F, T0 = v.stft_frames, B = v.n_bins;
    float *buf = sm, *spec = buf + N + P, *act0 = spec + 2 * B * T0, *act1 = act0 + v.act_max;
    const long long f = blockIdx.x, base = f * F;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        const long long s = base - C + i;        // the lookbehind is the tail of the previous frame (zeros before the signal)
        buf[i] = (s >= 0 && s < n_samples) ? audio[s] : 0.0f;
    }
    __syncthreads();
    for (int j = threadIdx.x; j < P; j += blockDim.x) buf[N + j] = buf[N - 2 - j];       // reflect pad on the right
    __syncthreads();
    // STFT as windows x basis (vad.c:330-336), then the magnitude
    for (int o = threadIdx.x; o < 2 * B * T0; o += blockDim.x) {
        const int r = o / T0, t = o % T0;
        const float *br = v.basis + (size_t)r * v.n_fft, *w = buf + t * v.hop;
        float acc = 0.0f;
        for (int k = 0; k < v.n_fft; k++) acc = fmaf(br[k], w[k], acc);
        spec[o] = acc;
    }
    __syncthreads();
    for (int o = threadIdx.x; o < B * T0; o += blockDim.x) {
        const float re = spec[o], im = spec[o + B * T0];
        act0[o] = sqrtf(re * re + im * im);
    }
    __syncthreads();
    float *in = act0, *out = act1;
    int t_in = T0;
    for (int l = 0; l < v.n_enc; l++) {
        const int t_out = conv_len(t_in, v.k[l], v.stride[l], v.pl[l], v.pr[l]), ck = v.cin[l] * v.k[l];
        for (int o = threadIdx.x; o < v.cout[l] * t_out; o += blockDim.x) {
            const int co = o / t_out, t = o % t_out;
            const float *w = v.enc_w[l] + (size_t)co * ck;
            float acc = 0.0f;
            for (int ci = 0; ci < v.cin[l]; ci++)
                for (int kk = 0; kk < v.k[l]; kk++) {
                    const int s = t * v.stride[l] - v.pl[l] + kk;
                    if (s >= 0 && s < t_in) acc = fmaf(w[ci * v.k[l] + kk], in[ci * t_in + s], acc);
                }
            const float x = acc + v.enc_b[l][co];
            out[o] = x > 0.0f ? x : 0.0f;
        }
        __syncthreads();
        float *sw = in; in = out; out = sw;
        t_in = t_out;
    }
    // the LSTM's input contribution for this frame: b_ih + b_hh + W_ih x (vad.c:357-359)
    const int H = v.hidden;
    for (int r = threadIdx.x; r < 4 * H; r += blockDim.x) {
        const float *w = v.w_ih + (size_t)r * H;
        float acc = 0.0f;
        for (int j = 0; j < H; j++) acc = fmaf(w[j], in[j], acc);
        xz[(size_t)f * 4 * H + r] = (v.b_ih[r] + v.b_hh[r]) + acc;
    }
}

__device__ __forceinline__ float vad_sigmoid(float x) {       // mynah_asr_sigmoid (src/qmat.h:31-35)
    if (x >= 0.0f) return 1.0f / (1.0f + expf(-x));
    const float e = expf(x);
    return e / (1.0f + e);
}

// One CTA of 4 H threads walks the frames: z = xz[f] + W_hh h, gates i f g o, head on ReLU(h).
template <int H>
__global__ void __launch_bounds__(4 * H)
vad_lstm_kernel(const VadDev v, const float *__restrict__ xz, int frames, float *__restrict__ probs) {
    // row r of W_hh: the first WR weights in registers, the rest in shared memory as [j][row] (conflict-free)
    constexpr int WR = 96, WS = H - WR;
    extern __shared__ float wsm[];
    __shared__ float h[H], z[4 * H];
    const int r = threadIdx.x;
    float w[WR];
#pragma unroll
    for (int j = 0; j < WR; j++) w[j] = v.w_hh[(size_t)r * H + j];
    for (int j = 0; j < WS; j++) wsm[j * 4 * H + r] = v.w_hh[(size_t)r * H + WR + j];
    float c = 0.0f;
    if (r < H) h[r] = 0.0f;
    __syncthreads();
    for (int f = 0; f < frames; f++) {
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < WR; j++) acc = fmaf(w[j], h[j], acc);
#pragma unroll
        for (int j = 0; j < WS; j++) acc = fmaf(wsm[j * 4 * H + r], h[WR + j], acc);
        z[r] = xz[(size_t)f * 4 * H + r] + acc;
        __syncthreads();
        if (r < H) {
            const float ig = vad_sigmoid(z[r]), fg = vad_sigmoid(z[H + r]), gg = tanhf(z[2 * H + r]), og = vad_sigmoid(z[3 * H + r]);
            c = fg * c + ig * gg;
            h[r] = og * tanhf(c);
        }
        __syncthreads();
        if (r == 0) {
            float a = v.head_b;
            for (int i = 0; i < H; i++) if (h[i] > 0.0f) a = fmaf(v.head_w[i], h[i], a);
            probs[f] = vad_sigmoid(a);
        }
    }
}

// e[j] = sum of squares (double) of the `win` samples from lo + j hop, added in order (find_split_point, src/mynah_asr.c:1183-1189)
__global__ void window_energy_kernel(const float *__restrict__ s, long long lo, int win, int hop, int n_windows, double *__restrict__ e) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n_windows) return;
    const float *p = s + lo + (long long)j * hop;
    double acc = 0.0;
    for (int i = 0; i < win; i++) { const double x = p[i]; acc += x * x; }
    e[j] = acc;
}

}  // namespace

struct mynah_b200_vad {
    mynah_b200_vad_config cfg;
    VadDev d;
    std::vector<void *> owned;
    cudaStream_t stream = nullptr;
    size_t smem = 0;
};

namespace {

float *vad_upload(mynah_b200_vad *v, const float *src, size_t n) {
    float *p = nullptr;
    if (!src || cudaMalloc((void **)&p, n * sizeof(float)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    v->owned.push_back(p);
    if (cudaMemcpy(p, src, n * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) return nullptr;
    return p;
}

// speech probabilities of the uploaded signal -> host vector
int vad_probs_dev(mynah_b200_vad *v, const float *audio_dev, size_t n, std::vector<float> &probs) {
    const int F = v->d.frame, H = v->d.hidden;
    const int frames = (int)((n + F - 1) / F);
    probs.assign((size_t)frames, 0.f);
    if (frames == 0) return 0;
    float *xz = nullptr, *pd = nullptr;
    MB_CUDA(cudaMallocAsync((void **)&xz, (size_t)frames * 4 * H * sizeof(float), v->stream));
    if (cudaMallocAsync((void **)&pd, (size_t)frames * sizeof(float), v->stream) != cudaSuccess) { cudaGetLastError(); cudaFreeAsync(xz, v->stream); set_error("vad: allocation failed"); return -1; }
    vad_encode_kernel<<<frames, 256, v->smem, v->stream>>>(v->d, audio_dev, (long long)n, xz);
    vad_lstm_kernel<128><<<1, 512, 32 * 512 * sizeof(float), v->stream>>>(v->d, xz, frames, pd);
    note_launch(2);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaMemcpyAsync(probs.data(), pd, (size_t)frames * sizeof(float), cudaMemcpyDeviceToHost, v->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(v->stream);
    cudaFreeAsync(xz, v->stream);
    cudaFreeAsync(pd, v->stream);
    if (e != cudaSuccess) { set_error("vad: %s", cudaGetErrorString(e)); return -1; }
    return frames;
}

struct Span { long long t0, t1; };

// mynah_asr_vad_seg_feed / _finish / mynah_asr_vad_pad_spans (src/vad.c:417-474) over a probability vector
std::vector<Span> spans_from_probs(const mynah_b200_vad_config &c, const std::vector<float> &probs, long long n_samples) {
    const double sr = 16000.0;
    auto ms = [&](int v) { return sr * (double)v / 1000.0; };
    std::vector<Span> out;
    bool trig = false;
    long long start = 0, temp_end = -1;
    for (size_t i = 0; i < probs.size(); i++) {
        const long long cur = (long long)c.frame_samples * (long long)i;
        const double p = (double)probs[i];
        if (p >= c.threshold) {
            temp_end = -1;
            if (!trig) { trig = true; start = cur; }
            continue;
        }
        if (p < c.neg_threshold && trig) {
            if (temp_end < 0) temp_end = cur;
            if ((double)(cur - temp_end) < ms(c.min_silence_ms)) continue;
            const long long end = temp_end;
            trig = false; temp_end = -1;
            if ((double)(end - start) > ms(c.min_speech_ms)) out.push_back(Span{start, end});
        }
    }
    if (trig && (double)(n_samples - start) > ms(c.min_speech_ms)) out.push_back(Span{start, n_samples});
    const long long pad = (long long)(sr * (double)c.speech_pad_ms / 1000.0);
    const int n = (int)out.size();
    for (int i = 0; i < n; i++) {
        if (i == 0) out[0].t0 = out[0].t0 - pad > 0 ? out[0].t0 - pad : 0;
        if (i != n - 1) {
            const long long gap = out[i + 1].t0 - out[i].t1;
            if (gap < 2 * pad) {
                out[i].t1 += gap / 2;
                const long long s1 = out[i + 1].t0 - gap / 2;
                out[i + 1].t0 = s1 > 0 ? s1 : 0;
            } else {
                out[i].t1 = out[i].t1 + pad < n_samples ? out[i].t1 + pad : n_samples;
                const long long s1 = out[i + 1].t0 - pad;
                out[i + 1].t0 = s1 > 0 ? s1 : 0;
            }
        } else {
            out[i].t1 = out[i].t1 + pad < n_samples ? out[i].t1 + pad : n_samples;
        }
    }
    return out;
}

// find_split_point (src/mynah_asr.c:1178-1192) on the resident signal: -1 on a device error
long long split_point_dev(const float *audio_dev, long long lo, long long hi, int sr, cudaStream_t st, std::vector<double> &host) {
    const int win = sr / 50, hop = win / 2;
    if (hop <= 0 || lo + win > hi) return hi;
    const int nw = (int)((hi - win - lo) / hop) + 1;
    double *e = nullptr;
    if (cudaMallocAsync((void **)&e, (size_t)nw * sizeof(double), st) != cudaSuccess) { cudaGetLastError(); set_error("plan_segments: allocation failed"); return -1; }
    window_energy_kernel<<<cdiv(nw, 128), 128, 0, st>>>(audio_dev, lo, win, hop, nw, e);
    note_launch();
    host.resize((size_t)nw);
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) err = cudaMemcpyAsync(host.data(), e, (size_t)nw * sizeof(double), cudaMemcpyDeviceToHost, st);
    if (err == cudaSuccess) err = cudaStreamSynchronize(st);
    cudaFreeAsync(e, st);
    if (err != cudaSuccess) { set_error("plan_segments: %s", cudaGetErrorString(err)); return -1; }
    double best = 1e300;
    long long pos = hi;
    for (int j = 0; j < nw; j++) if (host[(size_t)j] < best) { best = host[(size_t)j]; pos = lo + (long long)j * hop + win / 2; }
    return pos;
}

}  // namespace

extern "C" {

mynah_b200_vad *mynah_b200_vad_new(const mynah_b200_vad_config *c, const float *basis, const float *const *enc_w,
                                   const float *const *enc_b, const float *w_ih, const float *w_hh, const float *b_ih,
                                   const float *b_hh, const float *head_w, float head_b) {
    if (!mynah_b200_available()) { set_error("vad: no sm_100 CUDA device available"); return nullptr; }
    if (!c || !basis || !enc_w || !enc_b || !w_ih || !w_hh || !b_ih || !b_hh || !head_w) { set_error("vad_new: bad argument"); return nullptr; }
    if (c->n_enc < 1 || c->n_enc > VAD_MAX_ENC || c->lstm_hidden != 128 || c->frame_samples <= 0 || c->n_fft <= 0 || c->hop_length <= 0) {
        set_error("vad_new: unsupported geometry (1..%d encoder blocks, LSTM width 128)", VAD_MAX_ENC); return nullptr;
    }
    mynah_b200_vad *v = new mynah_b200_vad();
    v->cfg = *c;
    VadDev &d = v->d;
    memset(&d, 0, sizeof(d));
    d.frame = c->frame_samples; d.context = c->context_samples; d.pad = c->reflect_pad; d.n_fft = c->n_fft; d.hop = c->hop_length;
    d.n_bins = c->n_bins; d.hidden = c->lstm_hidden; d.n_enc = c->n_enc; d.head_b = head_b;
    d.stft_frames = (d.context + d.frame + d.pad - d.n_fft) / d.hop + 1;
    int t = d.stft_frames, cin = d.n_bins, act_max = d.n_bins * d.stft_frames;
    bool ok = d.stft_frames >= 1 && d.pad + 2 <= d.context + d.frame;
    d.basis = vad_upload(v, basis, (size_t)2 * d.n_bins * d.n_fft);
    ok = ok && d.basis;
    for (int i = 0; i < d.n_enc && ok; i++) {
        d.cin[i] = cin; d.cout[i] = c->enc_channels[i]; d.k[i] = c->enc_kernels[i]; d.stride[i] = c->enc_strides[i];
        d.pl[i] = c->enc_pads[2 * i]; d.pr[i] = c->enc_pads[2 * i + 1];
        if (d.cout[i] <= 0 || d.k[i] <= 0 || d.stride[i] <= 0) { ok = false; break; }
        t = (t + d.pl[i] + d.pr[i] - d.k[i]) / d.stride[i] + 1;
        if (t < 1) { ok = false; break; }
        if (d.cout[i] * t > act_max) act_max = d.cout[i] * t;
        d.enc_w[i] = vad_upload(v, enc_w[i], (size_t)d.cout[i] * cin * d.k[i]);
        d.enc_b[i] = vad_upload(v, enc_b[i], (size_t)d.cout[i]);
        ok = d.enc_w[i] && d.enc_b[i];
        cin = d.cout[i];
    }
    // the encoder must collapse to one timestep of the LSTM's width (vad.c:214-239)
    ok = ok && t == 1 && cin == d.hidden;
    const size_t H = (size_t)d.hidden;
    if (ok) {
        d.w_ih = vad_upload(v, w_ih, 4 * H * H); d.w_hh = vad_upload(v, w_hh, 4 * H * H);
        d.b_ih = vad_upload(v, b_ih, 4 * H); d.b_hh = vad_upload(v, b_hh, 4 * H); d.head_w = vad_upload(v, head_w, H);
        ok = d.w_ih && d.w_hh && d.b_ih && d.b_hh && d.head_w;
    }
    d.act_max = act_max;
    v->smem = ((size_t)d.context + d.frame + d.pad + 2 * (size_t)d.n_bins * d.stft_frames + 2 * (size_t)act_max) * sizeof(float);
    if (ok && v->smem > 200 * 1024) ok = false;
    if (ok && cudaStreamCreateWithFlags(&v->stream, cudaStreamNonBlocking) != cudaSuccess) ok = false;
    if (ok && cudaFuncSetAttribute(vad_lstm_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * 512 * (int)sizeof(float)) != cudaSuccess) ok = false;
    if (ok && v->smem > 48 * 1024 && cudaFuncSetAttribute(vad_encode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)v->smem) != cudaSuccess) ok = false;
    cudaDeviceSynchronize();
    if (!ok) { set_error("vad_new: the tensors contradict the geometry, or a device call failed"); mynah_b200_vad_free(v); return nullptr; }
    return v;
}

void mynah_b200_vad_free(mynah_b200_vad *v) {
    if (!v) return;
    for (void *p : v->owned) cudaFree(p);
    if (v->stream) cudaStreamDestroy(v->stream);
    delete v;
}

int mynah_b200_vad_frame_samples(const mynah_b200_vad *v) { return v ? v->d.frame : 0; }

// uploads the signal; the caller frees with cudaFree
static float *upload_signal(const float *samples, size_t n, cudaStream_t st) {
    float *a = nullptr;
    if (cudaMalloc((void **)&a, (n ? n : 1) * sizeof(float)) != cudaSuccess) { cudaGetLastError(); set_error("device allocation failed"); return nullptr; }
    if (n && (cudaMemcpyAsync(a, samples, n * sizeof(float), cudaMemcpyHostToDevice, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess)) {
        set_error("H2D copy failed"); cudaFree(a); return nullptr;
    }
    return a;
}

int mynah_b200_vad_probs(mynah_b200_vad *v, const float *samples, size_t n, float *probs, int cap) {
    if (!v || (!samples && n) || !probs) { set_error("vad_probs: bad argument"); return -1; }
    float *a = upload_signal(samples, n, v->stream);
    if (!a) return -1;
    std::vector<float> p;
    const int frames = vad_probs_dev(v, a, n, p);
    cudaFree(a);
    if (frames < 0) return -1;
    if (frames > cap) { set_error("vad_probs: %d frames, room for %d", frames, cap); return -1; }
    memcpy(probs, p.data(), (size_t)frames * sizeof(float));
    return frames;
}

int mynah_b200_vad_speech_spans(mynah_b200_vad *v, const float *samples, size_t n, long long *spans, int cap) {
    if (!v || (!samples && n) || !spans || cap < 0) { set_error("vad_speech_spans: bad argument"); return -1; }
    float *a = upload_signal(samples, n, v->stream);
    if (!a) return -1;
    std::vector<float> p;
    const int frames = vad_probs_dev(v, a, n, p);
    cudaFree(a);
    if (frames < 0) return -1;
    const std::vector<Span> sp = spans_from_probs(v->cfg, p, (long long)n);
    if ((int)sp.size() > cap) { set_error("vad_speech_spans: more than %d spans", cap); return -1; }
    for (size_t i = 0; i < sp.size(); i++) { spans[2 * i] = sp[i].t0; spans[2 * i + 1] = sp[i].t1; }
    return (int)sp.size();
}

int mynah_b200_plan_segments(mynah_b200_vad *v, const float *samples, size_t n_samples, int sample_rate, double seg_sec,
                             long long *segs, int cap) {
    if ((!samples && n_samples) || !segs || cap < 1 || sample_rate <= 0 || seg_sec <= 0) { set_error("plan_segments: bad argument"); return -1; }
    if (!mynah_b200_available()) { set_error("plan_segments: no sm_100 device"); return -1; }
    cudaStream_t st = v ? v->stream : nullptr;
    float *a = upload_signal(samples, n_samples, st);
    if (!a) return -1;
    const long long n = (long long)n_samples, sr = sample_rate, seg_max = (long long)(seg_sec * (double)sample_rate);
    std::vector<Span> ranges;                       // what gets cut: the whole signal, or the widened and merged speech spans
    bool vad_plan = false;
    if (v && n > 0) {
        std::vector<float> p;
        if (vad_probs_dev(v, a, n_samples, p) >= 0) {
            std::vector<Span> sp = spans_from_probs(v->cfg, p, n);
            const long long ctx = (long long)(0.6 * (double)sample_rate);      // MYNAH_ASR_VAD_CONTEXT_SEC (src/mynah_asr.c:67-68)
            for (Span &s : sp) { s.t0 = s.t0 > ctx ? s.t0 - ctx : 0; s.t1 = s.t1 + ctx < n ? s.t1 + ctx : n; }
            for (const Span &s : sp) {
                if (!ranges.empty() && s.t0 <= ranges.back().t1) { if (s.t1 > ranges.back().t1) ranges.back().t1 = s.t1; }
                else ranges.push_back(s);
            }
            vad_plan = true;
        }
    }
    if (!vad_plan) ranges.assign(1, Span{0, n});
    std::vector<long long> out;
    std::vector<double> scratch;
    int rc = 0;
    for (const Span &r : ranges) {
        long long cur = r.t0;
        while (cur < r.t1 && rc == 0) {
            long long end = r.t1;
            if (r.t1 - cur > seg_max + seg_max / 10) {                         // +10 %: no split for a small overrun
                const long long hi = cur + seg_max;
                long long lo = seg_max > 20 * sr ? hi - 20 * sr : cur + sr;    // the last 20 s of the window, at least 1 s in
                if (lo <= cur) lo = cur + 1;
                end = split_point_dev(a, lo, hi, sample_rate, st, scratch);
                if (end < 0) { rc = -1; break; }
                if (vad_plan && (end <= cur || end > r.t1)) end = hi;
            }
            if (end <= cur) end = cur + 1;
            out.push_back(cur); out.push_back(end - cur);
            cur = end;
        }
    }
    cudaFree(a);
    if (rc) return -1;
    if (out.empty()) { out.push_back(0); out.push_back(0); }                  // nothing to decode: one empty segment
    const int k = (int)(out.size() / 2);
    if (k > cap) { set_error("plan_segments: %d segments, room for %d", k, cap); return -1; }
    memcpy(segs, out.data(), out.size() * sizeof(long long));
    return k;
}

}  // extern "C"
