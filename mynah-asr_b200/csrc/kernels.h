// Host-callable launchers for the non-GEMM kernels of the hot path.
#pragma once
#include "common.cuh"
#include "gemm.h"

namespace mb {

// Weight formats accepted at the boundary (values are part of the C ABI).
enum {
    FMT_F32 = 0,
    FMT_MYNAH_Q8 = 1,    // per-row int8, f32 scales [n]            (src/qmat.h:6-9)
    FMT_MYNAH_Q4 = 2,    // per-32 nibbles, f32 scales [n,k/32]
    FMT_GGML_Q4_0 = 102, // 100 + ggml type id: 18-byte blocks of 32
    FMT_GGML_Q8_0 = 108, // 34-byte blocks of 32
    FMT_GGML_Q4_K = 112, // 144-byte super-blocks of 256
    FMT_GGML_Q6_K = 114, // 210-byte super-blocks of 256
};

// ---- dequant.cu
int dequant_to_f32(int fmt, const void *src, const float *scales, float *dst, int n, int k, cudaStream_t st);
size_t format_bytes(int fmt, int n, int k);
int format_block(int fmt);
// status (optional): device word that receives ST_RANGE when a value does not fit the planes (|v| >= 65504 or not finite)
int split_to_h16(const float *x, __half *hi, __half *lo, size_t n, cudaStream_t st, int *status = nullptr);

// ---- elementwise.cu
// Row LayerNorm (mean/var accumulated in double, eps 1e-5) with optional SiLU;
// writes f32 and/or fp16 (hi,lo) planes. out_f32 may alias x.
// chain: launched as a chained kernel (see chain_wait in common.cuh); the widths without a register kernel ignore it.
int layer_norm(const float *x, const float *w, const float *b, float *out_f32, H16 out_h, int T, int d, int act,
               cudaStream_t st, bool chain = false);
// the same with the row also (or only) written as int8 + per-row scale by the reference's activation rule
// (quantize_act_int8, src/qmat.c:186-202): the operand of an int8-activation contraction
int layer_norm_q8(const float *x, const float *w, const float *b, float *out_f32, H16 out_h, int8_t *q8, float *sx8, int T, int d,
                  int act, cudaStream_t st, bool chain = false);
// Conv-module middle: GLU over h2 [T,2d], depthwise conv k along time inside each
// segment, then either a per-channel affine (folded BatchNorm) + SiLU -> planes, or
// (affine null) the raw depthwise output as f32 for a following LayerNorm. With an affine, out_f32 (if given)
// receives the same values as the planes (either may be null).
int glu_dwconv(const float *h2, const float *dw_w, const float *dw_b, const float *scale, const float *shift,
               float *out_f32, H16 out_h, const int *seg_off, const int *seg_len, int batch, int max_len, int d,
               int k, int pad_left, cudaStream_t st);
int scale_inplace(float *x, size_t n, float s, cudaStream_t st);
int pos_emb(H16 pe, int T, int d, cudaStream_t st);            // [2T-1, d] planes

// ---- attention.cu
struct AttnArgs {
    const float *q;             // [rows, ldq] f32 (packed batch), bias_u / bias_v added inside
    int ldq;
    const __half *k, *v;        // [rows, d] fp16
    const __half *rk;           // [sum(2T-1), d] fp16: pos-emb projected by relative_k_proj
    const float *bias_u, *bias_v;   // [H, dk]
    float *ctx_f32;             // optional [rows, d]
    H16 ctx_h;                  // [rows, d] planes (operand of the output projection)
    const int *seg_off, *seg_len, *rk_off;   // device arrays [batch]
    int batch, max_len, d, H;
    int left, right;            // left < 0: full attention
    long long rows = 0, rk_rows = 0;   // rows of k / v and of rk (bounds of the TMA descriptors); 0: unknown
    int *status = nullptr;      // device status word for the bounded waits of the tcgen05 kernel
};
// impl 0 = tensor cores (tcgen05 kernel for full attention over 128-wide heads, else the warp-level tiled
// kernel), 1 = plain one-warp-per-query kernel, 2 = the warp-level tiled kernel
int attention_forward(const AttnArgs &a, int impl, cudaStream_t st);
// ---- attention_tc.cu
bool attention_tc_eligible(const AttnArgs &a);
int attention_tc(const AttnArgs &a, cudaStream_t st);

// ---- subsampling.cu
int conv_in_relu(const float *feats, const float *w, const float *b, float *out, int T, int F, int C, int To, int Fo,
                 int pl, cudaStream_t st);                         // [T,F] -> [To,Fo,C]
int conv_in_dw_fused(const float *feats, const float *w0, const float *b0, const float *w1, const float *b1, H16 out,
                     int T, int F, int C, int T1, int F1, int T2, int F2, int pl, cudaStream_t st);   // [T,F] -> planes [T2*F2, C]
int dwconv3x3_s2(const float *x, const float *w, const float *b, H16 out, int T, int F, int C, int To, int Fo, int pl,
                 cudaStream_t st);                                 // [T,F,C] -> planes [To*Fo, C]

// ---- mel.cu
struct MelCfg {
    int n_mels, n_fft, win_length, hop;
    double preemph, guard;
    int normalize;
};
int log_mel_device(const MelCfg &c, const float *audio, size_t n_samples, const float *mel_fb, const int *mel_lo,
                   const int *mel_hi, const double *win, const double *twiddle, float *feats, int T, int valid,
                   cudaStream_t st);

int log_mel_stream_device(const MelCfg &c, const float *tail, long long base, long long total, long long sig_stride, int n_sig,
                          const float *mel_fb, const int *mel_lo, const int *mel_hi, const double *win, const double *twiddle,
                          float *feats, long long feat_stride, int t0, int n_frames, cudaStream_t st);

// ---- qgemv.cu : out[T,n] = x[T,k] W^T for T <= 16 straight from the stored blocks
struct QWeight;
int qgemv(const QWeight &w, const float *x, int ldx, float *out, int ldo, const float *bias, int T, cudaStream_t st);
// ---- qgemv_mma.cu : the same product for Q4_0 / Q8_0 on mma.sync, from re-tiled blocks
int qgemv_mma_retile(const QWeight &w, uint8_t *qs, __half *ds, cudaStream_t st);
int qgemv_mma(const QWeight &w, const float *x, int ldx, float *out, int ldo, const float *bias, int T, cudaStream_t st);
// ---- qstream_tc.cu : the same product with the decode fused into the tcgen05 operand pipeline (T <= 8)
size_t qstream_tc_bytes(int fmt, int n, int k);
int qstream_tc_retile(const QWeight &w, uint8_t *dst, cudaStream_t st);
size_t qstream_tc_scratch_bytes(int n, int k);
int qstream_tc(const QWeight &w, const float *x, int ldx, float *out, int ldo, const float *bias, int T, int *status,
               cudaStream_t st);
// int8 activation rows by the reference's rule (quantize_act_int8, src/qmat.c:186-202): per row scale = amax / 127,
// q = round-half-away(x * 127 / amax) clamped to +-127; x [T, k] f32 -> qx [T, k] int8, sx [T]
int act_quant_rows(const float *x, int8_t *qx, float *sx, int T, int k, cudaStream_t st);
int qgemv_a8(const QWeight &w, const float *x, float *out, int T, int32_t *block_dots, float *sx_out, cudaStream_t st);

// ---- align.cu : CTC forced alignment (mynah_asr_align_ctc, src/align.c) with the scores resident
int align_min_frames(const int *tokens, int n);
int align_ctc_device(const float *scores_dev, int T, int V, const int *tokens, int n, int blank, int *t0, int *t1, cudaStream_t st);

// ---- launch accounting (model.cu): every kernel launch of the library is counted
void note_launch(int n = 1);
long long launch_count(bool reset);

// ---- decoder.cu
int argmax_rows(const float *logits, int ld, const float *bias, int T, int V, int *best, cudaStream_t st, bool chain = false);

}  // namespace mb
