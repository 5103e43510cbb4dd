/* TEST INFRASTRUCTURE ONLY — never linked into, loaded by or called from the
 * product library.
 *
 * A thin C shim compiled TOGETHER with the unmodified reference sources into
 * oracle/_ref/libmynah_ref.so. It owns the reference's structs (which ctypes
 * cannot lay out portably) and exposes the reference's own functions for the
 * hot path behind plain pointers:
 *
 *   src/features.c   mynah_asr_log_mel
 *   src/subsampling.c mynah_asr_subsampling_forward
 *   src/encoder.c    mynah_asr_encoder_{init,layer,forward,forward_raw,forward_batch,post},
 *                    mynah_asr_pos_emb, mynah_asr_enc_stream_*
 *   src/decoder.c    mynah_asr_greedy_decode (RNNT + TDT)
 *   src/decoder_ctc.c mynah_asr_ctc_decode
 *   src/decoder_aed.c mynah_asr_aed_{init,decode}
 *   src/qmat.c       mynah_asr_qmat_{init,mul}
 *   src/align.c      mynah_asr_align_ctc, mynah_asr_align_min_frames
 *
 * Every function below only forwards to the reference; no arithmetic lives
 * here. Weights arrive as a safetensors file with HF-verbatim tensor names,
 * opened by the reference's own loader (src/weights.c). */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "align.h"
#include "decoder.h"
#include "decoder_aed.h"
#include "decoder_ctc.h"
#include "encoder.h"
#include "features.h"
#include "qmat.h"
#include "subsampling.h"
#include "threads.h"
#include "weights.h"

typedef struct {
    mynah_asr_safetensors *st, *mel;
    mynah_asr_encoder enc;
    mynah_asr_decoder dec;
    mynah_asr_ctc ctc;
    mynah_asr_feat_cfg feat;
    mynah_asr_aed aed;
    int has_dec, has_ctc, has_feat, has_aed;
} ref_model;

void ref_close(ref_model *m) {
    if (!m) return;
    if (m->has_dec) mynah_asr_qmat_free(&m->dec.head);
    if (m->has_aed) mynah_asr_aed_free(&m->aed);
    mynah_asr_encoder_free(&m->enc);
    if (m->st) mynah_asr_st_close(m->st);
    if (m->mel) mynah_asr_st_close(m->mel);
    free(m);
}

/* quant: 0 f32, 1 int8, 2 int4 (mynah-native load-time quantisation); + 16 keeps the transducer
 * decoder's joint head in f32 while the encoder is quantised.
 * causal: -1 keeps what the tensor naming implies. durations NULL => RNNT. */
ref_model *ref_open(const char *weights, const char *mel_filters, int quant, int causal,
                    int xscaling, int n_mels, int normalize_per_feature, int blank,
                    int max_symbols, const int *durations, int n_durations) {
    ref_model *m = calloc(1, sizeof(*m));
    if (!m) return NULL;
    m->st = mynah_asr_st_open(weights);
    if (!m->st) { free(m); return NULL; }
    const int dec_quant = (quant & 16) ? 0 : quant;
    quant &= 15;
    if (mynah_asr_encoder_init(&m->enc, m->st, quant) != 0) { ref_close(m); return NULL; }
    if (causal >= 0) { m->enc.causal = causal; m->enc.ss.causal = causal; }
    if (xscaling) m->enc.xscale = sqrtf((float)m->enc.d_model);
    if (mynah_asr_st_get(m->st, "decoder.embedding.weight")) {
        if (mynah_asr_decoder_init(&m->dec, m->st, blank, max_symbols, dec_quant, durations,
                                   n_durations) != 0) { ref_close(m); return NULL; }
        m->has_dec = 1;
    }
    m->has_ctc = mynah_asr_ctc_init(&m->ctc, m->st) == 0;
    if (mel_filters) {
        m->mel = mynah_asr_st_open(mel_filters);
        if (!m->mel) { ref_close(m); return NULL; }
        const mynah_asr_tensor *fb = mynah_asr_st_get(m->mel, "mel_fb");
        const mynah_asr_tensor *win = mynah_asr_st_get(m->mel, "window");
        if (!fb || !win) { ref_close(m); return NULL; }
        m->feat = (mynah_asr_feat_cfg){
            .sample_rate = 16000, .n_mels = n_mels, .n_fft = 512,
            .win_length = (int)win->n_elems, .hop_length = 160, .preemphasis = 0.97,
            .log_zero_guard = 5.9604644775390625e-8,
            .normalize_per_feature = normalize_per_feature,
            .mel_fb = (const float *)fb->data, .window = (const float *)win->data};
        m->has_feat = 1;
    }
    return m;
}

/* AED decoder of the same safetensors file (mynah_asr_aed_init, src/decoder_aed.c:50-113). */
int ref_aed_open(ref_model *m, int n_layers, int n_heads, int max_seq, int max_gen_delta, int quant) {
    if (m->has_aed) return 0;
    if (mynah_asr_aed_init(&m->aed, m->st, n_layers, n_heads, max_seq, max_gen_delta, quant) != 0) {
        mynah_asr_aed_free(&m->aed);
        return -1;
    }
    m->has_aed = 1;
    return 0;
}

int ref_aed_decode(const ref_model *m, const float *enc, int T, const int *prompt, int n_prompt, int eos,
                   int *tokens, int cap) {
    if (!m->has_aed) return -1;
    return mynah_asr_aed_decode(&m->aed, enc, T, prompt, n_prompt, eos, tokens, cap);
}

/* dims[0..7] = d_model, n_layers, n_heads, ffn_dim, conv_k, d_out, causal, channels */
void ref_dims(const ref_model *m, int *dims) {
    dims[0] = m->enc.d_model; dims[1] = m->enc.n_layers; dims[2] = m->enc.n_heads;
    dims[3] = m->enc.ffn_dim; dims[4] = m->enc.conv_k; dims[5] = m->enc.d_out;
    dims[6] = m->enc.causal; dims[7] = m->enc.ss.channels;
}

void ref_free(void *p) { free(p); }
void ref_set_threads_env(void) { (void)mynah_asr_num_threads(); }

float *ref_log_mel(const ref_model *m, const float *audio, size_t n, int *n_frames, int *valid) {
    return m->has_feat ? mynah_asr_log_mel(&m->feat, audio, n, n_frames, valid) : NULL;
}

float *ref_subsampling(const ref_model *m, const float *feats, int T, int n_mels, int *t_out) {
    return mynah_asr_subsampling_forward(&m->enc.ss, feats, T, n_mels, t_out);
}

void ref_pos_emb(const ref_model *m, int T, float *pe) { mynah_asr_pos_emb(&m->enc, T, pe); }

int ref_encoder_layer(const ref_model *m, int li, float *x, int T, const float *pe, int left,
                      int right) {
    return mynah_asr_encoder_layer(&m->enc, li, x, T, pe, left, right);
}

void ref_encoder_post(const ref_model *m, const float *x, int T, float *out) {
    mynah_asr_encoder_post(&m->enc, x, T, 0, out);
}

float *ref_encoder_forward(const ref_model *m, const float *feats, int t_mel, int n_mels,
                           int left, int right, int raw, int *t_out) {
    return raw ? mynah_asr_encoder_forward_raw(&m->enc, feats, t_mel, n_mels, left, right, t_out)
               : mynah_asr_encoder_forward(&m->enc, feats, t_mel, n_mels, 0, left, right, t_out);
}

/* the same two with a prompt id (prompt-conditioned models, src/encoder.c:591-614) */
void ref_encoder_post_p(const ref_model *m, const float *x, int T, int prompt_id, float *out) {
    mynah_asr_encoder_post(&m->enc, x, T, prompt_id, out);
}
float *ref_encoder_forward_p(const ref_model *m, const float *feats, int t_mel, int n_mels, int prompt_id,
                             int left, int right, int *t_out) {
    return mynah_asr_encoder_forward(&m->enc, feats, t_mel, n_mels, prompt_id, left, right, t_out);
}
int ref_encoder_forward_batch_p(const ref_model *m, const float *const *feats, const int *t_mel,
                                int batch, int n_mels, const int *prompt_ids, int left, int right,
                                float **outs, int *t_outs) {
    return mynah_asr_encoder_forward_batch(&m->enc, feats, t_mel, batch, n_mels, prompt_ids, left,
                                           right, outs, t_outs);
}
int ref_stream_step_p(mynah_asr_enc_stream *es, const float *mel, int n_mel, int n_mels, int prompt_id,
                      int is_last, float *out) {
    return mynah_asr_enc_stream_step(es, mel, n_mel, n_mels, prompt_id, is_last, out);
}

int ref_encoder_forward_batch(const ref_model *m, const float *const *feats, const int *t_mel,
                              int batch, int n_mels, int left, int right, float **outs,
                              int *t_outs) {
    int *pids = calloc((size_t)batch, sizeof(int));
    if (!pids) return -1;
    const int rc = mynah_asr_encoder_forward_batch(&m->enc, feats, t_mel, batch, n_mels, pids,
                                                   left, right, outs, t_outs);
    free(pids);
    return rc;
}

int ref_ctc_decode(const ref_model *m, const float *enc, int T, int *tokens, int *frames,
                   int cap) {
    return m->has_ctc ? mynah_asr_ctc_decode(&m->ctc, enc, T, tokens, frames, cap) : -1;
}

/* Greedy RNNT/TDT from a fresh state (SOS = blank), as eng_decode_rnnt does
 * (src/mynah_asr.c:124-137). */
int ref_greedy_decode(const ref_model *m, const float *enc, int T, int *tokens, int *frames,
                      int cap) {
    if (!m->has_dec) return -1;
    mynah_asr_dec_state *s = malloc(sizeof(*s));
    if (!s) return -1;
    mynah_asr_dec_state_reset(&m->dec, s);
    const int n = mynah_asr_greedy_decode(&m->dec, s, enc, T, tokens, frames, cap);
    free(s);
    return n;
}

/* ---- cache-aware streaming encoder (src/encoder.c:619-872) ---- */
mynah_asr_enc_stream *ref_stream_open(const ref_model *m, int left, int right, int n_mels) {
    mynah_asr_enc_stream *es = calloc(1, sizeof(*es));
    if (!es) return NULL;
    if (mynah_asr_enc_stream_init(es, &m->enc, left, right, n_mels) != 0) {
        mynah_asr_enc_stream_free(es); free(es); return NULL;
    }
    return es;
}
int ref_stream_need(const mynah_asr_enc_stream *es) { return mynah_asr_enc_stream_need(es); }
int ref_stream_step(mynah_asr_enc_stream *es, const float *mel, int n_mel, int n_mels,
                    int is_last, float *out) {
    return mynah_asr_enc_stream_step(es, mel, n_mel, n_mels, 0, is_last, out);
}
void ref_stream_close(mynah_asr_enc_stream *es) {
    if (es) { mynah_asr_enc_stream_free(es); free(es); }
}

/* ---- CTC forced alignment (src/align.c) ---- */
int ref_align_ctc(const float *scores, int T, int V, const int *tokens, int n_tokens, int blank,
                  int *t0, int *t1) {
    return mynah_asr_align_ctc(scores, T, V, tokens, n_tokens, blank, t0, t1);
}
int ref_align_min_frames(const int *tokens, int n_tokens) {
    return mynah_asr_align_min_frames(tokens, n_tokens);
}

/* ---- one quantised linear: out[T,n] = x[T,k] W^T with W given as f32 and
 * quantised by the reference's own load-time quantiser (src/qmat.c:80-112) ---- */
int ref_qmat_mul_from_f32(const float *w, int n, int k, int qtype, const float *x, float *out,
                          int T) {
    /* qmat_init madvise()s the f32 pages away: hand it a private copy */
    float *wc = malloc((size_t)n * (size_t)k * sizeof(float));
    if (!wc) return -1;
    memcpy(wc, w, (size_t)n * (size_t)k * sizeof(float));
    mynah_asr_qmat m;
    if (mynah_asr_qmat_init(&m, wc, n, k, qtype) != 0) { free(wc); return -1; }
    mynah_asr_qmat_mul(&m, x, out, T);
    mynah_asr_qmat_free(&m);
    free(wc);
    return 0;
}
