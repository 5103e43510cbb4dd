/* mynah_b200 — B200 (sm_100a) compute backend for the mynah-asr hot path.
 *
 * A plain C ABI (pointers and sizes only) meant to sit behind the reference's
 * backend dispatch (src/backend.h, src/backend.c) and beside its qmat / encoder /
 * features / decoder entry points. Every function names the reference interface it
 * replaces. Conventions follow the reference: 0 = ok, -1 / NULL = error (the text is
 * available from mynah_b200_last_error()), never abort; host buffers returned to the
 * caller are malloc()'d and freed by the caller with free(); inputs are borrowed.
 * There is no CPU fallback inside: if the device path cannot run, the call fails.
 *
 * Threading: a model is immutable after mynah_b200_model_finalize() and may be shared by
 * several host threads. Every call that runs the encoder or a decoder takes one of the
 * model's execution contexts (its own CUDA stream, workspace arena and status word over the
 * shared weights) for its duration: up to max_contexts (default 4, env MYNAH_B200_CONTEXTS,
 * mynah_b200_model_set_max_contexts) calls run side by side, further ones wait for a free
 * context; there is no lock around the compute. A single-threaded caller always runs on the
 * first context. A stream group stays on the context that opened it. The result of a call does
 * not depend on the context it ran on nor on what runs beside it. One process drives one GPU
 * (cudaSetDevice by the caller, or MYNAH_B200_DEVICE / LOCAL_RANK through
 * mynah_b200_select_device); the model remembers its device and makes it current for the
 * calling thread.
 */
#ifndef MYNAH_B200_H
#define MYNAH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- weight formats ---------------------------------------------------------- */
enum {
    MYNAH_B200_F32 = 0,
    MYNAH_B200_MYNAH_Q8 = 1,   /* reference-native per-row int8 + f32 scales [n]      (src/qmat.h:6-9)  */
    MYNAH_B200_MYNAH_Q4 = 2,   /* reference-native 32-group nibbles + f32 scales [n,k/32]               */
    MYNAH_B200_GGML_Q4_0 = 102,/* ggml blocks, 100 + ggml type id (third_party/ingot/src/dequant.c)     */
    MYNAH_B200_GGML_Q8_0 = 108,
    MYNAH_B200_GGML_Q4_K = 112,
    MYNAH_B200_GGML_Q6_K = 114
};

/* qmat_mul flags */
enum {
    MYNAH_B200_A16 = 0,        /* float activations x exactly decoded weights (the reference's f32 path) */
    MYNAH_B200_A8 = 1,         /* int8 activations, integer block dots (src/qmat.c:186-202,285-364)      */
    MYNAH_B200_FAST = 2,       /* large T: single fp16 tensor-core pass instead of the 3-term split      */
    MYNAH_B200_SCALAR = 4,     /* small T: force the scalar-FMA streaming kernel; for cross-checks        */
    MYNAH_B200_MMA_SYNC = 8,   /* small T: force the warp-level (mma.sync) streaming kernel; Q4_0/Q8_0 with
                                  T <= 8 default to the tcgen05 streaming kernel                          */
    MYNAH_B200_FEW_ROWS = 16   /* any T: the operand-plane contraction of a decoder position (weights as the
                                  128-row side of the MMA, K slices over a thread-block cluster) — what the
                                  AED decoder runs its linears on; here for cross-checks and timing          */
};

/* ---- backend presence and errors --------------------------------------------- */
/* replaces mynah_asr_cuda_available (src/backend.c:24): 1 when the current device has compute capability 10.0
 * (the library holds sm_100a code only) */
int mynah_b200_available(void);
/* picks the GPU for this process: explicit index, else env MYNAH_B200_DEVICE, else LOCAL_RANK, else 0 */
int mynah_b200_select_device(int index);
const char *mynah_b200_last_error(void);

/* ---- f32 GEMM hook ------------------------------------------------------------ */
/* replaces mynah_asr_cuda_gemm_wt (src/backend.c:25, src/cuda_gemm.cu:144-190):
 * out[T,n] = x[T,k] W[n,k]^T, host pointers, synchronous. W is uploaded on every call
 * (no address-keyed cache: for a weight that may change between calls; mynah_asr_cuda_gemm_wt
 * below keeps the reference's cache-by-address convention). */
int mynah_b200_gemm_wt(const float *x, const float *w, float *out, int T, int n, int k);

/* The reference's own hook names (src/backend.c:23-26, defined by src/cuda_gemm.cu:62-90,144-190), so
 * that this library can stand where build/src/cuda_gemm.o stands in `make cuda`: same arguments, same
 * return values (1/0; 0 = done, -1 = the caller falls back to the CPU), and the same convention that W
 * is found again by its host address and must stay unchanged for the life of the process
 * ("W must stay stable", src/backend.h:16-18) — it is uploaded on the first call only. */
int mynah_asr_cuda_available(void);
int mynah_asr_cuda_gemm_wt(const float *x, const float *w, float *out, int T, int n, int k);

/* The same convention for a quantised operand, to be called at the top of mynah_asr_qmat_mul
 * (src/qmat.c:503) with the blocks the weight file holds: wq (and scales, native formats only) are
 * uploaded and re-tiled on the first call with this address and found by address afterwards.
 * Host pointers, synchronous; flags as for mynah_b200_qmat_mul. 0, or -1 with mynah_b200_last_error. */
int mynah_b200_qgemm(const void *wq, int fmt, const float *scales, int n, int k, const float *x, float *out,
                     int T, int flags);
/* Drops every weight the two calls above made resident; to be called where the reference drops its
 * Metal cache (mynah_asr_metal_weights_evict from mynah_asr_free, src/mynah_asr.c:358-361): after the
 * model file is unmapped the addresses mean nothing and a later load may reuse them. The reference's
 * CUDA file has no such call (src/cuda_gemm.cu:96-103 only ever appends). */
void mynah_b200_weights_evict(void);
int mynah_b200_weights_resident(void);        /* entries held, for tests */

/* ---- quantised weight matrix --------------------------------------------------- */
/* replaces mynah_asr_qmat + mynah_asr_qmat_init (src/qmat.h:39-47, src/qmat.c:80-143): the
 * stored blocks are copied to HBM once and stay resident. scales: native formats only. */
typedef struct mynah_b200_qmat mynah_b200_qmat;
mynah_b200_qmat *mynah_b200_qmat_create(int fmt, const void *data, const float *scales, int n, int k);
void mynah_b200_qmat_free(mynah_b200_qmat *m);
/* replaces mynah_asr_qmat_mul (src/qmat.c:503-651): out[T,n] = x[T,k] W^T, host x/out.
 * T <= 16 streams the stored blocks (bandwidth-bound); larger T runs on the tensor cores. */
int mynah_b200_qmat_mul(const mynah_b200_qmat *m, const float *x, float *out, int T, int flags);
/* A8 diagnostics: the exact int32 dot of every 32-block, dots[T][n][k/32], and the activation
 * scales sx[T] (the quantities the reference forms in dot_q8_* / dot_q4_*, src/qmat.c:285-364). */
int mynah_b200_qmat_block_dots(const mynah_b200_qmat *m, const float *x, int T, int32_t *dots, float *sx, float *out);
/* replaces mynah_asr_qmat_dequant (src/qmat.c:171-177): wd[n,k] f32 on the host */
int mynah_b200_qmat_dequant(const mynah_b200_qmat *m, float *wd);
/* same product with x, out already on the device (for callers that keep activations resident).
 * ASYNCHRONOUS: the work is queued on the handle's own stream (created non-blocking: it does not wait
 * for the legacy default stream, so x_dev must be complete before the call) and the return value only
 * says that it was queued. mynah_b200_qmat_sync waits for it and reports what the kernels found.
 * One handle owns one stream, one status word and one scratch area: do not use the same handle from
 * two threads at once (different handles are independent). */
int mynah_b200_qmat_mul_device(const mynah_b200_qmat *m, const float *x_dev, float *out_dev, int T, int flags);
/* waits for everything queued on the handle; -1 if a kernel reported a bounded wait that ran out or a
 * value outside the fp16 operand range (|v| >= 65504, inf, NaN) since the last sync, else 0 */
int mynah_b200_qmat_sync(const mynah_b200_qmat *m);

/* No counterpart in the reference. The int8-activation product of mynah_b200_qmat_mul(.., A8) for
 * hosts that must not allocate device memory while running (a real-time streaming thread, a process
 * with a fixed GPU memory budget): x_dev [T,k] and out_dev [T,n] are DEVICE pointers owned by the
 * caller, and the only scratch (quantised activations + scales) is a fixed ~128 KB array inside the
 * library, so the call makes no cudaMalloc/cudaFree and uses no allocating library routine.
 * Limits: T <= 16 rows and k <= 8192 per call, larger sizes are refused with -1; so are the formats
 * without an int8-activation mode (F32, Q4_K, Q6_K: only Q8_0, Q4_0 and the two native formats have
 * one). Every refusal happens before anything is launched. The first call on a device resolves the
 * array's address, and the first call with a given weight format on a device loads that format's
 * kernel: make one call per format you will use before any stream capture. All calls share the
 * array: it keeps the previous call's contents and calls that overlap on the GPU race — serialise
 * them. The kernels run on the handle's own non-blocking stream, which does not wait for the legacy
 * default stream: x_dev must be completely written (its producer synchronised) before the call.
 * Synchronous: out_dev is complete on return. */
int mynah_b200_qmat_mul_a8_static(const mynah_b200_qmat *m, const float *x_dev, float *out_dev, int T);

/* ---- model --------------------------------------------------------------------- */
typedef struct {
    int n_mels;                 /* mynah.json features.n_mels */
    int n_fft, win_length, hop_length;      /* 512, 400, 160 */
    double preemphasis, log_zero_guard;     /* 0.97, 2^-24 */
    int normalize_per_feature;  /* features.normalize == "per_feature" */
    int causal;                 /* -1: infer from tensor naming (src/subsampling.c:16-35); 0/1: config wins */
    int xscaling;               /* encoder.xscaling */
    int left_ctx, right_ctx;    /* default attention context; left < 0 = full attention */
    int blank_id, max_symbols;  /* decoder.blank_id, decoder.max_symbols_per_step */
    int n_durations;            /* TDT durations; 0 = RNNT */
    int durations[16];
    int strict;                 /* 1: 3-term fp16 split (f32-grade, default); 0: single fp16 pass */
    int attn_impl;              /* 0 tensor-core kernels (default: tcgen05 for full attention over 128-wide heads, else the warp-level tiled one), 1 plain kernel (cross-check), 2 warp-level tiled kernel */
    int aed_heads;              /* decoder.n_heads of an AED model (mynah_asr_aed_init's n_heads); layers, width,
                                 * vocabulary and max_seq are read off the tensors */
    int a8;                     /* 1: the ten linears of every encoder layer take int8 activations (quantize_act_int8,
                                 * src/qmat.c:186-202) and run as integer contractions on the tensor cores — the reference's
                                 * arithmetic with MYNAH_ASR_QGEMM=1 (src/qmat.c:598-643), bit-exact int32 sums. Needs those
                                 * weights in the reference-native per-row int8 format (MYNAH_B200_MYNAH_Q8) with k % 128 == 0.
                                 * 0 (default): float activations (the reference's default path above 16 rows). */
} mynah_b200_config;

void mynah_b200_config_default(mynah_b200_config *cfg);

typedef struct mynah_b200_model mynah_b200_model;
/* replaces the weight side of mynah_asr_load_quant (src/mynah_asr.c:167-350): tensors are handed over by their HF-verbatim names exactly as
 * src/weights.c exposes them (name, shape, data), but block-quantised tensors keep their ggml
 * type instead of being decoded to f32. fmt is one of the MYNAH_B200_* formats; data is
 * borrowed until mynah_b200_model_finalize returns. */
mynah_b200_model *mynah_b200_model_new(const mynah_b200_config *cfg);
int mynah_b200_model_add_tensor(mynah_b200_model *m, const char *name, int fmt, const int64_t *shape, int rank,
                                const void *data);
/* mel filterbank [n_fft/2+1, n_mels] and window [win_length] (mel_filters.safetensors) */
int mynah_b200_model_set_mel(mynah_b200_model *m, const float *mel_fb, const float *window);
/* resolves tensors like mynah_asr_encoder_init / subsampling_init / decoder_init / ctc_init
 * (src/encoder.c:56-183, src/subsampling.c:14-58, src/decoder.c:14-62, src/decoder_ctc.c:11-22),
 * uploads and decodes them; replaces the lazy per-pointer upload of src/cuda_gemm.cu:96-130 */
int mynah_b200_model_finalize(mynah_b200_model *m);
/* replaces mynah_asr_st_open + the loaders of mynah_asr_load_quant in one step (src/weights.c:60-117,
 * src/mynah_asr.c:167-350) for the device path: weights_path is a safetensors or GGUF file with the HF-verbatim
 * tensor names, mel_path the mel_filters.safetensors beside it (NULL: no front end). The file is mapped
 * read-only and every tensor goes from the mapping through pinned staging buffers into device memory; GGUF
 * block tensors (Q4_0, Q8_0, Q4_K, Q6_K) stay blocks and are re-tiled and decoded by kernels — the reference
 * decodes them to f32 on the host at load. quant as in mynah_asr_load_quant: 1 / 2 take the pre-quantised
 * "<name>.q8" / "<name>.q4" + "<name>.scales" tensors of a reference int8 / int4 checkpoint where present.
 * NULL on error. mynah_b200_model_load_stats: wall seconds of the load, host bytes copied, device bytes held. */
mynah_b200_model *mynah_b200_model_load(const char *weights_path, const char *mel_path, const mynah_b200_config *cfg,
                                        int quant);
void mynah_b200_model_load_stats(const mynah_b200_model *m, double *seconds, double *host_bytes, double *device_bytes);
/* upper bound of execution contexts (concurrent calls) of a model; contexts are created on demand, each
 * with its own workspace (sized by the largest call it has served). No counterpart in the reference, whose
 * per-thread state is thread-local (src/cuda_gemm.cu:50-60). */
int mynah_b200_model_set_max_contexts(mynah_b200_model *m, int n);
/* switches the numerics of the tensor-core contractions of later calls: 1 = three fp16 products per term
 * (f32-grade, the default), 0 = a single fp16 product. The weights serve both. A stream group keeps the
 * mode of the step it captured: do not switch while one is open. No counterpart in the reference (its
 * sgemm has one precision); used to report both modes against the same weights. */
int mynah_b200_model_set_strict(mynah_b200_model *m, int strict);
/* replaces mynah_asr_metal_weights_evict / mynah_asr_encoder_free */
void mynah_b200_model_free(mynah_b200_model *m);
/* dims[0..7] = d_model, n_layers, n_heads, ffn_dim, conv_k, d_out, causal, channels */
void mynah_b200_model_dims(const mynah_b200_model *m, int *dims);

/* ---- stages (host in, host out; everything in between stays on the device) ----- */
/* replaces mynah_asr_log_mel (src/features.h:28-29): returns feats [*n_frames, n_mels] */
float *mynah_b200_log_mel(mynah_b200_model *m, const float *audio, size_t n_samples, int *n_frames,
                          int *valid_frames);
/* replaces mynah_asr_subsampling_forward (src/subsampling.h:31-32) */
float *mynah_b200_subsampling_forward(mynah_b200_model *m, const float *feats, int T, int n_mels, int *t_out);
/* replaces mynah_asr_encoder_layer (src/encoder.h:57-58): one block in place on host x [T,d];
 * the positional embedding is computed inside (the reference's pe argument is a pure function of T) */
int mynah_b200_encoder_layer(mynah_b200_model *m, int li, float *x, int T, int left_ctx, int right_ctx);
/* replace mynah_asr_encoder_forward / _forward_raw (src/encoder.h:67-76) */
float *mynah_b200_encoder_forward(mynah_b200_model *m, const float *feats, int t_mel, int n_mels, int prompt_id,
                                  int left_ctx, int right_ctx, int *t_out);
float *mynah_b200_encoder_forward_raw(mynah_b200_model *m, const float *feats, int t_mel, int n_mels, int left_ctx,
                                      int right_ctx, int *t_out);
/* replaces mynah_asr_encoder_forward_batch (src/encoder.h:82-85): padding-free packed batch */
int mynah_b200_encoder_forward_batch(mynah_b200_model *m, const float *const *feats, const int *t_mel, int batch,
                                     int n_mels, const int *prompt_ids, int left_ctx, int right_ctx, float **outs,
                                     int *t_outs);
/* replaces mynah_asr_ctc_decode (src/decoder_ctc.h:28-29) */
int mynah_b200_ctc_decode(mynah_b200_model *m, const float *enc_out, int T, int *tokens, int *frames, int cap);
/* replaces mynah_asr_greedy_decode from a fresh state (src/decoder.h:51-52, as called by
 * eng_decode_rnnt, src/mynah_asr.c:124-137) */
int mynah_b200_greedy_decode(mynah_b200_model *m, const float *enc, int T, int *tokens, int *frames, int cap);

/* replaces mynah_asr_aed_decode (src/decoder_aed.h:44-48): greedy decode of the transformer decoder over
 * enc [T, d_out]; generated tokens (prompt and EOS excluded) in tokens[cap]; returns the count, -1 on error */
int mynah_b200_aed_decode(mynah_b200_model *m, const float *enc, int T, const int *prompt, int n_prompt, int eos,
                          int *tokens, int cap);
/* the same for several utterances decoded in lock step (the batched counterpart of batch_decode_worker,
 * src/mynah_asr.c:473-502, for the AED engine): utterance b has encs[b] [Ts[b], d_out], its own prompt and
 * budget caps[b]; tokens[b] is malloc()'d (caller frees). A batch gives the same tokens as each utterance alone. */
int mynah_b200_aed_decode_batch(mynah_b200_model *m, const float *const *encs, const int *Ts, int batch,
                                const int *const *prompts, const int *n_prompts, int eos, const int *caps, int **tokens,
                                int *n_tokens);

/* ---- CTC forced alignment (word timestamps of the AED engine) ----------------------- */
/* replaces mynah_asr_align_ctc / mynah_asr_align_min_frames (src/align.h:27-32): Viterbi alignment of `tokens`
 * (none of them `blank`) over scores [T, V] (raw logits do); t0[j] / t1[j] receive the first and last frame of
 * token j's run. Host pointers, synchronous; 0, or -1 for bad arguments or when no path exists (T shorter than
 * the tokens plus the blanks repeated labels need). Same result as the reference on the same scores, ties included. */
int mynah_b200_align_ctc(const float *scores, int T, int V, const int *tokens, int n_tokens, int blank, int *t0, int *t1);
int mynah_b200_align_min_frames(const int *tokens, int n_tokens);
/* the aligner step of align_words_ctc (src/mynah_asr.c:1102-1134) with the scores never leaving the device: the
 * model's CTC head over enc_out [T, d_model] (raw encoder output, blank = vocab - 1), then the alignment */
int mynah_b200_ctc_align(mynah_b200_model *m, const float *enc_out, int T, const int *tokens, int n_tokens, int *t0, int *t1);

/* ---- voice activity and offline segment planning ------------------------------------ */
/* the "vad" section of a VAD model's mynah.json (tools/convert_silero.py:192-215) */
typedef struct {
    int frame_samples, context_samples, reflect_pad, n_fft, hop_length, n_bins, lstm_hidden;
    int n_enc;                                   /* conv blocks (Silero v5: 4) */
    int enc_channels[8], enc_kernels[8], enc_strides[8], enc_pads[16];   /* pads: left, right per block */
    double threshold, neg_threshold;
    int min_speech_ms, min_silence_ms, speech_pad_ms;
} mynah_b200_vad_config;
typedef struct mynah_b200_vad mynah_b200_vad;
/* replaces mynah_asr_vad_open (src/vad.h:19-21) for tensors already read by the host: the STFT basis
 * [2 n_bins, n_fft], per block the conv weight [cout, cin, k] and bias, the LSTM (gate order i f g o, both
 * biases), the 1x1 head. NULL on error. */
mynah_b200_vad *mynah_b200_vad_new(const mynah_b200_vad_config *cfg, const float *basis, const float *const *enc_w,
                                   const float *const *enc_b, const float *w_ih, const float *w_hh, const float *b_ih,
                                   const float *b_hh, const float *head_w, float head_b);
void mynah_b200_vad_free(mynah_b200_vad *v);
int mynah_b200_vad_frame_samples(const mynah_b200_vad *v);
/* the probabilities mynah_asr_vad_feed (src/vad.h:29-31) returns frame by frame from a fresh state, for the whole
 * signal in one call: probs[ceil(n / frame_samples)]; returns the frame count, -1 on error */
int mynah_b200_vad_probs(mynah_b200_vad *v, const float *samples, size_t n_samples, float *probs, int cap);
/* replaces mynah_asr_vad_speech_spans (src/vad.h:80-84): padded speech spans as pairs t0, t1 (sample offsets,
 * [t0, t1)); returns their number, -1 on error or when there are more than cap */
int mynah_b200_vad_speech_spans(mynah_b200_vad *v, const float *samples, size_t n_samples, long long *spans, int cap);
/* replaces plan_segments (src/mynah_asr.c:1287-1323; with a VAD the plan of :1216-1280): the ranges the offline
 * path decodes independently, as pairs offset, length. v may be NULL (energy planner). seg_sec is the model's
 * segment limit (mynah_asr_segment_limit). Returns the number of segments (at least one), -1 on error. */
int mynah_b200_plan_segments(mynah_b200_vad *v, const float *samples, size_t n_samples, int sample_rate, double seg_sec,
                             long long *segs, int cap);

/* ---- cache-aware streaming (Nemotron-style causal encoders) ------------------------ */
/* replaces mynah_asr_enc_stream_init / _need / _step / _free (src/encoder.h:110-120) for n_streams
 * streams that advance in lock step: every step takes one chunk of mel frames from each stream and
 * returns q = right_ctx + 1 encoder frames per stream. The K/V caches (left_ctx frames per layer), the
 * conv caches and the subsampling's one-frame caches of all streams stay on the device; all streams of a
 * group start together (open one group per start time).
 * A stream's output does not depend on the other streams of its group. Groups come in two size classes, fixed when the
 * group opens: with n_streams * (right_ctx + 1) <= 128 rows per step the linears of the layers run on the few-row
 * kernel, larger groups on the many-row kernel; inside a class a stream's bits are the same whatever the group's size,
 * across the classes they agree to f32 rounding (relative 1e-5). */
typedef struct mynah_b200_stream_group mynah_b200_stream_group;
mynah_b200_stream_group *mynah_b200_stream_open(mynah_b200_model *m, int n_streams, int left_ctx, int right_ctx);
void mynah_b200_stream_close(mynah_b200_stream_group *g);
/* mel frames every stream must supply to the next step: 1 + 8 right_ctx first, then 8 (right_ctx + 1) */
int mynah_b200_stream_need(const mynah_b200_stream_group *g);
/* prompt-conditioned encoders (the prompt_id argument of mynah_asr_enc_stream_step, src/encoder.h:119-120): one id
 * per stream, to be set before the first step; without this call every stream uses prompt 0 */
int mynah_b200_stream_set_prompts(mynah_b200_stream_group *g, const int *prompt_ids);
/* mel [n_streams, n_mel, n_mels] -> out [n_streams, q, d_out] (host buffers, room for right_ctx + 3 frames
 * per stream as in the reference's callers); n_mel = stream_need() except
 * for the last, shorter chunk (is_last = 1: causal right padding as offline). Returns q, -1 on error. */
int mynah_b200_stream_step(mynah_b200_stream_group *g, const float *mel, int n_mel, int is_last, float *out);
/* replaces mynah_asr_mel_stream_feed / _finish (src/features.h:54-62) for the streams of a group: appends n
 * samples per stream (audio [n_streams, n], float in [-1, 1]) and writes the log-mel frames that became ready
 * to out [n_streams, frames, n_mels] (at most cap_frames; finish = 1 also emits the remaining valid frames,
 * zero-padded to the right). No per-feature normalisation, as in the reference's streaming front end; the
 * frames are bit-identical to mynah_b200_log_mel on the whole signal. Returns the frame count, -1 on error. */
int mynah_b200_stream_mel_feed(mynah_b200_stream_group *g, const float *audio, int n, int finish, float *out,
                               int cap_frames);
/* encoder step and greedy RNNT/TDT decoding of its q frames on the device, with the transducer state of every
 * stream carried from chunk to chunk (mynah_asr_greedy_decode on a persistent mynah_asr_dec_state, as
 * stream_flush_chunk calls it, src/mynah_asr.c:784-822): only the mel chunk and the new token ids cross PCIe.
 * tokens[s] / frames[s] (absolute encoder frames; frames may be NULL) are malloc()'d per stream. Returns q. */
int mynah_b200_stream_step_decode(mynah_b200_stream_group *g, const float *mel, int n_mel, int is_last, int **tokens,
                                  int **frames, int *n_tokens);
/* the same with device buffers on both sides (asynchronous on the model's stream) */
int mynah_b200_stream_step_device(mynah_b200_stream_group *g, const float *mel_dev, int n_mel, int is_last,
                                  float *out_dev);

/* ---- whole path, resident ------------------------------------------------------- */
/* audio in, token ids out: log-mel -> encoder (packed batch) -> greedy decoder, with only the
 * audio and the token ids crossing PCIe. The device-resident counterpart of one wave of
 * mynah_asr_transcribe_batch_ts (src/mynah_asr.c:624-679) up to detokenisation.
 * tokens[b] / frames[b] are malloc()'d (caller frees; frames may be NULL), n_tokens[b] set.
 * decoder: 0 = the model's transducer head (RNNT/TDT), 1 = CTC head (2 = AED: see mynah_b200_transcribe_batch_aed). */
int mynah_b200_transcribe_batch(mynah_b200_model *m, const float *const *audio, const size_t *n_samples, int batch,
                                int decoder, int **tokens, int **frames, int *n_tokens);

/* the same with one prompt id per utterance for prompt-conditioned encoders (the prompt_ids of
 * mynah_asr_encoder_forward_batch, src/encoder.h:82-85, as resolve_prompt fills them, src/mynah_asr.c:416-421);
 * prompt_ids NULL = 0 for all; ignored by models without a prompt projector */
int mynah_b200_transcribe_batch_prompts(mynah_b200_model *m, const float *const *audio, const size_t *n_samples, int batch,
                                        const int *prompt_ids, int decoder, int **tokens, int **frames, int *n_tokens);

/* The AED engine's wave (eng_decode_aed, src/mynah_asr.c:147-160): every utterance starts from the same prompt
 * and may generate T + max_gen_delta tokens (T = its encoder frames). */
int mynah_b200_transcribe_batch_aed(mynah_b200_model *m, const float *const *audio, const size_t *n_samples, int batch,
                                    const int *prompt, int n_prompt, int eos, int max_gen_delta, int **tokens,
                                    int *n_tokens);

/* Same, split for measurement: inputs already resident on the device. h = handle returned by
 * mynah_b200_batch_upload; run may be called repeatedly; results fetched once. */
typedef struct mynah_b200_batch mynah_b200_batch;
mynah_b200_batch *mynah_b200_batch_upload(mynah_b200_model *m, const float *const *audio, const size_t *n_samples,
                                          int batch);
/* one prompt id per utterance for prompt-conditioned encoders (NULL: back to 0 for all) */
void mynah_b200_batch_set_prompts(mynah_b200_batch *h, const int *prompt_ids);
/* decoder 2 (AED) needs its prompt, EOS id and generation allowance set on the handle first */
void mynah_b200_batch_set_aed(mynah_b200_batch *h, const int *prompt, int n_prompt, int eos, int max_gen_delta);
int mynah_b200_batch_run(mynah_b200_model *m, mynah_b200_batch *h, int decoder);
int mynah_b200_batch_fetch(mynah_b200_model *m, mynah_b200_batch *h, int **tokens, int **frames, int *n_tokens);
void mynah_b200_batch_free(mynah_b200_batch *h);

/* ---- introspection for tests and benchmarks ------------------------------------- */
/* number of kernels this library launched since the last reset (its own launches only) */
long long mynah_b200_launch_count(int reset);
/* CUDA stream of the model's first execution context (a cudaStream_t), for event timing by a single-threaded caller */
void *mynah_b200_model_stream(mynah_b200_model *m);
/* Per-category device timing of a model's launches (CUDA events recorded on the model's stream
 * around each launch): categories 0 contraction (tcgen05), 1 attention, 2 element-wise,
 * 3 subsampling convs, 4 log-mel, 5 greedy decoder. profile_end returns, per category, the summed
 * milliseconds, the algorithmic flops (contractions: 2*M*N*K) and the number of launches. */
void mynah_b200_profile_begin(mynah_b200_model *m);
int mynah_b200_profile_end(mynah_b200_model *m, double *ms, double *flops, long long *launches, int ncat);
/* Algorithmic DRAM bytes of the launches since profile_begin, per category (filled for the
 * contractions: both operands' fp16 planes read once, the output and any residual once). */
void mynah_b200_profile_bytes(mynah_b200_model *m, double *bytes, int ncat);
/* Phase clocks (SM cycles seen by CTA 0) of the last greedy-decoder launch made while profiling was
 * on: head, head barrier, select + barrier, LSTM layers + barriers, projector + barrier, then the
 * number of steps and of steps in which some utterance emitted. */
void mynah_b200_decoder_clocks(mynah_b200_model *m, long long *out8);
/* Times one large-T contraction with device-resident operands: returns the average milliseconds
 * of `iters` launches of out[T,n] = x[T,k] W^T (CUDA events on the launching stream). */
double mynah_b200_qmat_time(const mynah_b200_qmat *m, int T, int flags, int iters);

#ifdef __cplusplus
}
#endif
#endif
