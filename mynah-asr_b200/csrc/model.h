// Device-resident model: weights, workspace arena and the encoder / decoder drivers.
#pragma once
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/mynah_b200.h"
#include "kernels.h"
#include "qweight.h"

namespace mb {

static constexpr int DEC_MAX_LAYERS = 4;    // MYNAH_ASR_MAX_PRED_LAYERS (src/decoder.h:15)
static constexpr int DEC_MAX_DUR = 16;      // MYNAH_ASR_MAX_DURATIONS
static constexpr int DEC_MAX_B = 16;        // utterances decoded in lock step per launch

struct HostTensor {
    int fmt;
    std::vector<int64_t> shape;
    const void *data;
    size_t nelem() const { size_t n = 1; for (auto s : shape) n *= (size_t)s; return n; }
};

// Bump allocator over one cudaMalloc'd slab; reset at the start of every forward.
struct Arena {
    uint8_t *base = nullptr;
    size_t cap = 0, off = 0;
    int reserve(size_t bytes);
    void reset() { off = 0; }
    void *take(size_t bytes);
    template <typename T> T *get(size_t n) { return reinterpret_cast<T *>(take(n * sizeof(T))); }
    H16 planes(size_t n, bool with_lo = true) { H16 h; h.hi = get<__half>(n); h.lo = with_lo ? get<__half>(n) : nullptr; return h; }
    void release();
};

struct EncLayer {
    const float *ln_ff1_w, *ln_ff1_b, *ln_att_w, *ln_att_b, *ln_conv_w, *ln_conv_b, *ln_ff2_w, *ln_ff2_b, *ln_out_w, *ln_out_b;
    QWeight ff1_w1, ff1_w2, ff2_w1, ff2_w2, q_w, k_w, v_w, o_w, pw1_w, pw2_w, relk;
    const float *bias_u, *bias_v, *dw_w, *dw_b, *cnorm_w, *cnorm_b, *cnorm_scale, *cnorm_shift;
};

// One layer of the AED transformer decoder (mynah_asr_aed_layer, src/decoder_aed.h:13-24): the self-attention
// q/k/v projections and the cross-attention k/v projections are stored concatenated by rows.
struct AedLayer {
    const float *ln_self_w, *ln_self_b, *ln_cross_w, *ln_cross_b, *ln_ffn_w, *ln_ffn_b;
    QWeight sqkv, so, cq, ckv, co, ff1, ff2;
    const float *sqkv_b, *so_b, *cq_b, *ckv_b, *co_b, *ff1_b, *ff2_b;
};

// Cache-aware streaming state of S streams that advance in lock step (the device counterpart of S
// mynah_asr_enc_stream objects, src/encoder.h:93-108). K/V caches are rings of `left` slots: the j-th
// oldest valid frame of every stream sits in slot (start + j) % left.
struct StreamState {
    int S = 0, left = 0, right = 0, q = 1;
    int first = 1, valid = 0;
    // a group of at most 128 rows per regular step (S q <= 128) runs the linears of its layers on the few-row kernel
    // (gemm_skinny.cu), a larger one on the many-row kernel: fixed when the group opens, for its whole life
    bool few_rows = false;
    // rel-pos key projections rk = pos_emb(K) relk^T of every layer for the steady key count K = left + q: they depend on
    // nothing but the weights, so they are computed on the first full step with full caches and reused afterwards
    __half *rk_cache = nullptr;                         // [L][2 (left + q) - 1][d] fp16
    bool rk_ready = false;
    int *ln_count = nullptr;                            // row counters of the LayerNorms that run inside those contractions
    int *d_start = nullptr;                             // ring offset of the oldest frame, kept on the device
    // steady state (caches full, same buffers): one captured graph replays the whole step
    cudaGraphExec_t exec = nullptr;
    cudaGraph_t graph = nullptr;
    const void *g_mel = nullptr, *g_out = nullptr, *g_base = nullptr;
    size_t g_mark = 0;
    int g_launches = 0, g_q = 0, steady_runs = 0;
    // transducer state carried from chunk to chunk (mynah_asr_dec_state, src/decoder.h:31-38), one block per
    // DEC_MAX_B streams: h[2][L][B][H], c[L][B][H], g[B][H] floats; last_tok[B] and the h parity as ints
    float *dec_f = nullptr;
    int *dec_i = nullptr;
    int dec_started = 0;
    long long t_abs = 0;                                // encoder frames decoded so far (same for every stream)
    // incremental log-mel (mynah_asr_mel_stream, src/features.h:40-52): the tail of every stream's signal,
    // [S][MEL_CAP] floats in one of two buffers, samples [mel_base, mel_total) of the signal
    float *mel_buf[2] = {nullptr, nullptr};
    int mel_cur = 0;
    long long mel_base = 0, mel_total = 0, mel_next = 0;
    float *ss_cache[3] = {nullptr, nullptr, nullptr};   // last input frame of each subsampling stage: [S,F0], [S,F1,C], [S,F2,C]
    __half *k_cache = nullptr, *v_cache = nullptr;      // [L][S][H][left][dk] fp16: the ring of one (stream, head) is contiguous
    float *conv_cache = nullptr;                        // [L][S][k-1][d] GLU rows
    std::vector<int> prompt_ids;                        // prompt-conditioned encoders: one id per stream (empty = 0)
    std::vector<void *> owned;
};

struct Model {
    mynah_b200_config cfg;
    std::map<std::string, HostTensor> host;          // until finalize
    std::map<std::string, float *> f32;              // small f32 tensors on the device
    std::vector<void *> owned;                       // every device allocation of the model
    bool finalized = false;
    cudaStream_t stream = nullptr;                   // of this execution context (the weights are shared between contexts)
    Arena ws;
    int *status = nullptr;                           // device status word (bounded waits)

    // optional per-category device timing (CUDA events on `stream` around launches)
    enum { PROF_GEMM = 0, PROF_ATTN, PROF_ELEMWISE, PROF_SUBSAMPLING, PROF_MEL, PROF_DECODE, PROF_NCAT };
    struct ProfSpan { cudaEvent_t a, b; int cat; };
    bool prof_on = false;
    long long dec_dbg[8] = {0};                      // greedy-decoder phase clocks of the last profiled run
    std::vector<ProfSpan> prof_spans;
    size_t prof_used = 0;
    int prof_pending = -1;                           // decode span left open until the lanes have joined
    double prof_flops[PROF_NCAT] = {0}, prof_bytes[PROF_NCAT] = {0};
    long long prof_launches[PROF_NCAT] = {0};
    int prof_begin_span(int cat);                    // returns span index or -1
    void prof_end_span(int idx);

    // encoder
    int d_model = 0, n_layers = 0, n_heads = 0, d_head = 0, ffn_dim = 0, conv_k = 0, d_out = 0, channels = 0;
    int causal = 0, ss_freq[4] = {0, 0, 0, 0};
    float xscale = 1.0f;
    std::vector<EncLayer> layers;
    const float *conv_in_w = nullptr, *conv_in_b = nullptr, *dw_w[2] = {nullptr, nullptr}, *dw_b[2] = {nullptr, nullptr};
    QWeight pw[2], ss_lin, encproj;
    bool has_encproj = false;
    // prompt MLP of encoder_post (src/encoder.c:591-614): the one-hot columns of linear_1 are folded into a
    // per-prompt bias table, bias1[p] = b1 + W1[:, d + p]
    bool has_prompt = false;
    int num_prompts = 0, prompt_inter = 0;
    QWeight prompt_l1, prompt_l2;                    // [inter, d] (the first d columns of linear_1), [d, inter]
    float *prompt_bias1 = nullptr;                   // [num_prompts, inter]

    // decoders
    bool has_ctc = false, has_dec = false;
    QWeight ctc_head;
    int ctc_vocab = 0;
    const float *emb = nullptr, *proj_b = nullptr, *head_b = nullptr;
    H16 emb_planes{nullptr, nullptr};
    const float *b_ih[DEC_MAX_LAYERS], *b_hh[DEC_MAX_LAYERS];
    QWeight head, dec_proj, wcat[DEC_MAX_LAYERS];    // wcat[l] = [W_ih | W_hh] of LSTM layer l
    int vocab = 0, pred_hidden = 0, pred_layers = 0;

    // AED decoder (mynah_asr_aed, src/decoder_aed.h:26-38)
    bool has_aed = false, has_aed_proj = false;
    int aed_d = 0, aed_heads = 0, aed_ffn = 0, aed_vocab = 0, aed_max_seq = 0;
    const float *aed_emb = nullptr, *aed_pos = nullptr, *aed_embln_w = nullptr, *aed_embln_b = nullptr, *aed_fin_w = nullptr,
                *aed_fin_b = nullptr, *aed_head_b = nullptr, *aed_proj_b = nullptr;
    QWeight aed_head, aed_proj;
    std::vector<AedLayer> aed_layers;

    // mel
    std::vector<float> mel_fb_host, window_host;
    float *mel_fb = nullptr;
    int *mel_lo = nullptr, *mel_hi = nullptr;
    double *mel_win = nullptr, *mel_tw = nullptr;
    bool has_mel = false;

    // ---- load path: device memory for the weights comes from a few large slabs (one cudaMalloc per 256 MB instead
    // of one per tensor), host bytes reach the device through two pinned staging buffers (the copy of piece i + 1
    // into its buffer overlaps the DMA of piece i; nothing waits for the stream), and the f32 scratch of the block
    // decode is one buffer reused by every tensor
    struct Slab { uint8_t *base; size_t cap, off; };
    std::vector<Slab> slabs;
    bool use_slabs = false;                          // a whole model loads through slabs and staging; a single qmat handle does not
    uint8_t *stage[2] = {nullptr, nullptr};
    cudaEvent_t stage_ev[2] = {nullptr, nullptr};
    int stage_next = 0;
    float *load_tmp = nullptr;
    size_t load_tmp_cap = 0;
    double load_seconds = 0.0;                       // wall time of add_tensor .. finalize (or of model_load)
    size_t load_bytes = 0;                           // host bytes copied to the device while loading
    int upload_bytes(void *dst, const void *src, size_t n);
    float *decode_scratch(size_t nfloats);
    void release_load_buffers();

    // decode lanes: lock-step groups of DEC_MAX_B utterances run side by side on these streams, each on a share
    // of the SMs (a group's steps are latency-bound, not bandwidth-bound, so four groups on a quarter of the
    // SMs each finish sooner than four groups one after the other on all of them)
    static constexpr int DEC_LANES = 4;
    cudaStream_t lane[DEC_LANES] = {nullptr, nullptr, nullptr, nullptr};
    cudaEvent_t lane_done[DEC_LANES] = {nullptr, nullptr, nullptr, nullptr}, lane_fork = nullptr;
    int lanes_begin(int n_groups);                   // lanes in use (1 = everything stays on `stream`); forks them off `stream`
    cudaStream_t lane_stream(int lanes, int gi) const { return lanes > 1 ? lane[gi % lanes] : stream; }
    int lanes_join(int lanes);                       // `stream` waits for every lane

    ~Model();
    void *dev_alloc(size_t bytes);
    float *upload_f32(const float *src, size_t n);
    int upload_weight(QWeight &w, int fmt, const void *data, const float *scales, int n, int k, bool want_planes,
                      bool want_f32, const int *col_perm = nullptr);
    int check_status(const char *where);

    // drivers (device pointers in / out, all on `stream`)
    int gemm(const H16 &a, int lda, const QWeight &w, const GemmEpilogue &ep, int M, bool few_rows = false);   // few_rows: the decoder-position kernel (gemm_skinny.cu)
    // int8-activation mode: qa [M, w.k] int8 rows with their scales sx [M] times a reference-native int8 weight
    bool a8_ok(const QWeight &w) const { return w.fmt == FMT_MYNAH_Q8 && w.k % 128 == 0 && w.scales != nullptr; }
    bool a8_layers = false;                          // cfg.a8 and every encoder-layer linear is a8_ok
    int gemm_q8(const int8_t *qa, const float *sx, const QWeight &w, const GemmEpilogue &ep, int M);
    int subsample_item(const float *feats_dev, int t_mel, float *x_out, int *t_out);
    int encoder_layers(float *x, const std::vector<int> &lens, int left, int right, int first_layer, int n_run);
    // x [sum lens, d_model] -> out [sum lens, d_out]; prompt_ids (one per segment, may be null = all 0) select the
    // one-hot column of a prompt-conditioned model and are ignored otherwise
    int encoder_post(const float *x, const std::vector<int> &lens, const int *prompt_ids, float *out);
    int decode_ctc(const float *enc_dev, int T, std::vector<int> &tokens, std::vector<int> &frames);
    int decode_greedy(const float *enc_dev, const std::vector<int> &lens, std::vector<std::vector<int>> &tokens,
                      std::vector<std::vector<int>> &frames);
    // packed encoder output [sum T, d_out] -> generated tokens per utterance (prompt and EOS excluded); caps[b] bounds utterance b
    int decode_aed(const float *enc_dev, const std::vector<int> &lens, const std::vector<std::vector<int>> &prompts, int eos,
                   const std::vector<int> &caps, std::vector<std::vector<int>> &tokens);
    size_t aed_bytes(int total_T, int B, int max_len) const;
    // one chunk of every stream: mel_dev [S, n_mel, n_mels] -> out_dev [S, q, d_out]; returns q or -1
    int stream_open(StreamState &st, int S, int left, int right);
    void stream_close(StreamState &st);
    int stream_need(const StreamState &st) const { return st.valid == 0 && st.first ? 1 + 8 * st.right : 8 * (st.right + 1); }
    size_t stream_bytes(const StreamState &st, int n_mel) const;
    int stream_step(StreamState &st, const float *mel_dev, int n_mel, int is_last, float *out_dev);
    int stream_step_eager(StreamState &st, const float *mel_dev, int n_mel, int is_last, float *out_dev);
    // greedy RNNT/TDT over the q new frames of every stream with the state carried from the previous chunk
    // (mynah_asr_greedy_decode with a persistent mynah_asr_dec_state); frames are absolute
    // appends n samples per stream (host, [S][n]) and computes the mel frames that became ready (all of the
    // remaining valid ones with finish): out_host [S][frames][n_mels]; returns the frame count
    int stream_mel_feed(StreamState &st, const float *audio_host, int n, int finish, float *out_host, int cap_frames);
    int stream_decode(StreamState &st, const float *enc_dev, int q, std::vector<std::vector<int>> &tokens,
                      std::vector<std::vector<int>> &frames);
    int log_mel(const float *audio_dev, size_t n, float *feats_dev, int T, int valid);
    static int sub_len(int n, bool causal) { return (n + (causal ? 3 : 2) - 3) / 2 + 1; }
    int enc_len(int t_mel) const { int t = t_mel; for (int i = 0; i < 3; i++) t = sub_len(t, causal); return t; }
};

// Everything the lock-step greedy kernel needs (decoder.cu).
struct GreedyDev {
    // model
    const float *emb, *head_b, *proj_b;
    const __half *emb_hi, *emb_lo;                                 // embedding table as operand planes [V, H]
    const __half *head_hi, *head_lo, *proj_hi, *proj_lo;           // [V+ND, H], [H, H] operand planes
    const __half *wcat_hi[DEC_MAX_LAYERS], *wcat_lo[DEC_MAX_LAYERS];   // [4H, 2H] = [W_ih | W_hh]
    const float *b_ih[DEC_MAX_LAYERS], *b_hh[DEC_MAX_LAYERS];
    int V, ND, H, L, blank, max_symbols;
    int durations[DEC_MAX_DUR];
    // batch
    int B;
    const float *enc;            // packed [sum T, H]
    const int *enc_off, *enc_len;
    // state
    float *h[2], *c;             // h[parity]: fp16 planes (hi [L][B][H] then lo [L][B][H], 4 bytes per value); c[L][B][H] f32
    float *g;                    // [B][H]
    __half *jx_hi, *jx_lo;       // [16][H] each: relu(enc[t] + g) of the coming step as operand planes (written with g)
    int *t, *emitted_here, *n_out, *last_tok, *emit;
    int *tokens, *frames, cap;
    // scratch
    float *cand_v;               // [B][2][row blocks]  (token / duration candidates)
    int *cand_i;
    int *flags;                  // [2][2] {any_emit, all_done} by step parity, [4] final h parity
    int max_steps, init_state;
    int *par_state;              // optional: parity of h carried between launches on the same state
    long long *dbg;              // optional [8] phase timers (clock64 ticks of CTA 0), null = off
};

// blocks: CTAs of the cooperative grid (0 = one per SM); at least p.B
int greedy_launch(const GreedyDev &p, cudaStream_t st, int blocks = 0);
void set_load_seconds(mynah_b200_model *h, double seconds);     // capi.cu: the loader reports its whole wall time

}  // namespace mb
