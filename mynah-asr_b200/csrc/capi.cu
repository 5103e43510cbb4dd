// extern "C" boundary (include/mynah_b200.h): plain pointers and sizes in, host
// buffers out; resolves the reference's tensor names and drives the device path.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <chrono>
#include <condition_variable>
#include <memory>

#include "model.h"

using namespace mb;

namespace mb { long long launch_count(bool reset); }

// A model handle = the immutable weights + a small pool of execution contexts. Context 0 is `m` itself; further
// contexts are shallow copies of it made on demand (same device pointers to the weights, their own CUDA stream,
// workspace arena, status word and profiling state), so calls from several host threads run side by side on the
// same weights — the counterpart of the reference's per-thread cuBLAS handle / stream / buffers over a shared
// weight cache (src/cuda_gemm.cu:50-60,92-130).
struct mynah_b200_model {
    Model m;
    std::vector<std::unique_ptr<Model>> extra;      // contexts 1..
    std::vector<char> busy{0};                      // per context
    std::mutex pool_mu;
    std::condition_variable pool_cv;
    int max_ctx = 4;
    int device = 0;                                 // the GPU the model lives on
    Model &ctx(int i) { return i == 0 ? m : *extra[(size_t)i - 1]; }
    int n_ctx() const { return 1 + (int)extra.size(); }
};

namespace {
// Takes a free context for the duration of a call (lowest index first, so a single-threaded caller always runs on
// context 0); creates one while fewer than max_ctx exist, else waits. want >= 0: that context and no other (a
// stream group's caches and captured graph belong to the context that opened it).
class Lease {
public:
    explicit Lease(mynah_b200_model *h, int want = -1) : h_(h) {
        cudaSetDevice(h->device);                    // a fresh host thread starts on device 0
        std::unique_lock<std::mutex> lk(h->pool_mu);
        for (;;) {
            if (want >= 0) {
                if (want < h->n_ctx() && !h->busy[(size_t)want]) { idx_ = want; break; }
            } else {
                for (int i = 0; i < h->n_ctx(); i++) if (!h->busy[(size_t)i]) { idx_ = i; break; }
                if (idx_ >= 0) break;
                if (h->n_ctx() < h->max_ctx && h->m.finalized) {
                    if (Model *c = clone_context(h->m)) {
                        h->extra.emplace_back(c);
                        h->busy.push_back(0);
                        idx_ = h->n_ctx() - 1;
                        break;
                    }
                }
            }
            h->pool_cv.wait(lk);
        }
        h->busy[(size_t)idx_] = 1;
    }
    ~Lease() {
        { std::lock_guard<std::mutex> lk(h_->pool_mu); h_->busy[(size_t)idx_] = 0; }
        h_->pool_cv.notify_all();
    }
    Model &model() { return h_->ctx(idx_); }
    int index() const { return idx_; }
    Lease(const Lease &) = delete;
    Lease &operator=(const Lease &) = delete;

private:
    static Model *clone_context(const Model &src) {
        Model *c = new Model(src);                   // weights: the same device pointers
        c->owned.clear();                            // ... which only context 0 owns
        c->slabs.clear(); c->use_slabs = false;
        for (int i = 0; i < Model::DEC_LANES; i++) { c->lane[i] = nullptr; c->lane_done[i] = nullptr; }
        c->lane_fork = nullptr;
        c->prof_spans.clear(); c->prof_used = 0; c->prof_on = false;
        c->ws = Arena();
        c->stream = nullptr; c->status = nullptr;
        if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) { cudaGetLastError(); delete c; return nullptr; }
        c->status = (int *)c->dev_alloc(sizeof(int));
        if (!c->status || cudaMemset(c->status, 0, sizeof(int)) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) { delete c; return nullptr; }
        return c;
    }
    mynah_b200_model *h_;
    int idx_ = -1;
};

// Runs fn on every context while none of them is in a call.
template <typename F>
void with_all_contexts_idle(mynah_b200_model *h, F fn) {
    std::unique_lock<std::mutex> lk(h->pool_mu);
    h->pool_cv.wait(lk, [&] { for (char b : h->busy) if (b) return false; return true; });
    for (int i = 0; i < h->n_ctx(); i++) fn(h->ctx(i));
}
}  // namespace
struct mynah_b200_qmat {
    QWeight w;
    std::vector<void *> owned;
    cudaStream_t stream = nullptr;
    int *status = nullptr;
};
struct mynah_b200_batch {
    int batch = 0;
    std::vector<float *> audio;          // device
    std::vector<size_t> n_samples;
    std::vector<std::vector<int>> tokens, frames;
    std::vector<int> prompt_ids;         // prompt-conditioned encoders: one id per utterance (empty = 0 for all)
    std::vector<int> aed_prompt;         // decoder 2 (AED): the prompt every utterance starts from,
    int aed_eos = -1, aed_delta = 0;     // the end-of-sequence id and the generation allowance beyond T
};

struct mynah_b200_stream_group {
    mynah_b200_model *model = nullptr;
    int ctx = 0;                         // the execution context the group lives on
    mb::StreamState st;
};

namespace mb {
void set_load_seconds(mynah_b200_model *h, double seconds) { if (h) h->m.load_seconds = seconds; }
QmatView qmat_view(const void *handle) {
    const mynah_b200_qmat *q = static_cast<const mynah_b200_qmat *>(handle);
    return QmatView{&q->w, q->stream};
}
}  // namespace mb

static int internal_fmt(int fmt) {
    switch (fmt) {
    case MYNAH_B200_F32: return FMT_F32;
    case MYNAH_B200_MYNAH_Q8: return FMT_MYNAH_Q8;
    case MYNAH_B200_MYNAH_Q4: return FMT_MYNAH_Q4;
    case MYNAH_B200_GGML_Q4_0: return FMT_GGML_Q4_0;
    case MYNAH_B200_GGML_Q8_0: return FMT_GGML_Q8_0;
    case MYNAH_B200_GGML_Q4_K: return FMT_GGML_Q4_K;
    case MYNAH_B200_GGML_Q6_K: return FMT_GGML_Q6_K;
    default: return -1;
    }
}

extern "C" {

const char *mynah_b200_last_error(void) { return mb::last_error(); }

int mynah_b200_available(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) { cudaGetLastError(); return 0; }
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, dev) != cudaSuccess) { cudaGetLastError(); return 0; }
    return p.major == 10 && p.minor == 0 ? 1 : 0;      // the library holds sm_100a code only
}

int mynah_b200_select_device(int index) {
    if (index < 0) {
        const char *e = getenv("MYNAH_B200_DEVICE");
        if (!e) e = getenv("LOCAL_RANK");
        index = e ? atoi(e) : 0;
    }
    int n = 0;
    MB_CUDA(cudaGetDeviceCount(&n));
    if (index >= n) { set_error("device %d requested, %d present", index, n); return -1; }
    MB_CUDA(cudaSetDevice(index));
    return index;
}

long long mynah_b200_launch_count(int reset) { return mb::launch_count(reset != 0); }

void mynah_b200_config_default(mynah_b200_config *c) {
    memset(c, 0, sizeof(*c));
    c->n_mels = 128; c->n_fft = 512; c->win_length = 400; c->hop_length = 160;
    c->preemphasis = 0.97; c->log_zero_guard = 5.9604644775390625e-8;
    c->normalize_per_feature = 1; c->causal = -1; c->xscaling = 0;
    c->left_ctx = -1; c->right_ctx = -1; c->blank_id = 0; c->max_symbols = 10;
    c->n_durations = 0; c->strict = 1; c->attn_impl = 0; c->aed_heads = 8; c->a8 = 0;
}

// ------------------------------------------------------------------- model
mynah_b200_model *mynah_b200_model_new(const mynah_b200_config *cfg) {
    if (!mynah_b200_available()) { set_error("no sm_100 CUDA device available"); return nullptr; }
    mynah_b200_model *h = new mynah_b200_model();
    if (cfg) h->m.cfg = *cfg; else mynah_b200_config_default(&h->m.cfg);
    cudaGetDevice(&h->device);
    if (const char *e = getenv("MYNAH_B200_CONTEXTS")) { const int n = atoi(e); if (n >= 1 && n <= 64) h->max_ctx = n; }
    if (cudaStreamCreateWithFlags(&h->m.stream, cudaStreamNonBlocking) != cudaSuccess) {
        set_error("cudaStreamCreate failed"); delete h; return nullptr;
    }
    h->m.status = (int *)h->m.dev_alloc(sizeof(int));
    if (!h->m.status) { delete h; return nullptr; }
    h->m.use_slabs = true;
    cudaMemset(h->m.status, 0, sizeof(int));
    cudaDeviceSynchronize();
    return h;
}

int mynah_b200_model_add_tensor(mynah_b200_model *h, const char *name, int fmt, const int64_t *shape, int rank,
                                const void *data) {
    if (!h || !name || !data || rank <= 0 || rank > 8) { set_error("add_tensor: bad argument"); return -1; }
    if (h->m.finalized) { set_error("add_tensor after finalize"); return -1; }
    const int f = internal_fmt(fmt);
    if (f < 0) { set_error("add_tensor '%s': unknown format %d", name, fmt); return -1; }
    HostTensor t;
    t.fmt = f; t.data = data; t.shape.assign(shape, shape + rank);
    h->m.host[name] = t;
    return 0;
}

int mynah_b200_model_set_mel(mynah_b200_model *h, const float *mel_fb, const float *window) {
    if (!h || !mel_fb || !window) { set_error("set_mel: bad argument"); return -1; }
    Model &m = h->m;
    const int nb = m.cfg.n_fft / 2 + 1, nm = m.cfg.n_mels, nf = m.cfg.n_fft;
    m.mel_fb = m.upload_f32(mel_fb, (size_t)nb * nm);
    // non-zero bin range per filter, as mel_ranges does (src/features.c:50-61)
    std::vector<int> lo(nm), hi(nm);
    for (int k = 0; k < nm; k++) {
        int a = nb, z = 0;
        for (int b = 0; b < nb; b++) if (mel_fb[(size_t)b * nm + k] != 0.0f) { if (b < a) a = b; z = b + 1; }
        lo[k] = a; hi[k] = z;
    }
    std::vector<double> win(nf, 0.0), tw(nf);
    const int off = (nf - m.cfg.win_length) / 2;
    for (int i = 0; i < m.cfg.win_length; i++) win[off + i] = (double)window[i];
    for (int j = 0; j < nf / 2; j++) { const double a = -2.0 * M_PI * j / nf; tw[2 * j] = cos(a); tw[2 * j + 1] = sin(a); }
    m.mel_lo = (int *)m.dev_alloc(nm * sizeof(int));
    m.mel_hi = (int *)m.dev_alloc(nm * sizeof(int));
    m.mel_win = (double *)m.dev_alloc(nf * sizeof(double));
    m.mel_tw = (double *)m.dev_alloc(nf * sizeof(double));
    if (!m.mel_fb || !m.mel_lo || !m.mel_hi || !m.mel_win || !m.mel_tw) return -1;
    MB_CUDA(cudaMemcpy(m.mel_lo, lo.data(), nm * sizeof(int), cudaMemcpyHostToDevice));
    MB_CUDA(cudaMemcpy(m.mel_hi, hi.data(), nm * sizeof(int), cudaMemcpyHostToDevice));
    MB_CUDA(cudaMemcpy(m.mel_win, win.data(), nf * sizeof(double), cudaMemcpyHostToDevice));
    MB_CUDA(cudaMemcpy(m.mel_tw, tw.data(), nf * sizeof(double), cudaMemcpyHostToDevice));
    MB_CUDA(cudaDeviceSynchronize());     // these went through the legacy stream; the model's stream does not wait on it
    m.has_mel = true;
    return 0;
}

}  // extern "C"

// ---- name resolution helpers
static const HostTensor *find(Model &m, const std::string &name) {
    auto it = m.host.find(name);
    return it == m.host.end() ? nullptr : &it->second;
}
static const float *f32dev(Model &m, const std::string &name, bool required, int *err) {
    const HostTensor *t = find(m, name);
    if (!t) { if (required) { set_error("missing tensor '%s'", name.c_str()); *err = 1; } return nullptr; }
    if (t->fmt != FMT_F32) { set_error("tensor '%s' must be f32", name.c_str()); *err = 1; return nullptr; }
    float *d = m.upload_f32((const float *)t->data, t->nelem());
    if (!d) *err = 1;
    return d;
}
// a linear [n, k] or [n, k, 1]; bias looked up beside it
static int lin(Model &m, QWeight &w, const std::string &wname, bool planes, bool want_f32, const int *perm = nullptr) {
    const HostTensor *t = find(m, wname);
    if (!t || t->shape.empty() || t->shape[0] <= 0) { set_error("missing tensor '%s'", wname.c_str()); return -1; }
    const int n = (int)t->shape[0], k = (int)(t->nelem() / (size_t)t->shape[0]);
    const HostTensor *ts = find(m, wname + ".scales");     // native quantised checkpoints
    if (m.upload_weight(w, t->fmt, t->data, ts ? (const float *)ts->data : nullptr, n, k, planes, want_f32, perm)) return -1;
    std::string bname = wname;
    const size_t p = bname.rfind(".weight");
    if (p != std::string::npos) bname.replace(p, 7, ".bias");
    int err = 0;
    w.bias = const_cast<float *>(f32dev(m, bname, false, &err));
    return err ? -1 : 0;
}

// several linears over the same input, stored one below the other: [sum n, k] with the biases concatenated
// (block formats keep whole rows of blocks, so the stored bytes concatenate as they are)
static int lin_cat(Model &m, QWeight &w, const float **bias, const std::vector<std::string> &prefixes) {
    std::vector<uint8_t> bytes;
    std::vector<float> b;
    int fmt = -1, k = 0, n = 0;
    for (const std::string &pre : prefixes) {
        const HostTensor *t = find(m, pre + ".weight"), *tb = find(m, pre + ".bias");
        if (!t || t->shape.size() != 2 || !tb || tb->fmt != FMT_F32) { set_error("missing tensor '%s.weight' or its bias", pre.c_str()); return -1; }
        if (t->fmt == FMT_MYNAH_Q8 || t->fmt == FMT_MYNAH_Q4) { set_error("'%s': natively quantised AED weights are not supported", pre.c_str()); return -1; }
        if (fmt < 0) { fmt = t->fmt; k = (int)t->shape[1]; }
        if (t->fmt != fmt || (int)t->shape[1] != k) { set_error("'%s': projections of one attention differ in format or width", pre.c_str()); return -1; }
        const size_t nb = format_bytes(fmt, (int)t->shape[0], k);
        bytes.insert(bytes.end(), (const uint8_t *)t->data, (const uint8_t *)t->data + nb);
        b.insert(b.end(), (const float *)tb->data, (const float *)tb->data + t->shape[0]);
        n += (int)t->shape[0];
    }
    if (m.upload_weight(w, fmt, bytes.data(), nullptr, n, k, true, false)) return -1;
    *bias = m.upload_f32(b.data(), b.size());
    return *bias ? 0 : -1;
}

extern "C" {

int mynah_b200_model_finalize(mynah_b200_model *h) {
    if (!h) { set_error("finalize: null model"); return -1; }
    Model &m = h->m;
    if (m.finalized) return 0;
    const auto t_load0 = std::chrono::steady_clock::now();
    int err = 0;
    const std::string ss = "encoder.subsampling.";
    std::string cin, dwn[2], pwn[2];
    int causal_naming;
    if (find(m, ss + "conv_in.weight")) {           // Nemotron naming (src/subsampling.c:16-35)
        causal_naming = 1; cin = ss + "conv_in";
        for (int i = 0; i < 2; i++) { dwn[i] = ss + "layers." + std::to_string(i) + ".depthwise_conv"; pwn[i] = ss + "layers." + std::to_string(i) + ".pointwise_conv"; }
    } else {                                        // Parakeet naming (src/subsampling.c:36-52)
        causal_naming = 0; cin = ss + "layers.0";
        dwn[0] = ss + "layers.2"; dwn[1] = ss + "layers.5"; pwn[0] = ss + "layers.3"; pwn[1] = ss + "layers.6";
    }
    m.causal = m.cfg.causal >= 0 ? m.cfg.causal : causal_naming;
    const HostTensor *tc = find(m, cin + ".weight"), *tl = find(m, ss + "linear.weight");
    if (!tc || !tl) { set_error("missing subsampling tensors"); return -1; }
    m.channels = (int)tc->shape[0];
    m.d_model = (int)tl->shape[0];
    m.conv_in_w = f32dev(m, cin + ".weight", true, &err);
    m.conv_in_b = f32dev(m, cin + ".bias", true, &err);
    for (int i = 0; i < 2 && !err; i++) {
        m.dw_w[i] = f32dev(m, dwn[i] + ".weight", true, &err);
        m.dw_b[i] = f32dev(m, dwn[i] + ".bias", true, &err);
        if (lin(m, m.pw[i], pwn[i] + ".weight", true, false)) return -1;
        if (!m.pw[i].bias) { set_error("missing '%s.bias'", pwn[i].c_str()); return -1; }
    }
    if (err) return -1;
    {   // channel-major flatten c*F'+f  ->  f*C+c (see subsampling.cu)
        const int CF = (int)tl->shape[1], C = m.channels, F3 = CF / C;
        int f = m.cfg.n_mels;
        for (int i = 0; i < 3; i++) f = Model::sub_len(f, m.causal);
        if (f != F3) { set_error("subsampling linear expects %d freq bins, n_mels=%d gives %d", F3, m.cfg.n_mels, f); return -1; }
        std::vector<int> perm(CF);
        for (int ff = 0; ff < F3; ff++) for (int c = 0; c < C; c++) perm[ff * C + c] = c * F3 + ff;
        if (lin(m, m.ss_lin, ss + "linear.weight", true, false, perm.data())) return -1;
        if (!m.ss_lin.bias) { set_error("missing subsampling linear bias"); return -1; }
    }
    const HostTensor *bu = find(m, "encoder.layers.0.self_attn.bias_u");
    const HostTensor *dw = find(m, "encoder.layers.0.conv.depthwise_conv.weight");
    if (!bu || !dw) { set_error("missing encoder.layers.0 tensors"); return -1; }
    m.n_heads = (int)bu->shape[0]; m.d_head = (int)bu->shape[1]; m.conv_k = (int)dw->shape[2];
    if (m.cfg.xscaling) m.xscale = sqrtf((float)m.d_model);
    int nl = 0;
    while (find(m, "encoder.layers." + std::to_string(nl) + ".norm_out.weight")) nl++;
    if (nl == 0) { set_error("no encoder layers found"); return -1; }
    m.n_layers = nl;
    m.layers.resize(nl);
    const bool bn = find(m, "encoder.layers.0.conv.norm.running_mean") != nullptr;
    for (int li = 0; li < nl; li++) {
        EncLayer &L = m.layers[li];
        const std::string p = "encoder.layers." + std::to_string(li) + ".";
        L.ln_ff1_w = f32dev(m, p + "norm_feed_forward1.weight", true, &err); L.ln_ff1_b = f32dev(m, p + "norm_feed_forward1.bias", true, &err);
        L.ln_att_w = f32dev(m, p + "norm_self_att.weight", true, &err); L.ln_att_b = f32dev(m, p + "norm_self_att.bias", true, &err);
        L.ln_conv_w = f32dev(m, p + "norm_conv.weight", true, &err); L.ln_conv_b = f32dev(m, p + "norm_conv.bias", true, &err);
        L.ln_ff2_w = f32dev(m, p + "norm_feed_forward2.weight", true, &err); L.ln_ff2_b = f32dev(m, p + "norm_feed_forward2.bias", true, &err);
        L.ln_out_w = f32dev(m, p + "norm_out.weight", true, &err); L.ln_out_b = f32dev(m, p + "norm_out.bias", true, &err);
        L.bias_u = f32dev(m, p + "self_attn.bias_u", true, &err); L.bias_v = f32dev(m, p + "self_attn.bias_v", true, &err);
        L.dw_w = f32dev(m, p + "conv.depthwise_conv.weight", true, &err);
        L.dw_b = f32dev(m, p + "conv.depthwise_conv.bias", false, &err);
        L.cnorm_w = f32dev(m, p + "conv.norm.weight", true, &err); L.cnorm_b = f32dev(m, p + "conv.norm.bias", true, &err);
        L.cnorm_scale = L.cnorm_shift = nullptr;
        if (err) return -1;
        if (bn) {   // fold BatchNorm running stats (src/encoder.c:149-170)
            const HostTensor *mu = find(m, p + "conv.norm.running_mean"), *var = find(m, p + "conv.norm.running_var");
            const HostTensor *gw = find(m, p + "conv.norm.weight"), *gb = find(m, p + "conv.norm.bias");
            if (!mu || !var) { set_error("missing BatchNorm running stats at layer %d", li); return -1; }
            std::vector<float> sc(m.d_model), sh(m.d_model);
            for (int i = 0; i < m.d_model; i++) {
                sc[i] = (float)((double)((const float *)gw->data)[i] / sqrt((double)((const float *)var->data)[i] + 1e-5));
                sh[i] = ((const float *)gb->data)[i] - ((const float *)mu->data)[i] * sc[i];
            }
            L.cnorm_scale = m.upload_f32(sc.data(), m.d_model);
            L.cnorm_shift = m.upload_f32(sh.data(), m.d_model);
            if (!L.cnorm_scale || !L.cnorm_shift) return -1;
        }
        if (lin(m, L.ff1_w1, p + "feed_forward1.linear1.weight", true, false) || lin(m, L.ff1_w2, p + "feed_forward1.linear2.weight", true, false) ||
            lin(m, L.ff2_w1, p + "feed_forward2.linear1.weight", true, false) || lin(m, L.ff2_w2, p + "feed_forward2.linear2.weight", true, false) ||
            lin(m, L.q_w, p + "self_attn.q_proj.weight", true, false) || lin(m, L.k_w, p + "self_attn.k_proj.weight", true, false) ||
            lin(m, L.v_w, p + "self_attn.v_proj.weight", true, false) || lin(m, L.o_w, p + "self_attn.o_proj.weight", true, false) ||
            lin(m, L.relk, p + "self_attn.relative_k_proj.weight", true, false) ||
            lin(m, L.pw1_w, p + "conv.pointwise_conv1.weight", true, false) || lin(m, L.pw2_w, p + "conv.pointwise_conv2.weight", true, false))
            return -1;
    }
    m.ffn_dim = m.layers[0].ff1_w1.n;
    m.d_out = m.d_model;
    if (m.cfg.a8) {
        for (int li = 0; li < nl; li++) {
            const EncLayer &L = m.layers[li];
            const QWeight *ws[10] = {&L.ff1_w1, &L.ff1_w2, &L.ff2_w1, &L.ff2_w2, &L.q_w, &L.k_w, &L.v_w, &L.o_w, &L.pw1_w, &L.pw2_w};
            for (const QWeight *w : ws)
                if (!m.a8_ok(*w)) {
                    set_error("a8 mode: the linears of encoder layer %d must be reference-native int8 [n,k] with k %% 128 == 0 (got format %d, k=%d)", li, w->fmt, w->k);
                    return -1;
                }
        }
        m.a8_layers = true;
    }
    if (find(m, "encoder_projector.weight")) {
        if (lin(m, m.encproj, "encoder_projector.weight", true, false)) return -1;
        m.has_encproj = true;
        m.d_out = m.encproj.n;
    }
    if (const HostTensor *p1 = find(m, "prompt_projector.linear_1.weight")) {
        // Nemotron-style prompt MLP (mynah_asr_encoder_init, src/encoder.c:65-77,173-176): linear_1 is [inter, d + num_prompts]
        const HostTensor *b1 = find(m, "prompt_projector.linear_1.bias"), *p2 = find(m, "prompt_projector.linear_2.weight");
        const int d = m.d_model;
        if (!m.has_encproj || !b1 || !p2 || p1->fmt != FMT_F32 || b1->fmt != FMT_F32 || p1->shape.size() != 2 || (int)p1->shape[1] <= d) {
            set_error("prompt_projector needs f32 linear_1 [inter, d + prompts] with its bias, linear_2 and an encoder_projector"); return -1;
        }
        const int di = (int)p1->shape[0], dcat = (int)p1->shape[1], np = dcat - d;
        if (di % 64) { set_error("prompt_projector width %d must be a multiple of 64", di); return -1; }
        const float *w1 = (const float *)p1->data, *bb = (const float *)b1->data;
        std::vector<float> main((size_t)di * d), table((size_t)np * di);
        for (int i = 0; i < di; i++) {
            memcpy(&main[(size_t)i * d], w1 + (size_t)i * dcat, (size_t)d * sizeof(float));
            // the reference adds b1 to (x W^T + W[:, d + p]); the sum of the two constants first differs by an ulp at most
            for (int p = 0; p < np; p++) table[(size_t)p * di + i] = w1[(size_t)i * dcat + d + p] + bb[i];
        }
        if (m.upload_weight(m.prompt_l1, FMT_F32, main.data(), nullptr, di, d, true, false)) return -1;
        m.prompt_bias1 = m.upload_f32(table.data(), table.size());
        if (!m.prompt_bias1 || lin(m, m.prompt_l2, "prompt_projector.linear_2.weight", true, false)) return -1;
        if (!m.prompt_l2.bias || m.prompt_l2.n != d || m.prompt_l2.k != di) { set_error("prompt_projector.linear_2 must be [d, inter] with a bias"); return -1; }
        m.has_prompt = true; m.num_prompts = np; m.prompt_inter = di;
    }
    if (find(m, "ctc_head.weight")) {
        if (lin(m, m.ctc_head, "ctc_head.weight", true, false)) return -1;
        if (!m.ctc_head.bias) { set_error("missing ctc_head.bias"); return -1; }
        m.has_ctc = true;
        m.ctc_vocab = m.ctc_head.n;
    }
    if (const HostTensor *e = find(m, "decoder.embedding.weight")) {
        m.vocab = (int)e->shape[0]; m.pred_hidden = (int)e->shape[1];
        m.emb = f32dev(m, "decoder.embedding.weight", true, &err);
        if (m.emb) {                       // the same table as fp16 (hi, lo) planes: LSTM inputs are copied, not converted
            const size_t ne = (size_t)m.vocab * m.pred_hidden;
            m.emb_planes.hi = (__half *)m.dev_alloc(ne * 2); m.emb_planes.lo = (__half *)m.dev_alloc(ne * 2);
            if (!m.emb_planes.hi || !m.emb_planes.lo || split_to_h16(m.emb, m.emb_planes.hi, m.emb_planes.lo, ne, m.stream, m.status)) return -1;
        }
        m.proj_b = f32dev(m, "decoder.decoder_projector.bias", true, &err);
        m.head_b = f32dev(m, "joint.head.bias", true, &err);
        int n = 0;
        const int Hh = m.pred_hidden;
        for (; n < DEC_MAX_LAYERS; n++) {
            const std::string s = std::to_string(n);
            const HostTensor *wi = find(m, "decoder.lstm.weight_ih_l" + s), *wh = find(m, "decoder.lstm.weight_hh_l" + s);
            if (!wi) break;
            if (!wh || wi->fmt != FMT_F32 || wh->fmt != FMT_F32 || (int)wi->nelem() != 4 * Hh * Hh || (int)wh->nelem() != 4 * Hh * Hh) {
                set_error("LSTM layer %d is incomplete or has an unexpected shape", n); return -1;
            }
            m.b_ih[n] = f32dev(m, "decoder.lstm.bias_ih_l" + s, true, &err);
            m.b_hh[n] = f32dev(m, "decoder.lstm.bias_hh_l" + s, true, &err);
            // [W_ih | W_hh] side by side so one contraction over [input ; h] gives the gate pre-activations
            std::vector<float> cat((size_t)4 * Hh * 2 * Hh);
            for (int r = 0; r < 4 * Hh; r++) {
                memcpy(&cat[(size_t)r * 2 * Hh], (const float *)wi->data + (size_t)r * Hh, Hh * sizeof(float));
                memcpy(&cat[(size_t)r * 2 * Hh + Hh], (const float *)wh->data + (size_t)r * Hh, Hh * sizeof(float));
            }
            if (m.upload_weight(m.wcat[n], FMT_F32, cat.data(), nullptr, 4 * Hh, 2 * Hh, true, false)) return -1;
        }
        if (err) return -1;
        if (n == 0 || m.pred_hidden > 1024 || m.pred_hidden % 32) { set_error("unsupported prediction network (layers %d, hidden %d)", n, m.pred_hidden); return -1; }
        m.pred_layers = n;
        if (lin(m, m.dec_proj, "decoder.decoder_projector.weight", true, false)) return -1;
        if (lin(m, m.head, "joint.head.weight", true, false)) return -1;
        if (m.head.n != m.vocab + m.cfg.n_durations) { set_error("joint head has %d rows, expected vocab %d + %d durations", m.head.n, m.vocab, m.cfg.n_durations); return -1; }
        if (m.d_out != m.pred_hidden) { set_error("encoder output width %d != prediction hidden %d", m.d_out, m.pred_hidden); return -1; }
        m.has_dec = true;
    }
    if (const HostTensor *e = find(m, "aed.embedding.weight")) {
        // mynah_asr_aed_init (src/decoder_aed.c:50-113)
        if (e->fmt != FMT_F32 || e->shape.size() != 2) { set_error("aed.embedding.weight must be f32 [vocab, d]"); return -1; }
        m.aed_vocab = (int)e->shape[0]; m.aed_d = (int)e->shape[1];
        m.aed_heads = m.cfg.aed_heads > 0 ? m.cfg.aed_heads : 8;
        if (m.aed_d % m.aed_heads || m.aed_d % 64) { set_error("AED width %d must be a multiple of 64 and of its %d heads", m.aed_d, m.aed_heads); return -1; }
        const HostTensor *pe = find(m, "aed.pos_enc");
        if (!pe || pe->shape.size() != 2 || (int)pe->shape[1] != m.aed_d) { set_error("missing or misshapen aed.pos_enc"); return -1; }
        m.aed_max_seq = (int)pe->shape[0];
        m.aed_emb = f32dev(m, "aed.embedding.weight", true, &err);
        m.aed_pos = f32dev(m, "aed.pos_enc", true, &err);
        m.aed_embln_w = f32dev(m, "aed.emb_norm.weight", true, &err); m.aed_embln_b = f32dev(m, "aed.emb_norm.bias", true, &err);
        m.aed_fin_w = f32dev(m, "aed.final_norm.weight", true, &err); m.aed_fin_b = f32dev(m, "aed.final_norm.bias", true, &err);
        if (err) return -1;
        if (lin(m, m.aed_head, "aed.head.weight", true, false)) return -1;
        m.aed_head_b = m.aed_head.bias;
        if (!m.aed_head_b) { set_error("missing aed.head.bias"); return -1; }
        if (find(m, "enc_dec_proj.weight")) {
            if (lin(m, m.aed_proj, "enc_dec_proj.weight", true, false)) return -1;
            m.aed_proj_b = m.aed_proj.bias;
            m.has_aed_proj = true;
            if (m.aed_proj.n != m.aed_d || m.aed_proj.k != m.d_out) { set_error("enc_dec_proj is [%d,%d], expected [%d,%d]", m.aed_proj.n, m.aed_proj.k, m.aed_d, m.d_out); return -1; }
        } else if (m.d_out != m.aed_d) { set_error("encoder output width %d != AED width %d and no enc_dec_proj", m.d_out, m.aed_d); return -1; }
        int nl = 0;
        while (find(m, "aed.layers." + std::to_string(nl) + ".ln_self.weight")) nl++;
        if (nl == 0) { set_error("AED decoder without layers"); return -1; }
        m.aed_layers.resize(nl);
        for (int li = 0; li < nl; li++) {
            AedLayer &A = m.aed_layers[li];
            const std::string p = "aed.layers." + std::to_string(li) + ".";
            A.ln_self_w = f32dev(m, p + "ln_self.weight", true, &err); A.ln_self_b = f32dev(m, p + "ln_self.bias", true, &err);
            A.ln_cross_w = f32dev(m, p + "ln_cross.weight", true, &err); A.ln_cross_b = f32dev(m, p + "ln_cross.bias", true, &err);
            A.ln_ffn_w = f32dev(m, p + "ln_ffn.weight", true, &err); A.ln_ffn_b = f32dev(m, p + "ln_ffn.bias", true, &err);
            if (err) return -1;
            if (lin_cat(m, A.sqkv, &A.sqkv_b, {p + "self_attn.q_proj", p + "self_attn.k_proj", p + "self_attn.v_proj"}) ||
                lin_cat(m, A.ckv, &A.ckv_b, {p + "cross_attn.k_proj", p + "cross_attn.v_proj"}) ||
                lin_cat(m, A.so, &A.so_b, {p + "self_attn.o_proj"}) || lin_cat(m, A.cq, &A.cq_b, {p + "cross_attn.q_proj"}) ||
                lin_cat(m, A.co, &A.co_b, {p + "cross_attn.o_proj"}) || lin_cat(m, A.ff1, &A.ff1_b, {p + "ffn.linear1"}) ||
                lin_cat(m, A.ff2, &A.ff2_b, {p + "ffn.linear2"}))
                return -1;
            if (A.sqkv.n != 3 * m.aed_d || A.ckv.n != 2 * m.aed_d || A.sqkv.k != m.aed_d || A.ff2.n != m.aed_d || A.ff1.n % 64) {
                set_error("AED layer %d has unexpected shapes", li); return -1;
            }
        }
        m.aed_ffn = m.aed_layers[0].ff1.n;
        m.has_aed = true;
    }
    m.host.clear();
    MB_CUDA(cudaDeviceSynchronize());
    if (m.check_status("model_finalize (a weight does not fit the fp16 operand planes)")) return -1;
    m.release_load_buffers();
    m.load_seconds += std::chrono::duration<double>(std::chrono::steady_clock::now() - t_load0).count();
    m.finalized = true;
    return 0;
}

void mynah_b200_model_free(mynah_b200_model *h) { delete h; }

int mynah_b200_model_set_max_contexts(mynah_b200_model *h, int n) {
    if (!h || n < 1 || n > 64) { set_error("model_set_max_contexts: 1..64"); return -1; }
    std::lock_guard<std::mutex> lk(h->pool_mu);
    if (n < h->n_ctx()) { set_error("model_set_max_contexts: %d contexts already exist", h->n_ctx()); return -1; }
    h->max_ctx = n;
    return 0;
}

int mynah_b200_model_set_strict(mynah_b200_model *h, int strict) {
    if (!h) { set_error("model_set_strict: null model"); return -1; }
    with_all_contexts_idle(h, [&](Model &c) { c.cfg.strict = strict ? 1 : 0; });
    return 0;
}

void mynah_b200_model_dims(const mynah_b200_model *h, int *dims) {
    const Model &m = h->m;
    dims[0] = m.d_model; dims[1] = m.n_layers; dims[2] = m.n_heads; dims[3] = m.ffn_dim;
    dims[4] = m.conv_k; dims[5] = m.d_out; dims[6] = m.causal; dims[7] = m.channels;
}

void *mynah_b200_model_stream(mynah_b200_model *h) { return h ? (void *)h->m.stream : nullptr; }

void mynah_b200_model_load_stats(const mynah_b200_model *h, double *seconds, double *host_bytes, double *device_bytes) {
    if (!h) return;
    double dev = 0.0;
    for (const auto &sl : h->m.slabs) dev += (double)sl.off;
    if (seconds) *seconds = h->m.load_seconds;
    if (host_bytes) *host_bytes = (double)h->m.load_bytes;
    if (device_bytes) *device_bytes = dev;
}

}  // extern "C"

// -------------------------------------------------------------- workspace sizes
static size_t ss_bytes(const Model &m, int t_mel) {
    const int C = m.channels;
    const size_t T1 = Model::sub_len(t_mel, m.causal), F1 = Model::sub_len(m.cfg.n_mels, m.causal);
    const size_t T2 = Model::sub_len((int)T1, m.causal), F2 = Model::sub_len((int)F1, m.causal);
    const size_t T3 = Model::sub_len((int)T2, m.causal), F3 = Model::sub_len((int)F2, m.causal);
    return T1 * F1 * C * 4 + T2 * F2 * C * 8 + T3 * F3 * C * 8 + (1 << 16);
}
static size_t enc_bytes(const Model &m, size_t M, size_t rk_rows) {
    return M * ((size_t)m.d_model * 44 + (size_t)m.ffn_dim * 4) + rk_rows * m.d_model * 6 + (1 << 20) +
           (m.a8_layers ? M * ((size_t)m.d_model + 5 * (size_t)m.ffn_dim + 64) + 4096 : 0);
}
static size_t dec_bytes(const Model &m, int max_len) {
    const size_t B = DEC_MAX_B;
    return (size_t)max_len * m.cfg.max_symbols * B * 8 + B * 148 * 8 * 16 + 4 * (size_t)DEC_MAX_LAYERS * B * 1024 * 4 + B * (size_t)m.pred_hidden * 4 + (1 << 20);
}

// Full device pipeline for a packed batch whose mel features are already on the
// device: subsampling per item, layer stack on the packed rows, projector.
// x_out receives [sum T, d_model]; returns lens.
static int encode_batch_dev(Model &m, const std::vector<const float *> &feats_dev, const std::vector<int> &t_mel, int left,
                            int right, float *x, std::vector<int> &lens) {
    const int B = (int)t_mel.size();
    lens.resize(B);
    int off = 0;
    for (int b = 0; b < B; b++) {
        int t = 0;
        if (t_mel[b] > 0 && m.subsample_item(feats_dev[b], t_mel[b], x + (size_t)off * m.d_model, &t)) return -1;
        lens[b] = t;
        off += t;
    }
    return m.encoder_layers(x, lens, left, right, 0, m.n_layers);
}

extern "C" {

float *mynah_b200_log_mel(mynah_b200_model *h, const float *audio, size_t n, int *n_frames, int *valid_frames) {
    if (!h || !h->m.finalized || (!audio && n)) { set_error("log_mel: bad argument"); return nullptr; }
    Lease lease(h);
    Model &m = lease.model();
    const int hop = m.cfg.hop_length, T = 1 + (int)(n / hop), valid = (int)(n / hop), nm = m.cfg.n_mels;
    if (m.ws.reserve(n * 4 + (size_t)T * nm * 4 + (1 << 20))) return nullptr;
    m.ws.reset();
    float *a = m.ws.get<float>(n ? n : 1), *f = m.ws.get<float>((size_t)T * nm);
    if (!a || !f) return nullptr;
    MB_CUDA_NULL(cudaMemcpyAsync(a, audio, n * 4, cudaMemcpyHostToDevice, m.stream));
    if (m.log_mel(a, n, f, T, valid)) return nullptr;
    float *out = (float *)malloc((size_t)T * nm * sizeof(float));
    if (!out) { set_error("out of host memory"); return nullptr; }
    MB_CUDA_NULL(cudaMemcpyAsync(out, f, (size_t)T * nm * 4, cudaMemcpyDeviceToHost, m.stream));
    MB_CUDA_NULL(cudaStreamSynchronize(m.stream));
    *n_frames = T; *valid_frames = valid;
    return out;
}

float *mynah_b200_subsampling_forward(mynah_b200_model *h, const float *feats, int T, int n_mels, int *t_out) {
    if (!h || !h->m.finalized || !feats || T <= 0 || n_mels != h->m.cfg.n_mels) { set_error("subsampling_forward: bad argument"); return nullptr; }
    Lease lease(h);
    Model &m = lease.model();
    const int T3 = m.enc_len(T);
    if (m.ws.reserve(ss_bytes(m, T) + (size_t)T * n_mels * 4 + (size_t)T3 * m.d_model * 4 + (1 << 20))) return nullptr;
    m.ws.reset();
    float *f = m.ws.get<float>((size_t)T * n_mels), *x = m.ws.get<float>((size_t)T3 * m.d_model);
    MB_CUDA_NULL(cudaMemcpyAsync(f, feats, (size_t)T * n_mels * 4, cudaMemcpyHostToDevice, m.stream));
    int t = 0;
    if (m.subsample_item(f, T, x, &t) || m.check_status("subsampling")) return nullptr;
    float *out = (float *)malloc((size_t)t * m.d_model * sizeof(float));
    if (!out) { set_error("out of host memory"); return nullptr; }
    MB_CUDA_NULL(cudaMemcpyAsync(out, x, (size_t)t * m.d_model * 4, cudaMemcpyDeviceToHost, m.stream));
    MB_CUDA_NULL(cudaStreamSynchronize(m.stream));
    *t_out = t;
    return out;
}

int mynah_b200_encoder_layer(mynah_b200_model *h, int li, float *x, int T, int left, int right) {
    if (!h || !h->m.finalized || !x || T <= 0 || li < 0 || li >= h->m.n_layers) { set_error("encoder_layer: bad argument"); return -1; }
    Lease lease(h);
    Model &m = lease.model();
    if (m.ws.reserve(enc_bytes(m, T, 2 * T - 1) + (size_t)T * m.d_model * 4)) return -1;
    m.ws.reset();
    float *xd = m.ws.get<float>((size_t)T * m.d_model);
    MB_CUDA(cudaMemcpyAsync(xd, x, (size_t)T * m.d_model * 4, cudaMemcpyHostToDevice, m.stream));
    std::vector<int> lens{T};
    if (m.encoder_layers(xd, lens, left, right, li, 1) || m.check_status("encoder_layer")) return -1;
    MB_CUDA(cudaMemcpyAsync(x, xd, (size_t)T * m.d_model * 4, cudaMemcpyDeviceToHost, m.stream));
    MB_CUDA(cudaStreamSynchronize(m.stream));
    return 0;
}

int mynah_b200_encoder_forward_batch(mynah_b200_model *h, const float *const *feats, const int *t_mel, int batch,
                                     int n_mels, const int *prompt_ids, int left, int right, float **outs, int *t_outs) {
    if (!h || !h->m.finalized || batch <= 0 || n_mels != h->m.cfg.n_mels) { set_error("encoder_forward_batch: bad argument"); return -1; }
    Lease lease(h);
    Model &m = lease.model();
    size_t M = 0, rk = 0, fbytes = 0, ssmax = 0;
    for (int b = 0; b < batch; b++) {
        const size_t t = t_mel[b] > 0 ? m.enc_len(t_mel[b]) : 0;
        M += t; rk += 2 * t; fbytes += align_up((size_t)t_mel[b] * n_mels * 4, 256) + 256;
        if (t_mel[b] > 0 && ss_bytes(m, t_mel[b]) > ssmax) ssmax = ss_bytes(m, t_mel[b]);
    }
    if (m.ws.reserve(fbytes + ssmax + enc_bytes(m, M, rk) + M * ((size_t)m.d_model + m.d_out) * 4 + (1 << 20))) return -1;
    m.ws.reset();
    std::vector<const float *> fd(batch);
    std::vector<int> tm(t_mel, t_mel + batch), lens;
    for (int b = 0; b < batch; b++) {
        float *f = m.ws.get<float>((size_t)(t_mel[b] > 0 ? t_mel[b] : 1) * n_mels);
        if (!f) return -1;
        if (t_mel[b] > 0) MB_CUDA(cudaMemcpyAsync(f, feats[b], (size_t)t_mel[b] * n_mels * 4, cudaMemcpyHostToDevice, m.stream));
        fd[b] = f;
    }
    float *x = m.ws.get<float>((M ? M : 1) * m.d_model), *y = m.ws.get<float>((M ? M : 1) * m.d_out);
    if (!x || !y) return -1;
    if (encode_batch_dev(m, fd, tm, left, right, x, lens)) return -1;
    if (m.encoder_post(x, lens, prompt_ids, y) || m.check_status("encoder_forward_batch")) return -1;
    size_t off = 0;
    for (int b = 0; b < batch; b++) {
        t_outs[b] = lens[b];
        outs[b] = (float *)malloc((size_t)(lens[b] ? lens[b] : 1) * m.d_out * sizeof(float));
        if (!outs[b]) { set_error("out of host memory"); return -1; }
        MB_CUDA(cudaMemcpyAsync(outs[b], y + off * m.d_out, (size_t)lens[b] * m.d_out * 4, cudaMemcpyDeviceToHost, m.stream));
        off += lens[b];
    }
    MB_CUDA(cudaStreamSynchronize(m.stream));
    return 0;
}

static float *forward_one(mynah_b200_model *h, const float *feats, int t_mel, int n_mels, int prompt_id, int left, int right,
                          int raw, int *t_out) {
    if (!h || !h->m.finalized || !feats || t_mel <= 0 || n_mels != h->m.cfg.n_mels) { set_error("encoder_forward: bad argument"); return nullptr; }
    Lease lease(h);
    Model &m = lease.model();
    const size_t M = m.enc_len(t_mel);
    if (m.ws.reserve((size_t)t_mel * n_mels * 4 + ss_bytes(m, t_mel) + enc_bytes(m, M, 2 * M) + M * ((size_t)m.d_model + m.d_out) * 4 + (1 << 20))) return nullptr;
    m.ws.reset();
    float *f = m.ws.get<float>((size_t)t_mel * n_mels), *x = m.ws.get<float>(M * m.d_model), *y = m.ws.get<float>(M * m.d_out);
    if (!f || !x || !y) return nullptr;
    MB_CUDA_NULL(cudaMemcpyAsync(f, feats, (size_t)t_mel * n_mels * 4, cudaMemcpyHostToDevice, m.stream));
    std::vector<const float *> fd{f};
    std::vector<int> tm{t_mel}, lens;
    if (encode_batch_dev(m, fd, tm, left, right, x, lens)) return nullptr;
    const int wout = raw ? m.d_model : m.d_out;
    if (!raw && m.encoder_post(x, lens, &prompt_id, y)) return nullptr;
    if (m.check_status("encoder_forward")) return nullptr;
    float *out = (float *)malloc(M * wout * sizeof(float));
    if (!out) { set_error("out of host memory"); return nullptr; }
    MB_CUDA_NULL(cudaMemcpyAsync(out, raw ? x : y, M * wout * 4, cudaMemcpyDeviceToHost, m.stream));
    MB_CUDA_NULL(cudaStreamSynchronize(m.stream));
    *t_out = (int)M;
    return out;
}

float *mynah_b200_encoder_forward(mynah_b200_model *h, const float *feats, int t_mel, int n_mels, int prompt_id,
                                  int left, int right, int *t_out) {
    return forward_one(h, feats, t_mel, n_mels, prompt_id, left, right, 0, t_out);
}
float *mynah_b200_encoder_forward_raw(mynah_b200_model *h, const float *feats, int t_mel, int n_mels, int left,
                                      int right, int *t_out) {
    return forward_one(h, feats, t_mel, n_mels, 0, left, right, 1, t_out);
}

int mynah_b200_ctc_decode(mynah_b200_model *h, const float *enc_out, int T, int *tokens, int *frames, int cap) {
    if (!h || !h->m.finalized || !enc_out || T < 0) { set_error("ctc_decode: bad argument"); return -1; }
    Lease lease(h);
    Model &m = lease.model();
    if (T == 0) return 0;
    if (m.ws.reserve((size_t)T * (m.d_model * 8 + m.ctc_vocab * 4 + 8) + (1 << 20))) return -1;
    m.ws.reset();
    float *e = m.ws.get<float>((size_t)T * m.d_model);
    MB_CUDA(cudaMemcpyAsync(e, enc_out, (size_t)T * m.d_model * 4, cudaMemcpyHostToDevice, m.stream));
    std::vector<int> tk, fr;
    if (m.decode_ctc(e, T, tk, fr) || m.check_status("ctc_decode")) return -1;
    int n = 0;
    for (size_t i = 0; i < tk.size() && n < cap; i++, n++) { tokens[n] = tk[i]; if (frames) frames[n] = fr[i]; }
    return n;
}

int mynah_b200_greedy_decode(mynah_b200_model *h, const float *enc, int T, int *tokens, int *frames, int cap) {
    if (!h || !h->m.finalized || !enc || T < 0) { set_error("greedy_decode: bad argument"); return -1; }
    Lease lease(h);
    Model &m = lease.model();
    if (T == 0) return 0;
    if (m.ws.reserve((size_t)T * m.d_out * 4 + dec_bytes(m, T))) return -1;
    m.ws.reset();
    float *e = m.ws.get<float>((size_t)T * m.d_out);
    MB_CUDA(cudaMemcpyAsync(e, enc, (size_t)T * m.d_out * 4, cudaMemcpyHostToDevice, m.stream));
    std::vector<int> lens{T};
    std::vector<std::vector<int>> tk, fr;
    if (m.decode_greedy(e, lens, tk, fr)) return -1;
    int n = 0;
    for (size_t i = 0; i < tk[0].size() && n < cap; i++, n++) { tokens[n] = tk[0][i]; if (frames) frames[n] = fr[0][i]; }
    return n;
}

int mynah_b200_aed_decode_batch(mynah_b200_model *h, const float *const *encs, const int *Ts, int batch, const int *const *prompts,
                                const int *n_prompts, int eos, const int *caps, int **tokens, int *n_tokens) {
    if (!h || !h->m.finalized || !encs || !Ts || batch <= 0 || !prompts || !n_prompts || !caps || !tokens || !n_tokens) {
        set_error("aed_decode_batch: bad argument"); return -1;
    }
    Lease lease(h);
    Model &m = lease.model();
    if (!m.has_aed) { set_error("model has no AED decoder"); return -1; }
    size_t total = 0;
    int max_len = 0;
    std::vector<int> lens(Ts, Ts + batch), cp(caps, caps + batch);
    std::vector<std::vector<int>> pr(batch);
    for (int b = 0; b < batch; b++) {
        if (Ts[b] <= 0 || n_prompts[b] <= 0 || !prompts[b] || !encs[b]) { set_error("aed_decode_batch: utterance %d is empty or has no start token", b); return -1; }
        total += (size_t)Ts[b];
        pr[b].assign(prompts[b], prompts[b] + n_prompts[b]);
        const int ml = n_prompts[b] + (caps[b] > 0 ? caps[b] : 0);
        max_len = ml > max_len ? ml : max_len;
    }
    if (max_len > m.aed_max_seq) max_len = m.aed_max_seq;
    if (m.ws.reserve(total * m.d_out * 4 + m.aed_bytes((int)total, batch, max_len))) return -1;
    m.ws.reset();
    float *e = m.ws.get<float>(total * m.d_out);
    if (!e) return -1;
    size_t off = 0;
    for (int b = 0; b < batch; b++) {
        MB_CUDA(cudaMemcpyAsync(e + off * m.d_out, encs[b], (size_t)Ts[b] * m.d_out * 4, cudaMemcpyHostToDevice, m.stream));
        off += (size_t)Ts[b];
    }
    std::vector<std::vector<int>> tk;
    if (m.decode_aed(e, lens, pr, eos, cp, tk)) return -1;
    for (int b = 0; b < batch; b++) {
        n_tokens[b] = (int)tk[b].size();
        tokens[b] = (int *)malloc((tk[b].size() ? tk[b].size() : 1) * sizeof(int));
        if (!tokens[b]) { set_error("out of host memory"); return -1; }
        memcpy(tokens[b], tk[b].data(), tk[b].size() * sizeof(int));
    }
    return 0;
}

int mynah_b200_aed_decode(mynah_b200_model *h, const float *enc, int T, const int *prompt, int n_prompt, int eos, int *tokens, int cap) {
    if (!tokens || n_prompt <= 0 || !prompt) { set_error("aed_decode: bad argument (at least one start token is needed)"); return -1; }
    int *out = nullptr, n = 0;
    if (mynah_b200_aed_decode_batch(h, &enc, &T, 1, &prompt, &n_prompt, eos, &cap, &out, &n)) return -1;
    memcpy(tokens, out, (size_t)n * sizeof(int));
    free(out);
    return n;
}

void mynah_b200_batch_set_prompts(mynah_b200_batch *bt, const int *prompt_ids) {
    if (!bt) return;
    if (prompt_ids) bt->prompt_ids.assign(prompt_ids, prompt_ids + bt->batch); else bt->prompt_ids.clear();
}

void mynah_b200_batch_set_aed(mynah_b200_batch *bt, const int *prompt, int n_prompt, int eos, int max_gen_delta) {
    if (!bt) return;
    bt->aed_prompt.assign(prompt, prompt + (n_prompt > 0 ? n_prompt : 0));
    bt->aed_eos = eos; bt->aed_delta = max_gen_delta;
}

// ------------------------------------------------------------ CTC forced alignment
int mynah_b200_align_min_frames(const int *tokens, int n_tokens) { return tokens ? align_min_frames(tokens, n_tokens) : 0; }

int mynah_b200_align_ctc(const float *scores, int T, int V, const int *tokens, int n_tokens, int blank, int *t0, int *t1) {
    if (!scores || T <= 0 || V <= 0) { set_error("align_ctc: bad argument"); return -1; }
    if (!mynah_b200_available()) { set_error("align_ctc: no sm_100 device"); return -1; }
    float *d = nullptr;
    MB_CUDA(cudaMalloc((void **)&d, (size_t)T * V * sizeof(float)));
    int rc = -1;
    if (cudaMemcpy(d, scores, (size_t)T * V * sizeof(float), cudaMemcpyHostToDevice) == cudaSuccess)
        rc = align_ctc_device(d, T, V, tokens, n_tokens, blank, t0, t1, nullptr);
    else set_error("align_ctc: H2D copy failed");
    cudaFree(d);
    return rc;
}

int mynah_b200_ctc_align(mynah_b200_model *h, const float *enc_out, int T, const int *tokens, int n_tokens, int *t0, int *t1) {
    if (!h || !h->m.finalized || !enc_out || T <= 0 || !tokens || n_tokens <= 0) { set_error("ctc_align: bad argument"); return -1; }
    Lease lease(h);
    Model &m = lease.model();
    if (!m.has_ctc) { set_error("ctc_align: model has no CTC head"); return -1; }
    const int V = m.ctc_vocab, d = m.d_model;
    if (m.ws.reserve((size_t)T * ((size_t)d * 8 + (size_t)V * 4 + 8) + (1 << 20))) return -1;
    m.ws.reset();
    float *e = m.ws.get<float>((size_t)T * d), *logits = m.ws.get<float>((size_t)T * V);
    H16 hp = m.ws.planes((size_t)T * d);
    if (!e || !logits || !hp.lo) return -1;
    MB_CUDA(cudaMemcpyAsync(e, enc_out, (size_t)T * d * 4, cudaMemcpyHostToDevice, m.stream));
    if (split_to_h16(e, hp.hi, hp.lo, (size_t)T * d, m.stream, m.status)) return -1;
    note_launch();
    GemmEpilogue ep;
    memset(&ep, 0, sizeof(ep));
    ep.mode = OUT_F32; ep.act = ACT_NONE; ep.alpha = 1.f; ep.bias = m.ctc_head.bias; ep.out = logits; ep.ldo = V;
    if (m.gemm(hp, d, m.ctc_head, ep, T)) return -1;
    if (m.check_status("ctc_align")) return -1;
    return align_ctc_device(logits, T, V, tokens, n_tokens, V - 1, t0, t1, m.stream);
}

// ------------------------------------------------------------ cache-aware streaming
mynah_b200_stream_group *mynah_b200_stream_open(mynah_b200_model *h, int n_streams, int left_ctx, int right_ctx) {
    if (!h || !h->m.finalized) { set_error("stream_open: bad argument"); return nullptr; }
    Lease lease(h);
    Model &m = lease.model();
    mynah_b200_stream_group *g = new mynah_b200_stream_group();
    g->model = h;
    g->ctx = lease.index();
    if (m.stream_open(g->st, n_streams, left_ctx, right_ctx)) { m.stream_close(g->st); delete g; return nullptr; }
    return g;
}

void mynah_b200_stream_close(mynah_b200_stream_group *g) {
    if (!g) return;
    { Lease lease(g->model, g->ctx); lease.model().stream_close(g->st); }
    delete g;
}

int mynah_b200_stream_set_prompts(mynah_b200_stream_group *g, const int *prompt_ids) {
    if (!g || !prompt_ids) { set_error("stream_set_prompts: bad argument"); return -1; }
    Lease lease(g->model, g->ctx);
    Model &m = lease.model();
    if (g->st.exec) { set_error("stream_set_prompts: set the prompts before the first step"); return -1; }
    g->st.prompt_ids.assign(prompt_ids, prompt_ids + g->st.S);
    return 0;
}

int mynah_b200_stream_need(const mynah_b200_stream_group *g) { return g ? g->model->m.stream_need(g->st) : -1; }

int mynah_b200_stream_step_device(mynah_b200_stream_group *g, const float *mel_dev, int n_mel, int is_last, float *out_dev) {
    if (!g || !mel_dev || !out_dev) { set_error("stream_step: bad argument"); return -1; }
    Lease lease(g->model, g->ctx);
    Model &m = lease.model();
    if (n_mel != m.stream_need(g->st) && !is_last) { set_error("stream_step: %d mel frames given, %d needed", n_mel, m.stream_need(g->st)); return -1; }
    if (m.ws.reserve(m.stream_bytes(g->st, n_mel))) return -1;
    m.ws.reset();
    const int q = m.stream_step(g->st, mel_dev, n_mel, is_last, out_dev);
    if (q < 0 || m.check_status("stream_step")) return -1;
    return q;
}

int mynah_b200_stream_step(mynah_b200_stream_group *g, const float *mel, int n_mel, int is_last, float *out) {
    if (!g || !mel || !out || n_mel <= 0) { set_error("stream_step: bad argument"); return -1; }
    Lease lease(g->model, g->ctx);
    Model &m = lease.model();
    if (n_mel != m.stream_need(g->st) && !is_last) { set_error("stream_step: %d mel frames given, %d needed", n_mel, m.stream_need(g->st)); return -1; }
    const size_t S = g->st.S, nin = S * n_mel * m.cfg.n_mels, nout = S * (g->st.q + 2) * m.d_out;
    if (m.ws.reserve(m.stream_bytes(g->st, n_mel) + (nin + nout) * 4 + 4096)) return -1;
    m.ws.reset();
    float *md = m.ws.get<float>(nin), *od = m.ws.get<float>(nout);
    if (!md || !od) return -1;
    MB_CUDA(cudaMemcpyAsync(md, mel, nin * 4, cudaMemcpyHostToDevice, m.stream));
    const int q = m.stream_step(g->st, md, n_mel, is_last, od);
    if (q < 0) return -1;
    MB_CUDA(cudaMemcpyAsync(out, od, S * q * m.d_out * 4, cudaMemcpyDeviceToHost, m.stream));
    MB_CUDA(cudaStreamSynchronize(m.stream));
    if (m.check_status("stream_step")) return -1;
    return q;
}

int mynah_b200_stream_mel_feed(mynah_b200_stream_group *g, const float *audio, int n, int finish, float *out, int cap_frames) {
    if (!g || !out) { set_error("stream_mel_feed: bad argument"); return -1; }
    Lease lease(g->model, g->ctx);
    Model &m = lease.model();
    if (m.ws.reserve((size_t)g->st.S * (size_t)(cap_frames > 0 ? cap_frames : 1) * m.cfg.n_mels * 4 + (1 << 20))) return -1;
    m.ws.reset();
    return m.stream_mel_feed(g->st, audio, n, finish, out, cap_frames);
}

int mynah_b200_stream_step_decode(mynah_b200_stream_group *g, const float *mel, int n_mel, int is_last, int **tokens,
                                  int **frames, int *n_tokens) {
    if (!g || !mel || n_mel <= 0 || !tokens || !n_tokens) { set_error("stream_step_decode: bad argument"); return -1; }
    Lease lease(g->model, g->ctx);
    Model &m = lease.model();
    if (!m.has_dec) { set_error("stream_step_decode: model has no transducer decoder"); return -1; }
    if (n_mel != m.stream_need(g->st) && !is_last) { set_error("stream_step: %d mel frames given, %d needed", n_mel, m.stream_need(g->st)); return -1; }
    const size_t S = g->st.S, nin = S * n_mel * m.cfg.n_mels, nout = S * (g->st.q + 2) * m.d_out;
    const size_t nw = (size_t)(m.vocab + m.cfg.n_durations + 15) / 16, cap = (size_t)(g->st.q + 2) * m.cfg.max_symbols;
    const size_t decb = S * (24 + 4 * nw + 2 * cap) * 4 + ((S + 15) / 16) * (1024 + (size_t)DEC_MAX_B * m.pred_hidden * 4) + (1 << 20);
    if (m.ws.reserve(m.stream_bytes(g->st, n_mel) + (nin + nout) * 4 + decb + 4096)) return -1;
    m.ws.reset();
    float *md = m.ws.get<float>(nin), *od = m.ws.get<float>(nout);
    if (!md || !od) return -1;
    MB_CUDA(cudaMemcpyAsync(md, mel, nin * 4, cudaMemcpyHostToDevice, m.stream));
    const int q = m.stream_step(g->st, md, n_mel, is_last, od);
    if (q < 0) return -1;
    std::vector<std::vector<int>> tk, fr;
    if (m.stream_decode(g->st, od, q, tk, fr) || m.check_status("stream_step_decode")) return -1;
    for (size_t s = 0; s < S; s++) {
        n_tokens[s] = (int)tk[s].size();
        tokens[s] = (int *)malloc((tk[s].size() ? tk[s].size() : 1) * sizeof(int));
        if (frames) frames[s] = (int *)malloc((tk[s].size() ? tk[s].size() : 1) * sizeof(int));
        if (!tokens[s] || (frames && !frames[s])) { set_error("out of host memory"); return -1; }
        memcpy(tokens[s], tk[s].data(), tk[s].size() * sizeof(int));
        if (frames) memcpy(frames[s], fr[s].data(), fr[s].size() * sizeof(int));
    }
    return q;
}

// ------------------------------------------------------------ resident pipeline
mynah_b200_batch *mynah_b200_batch_upload(mynah_b200_model *h, const float *const *audio, const size_t *n_samples, int batch) {
    if (!h || !h->m.finalized || batch <= 0) { set_error("batch_upload: bad argument"); return nullptr; }
    mynah_b200_batch *bt = new mynah_b200_batch();
    bt->batch = batch;
    bt->audio.assign(batch, nullptr);
    bt->n_samples.assign(n_samples, n_samples + batch);
    for (int b = 0; b < batch; b++) {
        if (cudaMalloc(&bt->audio[b], (n_samples[b] ? n_samples[b] : 1) * sizeof(float)) != cudaSuccess) {
            set_error("batch_upload: cudaMalloc failed"); mynah_b200_batch_free(bt); return nullptr;
        }
        cudaMemcpyAsync(bt->audio[b], audio[b], n_samples[b] * sizeof(float), cudaMemcpyHostToDevice, h->m.stream);
    }
    cudaStreamSynchronize(h->m.stream);
    return bt;
}

void mynah_b200_batch_free(mynah_b200_batch *bt) {
    if (!bt) return;
    for (float *p : bt->audio) if (p) cudaFree(p);
    delete bt;
}

// Whole path for one batch. audio_dev: utterances already on the device, or null with
// audio_host set: then the audio is copied into the workspace arena first (no allocation
// on the hot path). Caller holds the model lock.
static int run_batch_locked(Model &m, mynah_b200_batch *bt, const float *const *audio_dev, const float *const *audio_host,
                            int decoder) {
    const int B = bt->batch, nm = m.cfg.n_mels, hop = m.cfg.hop_length;
    size_t M = 0, rk = 0, fbytes = 0, ssmax = 0, abytes = 0;
    int max_len = 0;
    std::vector<int> tmel(B), valid(B);
    for (int b = 0; b < B; b++) {
        tmel[b] = 1 + (int)(bt->n_samples[b] / hop); valid[b] = (int)(bt->n_samples[b] / hop);
        const int t = valid[b] > 0 ? m.enc_len(valid[b]) : 0;
        M += t; rk += 2 * (size_t)t; if (t > max_len) max_len = t;
        fbytes += align_up((size_t)tmel[b] * nm * 4, 256) + 256;
        abytes += align_up(bt->n_samples[b] * 4, 256) + 256;
        if (valid[b] > 0 && ss_bytes(m, valid[b]) > ssmax) ssmax = ss_bytes(m, valid[b]);
    }
    if (decoder == 2 && (!m.has_aed || bt->aed_prompt.empty())) { set_error("batch_run: AED decoding needs an AED model and mynah_b200_batch_set_aed"); return -1; }
    int aed_len = (int)bt->aed_prompt.size() + max_len + bt->aed_delta;
    if (decoder == 2 && aed_len > m.aed_max_seq) aed_len = m.aed_max_seq;
    const size_t decb = decoder == 1 ? M * ((size_t)m.d_model * 4 + (size_t)m.ctc_vocab * 4 + 8)
                      : decoder == 2 ? m.aed_bytes((int)M, B, aed_len) : dec_bytes(m, max_len);
    if (m.ws.reserve((audio_host ? abytes : 0) + fbytes + ssmax + enc_bytes(m, M, rk) + M * ((size_t)m.d_model + m.d_out) * 4 +
                     decb + (4 << 20))) return -1;
    m.ws.reset();
    std::vector<const float *> ad(B), fd(B);
    for (int b = 0; b < B; b++) {
        if (audio_host) {
            float *a = m.ws.get<float>(bt->n_samples[b] ? bt->n_samples[b] : 1);
            if (!a) return -1;
            MB_CUDA(cudaMemcpyAsync(a, audio_host[b], bt->n_samples[b] * sizeof(float), cudaMemcpyHostToDevice, m.stream));
            ad[b] = a;
        } else {
            ad[b] = audio_dev[b];
        }
    }
    for (int b = 0; b < B; b++) {
        float *f = m.ws.get<float>((size_t)tmel[b] * nm);
        if (!f) return -1;
        if (m.log_mel(ad[b], bt->n_samples[b], f, tmel[b], valid[b])) return -1;
        fd[b] = f;
    }
    float *x = m.ws.get<float>((M ? M : 1) * m.d_model), *y = m.ws.get<float>((M ? M : 1) * m.d_out);
    if (!x || !y) return -1;
    std::vector<int> lens;
    if (encode_batch_dev(m, fd, valid, m.cfg.left_ctx, m.cfg.right_ctx, x, lens)) return -1;
    bt->tokens.assign(B, {}); bt->frames.assign(B, {});
    if (decoder == 1) {
        size_t off = 0;
        for (int b = 0; b < B; b++) {      // CTC works on the raw encoder output (engine raw_encoder = 1)
            if (m.decode_ctc(x + off * m.d_model, lens[b], bt->tokens[b], bt->frames[b])) return -1;
            off += lens[b];
        }
    } else if (decoder == 2) {
        // AED engine: projected encoder output, generation budget T + max_gen_delta per utterance
        // (eng_decode_aed, src/mynah_asr.c:147-160, without timestamp tokens)
        if (m.encoder_post(x, lens, bt->prompt_ids.empty() ? nullptr : bt->prompt_ids.data(), y)) return -1;
        std::vector<std::vector<int>> pr(B, bt->aed_prompt);
        std::vector<int> caps(B);
        for (int b = 0; b < B; b++) caps[b] = lens[b] + bt->aed_delta;
        std::vector<int> idx;
        for (int b = 0; b < B; b++) if (lens[b] > 0) idx.push_back(b);
        if ((int)idx.size() == B) {
            if (m.decode_aed(y, lens, pr, bt->aed_eos, caps, bt->tokens)) return -1;
        } else {                           // utterances without a single encoder frame produce nothing
            std::vector<int> l2, c2;
            std::vector<std::vector<int>> p2, t2;
            for (int b : idx) { l2.push_back(lens[b]); c2.push_back(caps[b]); p2.push_back(pr[b]); }
            if (!idx.empty() && m.decode_aed(y, l2, p2, bt->aed_eos, c2, t2)) return -1;
            for (size_t i = 0; i < idx.size(); i++) bt->tokens[idx[i]] = t2[i];
        }
        for (int b = 0; b < B; b++) bt->frames[b].assign(bt->tokens[b].size(), 0);
    } else {
        if (m.encoder_post(x, lens, bt->prompt_ids.empty() ? nullptr : bt->prompt_ids.data(), y)) return -1;
        if (m.decode_greedy(y, lens, bt->tokens, bt->frames)) return -1;
    }
    return m.check_status("batch_run");
}

int mynah_b200_batch_run(mynah_b200_model *h, mynah_b200_batch *bt, int decoder) {
    if (!h || !bt) { set_error("batch_run: bad argument"); return -1; }
    Lease lease(h);
    return run_batch_locked(lease.model(), bt, bt->audio.data(), nullptr, decoder);
}

int mynah_b200_batch_fetch(mynah_b200_model *h, mynah_b200_batch *bt, int **tokens, int **frames, int *n_tokens) {
    (void)h;
    if (!bt || (int)bt->tokens.size() != bt->batch) { set_error("batch_fetch: nothing to fetch"); return -1; }
    for (int b = 0; b < bt->batch; b++) {
        const size_t n = bt->tokens[b].size();
        n_tokens[b] = (int)n;
        tokens[b] = (int *)malloc((n ? n : 1) * sizeof(int));
        if (!tokens[b]) { set_error("out of host memory"); return -1; }
        memcpy(tokens[b], bt->tokens[b].data(), n * sizeof(int));
        if (frames) {
            frames[b] = (int *)malloc((n ? n : 1) * sizeof(int));
            if (!frames[b]) { set_error("out of host memory"); return -1; }
            memcpy(frames[b], bt->frames[b].data(), n * sizeof(int));
        }
    }
    return 0;
}

int mynah_b200_transcribe_batch(mynah_b200_model *h, const float *const *audio, const size_t *n_samples, int batch,
                                int decoder, int **tokens, int **frames, int *n_tokens) {
    return mynah_b200_transcribe_batch_prompts(h, audio, n_samples, batch, nullptr, decoder, tokens, frames, n_tokens);
}

int mynah_b200_transcribe_batch_prompts(mynah_b200_model *h, const float *const *audio, const size_t *n_samples, int batch,
                                        const int *prompt_ids, int decoder, int **tokens, int **frames, int *n_tokens) {
    if (!h || !h->m.finalized || batch <= 0 || !audio || !n_samples) { set_error("transcribe_batch: bad argument"); return -1; }
    mynah_b200_batch bt;
    bt.batch = batch;
    bt.n_samples.assign(n_samples, n_samples + batch);
    mynah_b200_batch_set_prompts(&bt, prompt_ids);
    int rc;
    {
        Lease lease(h);
        rc = run_batch_locked(lease.model(), &bt, nullptr, audio, decoder);
    }
    if (rc == 0) rc = mynah_b200_batch_fetch(h, &bt, tokens, frames, n_tokens);
    return rc;
}

int mynah_b200_transcribe_batch_aed(mynah_b200_model *h, const float *const *audio, const size_t *n_samples, int batch,
                                    const int *prompt, int n_prompt, int eos, int max_gen_delta, int **tokens, int *n_tokens) {
    if (!h || !h->m.finalized || batch <= 0 || !audio || !n_samples || !prompt || n_prompt <= 0) { set_error("transcribe_batch_aed: bad argument"); return -1; }
    mynah_b200_batch bt;
    bt.batch = batch;
    bt.n_samples.assign(n_samples, n_samples + batch);
    mynah_b200_batch_set_aed(&bt, prompt, n_prompt, eos, max_gen_delta);
    int rc;
    {
        Lease lease(h);
        rc = run_batch_locked(lease.model(), &bt, nullptr, audio, 2);
    }
    if (rc == 0) rc = mynah_b200_batch_fetch(h, &bt, tokens, nullptr, n_tokens);
    return rc;
}

// ------------------------------------------------------------------- qmat API
mynah_b200_qmat *mynah_b200_qmat_create(int fmt, const void *data, const float *scales, int n, int k) {
    if (!mynah_b200_available()) { set_error("no sm_100 CUDA device available"); return nullptr; }
    const int f = internal_fmt(fmt);
    if (f < 0 || !data || n <= 0 || k <= 0) { set_error("qmat_create: bad argument"); return nullptr; }
    // a throw-away Model supplies the upload/dequant plumbing; ownership moves to the handle
    Model tmp;
    if (cudaStreamCreateWithFlags(&tmp.stream, cudaStreamNonBlocking) != cudaSuccess) { set_error("cudaStreamCreate failed"); return nullptr; }
    mynah_b200_qmat *q = new mynah_b200_qmat();
    const bool planes = (k % 64) == 0;
    tmp.status = q->status = (int *)tmp.dev_alloc(sizeof(int));
    if (!q->status) { delete q; return nullptr; }
    cudaMemset(q->status, 0, sizeof(int));
    cudaDeviceSynchronize();
    if (tmp.upload_weight(q->w, f, data, scales, n, k, planes, false)) { delete q; return nullptr; }
    cudaDeviceSynchronize();
    if (planes && tmp.check_status("qmat_create")) {
        // a weight value outside the fp16 operand range: the handle keeps the stored blocks (small-T products,
        // dequantisation) and drops the planes, so the many-row tensor-core product refuses instead of
        // returning inf / NaN
        q->w.hi = q->w.lo = nullptr;
    }
    q->owned.swap(tmp.owned);
    q->stream = tmp.stream;
    tmp.stream = nullptr;
    return q;
}

void mynah_b200_qmat_free(mynah_b200_qmat *q) {
    if (!q) return;
    for (void *p : q->owned) cudaFree(p);
    if (q->stream) cudaStreamDestroy(q->stream);
    delete q;
}

int mynah_b200_qmat_mul_device(const mynah_b200_qmat *q, const float *x, float *out, int T, int flags) {
    if (!q || !x || !out || T < 0) { set_error("qmat_mul: bad argument"); return -1; }
    if (T == 0) return 0;
    const QWeight &w = q->w;
    if (flags & MYNAH_B200_A8) {
        if (w.fmt == FMT_MYNAH_Q8 && T > 16 && w.k % 128 == 0) {
            // many rows: the same integers on the tensor cores (bit-identical to the row-dot kernel below)
            int8_t *qx = nullptr;
            float *sx = nullptr;
            MB_CUDA(cudaMallocAsync(&qx, (size_t)T * w.k, q->stream));
            if (cudaMallocAsync(&sx, (size_t)T * sizeof(float), q->stream) != cudaSuccess) {
                cudaGetLastError(); cudaFreeAsync(qx, q->stream); set_error("qmat_mul: device allocation failed"); return -1;
            }
            GemmEpilogue e;
            memset(&e, 0, sizeof(e));
            e.mode = OUT_F32; e.act = ACT_NONE; e.alpha = 1.f; e.out = out; e.ldo = w.n;
            int rc = act_quant_rows(x, qx, sx, T, w.k, q->stream);
            if (rc == 0) rc = gemm_i8(qx, w.k, sx, reinterpret_cast<const int8_t *>(w.raw), w.k, w.scales, e, T, w.n, w.k, q->status, q->stream);
            if (rc == 0) note_launch(2);
            cudaFreeAsync(qx, q->stream);
            cudaFreeAsync(sx, q->stream);
            return rc;
        }
        const int rc = qgemv_a8(w, x, out, T, nullptr, nullptr, q->stream);
        if (rc == 0) note_launch(2);
        return rc;
    }
    if (T <= 16 && w.k <= 8192 && !(flags & MYNAH_B200_FEW_ROWS)) {     // QMAT_SMALL_T / QMAT_K_MAX of the reference (src/qmat.c:180-181)
        if (w.tc_q && !(flags & (MYNAH_B200_SCALAR | MYNAH_B200_MMA_SYNC))) {
            int rc = 0;
            for (int t0 = 0; t0 < T && rc == 0; t0 += 8)
                rc = qstream_tc(w, x + (size_t)t0 * w.k, w.k, out + (size_t)t0 * w.n, w.n, nullptr, T - t0 < 8 ? T - t0 : 8,
                                q->status, q->stream);
            if (rc == 0) note_launch(((T + 7) / 8) * (w.tc_scratch ? 2 : 1));
            return rc;
        }
        if (w.mma_q && !(flags & MYNAH_B200_SCALAR)) {
            const int rc = qgemv_mma(w, x, w.k, out, w.n, nullptr, T, q->stream);
            if (rc == 0) note_launch((T + 3) / 4);
            return rc;
        }
        const int rc = qgemv(w, x, w.k, out, w.n, nullptr, T, q->stream);
        if (rc == 0) note_launch((T + 3) / 4);
        return rc;
    }
    if (!w.hi) { set_error("qmat_mul: the many-row path needs k %% 64 == 0 (k=%d) and weights below the fp16 operand limit 65504", w.k); return -1; }
    __half *hi = nullptr, *lo = nullptr;
    MB_CUDA(cudaMallocAsync(&hi, (size_t)T * w.k * 2, q->stream));
    if (cudaMallocAsync(&lo, (size_t)T * w.k * 2, q->stream) != cudaSuccess) {
        cudaGetLastError(); cudaFreeAsync(hi, q->stream); set_error("qmat_mul: device allocation failed"); return -1;
    }
    int rc = split_to_h16(x, hi, lo, (size_t)T * w.k, q->stream, q->status);
    GemmEpilogue e;
    memset(&e, 0, sizeof(e));
    e.mode = OUT_F32; e.act = ACT_NONE; e.alpha = 1.f; e.out = out; e.ldo = w.n;
    GemmOperand A{hi, lo, w.k}, B{w.hi, w.lo, w.k};
    if (rc == 0) rc = (flags & MYNAH_B200_FEW_ROWS) ? gemm_skinny(A, B, e, T, w.n, w.k, (flags & MYNAH_B200_FAST) ? 1 : 3, q->status, q->stream)
                                                    : gemm_tc(A, B, e, T, w.n, w.k, (flags & MYNAH_B200_FAST) ? 1 : 3, q->status, q->stream);
    if (rc == 0) note_launch(2);
    cudaFreeAsync(hi, q->stream);
    cudaFreeAsync(lo, q->stream);
    return rc;
}

int mynah_b200_qmat_sync(const mynah_b200_qmat *q) {
    if (!q) { set_error("qmat_sync: null handle"); return -1; }
    int st = 0;
    MB_CUDA(cudaMemcpyAsync(&st, q->status, sizeof(int), cudaMemcpyDeviceToHost, q->stream));
    MB_CUDA(cudaStreamSynchronize(q->stream));
    if (st != 0) {
        if (st == ST_RANGE) set_error("qmat: a value reached the fp16 operand range (|v| >= 65504) or was not finite");
        else set_error("qmat: a bounded wait inside the contraction kernel ran out (code %d)", st);
        cudaMemsetAsync(q->status, 0, sizeof(int), q->stream);
        cudaStreamSynchronize(q->stream);
        return -1;
    }
    return 0;
}

int mynah_b200_qmat_mul(const mynah_b200_qmat *q, const float *x, float *out, int T, int flags) {
    if (!q || !x || !out || T < 0) { set_error("qmat_mul: bad argument"); return -1; }
    if (T == 0) return 0;
    float *xd = nullptr, *od = nullptr;
    MB_CUDA(cudaMallocAsync(&xd, (size_t)T * q->w.k * 4, q->stream));
    if (cudaMallocAsync(&od, (size_t)T * q->w.n * 4, q->stream) != cudaSuccess) {
        cudaGetLastError(); cudaFreeAsync(xd, q->stream); set_error("qmat_mul: device allocation failed"); return -1;
    }
    int rc = 0;
    if (cudaMemcpyAsync(xd, x, (size_t)T * q->w.k * 4, cudaMemcpyHostToDevice, q->stream) != cudaSuccess) { set_error("qmat_mul: H2D copy failed"); rc = -1; }
    if (rc == 0) rc = mynah_b200_qmat_mul_device(q, xd, od, T, flags);
    if (rc == 0 && cudaMemcpyAsync(out, od, (size_t)T * q->w.n * 4, cudaMemcpyDeviceToHost, q->stream) != cudaSuccess) { set_error("qmat_mul: D2H copy failed"); rc = -1; }
    cudaFreeAsync(xd, q->stream);
    cudaFreeAsync(od, q->stream);
    if (mynah_b200_qmat_sync(q)) return -1;
    return rc;
}

int mynah_b200_qmat_block_dots(const mynah_b200_qmat *q, const float *x, int T, int32_t *dots, float *sx, float *out) {
    if (!q || !x || T <= 0) { set_error("qmat_block_dots: bad argument"); return -1; }
    const QWeight &w = q->w;
    const size_t nd = (size_t)T * w.n * (w.k / 32);
    float *xd = nullptr, *od = nullptr, *sd = nullptr;
    int32_t *dd = nullptr;
    if (cudaMalloc(&xd, (size_t)T * w.k * 4) != cudaSuccess || cudaMalloc(&od, (size_t)T * w.n * 4) != cudaSuccess ||
        cudaMalloc(&sd, (size_t)T * 4) != cudaSuccess || cudaMalloc(&dd, nd * 4) != cudaSuccess ||
        cudaMemcpyAsync(xd, x, (size_t)T * w.k * 4, cudaMemcpyHostToDevice, q->stream) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(xd); cudaFree(od); cudaFree(sd); cudaFree(dd);
        set_error("qmat_block_dots: device allocation or copy failed");
        return -1;
    }
    int rc = qgemv_a8(w, xd, od, T, dd, sd, q->stream);
    if (rc == 0) note_launch(2);
    cudaStreamSynchronize(q->stream);
    if (rc == 0 && dots) cudaMemcpy(dots, dd, nd * 4, cudaMemcpyDeviceToHost);
    if (rc == 0 && sx) cudaMemcpy(sx, sd, (size_t)T * 4, cudaMemcpyDeviceToHost);
    if (rc == 0 && out) cudaMemcpy(out, od, (size_t)T * w.n * 4, cudaMemcpyDeviceToHost);
    cudaFree(xd); cudaFree(od); cudaFree(sd); cudaFree(dd);
    if (rc == 0 && cudaGetLastError() != cudaSuccess) { set_error("qmat_block_dots: device error"); rc = -1; }
    return rc;
}

int mynah_b200_qmat_dequant(const mynah_b200_qmat *q, float *wd) {
    if (!q || !wd) { set_error("qmat_dequant: bad argument"); return -1; }
    const QWeight &w = q->w;
    float *d = nullptr;
    MB_CUDA(cudaMalloc(&d, (size_t)w.n * w.k * 4));
    int rc = dequant_to_f32(w.fmt, w.raw, w.scales, d, w.n, w.k, q->stream);
    if (rc == 0) note_launch();
    cudaStreamSynchronize(q->stream);
    if (rc == 0) cudaMemcpy(wd, d, (size_t)w.n * w.k * 4, cudaMemcpyDeviceToHost);
    cudaFree(d);
    return rc;
}

int mynah_b200_gemm_wt(const float *x, const float *w, float *out, int T, int n, int k) {
    if (!x || !w || !out || T <= 0 || n <= 0 || k <= 0) { set_error("gemm_wt: bad argument"); return -1; }
    mynah_b200_qmat *q = mynah_b200_qmat_create(MYNAH_B200_F32, w, nullptr, n, k);
    if (!q) return -1;
    const int rc = mynah_b200_qmat_mul(q, x, out, T, MYNAH_B200_A16);
    mynah_b200_qmat_free(q);
    return rc;
}

// ---- address-keyed resident weights: the calling convention of the reference's own CUDA hook
// (src/cuda_gemm.cu:92-130: every host weight pointer is uploaded once and found again by address).
// One entry per (pointer, format, shape); calls on the same weight take the entry's lock (its
// handle owns one stream and one scratch area), calls on different weights run side by side.
namespace {
// Entries are reference-counted: a call keeps its entry alive while it runs even if another thread
// evicts the cache meanwhile (the device memory goes when the last user lets go).
struct ResidentWeight {
    const void *host; int fmt, n, k;
    mynah_b200_qmat *q;
    std::mutex mu;
    ResidentWeight(const void *h, int f, int n_, int k_, mynah_b200_qmat *q_) : host(h), fmt(f), n(n_), k(k_), q(q_) {}
    ~ResidentWeight() { mynah_b200_qmat_free(q); }
};
std::mutex g_resident_mu;
std::vector<std::shared_ptr<ResidentWeight>> g_resident;

std::shared_ptr<ResidentWeight> resident_lookup(const void *host, int fmt, int n, int k) {
    for (auto &e : g_resident)
        if (e->host == host && e->fmt == fmt && e->n == n && e->k == k) return e;
    return nullptr;
}

std::shared_ptr<ResidentWeight> resident_weight(const void *host, int fmt, const float *scales, int n, int k) {
    {
        std::lock_guard<std::mutex> lk(g_resident_mu);
        if (auto e = resident_lookup(host, fmt, n, k)) return e;
    }
    // upload and re-tile outside the lock: first-touch calls on different weights run side by side
    mynah_b200_qmat *q = mynah_b200_qmat_create(fmt, host, scales, n, k);
    if (!q) return nullptr;
    auto fresh = std::make_shared<ResidentWeight>(host, fmt, n, k, q);
    std::lock_guard<std::mutex> lk(g_resident_mu);
    if (auto e = resident_lookup(host, fmt, n, k)) return e;      // another thread was first; ours is dropped
    g_resident.push_back(fresh);
    return fresh;
}
}  // namespace

int mynah_b200_qgemm(const void *wq, int fmt, const float *scales, int n, int k, const float *x, float *out, int T, int flags) {
    if (!wq || !x || !out || T < 0 || n <= 0 || k <= 0) { set_error("qgemm: bad argument"); return -1; }
    if (!mynah_b200_available()) { set_error("qgemm: no sm_100 device"); return -1; }
    std::shared_ptr<ResidentWeight> e = resident_weight(wq, fmt, scales, n, k);
    if (!e) return -1;
    std::lock_guard<std::mutex> lk(e->mu);
    return mynah_b200_qmat_mul(e->q, x, out, T, flags);
}

void mynah_b200_weights_evict(void) {
    std::vector<std::shared_ptr<ResidentWeight>> drop;
    {
        std::lock_guard<std::mutex> lk(g_resident_mu);
        drop.swap(g_resident);
    }
    // entries still in use by a running call are freed when that call returns
}

int mynah_b200_weights_resident(void) {
    std::lock_guard<std::mutex> lk(g_resident_mu);
    return (int)g_resident.size();
}

// the two symbols src/backend.c:23-26 declares and src/cuda_gemm.cu defines, same meaning:
// 1 / 0, and 0 = done, -1 = the caller falls back
int mynah_asr_cuda_available(void) { return mynah_b200_available(); }

int mynah_asr_cuda_gemm_wt(const float *x, const float *w, float *out, int T, int n, int k) {
    return mynah_b200_qgemm(w, MYNAH_B200_F32, nullptr, n, k, x, out, T, MYNAH_B200_A16);
}

void mynah_b200_profile_begin(mynah_b200_model *h) {
    if (!h) return;
    Lease lease(h, 0);      // the first context: the one a single-threaded caller always runs on
    Model &m = lease.model();
    m.prof_on = true; m.prof_used = 0;
    for (int i = 0; i < Model::PROF_NCAT; i++) { m.prof_flops[i] = 0; m.prof_bytes[i] = 0; m.prof_launches[i] = 0; }
}

int mynah_b200_profile_end(mynah_b200_model *h, double *ms, double *flops, long long *launches, int ncat) {
    if (!h) { set_error("profile_end: null model"); return -1; }
    Lease lease(h, 0);      // the first context: the one a single-threaded caller always runs on
    Model &m = lease.model();
    m.prof_on = false;
    MB_CUDA(cudaStreamSynchronize(m.stream));
    for (int i = 0; i < ncat; i++) { ms[i] = 0; flops[i] = 0; launches[i] = 0; }
    for (size_t i = 0; i < m.prof_used; i++) {
        float t = 0.f;
        if (cudaEventElapsedTime(&t, m.prof_spans[i].a, m.prof_spans[i].b) == cudaSuccess && m.prof_spans[i].cat < ncat)
            ms[m.prof_spans[i].cat] += t;
    }
    for (int i = 0; i < ncat && i < Model::PROF_NCAT; i++) { flops[i] = m.prof_flops[i]; launches[i] = m.prof_launches[i]; }
    m.prof_used = 0;
    return 0;
}

void mynah_b200_profile_bytes(mynah_b200_model *h, double *bytes, int ncat) {
    for (int i = 0; i < ncat; i++) bytes[i] = (h && i < Model::PROF_NCAT) ? h->m.prof_bytes[i] : 0.0;
}

void mynah_b200_decoder_clocks(mynah_b200_model *h, long long *out8) {
    for (int i = 0; i < 8; i++) out8[i] = h ? h->m.dec_dbg[i] : 0;
}

double mynah_b200_qmat_time(const mynah_b200_qmat *q, int T, int flags, int iters) {
    if (!q || T <= 0 || iters <= 0) { set_error("qmat_time: bad argument"); return -1.0; }
    const QWeight &w = q->w;
    float *x = nullptr, *out = nullptr;
    __half *hi = nullptr, *lo = nullptr;
    if (cudaMalloc(&x, (size_t)T * w.k * 4) != cudaSuccess || cudaMalloc(&out, (size_t)T * w.n * 4) != cudaSuccess) { set_error("qmat_time: cudaMalloc failed"); return -1.0; }
    cudaMemset(x, 0, (size_t)T * w.k * 4);
    cudaDeviceSynchronize();
    const bool i8 = (flags & MYNAH_B200_A8) && w.fmt == FMT_MYNAH_Q8 && T > 16 && w.k % 128 == 0;
    int8_t *qx = nullptr;
    float *sx = nullptr;
    if (i8) {          // the integer contraction alone: rows quantised once, outside the timed launches
        if (cudaMalloc((void **)&qx, (size_t)T * w.k) != cudaSuccess || cudaMalloc((void **)&sx, (size_t)T * 4) != cudaSuccess ||
            act_quant_rows(x, qx, sx, T, w.k, q->stream)) { cudaFree(x); cudaFree(out); cudaFree(qx); cudaFree(sx); set_error("qmat_time: setup failed"); return -1.0; }
    }
    const bool small = !i8 && !(flags & MYNAH_B200_FEW_ROWS) && ((T <= 16 && w.k <= 8192) || (flags & MYNAH_B200_A8));
    if (!small && !i8) {
        if (!w.hi) { set_error("qmat_time: no operand planes"); cudaFree(x); cudaFree(out); return -1.0; }
        cudaMalloc(&hi, (size_t)T * w.k * 2); cudaMalloc(&lo, (size_t)T * w.k * 2);
        split_to_h16(x, hi, lo, (size_t)T * w.k, q->stream);
    }
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    int rc = 0;
    for (int it = -2; it < iters && rc == 0; it++) {
        if (it == 0) cudaEventRecord(e0, q->stream);
        if (i8) {
            GemmEpilogue e;
            memset(&e, 0, sizeof(e));
            e.mode = OUT_F32; e.alpha = 1.f; e.out = out; e.ldo = w.n;
            rc = gemm_i8(qx, w.k, sx, reinterpret_cast<const int8_t *>(w.raw), w.k, w.scales, e, T, w.n, w.k, q->status, q->stream);
        } else if (small) rc = (flags & MYNAH_B200_A8) ? qgemv_a8(w, x, out, T, nullptr, nullptr, q->stream)
                   : (w.tc_q && T <= 8 && !(flags & (MYNAH_B200_SCALAR | MYNAH_B200_MMA_SYNC))) ? qstream_tc(w, x, w.k, out, w.n, nullptr, T, q->status, q->stream)
                   : (w.mma_q && !(flags & MYNAH_B200_SCALAR)) ? qgemv_mma(w, x, w.k, out, w.n, nullptr, T, q->stream)
                   : qgemv(w, x, w.k, out, w.n, nullptr, T, q->stream);
        else {
            GemmEpilogue e;
            memset(&e, 0, sizeof(e));
            e.mode = OUT_F32; e.alpha = 1.f; e.out = out; e.ldo = w.n;
            GemmOperand A{hi, lo, w.k}, B{w.hi, w.lo, w.k};
            rc = (flags & MYNAH_B200_FEW_ROWS) ? gemm_skinny(A, B, e, T, w.n, w.k, (flags & MYNAH_B200_FAST) ? 1 : 3, q->status, q->stream)
                                               : gemm_tc(A, B, e, T, w.n, w.k, (flags & MYNAH_B200_FAST) ? 1 : 3, q->status, q->stream);
        }
        if (it >= 0) note_launch();
    }
    cudaEventRecord(e1, q->stream);
    cudaEventSynchronize(e1);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    cudaFree(x); cudaFree(out); if (hi) cudaFree(hi); if (lo) cudaFree(lo); if (qx) cudaFree(qx); if (sx) cudaFree(sx);
    if (rc != 0 || cudaGetLastError() != cudaSuccess) { if (rc == 0) set_error("qmat_time: device error"); return -1.0; }
    return (double)ms / iters;
}

}  // extern "C"
