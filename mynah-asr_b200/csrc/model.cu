// Model container and the device-resident drivers of the hot path: weights are
// uploaded and decoded once (replacing the reference's lazy per-pointer upload,
// src/cuda_gemm.cu:96-130), activations never leave HBM between the mel input and
// the token ids (replacing its per-GEMM H2D/D2H round trip, src/cuda_gemm.cu:170-188).
#include "model.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>

namespace mb {

static std::atomic<long long> g_launches{0};
void note_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long launch_count(bool reset) { return reset ? g_launches.exchange(0) : g_launches.load(); }

// -------------------------------------------------------------------- arena
int Arena::reserve(size_t bytes) {
    bytes = align_up(bytes, 1 << 20);
    if (bytes <= cap) return 0;
    if (base) MB_CUDA(cudaFree(base));
    base = nullptr; cap = 0;
    MB_CUDA(cudaMalloc(&base, bytes));
    cap = bytes;
    return 0;
}
void *Arena::take(size_t bytes) {
    const size_t o = align_up(off, 256);
    if (o + bytes > cap) { set_error("workspace arena exhausted (%zu + %zu > %zu)", o, bytes, cap); return nullptr; }
    off = o + bytes;
    return base + o;
}
void Arena::release() { if (base) cudaFree(base); base = nullptr; cap = off = 0; }

// -------------------------------------------------------------------- model
static constexpr size_t SLAB_BYTES = 256u << 20;
static constexpr size_t STAGE_BYTES = 32u << 20;

Model::~Model() {
    release_load_buffers();
    for (void *p : owned) cudaFree(p);
    for (auto &s : prof_spans) { cudaEventDestroy(s.a); cudaEventDestroy(s.b); }
    ws.release();
    for (int i = 0; i < DEC_LANES; i++) {
        if (lane_done[i]) cudaEventDestroy(lane_done[i]);
        if (lane[i]) cudaStreamDestroy(lane[i]);
    }
    if (lane_fork) cudaEventDestroy(lane_fork);
    if (stream) cudaStreamDestroy(stream);
}
int Model::lanes_begin(int n_groups) {
    const int lanes = n_groups < DEC_LANES ? n_groups : DEC_LANES;
    if (lanes <= 1) return 1;
    if (!lane_fork) MB_CUDA(cudaEventCreateWithFlags(&lane_fork, cudaEventDisableTiming));
    MB_CUDA(cudaEventRecord(lane_fork, stream));
    for (int i = 0; i < lanes; i++) {
        if (!lane[i]) {
            MB_CUDA(cudaStreamCreateWithFlags(&lane[i], cudaStreamNonBlocking));
            MB_CUDA(cudaEventCreateWithFlags(&lane_done[i], cudaEventDisableTiming));
        }
        MB_CUDA(cudaStreamWaitEvent(lane[i], lane_fork, 0));
    }
    return lanes;
}
int Model::lanes_join(int lanes) {
    if (lanes <= 1) return 0;
    for (int i = 0; i < lanes; i++) {
        MB_CUDA(cudaEventRecord(lane_done[i], lane[i]));
        MB_CUDA(cudaStreamWaitEvent(stream, lane_done[i], 0));
    }
    return 0;
}
void Model::release_load_buffers() {
    for (int i = 0; i < 2; i++) {
        if (stage_ev[i]) { cudaEventSynchronize(stage_ev[i]); cudaEventDestroy(stage_ev[i]); stage_ev[i] = nullptr; }
        if (stage[i]) { cudaFreeHost(stage[i]); stage[i] = nullptr; }
    }
    if (load_tmp) { cudaStreamSynchronize(stream); cudaFree(load_tmp); load_tmp = nullptr; load_tmp_cap = 0; }
}
void *Model::dev_alloc(size_t bytes) {
    bytes = align_up(bytes ? bytes : 16, 256);
    if (use_slabs && bytes <= SLAB_BYTES / 4) {
        if (slabs.empty() || slabs.back().off + bytes > slabs.back().cap) {
            void *p = nullptr;
            if (cudaMalloc(&p, SLAB_BYTES) != cudaSuccess) { set_error("cudaMalloc(%zu) failed", SLAB_BYTES); cudaGetLastError(); return nullptr; }
            owned.push_back(p);
            slabs.push_back(Slab{(uint8_t *)p, SLAB_BYTES, 0});
        }
        Slab &sl = slabs.back();
        void *p = sl.base + sl.off;
        sl.off += bytes;
        return p;
    }
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) { set_error("cudaMalloc(%zu) failed", bytes); cudaGetLastError(); return nullptr; }
    owned.push_back(p);
    return p;
}
// Host bytes -> device through the pinned staging pair, asynchronously on the model's stream. The source is
// consumed before this returns (it may be a temporary); kernels launched later on the stream see the data.
int Model::upload_bytes(void *dst, const void *src, size_t n) {
    if (!use_slabs) {            // one matrix: a plain copy, waited for because src may be a temporary
        MB_CUDA(cudaMemcpyAsync(dst, src, n, cudaMemcpyHostToDevice, stream));
        MB_CUDA(cudaStreamSynchronize(stream));
        load_bytes += n;
        return 0;
    }
    for (int i = 0; i < 2; i++) {
        if (!stage[i]) {
            MB_CUDA(cudaMallocHost((void **)&stage[i], STAGE_BYTES));
            MB_CUDA(cudaEventCreateWithFlags(&stage_ev[i], cudaEventDisableTiming));
            MB_CUDA(cudaEventRecord(stage_ev[i], stream));
        }
    }
    for (size_t off = 0; off < n;) {
        const size_t piece = n - off < STAGE_BYTES ? n - off : STAGE_BYTES;
        const int b = stage_next;
        stage_next ^= 1;
        MB_CUDA(cudaEventSynchronize(stage_ev[b]));                 // the previous DMA out of this buffer has finished
        memcpy(stage[b], (const uint8_t *)src + off, piece);
        MB_CUDA(cudaMemcpyAsync((uint8_t *)dst + off, stage[b], piece, cudaMemcpyHostToDevice, stream));
        MB_CUDA(cudaEventRecord(stage_ev[b], stream));
        off += piece;
    }
    load_bytes += n;
    return 0;
}
float *Model::decode_scratch(size_t nfloats) {
    if (nfloats > load_tmp_cap) {
        if (load_tmp) { cudaStreamSynchronize(stream); cudaFree(load_tmp); load_tmp = nullptr; load_tmp_cap = 0; }
        const size_t want = nfloats > (16u << 20) ? nfloats : (16u << 20);
        if (cudaMalloc((void **)&load_tmp, want * sizeof(float)) != cudaSuccess) { set_error("cudaMalloc(%zu) failed", want * sizeof(float)); cudaGetLastError(); return nullptr; }
        load_tmp_cap = want;
    }
    return load_tmp;
}
float *Model::upload_f32(const float *src, size_t n) {
    float *d = (float *)dev_alloc(n * sizeof(float));
    if (!d) return nullptr;
    if (upload_bytes(d, src, n * sizeof(float))) return nullptr;
    return d;
}

__global__ void permute_cols_kernel(const float *__restrict__ in, float *__restrict__ out, const int *__restrict__ perm, int n, int k) {
    const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i >= (size_t)n * k) return;
    const int r = (int)(i / k), c = (int)(i % k);
    out[i] = in[(size_t)r * k + perm[c]];
}

int Model::upload_weight(QWeight &w, int fmt, const void *data, const float *scales, int n, int k, bool want_planes,
                         bool want_f32, const int *col_perm) {
    w.fmt = fmt; w.n = n; w.k = k;
    const int blk = format_block(fmt);
    if (k % blk) { set_error("weight [%d,%d]: k not a multiple of the %d-element block", n, k, blk); return -1; }
    w.raw_bytes = format_bytes(fmt, n, k);
    if (!w.raw_bytes) { set_error("unknown weight format %d", fmt); return -1; }
    w.raw = (uint8_t *)dev_alloc(w.raw_bytes + 64);          // slack for aligned over-reads
    if (!w.raw) return -1;
    if (upload_bytes(w.raw, data, w.raw_bytes)) return -1;
    MB_CUDA(cudaMemsetAsync(w.raw + w.raw_bytes, 0, 64, stream));
    if (fmt == FMT_MYNAH_Q8 || fmt == FMT_MYNAH_Q4) {
        if (!scales) { set_error("native quantised weight without scales"); return -1; }
        const size_t ns = fmt == FMT_MYNAH_Q8 ? (size_t)n : (size_t)n * (k / 32);
        w.scales = upload_f32(scales, ns);
        if (!w.scales) return -1;
    }
    if ((fmt == FMT_GGML_Q4_0 || fmt == FMT_GGML_Q8_0) && k % 128 == 0) {
        // re-tiled copy for the tensor-core small-T kernel (same bytes per parameter)
        w.mma_q = (uint8_t *)dev_alloc(fmt == FMT_GGML_Q4_0 ? (size_t)n * k / 2 : (size_t)n * k);
        w.mma_d = (__half *)dev_alloc((size_t)n * (k / 32) * sizeof(__half));
        if (!w.mma_q || !w.mma_d) return -1;
        if (qgemv_mma_retile(w, w.mma_q, w.mma_d, stream)) return -1;
        note_launch();
    }
    if (((fmt == FMT_GGML_Q4_0 || fmt == FMT_GGML_Q8_0) && k % 128 == 0) || (fmt == FMT_GGML_Q4_K && k % 256 == 0)) {
        w.tc_q = (uint8_t *)dev_alloc(qstream_tc_bytes(fmt, n, k));
        if (!w.tc_q) return -1;
        if (const size_t sb = qstream_tc_scratch_bytes(n, k)) {
            w.tc_scratch = (float *)dev_alloc(sb);
            if (!w.tc_scratch) return -1;
        }
        if (qstream_tc_retile(w, w.tc_q, stream)) return -1;
        note_launch();
    }
    if (!want_planes && !want_f32) return 0;
    // decode once on the device: into the reused scratch, or into a buffer of its own when the f32 copy is kept
    float *tmp = want_f32 ? (float *)dev_alloc((size_t)n * k * sizeof(float)) : decode_scratch((size_t)n * k);
    if (!tmp) return -1;
    int rc = dequant_to_f32(fmt, w.raw, w.scales, tmp, n, k, stream);
    note_launch();
    float *permuted = nullptr;
    if (rc == 0 && col_perm) {
        // column permutation (only the subsampling linear, once at load)
        int *perm_dev = nullptr;
        if (cudaMalloc((void **)&perm_dev, (size_t)k * sizeof(int)) != cudaSuccess || cudaMalloc((void **)&permuted, (size_t)n * k * sizeof(float)) != cudaSuccess) {
            cudaGetLastError(); cudaFree(perm_dev); set_error("cudaMalloc failed"); return -1;
        }
        rc = upload_bytes(perm_dev, col_perm, (size_t)k * sizeof(int));
        if (rc == 0) {
            permute_cols_kernel<<<(unsigned)(((size_t)n * k + 255) / 256), 256, 0, stream>>>(tmp, permuted, perm_dev, n, k);
            note_launch();
            if (want_f32) cudaMemcpyAsync(tmp, permuted, (size_t)n * k * sizeof(float), cudaMemcpyDeviceToDevice, stream);
        }
        cudaStreamSynchronize(stream);
        cudaFree(perm_dev);
    }
    if (rc == 0 && want_planes) {
        w.hi = (__half *)dev_alloc((size_t)n * k * 2);
        w.lo = (__half *)dev_alloc((size_t)n * k * 2);
        if (!w.hi || !w.lo) rc = -1;
        else { rc = split_to_h16(permuted ? permuted : tmp, w.hi, w.lo, (size_t)n * k, stream, status); note_launch(); }
    }
    if (permuted) { cudaStreamSynchronize(stream); cudaFree(permuted); }
    if (rc == 0 && want_f32) w.f32 = tmp;
    return rc;
}

int Model::prof_begin_span(int cat) {
    if (!prof_on) return -1;
    if (prof_used == prof_spans.size()) {
        ProfSpan s;
        if (cudaEventCreate(&s.a) != cudaSuccess || cudaEventCreate(&s.b) != cudaSuccess) return -1;
        prof_spans.push_back(s);
    }
    ProfSpan &s = prof_spans[prof_used];
    s.cat = cat;
    cudaEventRecord(s.a, stream);
    return (int)prof_used++;
}
void Model::prof_end_span(int idx) {
    if (idx >= 0) cudaEventRecord(prof_spans[idx].b, stream);
}

int Model::check_status(const char *where) {
    int st = 0;
    MB_CUDA(cudaMemcpyAsync(&st, status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    MB_CUDA(cudaStreamSynchronize(stream));
    if (st != 0) {
        if (st == ST_RANGE) set_error("%s: a value reached the fp16 operand range (|v| >= 65504) or was not finite", where);
        else set_error("%s: a bounded wait inside the contraction kernel ran out (code %d)", where, st);
        cudaMemsetAsync(status, 0, sizeof(int), stream);
        return -1;
    }
    return 0;
}

int Model::gemm(const H16 &a, int lda, const QWeight &w, const GemmEpilogue &ep, int M, bool few_rows) {
    if (!w.hi) { set_error("contraction on a weight without operand planes"); return -1; }
    GemmOperand A{a.hi, a.lo, lda}, B{w.hi, w.lo, w.k};
    const int sp = prof_begin_span(PROF_GEMM);
    const int rc = few_rows ? gemm_skinny(A, B, ep, M, w.n, w.k, cfg.strict ? 3 : 1, status, stream, true)
                            : gemm_tc(A, B, ep, M, w.n, w.k, cfg.strict ? 3 : 1, status, stream);
    prof_end_span(sp);
    if (sp >= 0) {
        prof_flops[PROF_GEMM] += 2.0 * M * (double)w.n * w.k;
        // operand planes read once (fp16 hi, and lo in strict mode) + what the epilogue reads and writes
        const double planes = cfg.strict ? 4.0 : 2.0;
        const double out_b = ep.mode == OUT_H16 ? (cfg.strict ? 4.0 : 2.0) : ep.mode == OUT_F32_H16 ? 8.0 : ep.mode == OUT_RESID ? 8.0 : 4.0;
        prof_bytes[PROF_GEMM] += planes * ((double)M * w.k + (double)w.n * w.k) + out_b * M * (double)w.n;
        prof_launches[PROF_GEMM]++;
    }
    if (rc == 0) note_launch();
    return rc;
}

int Model::gemm_q8(const int8_t *qa, const float *sx, const QWeight &w, const GemmEpilogue &ep, int M) {
    if (!a8_ok(w)) { set_error("int8-activation contraction on a weight that is not reference-native int8 with k %% 128 == 0"); return -1; }
    const int sp = prof_begin_span(PROF_GEMM);
    const int rc = gemm_i8(qa, w.k, sx, reinterpret_cast<const int8_t *>(w.raw), w.k, w.scales, ep, M, w.n, w.k, status, stream);
    prof_end_span(sp);
    if (sp >= 0) {
        prof_flops[PROF_GEMM] += 2.0 * M * (double)w.n * w.k;
        const double out_b = ep.mode == OUT_H16 ? 4.0 : ep.mode == OUT_F32_H16 ? 8.0 : ep.mode == OUT_RESID ? 8.0 : 4.0;
        prof_bytes[PROF_GEMM] += (double)M * w.k + (double)w.n * w.k + 4.0 * (M + w.n) + out_b * M * (double)w.n;
        prof_launches[PROF_GEMM]++;
    }
    if (rc == 0) note_launch();
    return rc;
}

static GemmEpilogue epi(int mode, int act, float alpha, const float *bias, float *out, int ldo, H16 h = H16{nullptr, nullptr},
                        int ldh = 0) {
    GemmEpilogue e;
    e.mode = mode; e.act = act; e.alpha = alpha; e.bias = bias; e.out = out; e.ldo = ldo;
    e.out_hi = h.hi; e.out_lo = h.lo; e.ldh = ldh;
    return e;
}

// ---------------------------------------------------------------- subsampling
// feats [t_mel, n_mels] on the device -> x_out [T3, d_model]; scratch from the arena
// (released on return: later kernels are ordered behind these on the same stream).
int Model::subsample_item(const float *feats, int t_mel, float *x_out, int *t_out) {
    const int C = channels, pl = causal ? 2 : 1, F0 = cfg.n_mels;
    const int T1 = sub_len(t_mel, causal), F1 = sub_len(F0, causal);
    const int T2 = sub_len(T1, causal), F2 = sub_len(F1, causal);
    const int T3 = sub_len(T2, causal), F3 = sub_len(F2, causal);
    const size_t mark = ws.off;
    H16 p1 = ws.planes((size_t)T2 * F2 * C);
    float *a1 = ws.get<float>((size_t)T2 * F2 * C);
    H16 p2 = ws.planes((size_t)T3 * F3 * C);
    H16 flat = ws.planes((size_t)T3 * F3 * C);
    if (!p1.hi || !p1.lo || !a1 || !p2.hi || !p2.lo || !flat.hi || !flat.lo) return -1;
    if (conv_in_dw_fused(feats, conv_in_w, conv_in_b, dw_w[0], dw_b[0], p1, t_mel, F0, C, T1, F1, T2, F2, pl, stream)) return -1;
    if (gemm(p1, C, pw[0], epi(OUT_F32, ACT_RELU, 1.f, pw[0].bias, a1, C), T2 * F2)) return -1;
    if (dwconv3x3_s2(a1, dw_w[1], dw_b[1], p2, T2, F2, C, T3, F3, pl, stream)) return -1;
    if (gemm(p2, C, pw[1], epi(OUT_H16, ACT_RELU, 1.f, pw[1].bias, nullptr, 0, flat, C), T3 * F3)) return -1;
    // flat is [T3, F3*C]: the linear's columns were permuted to this order at load
    if (gemm(flat, F3 * C, ss_lin, epi(OUT_F32, ACT_NONE, 1.f, ss_lin.bias, x_out, d_model), T3)) return -1;
    note_launch(2);
    if (xscale != 1.0f) { if (scale_inplace(x_out, (size_t)T3 * d_model, xscale, stream)) return -1; note_launch(); }
    ws.off = mark;
    *t_out = T3;
    return 0;
}

// ---------------------------------------------------------------- encoder stack
// x [sum(lens), d] in place. Runs layers [first_layer, first_layer + n_run).
int Model::encoder_layers(float *x, const std::vector<int> &lens, int left, int right, int first_layer, int n_run) {
    const int d = d_model, F = ffn_dim, B = (int)lens.size();
    int M = 0, max_len = 0;
    std::vector<int> seg_off(B), rk_off(B);
    std::vector<int> distinct, rk_base;        // distinct lengths and the row offset of their rk block
    int rk_rows = 0;
    for (int b = 0; b < B; b++) {
        seg_off[b] = M; M += lens[b];
        if (lens[b] > max_len) max_len = lens[b];
        int j = -1;
        for (size_t i = 0; i < distinct.size(); i++) if (distinct[i] == lens[b]) j = (int)i;
        if (j < 0) { distinct.push_back(lens[b]); rk_base.push_back(rk_rows); j = (int)distinct.size() - 1; rk_rows += 2 * lens[b] - 1; }
        rk_off[b] = rk_base[j];
    }
    if (M == 0) return 0;
    const size_t mark = ws.off;
    int *meta = ws.get<int>(3 * (size_t)B);
    if (!meta) return -1;
    std::vector<int> hmeta(3 * B);
    for (int b = 0; b < B; b++) { hmeta[b] = seg_off[b]; hmeta[B + b] = lens[b]; hmeta[2 * B + b] = rk_off[b]; }
    MB_CUDA(cudaMemcpyAsync(meta, hmeta.data(), hmeta.size() * sizeof(int), cudaMemcpyHostToDevice, stream));
    MB_CUDA(cudaStreamSynchronize(stream));      // hmeta is a stack-lifetime buffer
    const int *d_off = meta, *d_len = meta + B, *d_rk = meta + 2 * B;

    // the single-product mode never reads the lo planes: its producers do not write them (half the bytes of every
    // plane-writing epilogue, LayerNorm and conv-middle pass)
    const bool with_lo = cfg.strict != 0;
    H16 hA = ws.planes((size_t)M * d, with_lo), hC = ws.planes((size_t)M * d, with_lo), hF = ws.planes((size_t)M * F, with_lo);
    float *qbuf = ws.get<float>((size_t)M * d);
    H16 kbuf = ws.planes((size_t)M * d, false), vbuf = ws.planes((size_t)M * d, false);
    float *h2 = ws.get<float>((size_t)M * 2 * d);
    float *cbuf = ws.get<float>((size_t)M * d);
    H16 pe = ws.planes((size_t)rk_rows * d);
    H16 rk = ws.planes((size_t)rk_rows * d, false);
    if (!hA.hi || !hC.hi || !hF.hi || (with_lo && (!hA.lo || !hC.lo || !hF.lo)) || !qbuf || !kbuf.hi || !vbuf.hi || !h2 || !cbuf || !pe.lo || !rk.hi) return -1;

    // int8-activation mode: quantised rows of the LayerNorm outputs / attention context / conv middle (qA) and of
    // SiLU(FFN1) (qF), their scales, and the f32 values that get quantised
    const bool a8 = a8_layers;
    int8_t *qA = nullptr, *qF = nullptr;
    float *sxA = nullptr, *sxF = nullptr, *fF = nullptr;
    if (a8) {
        qA = ws.get<int8_t>((size_t)M * d); qF = ws.get<int8_t>((size_t)M * F);
        sxA = ws.get<float>(M); sxF = ws.get<float>(M); fF = ws.get<float>((size_t)M * F);
        if (!qA || !qF || !sxA || !sxF || !fF) return -1;
    }
    for (size_t i = 0; i < distinct.size(); i++) {
        H16 p{pe.hi + (size_t)rk_base[i] * d, pe.lo + (size_t)rk_base[i] * d};
        if (pos_emb(p, distinct[i], d, stream)) return -1;
        note_launch();
    }
    const int pad_left = causal ? conv_k - 1 : (conv_k - 1) / 2;
    const H16 none{nullptr, nullptr};
    for (int li = first_layer; li < first_layer + n_run; li++) {
        const EncLayer &L = layers[li];
        if (a8) {
            // the same block with int8 activations into every linear (the reference with MYNAH_ASR_QGEMM=1:
            // qmat_mul quantises the input rows of each of the ten linears, src/qmat.c:615-618)
            if (layer_norm_q8(x, L.ln_ff1_w, L.ln_ff1_b, nullptr, none, qA, sxA, M, d, ACT_NONE, stream)) return -1;
            if (gemm_q8(qA, sxA, L.ff1_w1, epi(OUT_F32, ACT_SILU, 1.f, L.ff1_w1.bias, fF, F), M)) return -1;
            if (act_quant_rows(fF, qF, sxF, M, F, stream)) return -1;
            if (gemm_q8(qF, sxF, L.ff1_w2, epi(OUT_RESID, ACT_NONE, 0.5f, L.ff1_w2.bias, x, d), M)) return -1;
            if (layer_norm_q8(x, L.ln_att_w, L.ln_att_b, nullptr, none, qA, sxA, M, d, ACT_NONE, stream)) return -1;
            if (gemm_q8(qA, sxA, L.q_w, epi(OUT_F32, ACT_NONE, 1.f, L.q_w.bias, qbuf, d), M)) return -1;
            if (gemm_q8(qA, sxA, L.k_w, epi(OUT_H16, ACT_NONE, 1.f, L.k_w.bias, nullptr, 0, kbuf, d), M)) return -1;
            if (gemm_q8(qA, sxA, L.v_w, epi(OUT_H16, ACT_NONE, 1.f, L.v_w.bias, nullptr, 0, vbuf, d), M)) return -1;
            if (gemm(pe, d, L.relk, epi(OUT_H16, ACT_NONE, 1.f, nullptr, nullptr, 0, rk, d), rk_rows)) return -1;
            AttnArgs at;
            at.q = qbuf; at.ldq = d; at.k = kbuf.hi; at.v = vbuf.hi; at.rk = rk.hi;
            at.bias_u = L.bias_u; at.bias_v = L.bias_v; at.ctx_f32 = cbuf; at.ctx_h = none;
            at.seg_off = d_off; at.seg_len = d_len; at.rk_off = d_rk;
            at.batch = B; at.max_len = max_len; at.d = d; at.H = n_heads; at.left = left; at.right = right;
            at.rows = M; at.rk_rows = rk_rows; at.status = status;
            { const int sp = prof_begin_span(PROF_ATTN);
              const int rc = attention_forward(at, cfg.attn_impl, stream);
              prof_end_span(sp);
              if (sp >= 0) prof_launches[PROF_ATTN]++;
              if (rc) return -1; }
            if (act_quant_rows(cbuf, qA, sxA, M, d, stream)) return -1;
            if (gemm_q8(qA, sxA, L.o_w, epi(OUT_RESID, ACT_NONE, 1.f, L.o_w.bias, x, d), M)) return -1;
            if (layer_norm_q8(x, L.ln_conv_w, L.ln_conv_b, nullptr, none, qA, sxA, M, d, ACT_NONE, stream)) return -1;
            if (gemm_q8(qA, sxA, L.pw1_w, epi(OUT_F32, ACT_NONE, 1.f, L.pw1_w.bias, h2, 2 * d), M)) return -1;
            if (L.cnorm_scale) {
                if (glu_dwconv(h2, L.dw_w, L.dw_b, L.cnorm_scale, L.cnorm_shift, cbuf, none, d_off, d_len, B, max_len, d,
                               conv_k, pad_left, stream)) return -1;
                if (act_quant_rows(cbuf, qA, sxA, M, d, stream)) return -1;
            } else {
                if (glu_dwconv(h2, L.dw_w, L.dw_b, nullptr, nullptr, cbuf, none, d_off, d_len, B, max_len, d, conv_k,
                               pad_left, stream)) return -1;
                if (layer_norm_q8(cbuf, L.cnorm_w, L.cnorm_b, nullptr, none, qA, sxA, M, d, ACT_SILU, stream)) return -1;
            }
            if (gemm_q8(qA, sxA, L.pw2_w, epi(OUT_RESID, ACT_NONE, 1.f, L.pw2_w.bias, x, d), M)) return -1;
            if (layer_norm_q8(x, L.ln_ff2_w, L.ln_ff2_b, nullptr, none, qA, sxA, M, d, ACT_NONE, stream)) return -1;
            if (gemm_q8(qA, sxA, L.ff2_w1, epi(OUT_F32, ACT_SILU, 1.f, L.ff2_w1.bias, fF, F), M)) return -1;
            if (act_quant_rows(fF, qF, sxF, M, F, stream)) return -1;
            if (gemm_q8(qF, sxF, L.ff2_w2, epi(OUT_RESID, ACT_NONE, 0.5f, L.ff2_w2.bias, x, d), M)) return -1;
            if (layer_norm(x, L.ln_out_w, L.ln_out_b, x, none, M, d, ACT_NONE, stream)) return -1;
            note_launch(11);   // 5 LayerNorms + attention + glu_dwconv + 4 activation quantisations (the contractions count themselves)
            continue;
        }
        // half FFN 1 (src/encoder.c:464-482,495-496)
        if (layer_norm(x, L.ln_ff1_w, L.ln_ff1_b, nullptr, hA, M, d, ACT_NONE, stream)) return -1;
        if (gemm(hA, d, L.ff1_w1, epi(OUT_H16, ACT_SILU, 1.f, L.ff1_w1.bias, nullptr, 0, hF, F), M)) return -1;
        if (gemm(hF, F, L.ff1_w2, epi(OUT_RESID, ACT_NONE, 0.5f, L.ff1_w2.bias, x, d), M)) return -1;
        // rel-pos MHSA (src/encoder.c:315-410,501-503)
        if (layer_norm(x, L.ln_att_w, L.ln_att_b, nullptr, hA, M, d, ACT_NONE, stream)) return -1;
        if (gemm(hA, d, L.q_w, epi(OUT_F32, ACT_NONE, 1.f, L.q_w.bias, qbuf, d), M)) return -1;
        if (gemm(hA, d, L.k_w, epi(OUT_H16, ACT_NONE, 1.f, L.k_w.bias, nullptr, 0, kbuf, d), M)) return -1;
        if (gemm(hA, d, L.v_w, epi(OUT_H16, ACT_NONE, 1.f, L.v_w.bias, nullptr, 0, vbuf, d), M)) return -1;
        if (gemm(pe, d, L.relk, epi(OUT_H16, ACT_NONE, 1.f, nullptr, nullptr, 0, rk, d), rk_rows)) return -1;
        AttnArgs at;
        at.q = qbuf; at.ldq = d; at.k = kbuf.hi; at.v = vbuf.hi; at.rk = rk.hi;
        at.bias_u = L.bias_u; at.bias_v = L.bias_v; at.ctx_f32 = nullptr; at.ctx_h = hC;
        at.seg_off = d_off; at.seg_len = d_len; at.rk_off = d_rk;
        at.batch = B; at.max_len = max_len; at.d = d; at.H = n_heads; at.left = left; at.right = right;
        at.rows = M; at.rk_rows = rk_rows; at.status = status;
        { const int sp = prof_begin_span(PROF_ATTN);
          const int rc = attention_forward(at, cfg.attn_impl, stream);
          prof_end_span(sp);
          if (sp >= 0) prof_launches[PROF_ATTN]++;
          if (rc) return -1; }
        if (gemm(hC, d, L.o_w, epi(OUT_RESID, ACT_NONE, 1.f, L.o_w.bias, x, d), M)) return -1;
        // conv module (src/encoder.c:413-460,506-508)
        if (layer_norm(x, L.ln_conv_w, L.ln_conv_b, nullptr, hA, M, d, ACT_NONE, stream)) return -1;
        if (gemm(hA, d, L.pw1_w, epi(OUT_F32, ACT_NONE, 1.f, L.pw1_w.bias, h2, 2 * d), M)) return -1;
        if (L.cnorm_scale) {
            if (glu_dwconv(h2, L.dw_w, L.dw_b, L.cnorm_scale, L.cnorm_shift, nullptr, hC, d_off, d_len, B, max_len, d,
                           conv_k, pad_left, stream)) return -1;
        } else {
            if (glu_dwconv(h2, L.dw_w, L.dw_b, nullptr, nullptr, cbuf, none, d_off, d_len, B, max_len, d, conv_k,
                           pad_left, stream)) return -1;
            if (layer_norm(cbuf, L.cnorm_w, L.cnorm_b, nullptr, hC, M, d, ACT_SILU, stream)) return -1;
            note_launch();
        }
        if (gemm(hC, d, L.pw2_w, epi(OUT_RESID, ACT_NONE, 1.f, L.pw2_w.bias, x, d), M)) return -1;
        // half FFN 2 + output LayerNorm (src/encoder.c:510-516)
        if (layer_norm(x, L.ln_ff2_w, L.ln_ff2_b, nullptr, hA, M, d, ACT_NONE, stream)) return -1;
        if (gemm(hA, d, L.ff2_w1, epi(OUT_H16, ACT_SILU, 1.f, L.ff2_w1.bias, nullptr, 0, hF, F), M)) return -1;
        if (gemm(hF, F, L.ff2_w2, epi(OUT_RESID, ACT_NONE, 0.5f, L.ff2_w2.bias, x, d), M)) return -1;
        if (layer_norm(x, L.ln_out_w, L.ln_out_b, x, none, M, d, ACT_NONE, stream)) return -1;
        note_launch(7);   // 5 LayerNorms + attention + glu_dwconv (the contractions count themselves)
    }
    ws.off = mark;
    return 0;
}

// encoder_projector when present, else copy (src/encoder.c:573-590)
int Model::encoder_post(const float *x, const std::vector<int> &lens, const int *prompt_ids, float *out) {
    int M = 0;
    for (int l : lens) M += l;
    if (M == 0) return 0;
    if (!has_encproj) {
        MB_CUDA(cudaMemcpyAsync(out, x, (size_t)M * d_model * sizeof(float), cudaMemcpyDeviceToDevice, stream));
        return 0;
    }
    const size_t mark = ws.off;
    H16 h = ws.planes((size_t)M * d_model);
    if (!h.lo) return -1;
    if (split_to_h16(x, h.hi, h.lo, (size_t)M * d_model, stream, status)) return -1;
    note_launch();
    if (has_prompt) {
        // concat(x, onehot(p)) W1^T + b1 = x W1[:, :d]^T + bias1[p]; ReLU; W2 (+b2); then the projector
        // (src/encoder.c:591-614). Runs of segments with the same prompt share one contraction.
        const int di = prompt_inter;
        H16 mid = ws.planes((size_t)M * di), fused = ws.planes((size_t)M * d_model);
        if (!mid.lo || !fused.lo) return -1;
        int row = 0;
        for (size_t b = 0; b < lens.size();) {
            const int pid = prompt_ids ? prompt_ids[b] : 0;
            if (pid < 0 || pid >= num_prompts) { set_error("encoder_post: prompt id %d outside [0, %d)", pid, num_prompts); return -1; }
            int rows = 0;
            size_t e = b;
            while (e < lens.size() && (prompt_ids ? prompt_ids[e] : 0) == pid) rows += lens[e++];
            if (rows > 0) {
                H16 hs{h.hi + (size_t)row * d_model, h.lo + (size_t)row * d_model};
                H16 ms{mid.hi + (size_t)row * di, mid.lo + (size_t)row * di};
                if (gemm(hs, d_model, prompt_l1, epi(OUT_H16, ACT_RELU, 1.f, prompt_bias1 + (size_t)pid * di, nullptr, 0, ms, di), rows)) return -1;
            }
            row += rows;
            b = e;
        }
        if (gemm(mid, di, prompt_l2, epi(OUT_H16, ACT_NONE, 1.f, prompt_l2.bias, nullptr, 0, fused, d_model), M)) return -1;
        h = fused;
    }
    if (gemm(h, d_model, encproj, epi(OUT_F32, ACT_NONE, 1.f, encproj.bias, out, d_out), M)) return -1;
    ws.off = mark;
    return 0;
}

int Model::log_mel(const float *audio_dev, size_t n, float *feats_dev, int T, int valid) {
    if (!has_mel) { set_error("log_mel: mel filterbank not set"); return -1; }
    MelCfg c{cfg.n_mels, cfg.n_fft, cfg.win_length, cfg.hop_length, cfg.preemphasis, cfg.log_zero_guard,
             cfg.normalize_per_feature};
    const int sp = prof_begin_span(PROF_MEL);
    const int rc = log_mel_device(c, audio_dev, n, mel_fb, mel_lo, mel_hi, mel_win, mel_tw, feats_dev, T, valid, stream);
    prof_end_span(sp);
    if (sp >= 0) prof_launches[PROF_MEL]++;
    if (rc == 0) note_launch(valid > 0 ? (c.normalize && valid > 1 ? 2 : 1) : 0);
    return rc;
}

// ---------------------------------------------------------------- decoders
int Model::decode_ctc(const float *enc_dev, int T, std::vector<int> &tokens, std::vector<int> &frames) {
    tokens.clear(); frames.clear();
    if (!has_ctc) { set_error("model has no CTC head"); return -1; }
    if (T <= 0) return 0;
    const int V = ctc_vocab, d = d_model;
    const size_t mark = ws.off;
    H16 h = ws.planes((size_t)T * d);
    float *logits = ws.get<float>((size_t)T * V);
    int *best = ws.get<int>(T);
    if (!h.lo || !logits || !best) return -1;
    if (split_to_h16(enc_dev, h.hi, h.lo, (size_t)T * d, stream, status)) return -1;
    if (gemm(h, d, ctc_head, epi(OUT_F32, ACT_NONE, 1.f, ctc_head.bias, logits, V), T)) return -1;
    if (argmax_rows(logits, V, nullptr, T, V, best, stream)) return -1;
    note_launch(2);
    std::vector<int> hb(T);
    MB_CUDA(cudaMemcpyAsync(hb.data(), best, T * sizeof(int), cudaMemcpyDeviceToHost, stream));
    MB_CUDA(cudaStreamSynchronize(stream));
    ws.off = mark;
    // collapse repeats, drop blank = V-1, keep the first frame (src/decoder_ctc.c:43-58)
    int prev = -1;
    for (int t = 0; t < T; t++) {
        if (hb[t] != prev && hb[t] != V - 1) { tokens.push_back(hb[t]); frames.push_back(t); }
        prev = hb[t];
    }
    return 0;
}

int Model::decode_greedy(const float *enc_dev, const std::vector<int> &lens, std::vector<std::vector<int>> &tokens,
                         std::vector<std::vector<int>> &frames) {
    const int Ball = (int)lens.size(), H = pred_hidden, L = pred_layers;
    tokens.assign(Ball, {}); frames.assign(Ball, {});
    if (!has_dec) { set_error("model has no transducer decoder"); return -1; }
    std::vector<int> offs(Ball);
    for (int b = 0, o = 0; b < Ball; o += lens[b], b++) offs[b] = o;
    const int nw = (vocab + cfg.n_durations + 15) / 16;     // candidate slots: one per 16-row block of the head
    // lock-step groups of DEC_MAX_B utterances; with several groups they run side by side on the decode lanes
    struct Group { int g0, B, cap; int *n_out, *tokens, *frames; long long *dbg; };
    std::vector<Group> groups;
    for (int g0 = 0; g0 < Ball; g0 += DEC_MAX_B) {
        const int B = Ball - g0 < DEC_MAX_B ? Ball - g0 : DEC_MAX_B;
        int max_len = 0;
        for (int b = 0; b < B; b++) if (lens[g0 + b] > max_len) max_len = lens[g0 + b];
        if (max_len > 0) groups.push_back(Group{g0, B, max_len * cfg.max_symbols, nullptr, nullptr, nullptr, nullptr});
    }
    if (groups.empty()) return 0;
    const size_t mark = ws.off;
    int *hm_dev = ws.get<int>(2 * (size_t)Ball);
    if (!hm_dev) return -1;
    std::vector<int> hm(2 * (size_t)Ball);
    for (int b = 0; b < Ball; b++) { hm[b] = offs[b]; hm[Ball + b] = lens[b]; }
    MB_CUDA(cudaMemcpyAsync(hm_dev, hm.data(), hm.size() * sizeof(int), cudaMemcpyHostToDevice, stream));
    MB_CUDA(cudaStreamSynchronize(stream));          // hm is a stack-lifetime buffer
    const int lanes = lanes_begin((int)groups.size());
    if (lanes < 1) return -1;
    const int lane_blocks = lanes > 1 ? (device_sm_count() / lanes > DEC_MAX_B ? device_sm_count() / lanes : DEC_MAX_B) : 0;
    for (size_t gi = 0; gi < groups.size(); gi++) {
        Group &G = groups[gi];
        const int B = G.B, cap = G.cap;
        cudaStream_t ls = lane_stream(lanes, (int)gi);
        const size_t nstate = (size_t)L * B * H;
        float *fz = ws.get<float>(3 * nstate + (size_t)B * H + 2 * (size_t)B * nw + (size_t)DEC_MAX_B * H);
        int *iz = ws.get<int>(8 * (size_t)B + 2 * (size_t)B * nw + 2 * (size_t)B * cap + 16);
        if (!fz || !iz) return -1;
        MB_CUDA(cudaMemsetAsync(fz, 0, (3 * nstate + (size_t)B * H) * sizeof(float), ls));
        MB_CUDA(cudaMemsetAsync(iz, 0, (8 * (size_t)B + 16) * sizeof(int), ls));
        GreedyDev p;
        memset(&p, 0, sizeof(p));
        p.emb = emb; p.head_b = head_b; p.proj_b = proj_b;
        p.emb_hi = emb_planes.hi; p.emb_lo = emb_planes.lo;
        p.head_hi = head.hi; p.head_lo = head.lo; p.proj_hi = dec_proj.hi; p.proj_lo = dec_proj.lo;
        for (int l = 0; l < L; l++) { p.wcat_hi[l] = wcat[l].hi; p.wcat_lo[l] = wcat[l].lo; p.b_ih[l] = b_ih[l]; p.b_hh[l] = b_hh[l]; }
        p.V = vocab; p.ND = cfg.n_durations; p.H = H; p.L = L; p.blank = cfg.blank_id; p.max_symbols = cfg.max_symbols;
        for (int i = 0; i < cfg.n_durations; i++) p.durations[i] = cfg.durations[i];
        p.B = B; p.enc = enc_dev;
        p.h[0] = fz; p.h[1] = fz + nstate; p.c = fz + 2 * nstate; p.g = fz + 3 * nstate;
        // the planes first: they are copied in 16-byte pieces and B * H floats keep that alignment
        p.jx_hi = reinterpret_cast<__half *>(p.g + (size_t)B * H); p.jx_lo = p.jx_hi + (size_t)DEC_MAX_B * H;
        p.cand_v = p.g + (size_t)B * H + (size_t)DEC_MAX_B * H;
        int *q = iz;
        p.flags = q; q += 16;
        p.t = q; q += B; p.emitted_here = q; q += B; p.n_out = q; q += B; p.last_tok = q; q += B; p.emit = q; q += B;
        q += 3 * B;
        p.cand_i = q; q += 2 * (size_t)B * nw;
        p.tokens = q; q += (size_t)B * cap; p.frames = q;
        p.cap = cap; p.enc_off = hm_dev + G.g0; p.enc_len = hm_dev + Ball + G.g0;
        int max_len = cap / cfg.max_symbols;
        p.max_steps = max_len * (cfg.max_symbols + 1) + 8; p.init_state = 1;
        if (prof_on && gi == 0) { G.dbg = reinterpret_cast<long long *>(ws.get<long long>(8)); if (G.dbg) MB_CUDA(cudaMemsetAsync(G.dbg, 0, 64, ls)); }
        p.dbg = G.dbg;
        G.n_out = p.n_out; G.tokens = p.tokens; G.frames = p.frames;
        { const int sp = gi == 0 ? prof_begin_span(PROF_DECODE) : -1;       // the span of group 0 brackets the fork; the rest overlap it
          const int rc = greedy_launch(p, ls, lane_blocks);
          if (sp >= 0 && lanes <= 1) { prof_end_span(sp); prof_launches[PROF_DECODE]++; }
          else if (sp >= 0) prof_pending = sp;
          if (rc) return -1; }
        note_launch();
    }
    if (lanes_join(lanes)) return -1;
    if (prof_pending >= 0) { prof_end_span(prof_pending); prof_launches[PROF_DECODE] += (long long)groups.size(); prof_pending = -1; }
    for (const Group &G : groups) {
        const int B = G.B, cap = G.cap;
        std::vector<int> hn(B), ht((size_t)B * cap), hf((size_t)B * cap);
        MB_CUDA(cudaMemcpyAsync(hn.data(), G.n_out, B * sizeof(int), cudaMemcpyDeviceToHost, stream));
        MB_CUDA(cudaMemcpyAsync(ht.data(), G.tokens, ht.size() * sizeof(int), cudaMemcpyDeviceToHost, stream));
        MB_CUDA(cudaMemcpyAsync(hf.data(), G.frames, hf.size() * sizeof(int), cudaMemcpyDeviceToHost, stream));
        if (G.dbg) MB_CUDA(cudaMemcpyAsync(dec_dbg, G.dbg, 64, cudaMemcpyDeviceToHost, stream));
        MB_CUDA(cudaStreamSynchronize(stream));
        for (int b = 0; b < B; b++) {
            tokens[G.g0 + b].assign(ht.begin() + (size_t)b * cap, ht.begin() + (size_t)b * cap + hn[b]);
            frames[G.g0 + b].assign(hf.begin() + (size_t)b * cap, hf.begin() + (size_t)b * cap + hn[b]);
        }
    }
    ws.off = mark;
    return 0;
}

}  // namespace mb
