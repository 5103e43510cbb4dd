// CTC forced alignment on the device: Viterbi over the extended label sequence blank, tok0, blank, tok1, ..., blank
// against per-frame scores [T, V] — the reference's mynah_asr_align_ctc (src/align.c:32-97), which gives the AED
// engine its word timestamps (align_words_ctc, src/mynah_asr.c:1102-1134) — with the scores already in HBM, where
// the aligner model's CTC head leaves them.
//
// One CTA per utterance. The recurrence is sequential in time and parallel over the S = 2N + 1 states: a thread
// owns states s, s + blockDim, ...; the two score vectors live in shared memory (double-buffered, one barrier per
// frame), the backpointers (one byte per frame and state) go to global memory, and thread 0 walks them back. The
// arithmetic and every comparison are the reference's: candidates stay / from s-1 / from s-2 (only into a label
// that differs from the label two states back), a later candidate wins only when strictly greater, pruned or
// unreachable states carry the finite sentinel -1e30, a path is "none" below -1e29, raw logits serve as scores.
// Given the same scores the result is identical to the reference's, ties included.
#include "kernels.h"

namespace mb {

static constexpr float ALIGN_NEG_BIG = -1.0e30f;
static constexpr float ALIGN_UNREACHABLE = -1.0e29f;

struct AlignItem {
    const float *scores;     // [T, V] on the device
    const int *tokens;       // [n] on the device
    unsigned char *bp;       // [T, 2n + 1] scratch
    int *t0, *t1;            // [n] out
    int *rc;                 // out: 0 ok, -1 no path
    int T, V, n, blank;
};

__global__ void __launch_bounds__(256)
align_ctc_kernel(const AlignItem *__restrict__ items) {
    extern __shared__ float sm[];
    const AlignItem it = items[blockIdx.x];
    const int S = 2 * it.n + 1, T = it.T, V = it.V;
    float *prv = sm, *cur = sm + S;
    int *ext = reinterpret_cast<int *>(sm + 2 * S);
    for (int s = threadIdx.x; s < S; s += blockDim.x) {
        ext[s] = (s & 1) ? it.tokens[s >> 1] : it.blank;
        it.bp[s] = 0;
    }
    __syncthreads();
    for (int s = threadIdx.x; s < S; s += blockDim.x)
        prv[s] = s < 2 ? it.scores[ext[s]] : ALIGN_NEG_BIG;       // frame 0: the leading blank or the first token
    __syncthreads();
    for (int t = 1; t < T; t++) {
        const float *row = it.scores + (size_t)t * V;
        unsigned char *bpt = it.bp + (size_t)t * S;
        const int s_lo = S - 2 * (T - t) > 0 ? S - 2 * (T - t) : 0;
        const int s_hi = 2 * t + 1 < S - 1 ? 2 * t + 1 : S - 1;
        for (int s = threadIdx.x; s < S; s += blockDim.x) {
            float v = ALIGN_NEG_BIG;
            unsigned char from = 0;
            if (s >= s_lo && s <= s_hi) {
                float best = prv[s];
                if (s >= 1 && prv[s - 1] > best) { best = prv[s - 1]; from = 1; }
                if (s >= 2 && ext[s] != it.blank && ext[s] != ext[s - 2] && prv[s - 2] > best) { best = prv[s - 2]; from = 2; }
                v = best > ALIGN_UNREACHABLE ? __fadd_rn(best, row[ext[s]]) : ALIGN_NEG_BIG;
            }
            cur[s] = v;
            bpt[s] = from;
        }
        __syncthreads();
        float *sw = prv; prv = cur; cur = sw;
    }
    for (int j = threadIdx.x; j < it.n; j += blockDim.x) { it.t0[j] = -1; it.t1[j] = -1; }
    __syncthreads();
    if (threadIdx.x == 0) {
        int s = prv[S - 1] >= prv[S - 2] ? S - 1 : S - 2;        // ends on the trailing blank or on the last token
        int rc = prv[s] <= ALIGN_UNREACHABLE ? -1 : 0;
        if (rc == 0) {
            for (int t = T - 1; t >= 0; t--) {
                if (s & 1) {
                    const int j = s >> 1;
                    if (it.t1[j] < 0) it.t1[j] = t;
                    it.t0[j] = t;
                }
                s -= it.bp[(size_t)t * S + s];
            }
            for (int j = 0; j < it.n; j++) if (it.t0[j] < 0) rc = -1;
        }
        *it.rc = rc;
    }
}

int align_min_frames(const int *tokens, int n) {
    if (n <= 0) return 0;
    int need = n;
    for (int i = 1; i < n; i++) if (tokens[i] == tokens[i - 1]) need++;
    return need;
}

// scores_dev [T, V] resident; tokens on the host. Synchronous on `st`. Returns 0 / -1 like the reference.
int align_ctc_device(const float *scores_dev, int T, int V, const int *tokens, int n, int blank, int *t0, int *t1, cudaStream_t st) {
    if (!scores_dev || !tokens || !t0 || !t1 || T <= 0 || V <= 0 || n <= 0 || blank < 0 || blank >= V) { set_error("align_ctc: bad argument"); return -1; }
    for (int i = 0; i < n; i++) if (tokens[i] < 0 || tokens[i] >= V || tokens[i] == blank) { set_error("align_ctc: token %d is not a label", tokens[i]); return -1; }
    if (T < align_min_frames(tokens, n)) { set_error("align_ctc: %d frames cannot hold %d tokens", T, n); return -1; }
    const int S = 2 * n + 1;
    const size_t smem = (size_t)S * (2 * sizeof(float) + sizeof(int));
    if (smem > 200 * 1024) { set_error("align_ctc: %d tokens exceed the shared-memory budget", n); return -1; }
    uint8_t *buf = nullptr;
    const size_t off_tok = align_up(sizeof(AlignItem), 256), off_t0 = off_tok + align_up((size_t)n * 4, 256), off_t1 = off_t0 + align_up((size_t)n * 4, 256);
    const size_t off_rc = off_t1 + align_up((size_t)n * 4, 256), off_bp = off_rc + 256, total = off_bp + (size_t)T * S;
    MB_CUDA(cudaMallocAsync((void **)&buf, total, st));
    AlignItem it;
    it.scores = scores_dev; it.tokens = (const int *)(buf + off_tok); it.bp = buf + off_bp;
    it.t0 = (int *)(buf + off_t0); it.t1 = (int *)(buf + off_t1); it.rc = (int *)(buf + off_rc);
    it.T = T; it.V = V; it.n = n; it.blank = blank;
    int rc = -1;
    cudaError_t e = cudaMemcpyAsync(buf, &it, sizeof(it), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(buf + off_tok, tokens, (size_t)n * 4, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) {
        static PerDevice configured = {};
        int dev = 0;
        if (smem > 48 * 1024 && configured.below(smem, &dev)) {
            e = cudaFuncSetAttribute(align_ctc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            configured.record(dev, smem);
        }
    }
    if (e == cudaSuccess) {
        align_ctc_kernel<<<1, 256, smem, st>>>((const AlignItem *)buf);
        note_launch();
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(&rc, buf + off_rc, 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(t0, buf + off_t0, (size_t)n * 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(t1, buf + off_t1, (size_t)n * 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFreeAsync(buf, st);
    if (e != cudaSuccess) { set_error("align_ctc: %s", cudaGetErrorString(e)); return -1; }
    if (rc != 0) set_error("align_ctc: no path");
    return rc;
}

}  // namespace mb
