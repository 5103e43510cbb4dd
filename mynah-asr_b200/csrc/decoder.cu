// Greedy decoders on device.
//
// CTC (the reference's mynah_asr_ctc_decode, src/decoder_ctc.c:36-61): the head
// GEMM runs on the contraction kernel; argmax_rows picks the first maximum of
// logit + bias per frame; the collapse (drop repeats, drop blank = V-1) is a scan
// over T integers done by the caller.
//
// RNNT / TDT (mynah_asr_greedy_decode and greedy_decode_tdt, src/decoder.c:129-265):
// strictly sequential per utterance, so a batch of up to 16 utterances advances in
// lock step inside ONE persistent cooperative kernel — no launch or host round trip
// per step. Every step is a few grid-wide phases separated by grid syncs:
//   head    logits[b] = head . relu(enc[b][t_b] + g[b]), every warp owning a slice
//           of the V (+durations) rows and keeping a running first-argmax per b
//   select  one CTA per utterance merges the candidates and applies the emission
//           rule: non-blank -> emit, advance by the predicted duration (RNNT: 0),
//           blank with duration 0 -> 1, max_symbols guard (src/decoder.c:161-176)
//   lstm    (only if some utterance emitted) one warp per hidden unit computes the
//           four gate rows of W_ih and W_hh for all emitting utterances and applies
//           the cell update; layers are separated by a grid sync
//   proj    g[b] = decoder_projector(h_last[b])
// All arithmetic is f32 FMA over the exactly decoded f32 weights, like the
// reference's sgemv/sgemm path.
#include <cooperative_groups.h>

#include "kernels.h"
#include "model.h"

namespace cg = cooperative_groups;

namespace mb {

// -------------------------------------------------------------- argmax per row
__global__ void __launch_bounds__(256)
argmax_kernel(const float *__restrict__ logits, int ld, const float *__restrict__ bias, int V, int *__restrict__ best) {
    __shared__ float sv[256];
    __shared__ int si[256];
    const float *row = logits + (size_t)blockIdx.x * ld;
    float bv = -3.0e38f;
    int bi = 0x7fffffff;
    for (int k = threadIdx.x; k < V; k += 256) {
        const float v = row[k] + (bias ? bias[k] : 0.0f);
        if (v > bv) { bv = v; bi = k; }          // ascending k per thread: first maximum kept
    }
    sv[threadIdx.x] = bv; si[threadIdx.x] = bi;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) {
            const float v = sv[threadIdx.x + o];
            const int i = si[threadIdx.x + o];
            if (v > sv[threadIdx.x] || (v == sv[threadIdx.x] && i < si[threadIdx.x])) { sv[threadIdx.x] = v; si[threadIdx.x] = i; }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) best[blockIdx.x] = si[0];
}

int argmax_rows(const float *logits, int ld, const float *bias, int T, int V, int *best, cudaStream_t st) {
    if (T <= 0) return 0;
    argmax_kernel<<<T, 256, 0, st>>>(logits, ld, bias, V, best);
    MB_CUDA(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------- RNNT / TDT lock-step

__device__ __forceinline__ float dotrow(const float *__restrict__ w, const float *__restrict__ x, int H, int lane) {
    float s = 0.0f;
    for (int k = lane * 4; k < H; k += 128) {
        const float4 a = *reinterpret_cast<const float4 *>(w + k);
        const float4 b = *reinterpret_cast<const float4 *>(x + k);
        s += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
    }
    return warp_sum(s);
}

// One stacked-LSTM layer for the utterances whose emit flag is set (pred_step,
// src/decoder.c:73-99). Reads h[par], writes h[par^1]; c is updated in place
// (each (b, unit) has one owner). Non-emitting utterances copy h through.
__device__ void lstm_layer(const GreedyDev &p, int l, int par, float *xs, int gw, int nw, int lane) {
    const int H = p.H, B = p.B;
    const float *hold = p.h[par] + (size_t)l * B * H;
    float *hnew = p.h[par ^ 1] + (size_t)l * B * H;
    float *cc = p.c + (size_t)l * B * H;
    for (int idx = gw; idx < H * B; idx += nw) {
        const int b = idx / H, i = idx % H;
        if (!p.emit[b]) { if (lane == 0) hnew[(size_t)b * H + i] = hold[(size_t)b * H + i]; continue; }
        const float *x = l == 0 ? p.emb + (size_t)p.last_tok[b] * H : p.h[par ^ 1] + ((size_t)(l - 1) * B + b) * H;
        const float *hp = hold + (size_t)b * H;
        float z[4];
#pragma unroll
        for (int gte = 0; gte < 4; gte++) {
            const size_t r = (size_t)(gte * H + i);
            z[gte] = p.b_ih[l][r] + p.b_hh[l][r] + dotrow(p.w_ih[l] + r * H, x, H, lane) +
                     dotrow(p.w_hh[l] + r * H, hp, H, lane);
        }
        if (lane == 0) {
            const float ig = sigmoid_stable(z[0]), fg = sigmoid_stable(z[1]);
            const float gg = tanhf(z[2]), og = sigmoid_stable(z[3]);
            const float cn = fg * cc[(size_t)b * H + i] + ig * gg;
            cc[(size_t)b * H + i] = cn;
            hnew[(size_t)b * H + i] = og * tanhf(cn);
        }
    }
    (void)xs;
}

__global__ void __launch_bounds__(256, 1)
greedy_kernel(GreedyDev p) {
    cg::grid_group grid = cg::this_grid();
    extern __shared__ float joint[];                 // [B][H]
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int nw = gridDim.x * 8, gw = blockIdx.x * 8 + wib;
    const int H = p.H, B = p.B, V = p.V, VL = p.V + p.ND;
    int par = 0;

    if (p.init_state) {
        // SOS = blank on a zero state (src/decoder.c:151): run the prediction net once
        if (blockIdx.x == 0 && threadIdx.x < B) { p.emit[threadIdx.x] = 1; p.last_tok[threadIdx.x] = p.blank; }
        grid.sync();
        for (int l = 0; l < p.L; l++) { lstm_layer(p, l, par, joint, gw, nw, lane); grid.sync(); }
        par ^= 1;
        for (int i = gw; i < B * H; i += nw) {
            const int b = i / H, u = i % H;
            const float v = p.proj_b[u] + dotrow(p.proj_w + (size_t)u * H, p.h[par] + ((size_t)(p.L - 1) * B + b) * H, H, lane);
            if (lane == 0) p.g[i] = v;
        }
        grid.sync();
    }

    for (int step = 0; step < p.max_steps; step++) {
        // ---- head: joint = relu(enc[t] + g), logits, running first-argmax per warp
        for (int i = threadIdx.x; i < B * H; i += blockDim.x) {
            const int b = i / H, u = i % H;
            const int tb = p.t[b];
            joint[i] = tb < p.enc_len[b] ? fmaxf(p.enc[(size_t)(p.enc_off[b] + tb) * H + u] + p.g[i], 0.0f) : 0.0f;
        }
        __syncthreads();
        float bvt[DEC_MAX_B], bvd[DEC_MAX_B];
        int bit[DEC_MAX_B], bid[DEC_MAX_B];
#pragma unroll
        for (int b = 0; b < DEC_MAX_B; b++) { bvt[b] = bvd[b] = -3.0e38f; bit[b] = bid[b] = 0x7fffffff; }
        for (int r = gw; r < VL; r += nw) {
            const float *wr = p.head_w + (size_t)r * H;
            const float hb = p.head_b[r];
            const bool is_dur = r >= V;
#pragma unroll
            for (int b = 0; b < DEC_MAX_B; b++) {
                if (b < B) {
                    const float v = dotrow(wr, joint + b * H, H, lane) + hb;
                    // rows ascend within a warp, so ">" keeps the first maximum
                    if (is_dur) { if (v > bvd[b]) { bvd[b] = v; bid[b] = r; } }
                    else { if (v > bvt[b]) { bvt[b] = v; bit[b] = r; } }
                }
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int b = 0; b < DEC_MAX_B; b++) {
                if (b < B) {
                    p.cand_v[((size_t)b * 2 + 0) * nw + gw] = bvt[b]; p.cand_i[((size_t)b * 2 + 0) * nw + gw] = bit[b];
                    p.cand_v[((size_t)b * 2 + 1) * nw + gw] = bvd[b]; p.cand_i[((size_t)b * 2 + 1) * nw + gw] = bid[b];
                }
            }
        }
        // flags are double-buffered by step parity: a CTA that runs ahead into the next
        // step must not overwrite what a slower CTA is still reading
        int *fl = p.flags + (step & 1) * 2;
        if (blockIdx.x == 0 && threadIdx.x == 0) { fl[0] = 0; fl[1] = 1; }
        grid.sync();
        // ---- select: CTA b merges candidates and applies the emission rule
        if (blockIdx.x < B) {
            const int b = blockIdx.x;
            __shared__ float sv[2][256];
            __shared__ int si[2][256];
            for (int kind = 0; kind < 2; kind++) {
                float v = -3.0e38f; int ix = 0x7fffffff;
                for (int w = threadIdx.x; w < nw; w += blockDim.x) {
                    const float cv = p.cand_v[((size_t)b * 2 + kind) * nw + w];
                    const int ci = p.cand_i[((size_t)b * 2 + kind) * nw + w];
                    if (cv > v || (cv == v && ci < ix)) { v = cv; ix = ci; }
                }
                sv[kind][threadIdx.x] = v; si[kind][threadIdx.x] = ix;
            }
            __syncthreads();
            for (int o = 128; o > 0; o >>= 1) {
                if (threadIdx.x < o)
                    for (int kind = 0; kind < 2; kind++) {
                        const float v = sv[kind][threadIdx.x + o]; const int ix = si[kind][threadIdx.x + o];
                        if (v > sv[kind][threadIdx.x] || (v == sv[kind][threadIdx.x] && ix < si[kind][threadIdx.x])) {
                            sv[kind][threadIdx.x] = v; si[kind][threadIdx.x] = ix;
                        }
                    }
                __syncthreads();
            }
            if (threadIdx.x == 0) {
                int tb = p.t[b];
                int em = 0;
                if (tb < p.enc_len[b]) {
                    const int k = si[0][0];
                    int dur = p.ND > 0 ? p.durations[si[1][0] - V] : (k == p.blank ? 1 : 0);
                    if (k != p.blank) {
                        const int no = p.n_out[b];
                        if (no < p.cap) { p.tokens[(size_t)b * p.cap + no] = k; p.frames[(size_t)b * p.cap + no] = tb; p.n_out[b] = no + 1; }
                        em = 1;
                        p.last_tok[b] = k;
                        const int eh = p.emitted_here[b] + 1;
                        p.emitted_here[b] = eh;
                        if (dur == 0 && eh >= p.max_symbols) dur = 1;
                    } else if (dur == 0) {
                        dur = 1;
                    }
                    if (dur > 0) p.emitted_here[b] = 0;
                    tb += dur;
                    p.t[b] = tb;
                }
                p.emit[b] = em;
                if (em) atomicExch(&fl[0], 1);
                if (tb < p.enc_len[b]) atomicExch(&fl[1], 0);
            }
        }
        grid.sync();
        const int any_emit = *reinterpret_cast<volatile int *>(&fl[0]);
        const int all_done = *reinterpret_cast<volatile int *>(&fl[1]);
        if (any_emit) {
            for (int l = 0; l < p.L; l++) { lstm_layer(p, l, par, joint, gw, nw, lane); grid.sync(); }
            par ^= 1;
            for (int i = gw; i < B * H; i += nw) {
                const int b = i / H, u = i % H;
                if (!p.emit[b]) continue;
                const float v = p.proj_b[u] + dotrow(p.proj_w + (size_t)u * H, p.h[par] + ((size_t)(p.L - 1) * B + b) * H, H, lane);
                if (lane == 0) p.g[i] = v;
            }
            grid.sync();
        }
        if (all_done) break;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) p.flags[4] = par;
}

int greedy_launch(const GreedyDev &p, cudaStream_t st) {
    int dev = 0, sms = 0, coop = 0;
    MB_CUDA(cudaGetDevice(&dev));
    MB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    MB_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    if (!coop) { set_error("greedy decode: device lacks cooperative launch"); return -1; }
    const size_t smem = (size_t)p.B * p.H * sizeof(float);
    if (smem > 48 * 1024)
        MB_CUDA(cudaFuncSetAttribute(greedy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int per_sm = 0;
    MB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, greedy_kernel, 256, smem));
    if (per_sm < 1) { set_error("greedy decode: kernel does not fit an SM"); return -1; }
    int blocks = sms;
    if (blocks < p.B) { set_error("greedy decode: batch %d exceeds SM count", p.B); return -1; }
    GreedyDev pc = p;
    void *args[] = {&pc};
    MB_CUDA(cudaLaunchCooperativeKernel((void *)greedy_kernel, dim3(blocks), dim3(256), args, smem, st));
    return 0;
}

}  // namespace mb
