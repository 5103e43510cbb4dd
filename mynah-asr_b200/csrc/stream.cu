// Cache-aware streaming encoder step for S streams in lock step: the device counterpart of
// mynah_asr_enc_stream_step (src/encoder.c:809-872) with ss_stream_step (src/subsampling.c:320-370),
// stream_attention (:695-760), update_kv_cache (:763-776) and stream_conv_module (:779-807).
// Where the reference runs 240 weight-streaming GEMVs per stream and chunk, the streams of a group are
// stacked: every linear is one contraction over M = S * q rows, so the weights cross HBM once per
// chunk for all streams. Only the parts that touch per-stream state are kernels of their own.
#include "model.h"

namespace mb {

// ---- subsampling stages on a chunk (time axis = [zero if first][cached frame][chunk][zero if last], valid
// stride-2 conv in time, (2,1) zero padding in frequency: stream_stage, src/subsampling.c:289-318)
// stage 0: mel [S, T, F] (one channel) -> out [S, To, Fo, C] with ReLU
__global__ void ss_stream_stage0_kernel(const float *__restrict__ mel, const float *__restrict__ cache, const float *__restrict__ w,
                                        const float *__restrict__ b, float *__restrict__ out, int S, int T, int F, int C, int To, int Fo,
                                        int lp) {
    const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (idx >= (size_t)S * To * Fo * C) return;
    const int c = (int)(idx % C);
    size_t r = idx / C;
    const int fo = (int)(r % Fo); r /= Fo;
    const int to = (int)(r % To);
    const int s = (int)(r / To);
    float acc = b[c];
    for (int dt = 0; dt < 3; dt++) {
        const int tp = 2 * to + dt - lp;                 // index into the chunk; -1 = cached frame, below = zero, >= T = zero
        if (tp < -1 || tp >= T) continue;
        const float *row = tp < 0 ? cache + (size_t)s * F : mel + ((size_t)s * T + tp) * F;
        for (int df = 0; df < 3; df++) {
            const int f = 2 * fo + df - 2;
            if (f >= 0 && f < F) acc = fmaf(w[c * 9 + dt * 3 + df], row[f], acc);
        }
    }
    out[idx] = fmaxf(acc, 0.f);
}

// depthwise stage: a [S, T, F, C] -> planes [S, To, Fo, C] (operand of the pointwise contraction)
__global__ void ss_stream_dw_kernel(const float *__restrict__ a, const float *__restrict__ cache, const float *__restrict__ w,
                                    const float *__restrict__ b, H16 out, int S, int T, int F, int C, int To, int Fo, int lp) {
    const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (idx >= (size_t)S * To * Fo * C) return;
    const int c = (int)(idx % C);
    size_t r = idx / C;
    const int fo = (int)(r % Fo); r /= Fo;
    const int to = (int)(r % To);
    const int s = (int)(r / To);
    float acc = b[c];
    for (int dt = 0; dt < 3; dt++) {
        const int tp = 2 * to + dt - lp;
        if (tp < -1 || tp >= T) continue;
        const float *row = tp < 0 ? cache + (size_t)s * F * C : a + ((size_t)s * T + tp) * F * C;
        for (int df = 0; df < 3; df++) {
            const int f = 2 * fo + df - 2;
            if (f >= 0 && f < F) acc = fmaf(w[c * 9 + dt * 3 + df], row[(size_t)f * C + c], acc);
        }
    }
    __half hi, lo;
    split_h16(acc, hi, lo);
    out.hi[idx] = hi;
    out.lo[idx] = lo;
}

// cache[s] = last time row of x [S, T, W]
__global__ void ss_stream_cache_kernel(const float *__restrict__ x, float *__restrict__ cache, int S, int T, int W) {
    const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (idx >= (size_t)S * W) return;
    const int s = (int)(idx / W), i = (int)(idx % W);
    cache[idx] = x[((size_t)s * T + (T - 1)) * W + i];
}

// ---- attention of the chunk's Q rows over [valid cached frames ; chunk], no mask. Grid (H, S), STREAM_ATTN_WARPS warps.
// score[t][j] = ((q_t + u) . k_j + (q_t + v) . rk[K-1-valid-t+j]) / sqrt(dk); ctx planes [S*Q, d]. dk is a multiple of 4.
// Scores: a warp takes STREAM_ATTN_KU keys at a time, a lane four consecutive elements of each k and rk row (8-byte
// loads). Context: warp w sums the keys j = w, w + warps, ... for the lane's four columns (as many keys in flight);
// the partial sums are added in warp order.
// update != 0: afterwards the chunk's k / v rows of this head go to their ring slots (update_kv_cache,
// src/encoder.c:763-776) — the columns of head h of stream s are read by this block alone, so it may overwrite them
// once its own reads are done.
static constexpr int STREAM_ATTN_WARPS = 8;                // (16 measured slower: 20.1 against 17.1 ms per step at 512 streams)
static constexpr int STREAM_ATTN_KU = 4;               // keys a warp has in flight (8 measured slower: 19.1 against 17.2 ms per step at 512 streams)
__device__ __forceinline__ float4 ld_half4(const __half *p) {
    const uint2 a = *reinterpret_cast<const uint2 *>(p);
    const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&a.x)), hi = __half22float2(*reinterpret_cast<const __half2 *>(&a.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__global__ void __launch_bounds__(STREAM_ATTN_WARPS * 32)
stream_attn_kernel(const float *__restrict__ q, const __half *__restrict__ kn, const __half *__restrict__ vn,
                   __half *kc, __half *vc, const __half *__restrict__ rk,
                   const float *__restrict__ bias_u, const float *__restrict__ bias_v, H16 ctx, int Q, int valid,
                   const int *__restrict__ d_start, int left, int d, int dk, int update) {
    extern __shared__ float sm[];
    chain_trigger();                   // a chained contraction behind this kernel may start fetching its weights
    chain_wait();
    constexpr int NW = STREAM_ATTN_WARPS;
    const int K = valid + Q, start = *d_start;
    float *sc = sm;                                    // [K] (rounded up to a multiple of 4)
    float *qu = sc + ((K + 3) & ~3), *qv = qu + dk;    // [dk] each
    float *red = qv + dk;                              // [32]
    float *part = red + 32;                            // [NW][dk]
    const int h = blockIdx.x, s = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float scale = 1.0f / sqrtf((float)dk);
    // the ring of (stream s, head h) is one contiguous block of left x dk halves: [S][H][left][dk]
    const size_t cbase = ((size_t)s * gridDim.x + h) * left * dk, nbase = (size_t)s * Q * d + h * dk;
    // row j of the keys / values: a cached frame in its ring slot, or a row of the chunk
    auto krow = [&](int j) { int x = start + j; if (x >= left) x -= left; return j < valid ? kc + cbase + (size_t)x * dk : kn + nbase + (size_t)(j - valid) * d; };
    auto vrow = [&](int j) { int x = start + j; if (x >= left) x -= left; return j < valid ? vc + cbase + (size_t)x * dk : vn + nbase + (size_t)(j - valid) * d; };
    for (int t = 0; t < Q; t++) {
        const size_t row = (size_t)s * Q + t;
        for (int i = threadIdx.x; i < dk; i += blockDim.x) {
            const float v = q[row * d + h * dk + i];
            qu[i] = v + bias_u[h * dk + i];
            qv[i] = v + bias_v[h * dk + i];
        }
        __syncthreads();
        const int base = K - 1 - valid - t;
        constexpr int KU = STREAM_ATTN_KU;
        for (int j0 = warp * KU; j0 < K; j0 += KU * NW) {
            float a[KU];
#pragma unroll
            for (int u = 0; u < KU; u++) a[u] = 0.f;
            for (int i0 = lane * 4; i0 < dk; i0 += 128) {
                float4 kk[KU], rr[KU];
#pragma unroll
                for (int u = 0; u < KU; u++) {
                    const int j = j0 + u < K ? j0 + u : K - 1;
                    kk[u] = ld_half4(krow(j) + i0);
                    rr[u] = ld_half4(rk + (size_t)(base + j) * d + h * dk + i0);
                }
                const float4 u4 = *reinterpret_cast<const float4 *>(qu + i0), v4 = *reinterpret_cast<const float4 *>(qv + i0);
#pragma unroll
                for (int u = 0; u < KU; u++) {
                    a[u] = fmaf(u4.x, kk[u].x, a[u]); a[u] = fmaf(v4.x, rr[u].x, a[u]);
                    a[u] = fmaf(u4.y, kk[u].y, a[u]); a[u] = fmaf(v4.y, rr[u].y, a[u]);
                    a[u] = fmaf(u4.z, kk[u].z, a[u]); a[u] = fmaf(v4.z, rr[u].z, a[u]);
                    a[u] = fmaf(u4.w, kk[u].w, a[u]); a[u] = fmaf(v4.w, rr[u].w, a[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < KU; u++) {
                const float r = warp_sum(a[u]);
                if (lane == 0 && j0 + u < K) sc[j0 + u] = r * scale;
            }
        }
        __syncthreads();
        float m = -INFINITY;
        for (int j = threadIdx.x; j < K; j += blockDim.x) m = fmaxf(m, sc[j]);
        m = warp_max(m);
        if (lane == 0) red[warp] = m;
        __syncthreads();
        m = red[0];
        for (int i = 1; i < NW; i++) m = fmaxf(m, red[i]);
        __syncthreads();
        float sum = 0.f;
        for (int j = threadIdx.x; j < K; j += blockDim.x) { const float e = expf(sc[j] - m); sc[j] = e; sum += e; }
        sum = warp_sum(sum);
        if (lane == 0) red[warp] = sum;
        __syncthreads();
        sum = 0.f;
        for (int i = 0; i < NW; i++) sum += red[i];
        const float inv = 1.0f / sum;
        for (int c0 = lane * 4; c0 < dk; c0 += 128) {
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
            int j = warp;
            for (; j + (KU - 1) * NW < K; j += KU * NW) {
                float4 v[KU];
#pragma unroll
                for (int u = 0; u < KU; u++) v[u] = ld_half4(vrow(j + NW * u) + c0);
#pragma unroll
                for (int u = 0; u < KU; u++) {
                    const float w = sc[j + NW * u] * inv;
                    o.x = fmaf(w, v[u].x, o.x); o.y = fmaf(w, v[u].y, o.y); o.z = fmaf(w, v[u].z, o.z); o.w = fmaf(w, v[u].w, o.w);
                }
            }
            for (; j < K; j += NW) {
                const float4 v = ld_half4(vrow(j) + c0);
                const float w = sc[j] * inv;
                o.x = fmaf(w, v.x, o.x); o.y = fmaf(w, v.y, o.y); o.z = fmaf(w, v.z, o.z); o.w = fmaf(w, v.w, o.w);
            }
            *reinterpret_cast<float4 *>(part + warp * dk + c0) = o;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < dk; i += blockDim.x) {
            float o = part[i];
            for (int w = 1; w < NW; w++) o += part[w * dk + i];
            __half hi, lo;
            split_h16(o, hi, lo);
            ctx.hi[row * d + h * dk + i] = hi;
            ctx.lo[row * d + h * dk + i] = lo;
        }
        __syncthreads();
    }
    if (update) {
        for (int idx = threadIdx.x; idx < Q * dk; idx += blockDim.x) {
            const int t = idx / dk, i = idx - t * dk;
            int x = start + valid + t;
            x %= left;
            kc[cbase + (size_t)x * dk + i] = kn[nbase + (size_t)t * d + i];
            vc[cbase + (size_t)x * dk + i] = vn[nbase + (size_t)t * d + i];
        }
    }
}

// after the last layer: the ring's oldest frame moves on by the frames that were overwritten
__global__ void stream_advance_kernel(int *d_start, int valid, int Q, int left) {
    const int total = valid + Q;
    if (total > left) *d_start = (*d_start + (total - left)) % left;
}

// GLU rows appended to the k-1 cached ones, depthwise conv over the k rows ending at each new row, cache
// refreshed with the last k-1 rows (stream_conv_module, src/encoder.c:779-800). One thread per (stream, channel).
template <int KMAX>
__global__ void stream_conv_kernel(const float *__restrict__ h2, const float *__restrict__ dw_w, float *__restrict__ cache,
                                   float *__restrict__ out, int S, int Q, int d, int k) {
    chain_trigger();
    chain_wait();
    const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (idx >= (size_t)S * d) return;
    const int s = (int)(idx / d), i = (int)(idx % d);
    float seq[KMAX];                                     // k-1 cached rows then the Q new ones (k - 1 + Q <= KMAX)
    float *cc = cache + (size_t)s * (k - 1) * d + i;
    for (int j = 0; j < k - 1; j++) seq[j] = cc[(size_t)j * d];
    for (int t = 0; t < Q; t++) {
        const float *r = h2 + ((size_t)s * Q + t) * 2 * d;
        seq[k - 1 + t] = r[i] * sigmoid_fast(r[d + i]);
    }
    for (int t = 0; t < Q; t++) {
        float o = 0.f;
        for (int j = 0; j < k; j++) o = fmaf(dw_w[(size_t)i * k + j], seq[t + j], o);
        out[((size_t)s * Q + t) * d + i] = o;
    }
    for (int j = 0; j < k - 1; j++) cc[(size_t)j * d] = seq[Q + j];
}

static GemmEpilogue st_epi(int mode, int act, float alpha, const float *bias, float *out, int ldo, H16 h = H16{nullptr, nullptr}, int ldh = 0) {
    GemmEpilogue e;
    memset(&e, 0, sizeof(e));
    e.mode = mode; e.act = act; e.alpha = alpha; e.bias = bias; e.out = out; e.ldo = ldo; e.out_hi = h.hi; e.out_lo = h.lo; e.ldh = ldh;
    return e;
}

static constexpr int STREAM_CONV_MAX = 48;               // k - 1 + q rows held in registers by stream_conv_kernel

// Device memory of a stream group belongs to the group (plain allocations, freed at close), not to the model's slabs.
static void *stream_alloc(StreamState &st, size_t bytes) {
    void *p = nullptr;
    if (cudaMalloc(&p, bytes ? bytes : 16) != cudaSuccess) { cudaGetLastError(); set_error("cudaMalloc(%zu) failed", bytes); return nullptr; }
    st.owned.push_back(p);
    return p;
}

int Model::stream_open(StreamState &st, int S, int left, int right) {
    if (!causal) { set_error("stream_open: cache-aware streaming needs a causal (Nemotron-style) encoder"); return -1; }
    if (S <= 0 || left < 0 || right < 0) { set_error("stream_open: bad argument"); return -1; }
    if (left > 0 && right + 1 > left) { set_error("stream_open: chunk of %d frames exceeds the left context %d", right + 1, left); return -1; }
    if (conv_k - 1 + right + 1 > STREAM_CONV_MAX) { set_error("stream_open: conv kernel %d with chunks of %d frames is too long", conv_k, right + 1); return -1; }
    for (const EncLayer &L : layers) if (L.cnorm_scale) { set_error("stream_open: streaming needs the LayerNorm conv norm"); return -1; }
    st = StreamState();
    st.S = S; st.left = left; st.right = right; st.q = right + 1;
    st.few_rows = S * st.q <= 128;
    if (st.few_rows) {
        const size_t rows = (size_t)S * (st.q + 2);
        st.ln_count = (int *)stream_alloc(st, rows * sizeof(int));
        if (!st.ln_count) return -1;
        MB_CUDA(cudaMemsetAsync(st.ln_count, 0, rows * sizeof(int), stream));
    }
    const int C = channels;
    int F = cfg.n_mels;
    for (int s = 0; s < 3; s++) {
        const size_t n = (size_t)S * F * (s == 0 ? 1 : C);
        st.ss_cache[s] = (float *)stream_alloc(st, n * sizeof(float));
        if (!st.ss_cache[s]) return -1;
        MB_CUDA(cudaMemsetAsync(st.ss_cache[s], 0, n * sizeof(float), stream));
        F = F / 2 + 1;
    }
    const size_t kv = (size_t)n_layers * S * (left > 0 ? left : 1) * d_model, cv = (size_t)n_layers * S * (conv_k - 1) * d_model;
    st.k_cache = (__half *)stream_alloc(st, kv * sizeof(__half));
    st.v_cache = (__half *)stream_alloc(st, kv * sizeof(__half));
    st.conv_cache = (float *)stream_alloc(st, cv * sizeof(float));
    if (!st.k_cache || !st.v_cache || !st.conv_cache) return -1;
    st.d_start = (int *)stream_alloc(st, sizeof(int));
    if (!st.d_start) return -1;
    if (left > 0) {
        st.rk_cache = (__half *)stream_alloc(st, (size_t)n_layers * (2 * (size_t)(left + st.q) - 1) * d_model * sizeof(__half));
        if (!st.rk_cache) return -1;
    }
    MB_CUDA(cudaMemsetAsync(st.d_start, 0, sizeof(int), stream));
    MB_CUDA(cudaMemsetAsync(st.k_cache, 0, kv * sizeof(__half), stream));
    MB_CUDA(cudaMemsetAsync(st.v_cache, 0, kv * sizeof(__half), stream));
    MB_CUDA(cudaMemsetAsync(st.conv_cache, 0, cv * sizeof(float), stream));
    MB_CUDA(cudaStreamSynchronize(stream));
    return 0;
}

void Model::stream_close(StreamState &st) {
    if (st.exec) cudaGraphExecDestroy(st.exec);
    if (st.graph) cudaGraphDestroy(st.graph);
    for (void *p : st.owned) cudaFree(p);
    st = StreamState();
}

size_t Model::stream_bytes(const StreamState &st, int n_mel) const {
    const size_t S = st.S, C = channels, d = d_model, Q = st.q + 2, M = S * Q, P = 2 * ((size_t)st.left + Q) - 1;
    const size_t T1 = n_mel / 2 + 2, F1 = cfg.n_mels / 2 + 2;
    return S * T1 * F1 * C * 4 * 4 + M * (d * 44 + (size_t)ffn_dim * 4) + P * d * 8 + (4 << 20);
}

// In steady state (caches full, full-size chunk, same input / output / workspace addresses as last time, no
// profiling spans wanted) the few hundred launches of a step are replayed from one captured graph: nothing the host
// passes changes from step to step any more — the ring offset lives in device memory.
int Model::stream_step(StreamState &st, const float *mel, int n_mel, int is_last, float *out) {
    const bool steady = !st.first && !is_last && st.left > 0 && st.valid == st.left && n_mel == stream_need(st) && !prof_on;
    if (!steady) return stream_step_eager(st, mel, n_mel, is_last, out);
    const bool same = st.g_mel == mel && st.g_out == out && st.g_base == ws.base && st.g_mark == ws.off;
    if (st.exec && same) {
        if (cudaGraphLaunch(st.exec, stream) != cudaSuccess) { set_error("stream_step: graph launch failed"); return -1; }
        note_launch(st.g_launches);
        return st.g_q;
    }
    if (st.steady_runs++ == 0 || (st.exec && !same)) {       // first steady step eagerly (launch attributes), or other buffers: re-capture next time
        if (st.exec) { cudaGraphExecDestroy(st.exec); cudaGraphDestroy(st.graph); st.exec = nullptr; st.graph = nullptr; }
        return stream_step_eager(st, mel, n_mel, is_last, out);
    }
    const long long before = launch_count(false);
    if (cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { cudaGetLastError(); return stream_step_eager(st, mel, n_mel, is_last, out); }
    const size_t mark = ws.off;
    const int q = stream_step_eager(st, mel, n_mel, is_last, out);
    cudaGraph_t g = nullptr;
    const cudaError_t e = cudaStreamEndCapture(stream, &g);
    const int recorded = (int)(launch_count(false) - before);
    note_launch(-recorded);                                  // recorded, not launched
    if (q < 0 || e != cudaSuccess || !g || cudaGraphInstantiate(&st.exec, g, 0) != cudaSuccess) {
        if (g) cudaGraphDestroy(g);
        st.exec = nullptr;
        cudaGetLastError();
        return q < 0 ? -1 : stream_step_eager(st, mel, n_mel, is_last, out);
    }
    st.graph = g; st.g_mel = mel; st.g_out = out; st.g_base = ws.base; st.g_mark = mark; st.g_launches = recorded; st.g_q = q;
    if (cudaGraphLaunch(st.exec, stream) != cudaSuccess) { set_error("stream_step: graph launch failed"); return -1; }
    note_launch(recorded);
    return q;
}

int Model::stream_step_eager(StreamState &st, const float *mel, int n_mel, int is_last, float *out) {
    const int S = st.S, C = channels, d = d_model, F = ffn_dim, H = n_heads, dk = d_head;
    if (n_mel <= 0) { set_error("stream_step: empty chunk"); return -1; }
    const int lp = st.first ? 2 : 1, rp = is_last ? 1 : 0;
    // ---- subsampling on the chunk (src/subsampling.c:320-370)
    const int F0 = cfg.n_mels, F1 = F0 / 2 + 1, F2 = F1 / 2 + 1, F3 = F2 / 2 + 1;
    auto stage_len = [&](int T) { return T + lp + rp >= 3 ? (T + lp + rp - 3) / 2 + 1 : 0; };
    const int T1 = stage_len(n_mel), T2 = T1 > 0 ? stage_len(T1) : 0, T3 = T2 > 0 ? stage_len(T2) : 0;
    if (T1 <= 0 || T2 <= 0 || T3 <= 0) { set_error("stream_step: a chunk of %d mel frames yields no encoder frame", n_mel); return -1; }
    const int Q = T3, M = S * Q;
    if (Q > st.q + 2 || conv_k - 1 + Q > STREAM_CONV_MAX || (st.left > 0 && Q > st.left)) { set_error("stream_step: chunk of %d encoder frames is too long", Q); return -1; }
    const size_t mark = ws.off;
    float *a0 = ws.get<float>((size_t)S * T1 * F1 * C);
    H16 p1 = ws.planes((size_t)S * T2 * F2 * C);
    float *a1 = ws.get<float>((size_t)S * T2 * F2 * C);
    H16 p2 = ws.planes((size_t)S * T3 * F3 * C), flat = ws.planes((size_t)S * T3 * F3 * C);
    float *x = ws.get<float>((size_t)M * d);
    if (!a0 || !p1.lo || !a1 || !p2.lo || !flat.lo || !x) return -1;
    const int TPB = 256;
    {
        const size_t n0 = (size_t)S * T1 * F1 * C, n1 = (size_t)S * T2 * F2 * C, n2 = (size_t)S * T3 * F3 * C;
        ss_stream_stage0_kernel<<<(unsigned)cdiv(n0, TPB), TPB, 0, stream>>>(mel, st.ss_cache[0], conv_in_w, conv_in_b, a0, S, n_mel, F0, C, T1, F1, lp);
        ss_stream_cache_kernel<<<(unsigned)cdiv((size_t)S * F0, TPB), TPB, 0, stream>>>(mel, st.ss_cache[0], S, n_mel, F0);
        ss_stream_dw_kernel<<<(unsigned)cdiv(n1, TPB), TPB, 0, stream>>>(a0, st.ss_cache[1], dw_w[0], dw_b[0], p1, S, T1, F1, C, T2, F2, lp);
        ss_stream_cache_kernel<<<(unsigned)cdiv((size_t)S * F1 * C, TPB), TPB, 0, stream>>>(a0, st.ss_cache[1], S, T1, F1 * C);
        MB_CUDA(cudaGetLastError());
        if (gemm(p1, C, pw[0], st_epi(OUT_F32, ACT_RELU, 1.f, pw[0].bias, a1, C), S * T2 * F2)) return -1;
        ss_stream_dw_kernel<<<(unsigned)cdiv(n2, TPB), TPB, 0, stream>>>(a1, st.ss_cache[2], dw_w[1], dw_b[1], p2, S, T2, F2, C, T3, F3, lp);
        ss_stream_cache_kernel<<<(unsigned)cdiv((size_t)S * F2 * C, TPB), TPB, 0, stream>>>(a1, st.ss_cache[2], S, T2, F2 * C);
        MB_CUDA(cudaGetLastError());
        if (gemm(p2, C, pw[1], st_epi(OUT_H16, ACT_RELU, 1.f, pw[1].bias, nullptr, 0, flat, C), S * T3 * F3)) return -1;
        // flat is [S*Q, F3*C]: the linear's columns were permuted to this order at load. No xscale here, as in the reference's step.
        if (gemm(flat, F3 * C, ss_lin, st_epi(OUT_F32, ACT_NONE, 1.f, ss_lin.bias, x, d), M, st.few_rows)) return -1;
        note_launch(6);
    }
    // ---- layers (src/encoder.c:826-866)
    const int valid = st.valid, K = valid + Q, P = 2 * K - 1;
    H16 hA = ws.planes((size_t)M * d), hC = ws.planes((size_t)M * d), hF = ws.planes((size_t)M * F);
    float *qbuf = ws.get<float>((size_t)M * d), *h2 = ws.get<float>((size_t)M * 2 * d), *cbuf = ws.get<float>((size_t)M * d);
    H16 kn = ws.planes((size_t)M * d, false), vn = ws.planes((size_t)M * d, false);
    H16 pe = ws.planes((size_t)P * d), rk = ws.planes((size_t)P * d, false);
    if (!hA.lo || !hC.lo || !hF.lo || !qbuf || !h2 || !cbuf || !kn.hi || !vn.hi || !pe.lo || !rk.hi) return -1;
    // full caches and a full-size chunk: the key count of every later step, whose rk the group keeps
    const bool rk_keep = st.rk_cache && valid == st.left && Q == st.q;
    const bool rk_have = rk_keep && st.rk_ready;
    if (!rk_have) {
        if (pos_emb(pe, K, d, stream)) return -1;
        note_launch();
    }
    const size_t attn_smem = ((size_t)K + 4 + (2 + STREAM_ATTN_WARPS) * (size_t)dk + 32) * sizeof(float);
    if (dk % 4) { set_error("stream_step: head width %d must be a multiple of 4", dk); return -1; }
    if (attn_smem > 200 * 1024) { set_error("stream_step: context too long for the attention kernel"); return -1; }
    static PerDevice attn_smem_set = {};
    int cur_dev = 0;
    if (attn_smem_set.below(attn_smem, &cur_dev)) {
        MB_CUDA(cudaFuncSetAttribute(stream_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)attn_smem));
        attn_smem_set.record(cur_dev, attn_smem);
    }
    const H16 none{nullptr, nullptr};
    const int leftn = st.left > 0 ? st.left : 1;
    // In a few-row group the LayerNorm that follows a residual update runs inside the contraction that makes it
    const bool tail = st.few_rows && st.ln_count && gemm_skinny_ln_width(d);
    auto resid = [&](float alpha, const float *bias, const float *nw, const float *nb) {
        GemmEpilogue e = st_epi(OUT_RESID, ACT_NONE, alpha, bias, x, d);
        if (tail) { e.ln_w = nw; e.ln_b = nb; e.ln_hi = hA.hi; e.ln_lo = hA.lo; e.ln_count = st.ln_count; }
        return e;
    };
    for (int li = 0; li < n_layers; li++) {
        const EncLayer &L = layers[li];
        __half *kc = st.k_cache + (size_t)li * S * leftn * d, *vc = st.v_cache + (size_t)li * S * leftn * d;
        float *cc = st.conv_cache + (size_t)li * S * (conv_k - 1) * d;
        // (with the tails, a layer's opening LayerNorm comes out of the contraction that closes the layer before it)
        if ((!tail || li == 0) && layer_norm(x, L.ln_ff1_w, L.ln_ff1_b, nullptr, hA, M, d, ACT_NONE, stream, true)) return -1;
        if (gemm(hA, d, L.ff1_w1, st_epi(OUT_H16, ACT_SILU, 1.f, L.ff1_w1.bias, nullptr, 0, hF, F), M, st.few_rows)) return -1;
        if (gemm(hF, F, L.ff1_w2, resid(0.5f, L.ff1_w2.bias, L.ln_att_w, L.ln_att_b), M, st.few_rows)) return -1;
        if (!tail && layer_norm(x, L.ln_att_w, L.ln_att_b, nullptr, hA, M, d, ACT_NONE, stream, true)) return -1;
        if (gemm(hA, d, L.q_w, st_epi(OUT_F32, ACT_NONE, 1.f, L.q_w.bias, qbuf, d), M, st.few_rows)) return -1;
        if (gemm(hA, d, L.k_w, st_epi(OUT_H16, ACT_NONE, 1.f, L.k_w.bias, nullptr, 0, kn, d), M, st.few_rows)) return -1;
        if (gemm(hA, d, L.v_w, st_epi(OUT_H16, ACT_NONE, 1.f, L.v_w.bias, nullptr, 0, vn, d), M, st.few_rows)) return -1;
        __half *rk_l = rk_keep ? st.rk_cache + (size_t)li * P * d : rk.hi;
        if (!rk_have && gemm(pe, d, L.relk, st_epi(OUT_H16, ACT_NONE, 1.f, nullptr, nullptr, 0, H16{rk_l, nullptr}, d), P)) return -1;
        MB_CUDA(launch_kernel(stream_attn_kernel, dim3(H, S), dim3(STREAM_ATTN_WARPS * 32), attn_smem, stream, true, 1, (const float *)qbuf, (const __half *)kn.hi, (const __half *)vn.hi,
                              kc, vc, (const __half *)rk_l, L.bias_u, L.bias_v, hC, Q, valid, (const int *)st.d_start, leftn, d, dk, st.left > 0 ? 1 : 0));
        if (gemm(hC, d, L.o_w, resid(1.f, L.o_w.bias, L.ln_conv_w, L.ln_conv_b), M, st.few_rows)) return -1;
        if (!tail && layer_norm(x, L.ln_conv_w, L.ln_conv_b, nullptr, hA, M, d, ACT_NONE, stream, true)) return -1;
        if (gemm(hA, d, L.pw1_w, st_epi(OUT_F32, ACT_NONE, 1.f, L.pw1_w.bias, h2, 2 * d), M, st.few_rows)) return -1;
        MB_CUDA(launch_kernel(stream_conv_kernel<STREAM_CONV_MAX>, dim3((unsigned)cdiv((size_t)S * d, 128)), dim3(128), 0, stream, true, 1, (const float *)h2, L.dw_w, cc, cbuf,
                              S, Q, d, conv_k));
        if (layer_norm(cbuf, L.cnorm_w, L.cnorm_b, nullptr, hC, M, d, ACT_SILU, stream, true)) return -1;
        if (gemm(hC, d, L.pw2_w, resid(1.f, L.pw2_w.bias, L.ln_ff2_w, L.ln_ff2_b), M, st.few_rows)) return -1;
        if (!tail && layer_norm(x, L.ln_ff2_w, L.ln_ff2_b, nullptr, hA, M, d, ACT_NONE, stream, true)) return -1;
        if (gemm(hA, d, L.ff2_w1, st_epi(OUT_H16, ACT_SILU, 1.f, L.ff2_w1.bias, nullptr, 0, hF, F), M, st.few_rows)) return -1;
        {
            GemmEpilogue e = st_epi(OUT_RESID, ACT_NONE, 0.5f, L.ff2_w2.bias, x, d);
            if (tail) {                    // x = LN_out(x) in place, then the next layer's LN_ff1 of it into hA
                e.ln_w = L.ln_out_w; e.ln_b = L.ln_out_b; e.ln_count = st.ln_count;
                if (li + 1 < n_layers) { e.ln2_w = layers[li + 1].ln_ff1_w; e.ln2_b = layers[li + 1].ln_ff1_b; e.ln_hi = hA.hi; e.ln_lo = hA.lo; }
            }
            if (gemm(hF, F, L.ff2_w2, e, M, st.few_rows)) return -1;
        }
        if (!tail && layer_norm(x, L.ln_out_w, L.ln_out_b, x, none, M, d, ACT_NONE, stream, true)) return -1;
        note_launch((tail ? (li == 0 ? 4 : 3) : 8));
    }
    {   // rows are stream-major: Q rows per stream, each stream with its own prompt id
        const std::vector<int> post_lens((size_t)st.S, Q);
        if (encoder_post(x, post_lens, st.prompt_ids.empty() ? nullptr : st.prompt_ids.data(), out)) return -1;
    }
    // cache bookkeeping of the host side (src/encoder.c:868 and the ring's start)
    if (st.left > 0) {
        const int total = valid + Q;
        stream_advance_kernel<<<1, 1, 0, stream>>>(st.d_start, valid, Q, st.left);
        MB_CUDA(cudaGetLastError());
        note_launch();
        st.valid = total < st.left ? total : st.left;
    }
    if (rk_keep) st.rk_ready = true;
    st.first = 0;
    ws.off = mark;
    return Q;
}

// ---- incremental log-mel for the streams of a group (mynah_asr_mel_stream_feed / _finish, src/features.c:229-272):
// frame t is ready once the signal covers t*hop + n_fft/2; finish emits the remaining valid frames with
// zeros to the right. Same frame kernel as the offline front end, so ready frames are bit-identical to it.
static constexpr int MEL_CAP = 1 << 16;                  // samples of signal tail kept per stream

int Model::stream_mel_feed(StreamState &st, const float *audio, int n, int finish, float *out, int cap_frames) {
    if (!has_mel) { set_error("stream_mel_feed: mel filterbank not set"); return -1; }
    if (n < 0 || (n > 0 && !audio) || cap_frames < 0) { set_error("stream_mel_feed: bad argument"); return -1; }
    const int S = st.S, hop = cfg.hop_length, nf = cfg.n_fft, nm = cfg.n_mels;
    if (!st.mel_buf[0]) {
        for (int i = 0; i < 2; i++) {
            st.mel_buf[i] = (float *)stream_alloc(st, (size_t)S * MEL_CAP * sizeof(float));
            if (!st.mel_buf[i]) return -1;
        }
    }
    // drop what no later frame needs (one sample more than the window: the pre-emphasis reads s - 1)
    const long long min_keep = st.mel_next * hop - nf / 2 - 1;
    if (min_keep > st.mel_base) {
        const long long tail = st.mel_total - min_keep;
        if (tail > 0)
            MB_CUDA(cudaMemcpy2DAsync(st.mel_buf[st.mel_cur ^ 1], (size_t)MEL_CAP * 4, st.mel_buf[st.mel_cur] + (min_keep - st.mel_base),
                                      (size_t)MEL_CAP * 4, (size_t)tail * 4, S, cudaMemcpyDeviceToDevice, stream));
        st.mel_cur ^= 1;
        st.mel_base = min_keep;
    }
    if (st.mel_total - st.mel_base + n > MEL_CAP) { set_error("stream_mel_feed: %d samples at once exceed the %d-sample window", n, MEL_CAP); return -1; }
    if (n > 0) {
        MB_CUDA(cudaMemcpy2DAsync(st.mel_buf[st.mel_cur] + (st.mel_total - st.mel_base), (size_t)MEL_CAP * 4, audio, (size_t)n * 4,
                                  (size_t)n * 4, S, cudaMemcpyHostToDevice, stream));
        st.mel_total += n;
    }
    long long t_end = st.mel_total >= nf / 2 ? (st.mel_total - nf / 2) / hop + 1 : 0;
    if (finish) { const long long valid = st.mel_total / hop; if (valid > t_end) t_end = valid; else if (valid < t_end) t_end = valid > st.mel_next ? valid : st.mel_next; }
    long long n_new = t_end - st.mel_next;
    if (n_new > cap_frames) n_new = cap_frames;
    if (n_new <= 0) { MB_CUDA(cudaStreamSynchronize(stream)); return 0; }
    const size_t mark = ws.off;
    float *fd = ws.get<float>((size_t)S * n_new * nm);
    if (!fd) return -1;
    MelCfg c{nm, nf, cfg.win_length, hop, cfg.preemphasis, cfg.log_zero_guard, 0};
    if (log_mel_stream_device(c, st.mel_buf[st.mel_cur], st.mel_base, st.mel_total, MEL_CAP, S, mel_fb, mel_lo, mel_hi, mel_win, mel_tw, fd,
                              (long long)n_new * nm, (int)st.mel_next, (int)n_new, stream)) return -1;
    note_launch();
    MB_CUDA(cudaMemcpyAsync(out, fd, (size_t)S * n_new * nm * sizeof(float), cudaMemcpyDeviceToHost, stream));
    MB_CUDA(cudaStreamSynchronize(stream));
    st.mel_next += n_new;
    ws.off = mark;
    return (int)n_new;
}

// ---- per-chunk transducer decoding with carried state (src/decoder.c:112-265 called chunk by chunk, as
// stream_flush_chunk does, src/mynah_asr.c:784-822). Streams are decoded DEC_MAX_B at a time by the lock-step
// greedy kernel; every group keeps its LSTM state, pred-net output and last token on the device.
int Model::stream_decode(StreamState &st, const float *enc_dev, int q, std::vector<std::vector<int>> &tokens,
                         std::vector<std::vector<int>> &frames) {
    const int S = st.S, H = pred_hidden, L = pred_layers;
    tokens.assign(S, {}); frames.assign(S, {});
    if (!has_dec) { set_error("stream_decode: model has no transducer decoder"); return -1; }
    if (q <= 0) return 0;
    const int ngroups = cdiv(S, DEC_MAX_B);
    const size_t fblock = (size_t)(3 * L + 1) * DEC_MAX_B * H, iblock = DEC_MAX_B + 8;
    if (!st.dec_f) {
        st.dec_f = (float *)stream_alloc(st, ngroups * fblock * sizeof(float));
        st.dec_i = (int *)stream_alloc(st, ngroups * iblock * sizeof(int));
        if (!st.dec_f || !st.dec_i) return -1;
        MB_CUDA(cudaMemsetAsync(st.dec_f, 0, ngroups * fblock * sizeof(float), stream));
        MB_CUDA(cudaMemsetAsync(st.dec_i, 0, ngroups * iblock * sizeof(int), stream));
    }
    const int nw = (vocab + cfg.n_durations + 15) / 16, cap = q * cfg.max_symbols;
    const size_t mark = ws.off;
    struct Out { int *n_out, *tokens, *frames; int B; };
    std::vector<Out> outs(ngroups);
    std::vector<int> hm(2 * (size_t)S);                      // per group: B frame offsets, then B lengths
    for (int gi = 0, o = 0; gi < ngroups; gi++) {
        const int g0 = gi * DEC_MAX_B, B = S - g0 < DEC_MAX_B ? S - g0 : DEC_MAX_B;
        for (int b = 0; b < B; b++) { hm[o + b] = (g0 + b) * q; hm[o + B + b] = q; }
        o += 2 * B;
    }
    // every group's integer block (flags, per-utterance state, candidates, emitted tokens and frames) sits in one
    // region so that a single copy brings all results back
    const size_t ipg = 8 * (size_t)DEC_MAX_B + 2 * (size_t)DEC_MAX_B * nw + 2 * (size_t)DEC_MAX_B * cap + 16;
    int *iz_all = ws.get<int>(ipg * ngroups);
    if (!iz_all) return -1;
    MB_CUDA(cudaMemsetAsync(iz_all, 0, ipg * ngroups * sizeof(int), stream));
    int *hm_dev = ws.get<int>(hm.size());
    if (!hm_dev) return -1;
    MB_CUDA(cudaMemcpyAsync(hm_dev, hm.data(), hm.size() * sizeof(int), cudaMemcpyHostToDevice, stream));
    MB_CUDA(cudaStreamSynchronize(stream));          // hm is a stack-lifetime buffer
    const int lanes = lanes_begin(ngroups);
    if (lanes < 1) return -1;
    const int lane_blocks = lanes > 1 ? (device_sm_count() / lanes > DEC_MAX_B ? device_sm_count() / lanes : DEC_MAX_B) : 0;
    for (int gi = 0; gi < ngroups; gi++) {
        const int g0 = gi * DEC_MAX_B, B = S - g0 < DEC_MAX_B ? S - g0 : DEC_MAX_B;
        const size_t nstate = (size_t)L * B * H;
        float *fs = st.dec_f + gi * fblock;
        int *is = st.dec_i + gi * iblock;
        float *cand = ws.get<float>(2 * (size_t)B * nw + (size_t)DEC_MAX_B * H);
        int *iz = iz_all + gi * ipg;
        if (!cand) return -1;
        GreedyDev p;
        memset(&p, 0, sizeof(p));
        p.emb = emb; p.head_b = head_b; p.proj_b = proj_b;
        p.emb_hi = emb_planes.hi; p.emb_lo = emb_planes.lo;
        p.head_hi = head.hi; p.head_lo = head.lo; p.proj_hi = dec_proj.hi; p.proj_lo = dec_proj.lo;
        for (int l = 0; l < L; l++) { p.wcat_hi[l] = wcat[l].hi; p.wcat_lo[l] = wcat[l].lo; p.b_ih[l] = b_ih[l]; p.b_hh[l] = b_hh[l]; }
        p.V = vocab; p.ND = cfg.n_durations; p.H = H; p.L = L; p.blank = cfg.blank_id; p.max_symbols = cfg.max_symbols;
        for (int i = 0; i < cfg.n_durations; i++) p.durations[i] = cfg.durations[i];
        p.B = B; p.enc = enc_dev;
        p.h[0] = fs; p.h[1] = fs + nstate; p.c = fs + 2 * nstate; p.g = fs + 3 * nstate;
        p.jx_hi = reinterpret_cast<__half *>(cand); p.jx_lo = p.jx_hi + (size_t)DEC_MAX_B * H;
        p.cand_v = cand + (size_t)DEC_MAX_B * H;
        int *qi = iz;
        p.flags = qi; qi += 16;
        p.t = qi; qi += B; p.emitted_here = qi; qi += B; p.n_out = qi; qi += B; p.emit = qi; qi += B;
        qi += 4 * B;
        p.cand_i = qi; qi += 2 * (size_t)B * nw;
        p.tokens = qi; qi += (size_t)B * cap; p.frames = qi;
        p.last_tok = is; p.par_state = is + DEC_MAX_B;
        p.cap = cap; p.enc_off = hm_dev + 2 * (size_t)g0; p.enc_len = hm_dev + 2 * (size_t)g0 + B;
        p.max_steps = q * (cfg.max_symbols + 1) + 8; p.init_state = st.dec_started ? 0 : 1;
        if (greedy_launch(p, lane_stream(lanes, gi), lane_blocks)) return -1;
        note_launch();
        outs[gi] = Out{p.n_out, p.tokens, p.frames, B};
    }
    if (lanes_join(lanes)) return -1;
    std::vector<int> hz(ipg * ngroups);
    MB_CUDA(cudaMemcpyAsync(hz.data(), iz_all, hz.size() * sizeof(int), cudaMemcpyDeviceToHost, stream));
    MB_CUDA(cudaStreamSynchronize(stream));
    for (int gi = 0; gi < ngroups; gi++) {
        const Out &o = outs[gi];
        const int *hn = hz.data() + (o.n_out - iz_all), *ht = hz.data() + (o.tokens - iz_all), *hf = hz.data() + (o.frames - iz_all);
        for (int b = 0; b < o.B; b++) {
            const int s = gi * DEC_MAX_B + b;
            tokens[s].assign(ht + (size_t)b * cap, ht + (size_t)b * cap + hn[b]);
            frames[s].resize(hn[b]);
            for (int i = 0; i < hn[b]; i++) frames[s][i] = (int)(st.t_abs + hf[(size_t)b * cap + i]);
        }
    }
    st.dec_started = 1;
    st.t_abs += q;
    ws.off = mark;
    return 0;
}

}  // namespace mb
