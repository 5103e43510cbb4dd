// Greedy AED decode (pre-LN transformer decoder with a self-attention KV cache and
// cross-attention over the projected encoder output): the device counterpart of
// mynah_asr_aed_decode (src/decoder_aed.c:139-232) for B utterances in lock step.
// All utterances sit at the same position p; each row of every kernel depends only on its own
// utterance, so a batch decodes to the same bits as each utterance alone.
// The linears run on the tcgen05 contractions (the cross K/V projections over all frames on the many-row kernel, a
// position's linears on the few-row kernel, gemm_skinny.cu); this file holds what sits between them: the two
// single-query attentions and the turn from one position to the next (selection, embedding, opening LayerNorms).
#include "model.h"
#include "ln_row.cuh"

namespace mb {

// The position p lives in device memory (pd) so that one captured CUDA graph serves every position.
// x[b] = emb[cur[b]] + pos[p]   (src/decoder_aed.c:183-184; the LayerNorm follows as its own launch)
__global__ void aed_embed_kernel(const float *__restrict__ emb, const float *__restrict__ pos, const int *__restrict__ cur,
                                 const int *__restrict__ pd, float *__restrict__ x, int D) {
    chain_trigger();
    chain_wait();
    const int b = blockIdx.x, p = *pd;
    const float *e = emb + (size_t)cur[b] * D, *pe = pos + (size_t)p * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) x[(size_t)b * D + i] = e[i] + pe[i];
}

// Block-wide max / sum over `n` values held in shared memory (blockDim.x <= 1024).
__device__ __forceinline__ float block_reduce(float v, float *red, bool is_max) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = is_max ? warp_max(v) : warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = is_max ? -INFINITY : 0.f;
    for (int i = 0; i < nw; i++) r = is_max ? fmaxf(r, red[i]) : r + red[i];
    __syncthreads();
    return r;
}

// Causal self-attention of one new position (src/decoder_aed.c:191-196 with attend, :117-131):
// appends this step's k, v to the cache and attends over positions 0..p. Grid (H, B), SELF_WARPS warps.
// qkv [B, 3D] = (q | k | v) with biases already added; cache [B, max_len, D] each. dk is a multiple of 4.
// Scores: a warp takes a key at a time, a lane four consecutive elements of it (one 16-byte load; four keys in
// flight). Context: warp w sums the keys j = w, w + SELF_WARPS, ... for the lane's four columns; the partial sums are
// added in warp order.
static constexpr int SELF_WARPS = 16;
__global__ void __launch_bounds__(SELF_WARPS * 32)
aed_self_attn_kernel(const float *__restrict__ qkv, float *__restrict__ ck, float *__restrict__ cv,
                     const int *__restrict__ pd, int pd_stride, int max_len, int D, int dk, H16 out) {
    extern __shared__ float sm[];
    chain_trigger();
    chain_wait();
    const int p = pd[blockIdx.y * pd_stride];         // one position for all (stride 0) or a copy per utterance
    float *sc = sm, *q = sm + ((max_len + 3) & ~3), *red = q + dk, *part = red + 32;     // part: [SELF_WARPS][dk]
    const int h = blockIdx.x, b = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float *row = qkv + (size_t)b * 3 * D + h * dk;
    float *K = ck + (size_t)b * max_len * D + h * dk, *V = cv + (size_t)b * max_len * D + h * dk;
    for (int i = threadIdx.x; i < dk; i += blockDim.x) {
        q[i] = row[i];
        K[(size_t)p * D + i] = row[D + i];
        V[(size_t)p * D + i] = row[2 * D + i];
    }
    __syncthreads();
    const float scale = 1.0f / sqrtf((float)dk);
    for (int j0 = warp * 4; j0 <= p; j0 += 4 * SELF_WARPS) {
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        for (int i0 = lane * 4; i0 < dk; i0 += 128) {
            float4 k[4];
#pragma unroll
            for (int u = 0; u < 4; u++) k[u] = *reinterpret_cast<const float4 *>(K + (size_t)(j0 + u <= p ? j0 + u : p) * D + i0);
            const float4 qq = *reinterpret_cast<const float4 *>(q + i0);
#pragma unroll
            for (int u = 0; u < 4; u++) s[u] = fmaf(qq.x, k[u].x, fmaf(qq.y, k[u].y, fmaf(qq.z, k[u].z, fmaf(qq.w, k[u].w, s[u]))));
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const float t = warp_sum(s[u]);
            if (lane == 0 && j0 + u <= p) sc[j0 + u] = t * scale;
        }
    }
    __syncthreads();
    float m = -INFINITY;
    for (int j = threadIdx.x; j <= p; j += blockDim.x) m = fmaxf(m, sc[j]);
    m = block_reduce(m, red, true);
    float sum = 0.f;
    for (int j = threadIdx.x; j <= p; j += blockDim.x) { const float e = expf(sc[j] - m); sc[j] = e; sum += e; }
    sum = block_reduce(sum, red, false);
    const float inv = 1.0f / sum;
    for (int c0 = lane * 4; c0 < dk; c0 += 128) {
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        int j = warp;
        for (; j + 3 * SELF_WARPS <= p; j += 4 * SELF_WARPS) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) v[u] = *reinterpret_cast<const float4 *>(V + (size_t)(j + SELF_WARPS * u) * D + c0);
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const float w = sc[j + SELF_WARPS * u] * inv;
                o.x = fmaf(w, v[u].x, o.x); o.y = fmaf(w, v[u].y, o.y); o.z = fmaf(w, v[u].z, o.z); o.w = fmaf(w, v[u].w, o.w);
            }
        }
        for (; j <= p; j += SELF_WARPS) {
            const float4 v = *reinterpret_cast<const float4 *>(V + (size_t)j * D + c0);
            const float w = sc[j] * inv;
            o.x = fmaf(w, v.x, o.x); o.y = fmaf(w, v.y, o.y); o.z = fmaf(w, v.z, o.z); o.w = fmaf(w, v.w, o.w);
        }
        *reinterpret_cast<float4 *>(part + warp * dk + c0) = o;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < dk; i += blockDim.x) {
        float t = part[i];
        for (int w = 1; w < SELF_WARPS; w++) t += part[w * dk + i];
        __half hi, lo;
        split_h16(t, hi, lo);
        out.hi[(size_t)b * D + h * dk + i] = hi;
        if (out.lo) out.lo[(size_t)b * D + h * dk + i] = lo;
    }
}

// The cross K / V of a layer leave their contraction as planes [sum T, 2D] = (K | V) per frame; a (head, utterance) block
// of the cross-attention would read 2 dk bytes out of every 4 D. Once per decode they are regrouped so that the T_b rows
// of one (utterance, head) follow each other: K at ((off_b H + h T_b + j) dk), V the same v_off halves further on.
// Grid (H, B); 16-byte copies.
__global__ void aed_kv_by_head_kernel(const __half *__restrict__ src, __half *__restrict__ dst, size_t v_off, const int *__restrict__ enc_off,
                                      const int *__restrict__ enc_len, int D, int dk) {
    const int h = blockIdx.x, b = blockIdx.y, T = enc_len[b], c8 = dk >> 3;
    const size_t r0 = (size_t)enc_off[b], kb = (r0 * gridDim.x + (size_t)h * T) * dk;
    for (int idx = threadIdx.x; idx < T * c8; idx += blockDim.x) {
        const int j = idx / c8, c = idx - j * c8;
        const uint4 *s = reinterpret_cast<const uint4 *>(src + (r0 + j) * 2 * (size_t)D + h * dk) + c;
        reinterpret_cast<uint4 *>(dst + kb + (size_t)j * dk)[c] = s[0];
        reinterpret_cast<uint4 *>(dst + kb + v_off + (size_t)j * dk)[c] = *reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(s) + D);
    }
}

// Cross-attention of one query per utterance over its T_b projected encoder frames
// (src/decoder_aed.c:199-202). Grid (H, B), 512 threads. kv: the layer's K and V planes grouped by (utterance, head),
// fp16 hi (+ lo * 2^-11 when present). q [B, D] f32 with bias. dk is a multiple of 4.
// Scores: a warp takes four key rows at a time, a lane four consecutive elements of each (8-byte loads,
// eight in flight per lane). Context: a warp owns every sixteenth key, a lane four adjacent columns.
__device__ __forceinline__ float4 ld_h4(const __half *hi, const __half *lo, size_t o) {
    const uint2 a = *reinterpret_cast<const uint2 *>(hi + o);
    const float2 a0 = __half22float2(*reinterpret_cast<const __half2 *>(&a.x)), a1 = __half22float2(*reinterpret_cast<const __half2 *>(&a.y));
    float4 r = make_float4(a0.x, a0.y, a1.x, a1.y);
    if (lo) {
        const uint2 b = *reinterpret_cast<const uint2 *>(lo + o);
        const float2 b0 = __half22float2(*reinterpret_cast<const __half2 *>(&b.x)), b1 = __half22float2(*reinterpret_cast<const __half2 *>(&b.y));
        r.x = fmaf(b0.x, H16_LO_INV, r.x); r.y = fmaf(b0.y, H16_LO_INV, r.y); r.z = fmaf(b1.x, H16_LO_INV, r.z); r.w = fmaf(b1.y, H16_LO_INV, r.w);
    }
    return r;
}
static constexpr int CROSS_WARPS = 16;
static constexpr int CROSS_KU = 8;              // key rows a warp has in flight
__global__ void __launch_bounds__(CROSS_WARPS * 32)
aed_cross_attn_kernel(const float *__restrict__ qm, const __half *__restrict__ kv_hi, const __half *__restrict__ kv_lo, size_t v_off,
                      const int *__restrict__ enc_off, const int *__restrict__ enc_len, int max_T, int D, int dk, H16 out) {
    extern __shared__ float sm[];
    chain_trigger();
    chain_wait();
    float *sc = sm, *q = sm + ((max_T + 3) & ~3), *red = q + dk, *part = red + 32;     // part: [CROSS_WARPS][dk] partial outputs
    const int h = blockIdx.x, b = blockIdx.y;
    const int T = enc_len[b], lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // K rows of (utterance b, head h) lie one after the other (aed_kv_by_head_kernel), V rows likewise v_off halves further on
    const size_t kb = ((size_t)enc_off[b] * gridDim.x + (size_t)h * T) * dk, vb = kb + v_off;
    for (int i = threadIdx.x; i < dk; i += blockDim.x) q[i] = qm[(size_t)b * D + h * dk + i];
    __syncthreads();
    const float scale = 1.0f / sqrtf((float)dk);
    for (int j0 = warp * CROSS_KU; j0 < T; j0 += CROSS_KU * CROSS_WARPS) {
        float s[CROSS_KU];
#pragma unroll
        for (int u = 0; u < CROSS_KU; u++) s[u] = 0.f;
        for (int i0 = lane * 4; i0 < dk; i0 += 128) {
            float4 k[CROSS_KU];
#pragma unroll
            for (int u = 0; u < CROSS_KU; u++) {
                const int j = j0 + u < T ? j0 + u : T - 1;
                k[u] = ld_h4(kv_hi, kv_lo, kb + (size_t)j * dk + i0);
            }
            const float4 qq = *reinterpret_cast<const float4 *>(q + i0);
#pragma unroll
            for (int u = 0; u < CROSS_KU; u++) s[u] = fmaf(qq.x, k[u].x, fmaf(qq.y, k[u].y, fmaf(qq.z, k[u].z, fmaf(qq.w, k[u].w, s[u]))));
        }
#pragma unroll
        for (int u = 0; u < CROSS_KU; u++) {
            const float t = warp_sum(s[u]);
            if (lane == 0 && j0 + u < T) sc[j0 + u] = t * scale;
        }
    }
    __syncthreads();
    float m = -INFINITY;
    for (int j = threadIdx.x; j < T; j += blockDim.x) m = fmaxf(m, sc[j]);
    m = block_reduce(m, red, true);
    float sum = 0.f;
    for (int j = threadIdx.x; j < T; j += blockDim.x) { const float e = expf(sc[j] - m); sc[j] = e; sum += e; }
    sum = block_reduce(sum, red, false);
    const float inv = 1.0f / sum;
    // context: warp w sums the keys j = w, w + CROSS_WARPS, ... for the lane's four columns (8-byte loads of each plane,
    // CROSS_KU keys in flight); the partial sums are added in warp order
    for (int c0 = lane * 4; c0 < dk; c0 += 128) {
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        int j = warp;
        for (; j + (CROSS_KU - 1) * CROSS_WARPS < T; j += CROSS_KU * CROSS_WARPS) {
            float4 v[CROSS_KU];
#pragma unroll
            for (int u = 0; u < CROSS_KU; u++) v[u] = ld_h4(kv_hi, kv_lo, vb + (size_t)(j + CROSS_WARPS * u) * dk + c0);
#pragma unroll
            for (int u = 0; u < CROSS_KU; u++) {
                const float w = sc[j + CROSS_WARPS * u] * inv;
                o.x = fmaf(w, v[u].x, o.x); o.y = fmaf(w, v[u].y, o.y); o.z = fmaf(w, v[u].z, o.z); o.w = fmaf(w, v[u].w, o.w);
            }
        }
        for (; j < T; j += CROSS_WARPS) {
            const float4 v = ld_h4(kv_hi, kv_lo, vb + (size_t)j * dk + c0);
            const float w = sc[j] * inv;
            o.x = fmaf(w, v.x, o.x); o.y = fmaf(w, v.y, o.y); o.z = fmaf(w, v.z, o.z); o.w = fmaf(w, v.w, o.w);
        }
        *reinterpret_cast<float4 *>(part + warp * dk + c0) = o;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < dk; i += blockDim.x) {
        float t = part[i];
        for (int w = 1; w < CROSS_WARPS; w++) t += part[w * dk + i];
        __half hi, lo;
        split_h16(t, hi, lo);
        out.hi[(size_t)b * D + h * dk + i] = hi;
        if (out.lo) out.lo[(size_t)b * D + h * dk + i] = lo;
    }
}

// Greedy selection at position p (src/decoder_aed.c:211-223), then p += 1. One block.
// st: [cur | n_out | done | n_prompt | max_len | cap] x B, then n_done, p.
__global__ void aed_select_kernel(const int *__restrict__ best, int eos, int cap_stride, int B, int *st, const int *__restrict__ prompts,
                                  int max_prompt, int *__restrict__ tokens) {
    chain_trigger();
    chain_wait();
    const int b = threadIdx.x;
    int *cur = st, *n_out = st + B, *done = st + 2 * B, *n_prompt = st + 3 * B, *max_len = st + 4 * B, *n_done = st + 6 * B;
    const int p = st[6 * B + 1];
    __syncthreads();
    if (b == 0) st[6 * B + 1] = p + 1;
    if (b >= B) return;
    const int cap = st[5 * B + b];
    if (done[b]) return;
    bool fin = false;
    if (p + 1 < n_prompt[b]) {
        cur[b] = prompts[b * max_prompt + p + 1];
    } else {
        const int t = best[b];
        if (t == eos || n_out[b] >= cap) fin = true;
        else { tokens[(size_t)b * cap_stride + n_out[b]] = t; n_out[b]++; cur[b] = t; }
    }
    if (p + 1 >= max_len[b]) fin = true;
    if (fin) { done[b] = 1; atomicAdd(n_done, 1); }
}

// The turn from one position to the next in one launch, one block per utterance: greedy selection at position p
// (src/decoder_aed.c:211-223; the first maximum of the logits row, as argmax_kernel finds it), then the next position's
// input x[b] = emb[cur[b]] + pos[p + 1] (:183-184) with the embedding LayerNorm in place and the first layer's opening
// LayerNorm into the planes xn — the same row arithmetic as ln_reg_kernel (ln_row). first != 0: no selection, position 0.
// st: [cur | n_out | done | n_prompt | max_len | cap] x B, then n_done, (unused), .., then at 6B + 4 the position of
// every utterance (all equal; a copy each, so that no block reads what another one writes).
template <int NV>
__global__ void __launch_bounds__(256)
aed_next_kernel(const float *__restrict__ logits, int V, int eos, int cap_stride, int B, int *st, const int *__restrict__ prompts, int max_prompt,
                int *__restrict__ tokens, const float *__restrict__ emb, const float *__restrict__ pos, int max_seq,
                const float *__restrict__ ln1_w, const float *__restrict__ ln1_b, const float *__restrict__ ln2_w, const float *__restrict__ ln2_b,
                float *__restrict__ x, H16 xn, int first) {
    constexpr int D = NV * 128;
    __shared__ float sv[256];
    __shared__ int si[256];
    chain_trigger();
    chain_wait();
    const int b = blockIdx.x;
    int *cur = st, *n_out = st + B, *done = st + 2 * B, *n_prompt = st + 3 * B, *max_len = st + 4 * B, *n_done = st + 6 * B, *pos_b = st + 6 * B + 4;
    int p = pos_b[b];
    if (!first) {
        const float *row = logits + (size_t)b * V;
        float bv = -3.0e38f;
        int bi = 0x7fffffff;
        for (int k = threadIdx.x; k < V; k += 256) {
            const float v = row[k];
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
        if (threadIdx.x == 0) {
            if (!done[b]) {
                const int cap = st[5 * B + b];
                bool fin = false;
                if (p + 1 < n_prompt[b]) {
                    cur[b] = prompts[b * max_prompt + p + 1];
                } else {
                    const int t = si[0];
                    if (t == eos || n_out[b] >= cap) fin = true;
                    else { tokens[(size_t)b * cap_stride + n_out[b]] = t; n_out[b]++; cur[b] = t; }
                }
                if (p + 1 >= max_len[b]) fin = true;
                if (fin) { done[b] = 1; atomicAdd(n_done, 1); }
            }
            pos_b[b] = p + 1;
        }
        __syncthreads();                              // cur[b] is final for the threads below
        p += 1;
    }
    if (p >= max_seq) return;                         // beyond the position table: no further position is decoded
    const float *e = emb + (size_t)cur[b] * D, *pe = pos + (size_t)p * D;
    for (int i = threadIdx.x; i < D; i += 256) x[(size_t)b * D + i] = e[i] + pe[i];
    __syncthreads();
    if (threadIdx.x < 32) {
        ln_row<NV, false>(x, ln1_w, ln1_b, x, nullptr, nullptr, nullptr, nullptr, b, ACT_NONE, threadIdx.x);
        __syncwarp();
        ln_row<NV, false>(x, ln2_w, ln2_b, nullptr, xn.hi, xn.lo, nullptr, nullptr, b, ACT_NONE, threadIdx.x);
    }
}

static GemmEpilogue aed_epi(int mode, int act, float alpha, const float *bias, float *out, int ldo, H16 h = {nullptr, nullptr}, int ldh = 0) {
    GemmEpilogue e;
    memset(&e, 0, sizeof(e));
    e.mode = mode; e.act = act; e.alpha = alpha; e.bias = bias; e.out = out; e.ldo = ldo; e.out_hi = h.hi; e.out_lo = h.lo; e.ldh = ldh;
    return e;
}

size_t Model::aed_bytes(int total_T, int B, int max_len) const {
    const size_t D = aed_d, F = aed_ffn, L = aed_layers.size();
    return (size_t)total_T * (d_out * 4 + D * 4 + (L + 1) * 2 * D * 4) + L * 2 * (size_t)B * max_len * D * 4 +
           (size_t)B * (D * 24 + 3 * D * 4 + F * 4 + (size_t)aed_vocab * 4) + (size_t)B * (max_len + 64) * 8 + (1 << 20);
}

int Model::decode_aed(const float *enc_dev, const std::vector<int> &lens, const std::vector<std::vector<int>> &prompts, int eos,
                      const std::vector<int> &caps, std::vector<std::vector<int>> &tokens) {
    const int B = (int)lens.size(), D = aed_d, H = aed_heads, dk = D / H, L = (int)aed_layers.size(), V = aed_vocab, F = aed_ffn;
    tokens.assign(B, {});
    if (!has_aed) { set_error("model has no AED decoder"); return -1; }
    if (B == 0) return 0;
    if (dk > 256 || dk % 4) { set_error("aed_decode: head width %d must be a multiple of 4 up to 256", dk); return -1; }
    if ((int)prompts.size() != B || (int)caps.size() != B) { set_error("aed_decode: one prompt and one cap per utterance"); return -1; }
    int cap = 0;
    for (int c : caps) cap = c > cap ? c : cap;
    std::vector<int> off(B), mlen(B);
    int total_T = 0, max_T = 0, max_len = 0, max_prompt = 0, min_prompt = 1 << 30;
    for (int b = 0; b < B; b++) {
        if (prompts[b].empty()) { set_error("aed_decode: empty prompt (a start token is needed)"); return -1; }   // :143
        if (lens[b] <= 0) { set_error("aed_decode: utterance %d has no encoder frames", b); return -1; }
        for (int t : prompts[b]) if (t < 0 || t >= V) { set_error("aed_decode: prompt token %d outside the vocabulary", t); return -1; }
        off[b] = total_T; total_T += lens[b];
        max_T = lens[b] > max_T ? lens[b] : max_T;
        const int np = (int)prompts[b].size();
        const int cb = caps[b] > 0 ? caps[b] : 0;
        mlen[b] = np + cb < aed_max_seq ? np + cb : aed_max_seq;                 // :145-146
        max_len = mlen[b] > max_len ? mlen[b] : max_len;
        max_prompt = np > max_prompt ? np : max_prompt;
        min_prompt = np < min_prompt ? np : min_prompt;
    }
    const size_t mark = ws.off;
    const int capn = cap > 0 ? cap : 1;
    // ---- projected encoder output and the per-layer cross K/V, once (:149-178)
    H16 enc_h = ws.planes((size_t)total_T * d_out);
    H16 encp = enc_h;
    if (!enc_h.hi) return -1;
    if (split_to_h16(enc_dev, enc_h.hi, enc_h.lo, (size_t)total_T * d_out, stream, status)) return -1;
    note_launch();
    if (has_aed_proj) {
        encp = ws.planes((size_t)total_T * D);
        if (!encp.hi) return -1;
        if (gemm(enc_h, d_out, aed_proj, aed_epi(OUT_H16, ACT_NONE, 1.f, aed_proj_b, nullptr, 0, encp, D), total_T)) return -1;
    }
    int *d_off = ws.get<int>(2 * (size_t)B);
    if (!d_off) return -1;
    std::vector<int> ho(2 * (size_t)B);
    for (int b = 0; b < B; b++) { ho[b] = off[b]; ho[B + b] = lens[b]; }
    MB_CUDA(cudaMemcpyAsync(d_off, ho.data(), ho.size() * sizeof(int), cudaMemcpyHostToDevice, stream));
    const bool by_head = dk % 8 == 0 && D % 8 == 0;           // 16-byte copies
    if (!by_head) { set_error("aed_decode: head width %d must be a multiple of 8", dk); return -1; }
    const size_t v_off = (size_t)total_T * D;
    std::vector<H16> ckv(L);
    H16 kv_rows = ws.planes((size_t)total_T * 2 * D);          // one layer's (K | V) rows as the contraction writes them
    if (!kv_rows.hi) return -1;
    for (int l = 0; l < L; l++) {
        ckv[l] = ws.planes((size_t)total_T * 2 * D);
        if (!ckv[l].hi) return -1;
        if (gemm(encp, D, aed_layers[l].ckv, aed_epi(OUT_H16, ACT_NONE, 1.f, aed_layers[l].ckv_b, nullptr, 0, kv_rows, 2 * D), total_T)) return -1;
        aed_kv_by_head_kernel<<<dim3(H, B), 256, 0, stream>>>(kv_rows.hi, ckv[l].hi, v_off, d_off, d_off + B, D, dk);
        if (kv_rows.lo) aed_kv_by_head_kernel<<<dim3(H, B), 256, 0, stream>>>(kv_rows.lo, ckv[l].lo, v_off, d_off, d_off + B, D, dk);
        MB_CUDA(cudaGetLastError());
        note_launch(kv_rows.lo ? 2 : 1);
    }
    // ---- state
    float *sk = ws.get<float>((size_t)L * 2 * B * max_len * D);
    float *x = ws.get<float>((size_t)B * D), *qkv = ws.get<float>((size_t)B * 3 * D), *q = ws.get<float>((size_t)B * D);
    float *logits = ws.get<float>((size_t)B * V);
    H16 xn = ws.planes((size_t)B * D), att = ws.planes((size_t)B * D), ff = ws.planes((size_t)B * F);
    int *st = ws.get<int>(7 * (size_t)B + 4), *best = ws.get<int>(B), *d_prompts = ws.get<int>((size_t)B * max_prompt);
    int *d_tokens = ws.get<int>((size_t)B * capn);
    if (!sk || !x || !qkv || !q || !logits || !xn.hi || !att.hi || !ff.hi || !st || !best || !d_prompts || !d_tokens) return -1;
    std::vector<int> hst(7 * (size_t)B + 4, 0), hp((size_t)B * max_prompt, 0);
    for (int b = 0; b < B; b++) {
        hst[b] = prompts[b][0];                              // cur
        hst[3 * B + b] = (int)prompts[b].size();
        hst[4 * B + b] = mlen[b];
        hst[5 * B + b] = caps[b] > 0 ? caps[b] : 0;
        for (size_t i = 0; i < prompts[b].size(); i++) hp[(size_t)b * max_prompt + i] = prompts[b][i];
    }
    MB_CUDA(cudaMemcpyAsync(st, hst.data(), hst.size() * sizeof(int), cudaMemcpyHostToDevice, stream));
    MB_CUDA(cudaMemcpyAsync(d_prompts, hp.data(), hp.size() * sizeof(int), cudaMemcpyHostToDevice, stream));
    const size_t self_smem = ((size_t)max_len + 4 + (1 + SELF_WARPS) * (size_t)dk + 32) * sizeof(float);
    const int cross_threads = CROSS_WARPS * 32;
    const size_t cross_smem = ((size_t)max_T + 4 + (1 + CROSS_WARPS) * (size_t)dk + 32) * sizeof(float);
    if (self_smem > 200 * 1024 || cross_smem > 200 * 1024) { set_error("aed_decode: sequence too long for the attention kernels"); return -1; }
    MB_CUDA(cudaFuncSetAttribute(aed_self_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)self_smem));
    MB_CUDA(cudaFuncSetAttribute(aed_cross_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cross_smem));
    const int sp = prof_begin_span(PROF_DECODE);
    const int *pd = st + 6 * B + 1;
    // everything one position needs, in stream order; no host value changes between positions
    // The LayerNorm that follows a residual update runs inside the contraction that makes the update (GemmEpilogue::ln_*)
    // when the width is one the register LayerNorm serves; otherwise as a launch of its own.
    const bool ln_tail = gemm_skinny_ln_width(D);
    int *ln_count = ws.get<int>(B);
    if (!ln_count) return -1;
    MB_CUDA(cudaMemsetAsync(ln_count, 0, (size_t)B * sizeof(int), stream));
    auto resid = [&](const float *bias, const float *nw, const float *nb) {     // x += y, then xn = LN(x; nw, nb)
        GemmEpilogue e = aed_epi(OUT_RESID, ACT_NONE, 1.f, bias, x, D);
        if (ln_tail) { e.ln_w = nw; e.ln_b = nb; e.ln_hi = xn.hi; e.ln_lo = xn.lo; e.ln_count = ln_count; }
        return e;
    };
    // With those widths the turn between positions is one launch too (aed_next_kernel): selection, next embedding and the
    // two LayerNorms that open a position; it also prepares position 0 (first = 1).
    auto next = [&](int first) -> int {
#define AED_NEXT(NV) MB_CUDA(launch_kernel(aed_next_kernel<NV>, dim3(B), dim3(256), 0, stream, true, 1, (const float *)logits, V, eos, capn, B, st, (const int *)d_prompts, \
                                           max_prompt, d_tokens, aed_emb, aed_pos, aed_max_seq, aed_embln_w, aed_embln_b, aed_layers[0].ln_self_w, aed_layers[0].ln_self_b, x, xn, first))
        switch (D) {
            case 128: AED_NEXT(1); break;
            case 256: AED_NEXT(2); break;
            case 512: AED_NEXT(4); break;
            case 640: AED_NEXT(5); break;
            case 1024: AED_NEXT(8); break;
            default: AED_NEXT(16); break;            // 2048: the last of gemm_skinny_ln_width's widths
        }
#undef AED_NEXT
        return 0;
    };
    const int *pos_b = st + 6 * B + 4;
    auto position = [&]() -> int {
        // every launch of a position is chained: blocks of the next kernel are placed while the one before drains
        if (!ln_tail) {
            MB_CUDA(launch_kernel(aed_embed_kernel, dim3(B), dim3(128), 0, stream, true, 1, aed_emb, aed_pos, (const int *)st, pd, x, D));
            if (layer_norm(x, aed_embln_w, aed_embln_b, x, H16{nullptr, nullptr}, B, D, 0, stream, true)) return -1;
            if (layer_norm(x, aed_layers[0].ln_self_w, aed_layers[0].ln_self_b, nullptr, xn, B, D, 0, stream, true)) return -1;
        }
        for (int l = 0; l < L; l++) {
            const AedLayer &A = aed_layers[l];
            float *K = sk + (size_t)(2 * l) * B * max_len * D, *Vc = K + (size_t)B * max_len * D;
            // LayerNorm after the last contraction of this layer: the next layer's first one, or the final one
            const float *nw = l + 1 < L ? aed_layers[l + 1].ln_self_w : aed_fin_w, *nb = l + 1 < L ? aed_layers[l + 1].ln_self_b : aed_fin_b;
            if (gemm(xn, D, A.sqkv, aed_epi(OUT_F32, ACT_NONE, 1.f, A.sqkv_b, qkv, 3 * D), B, true)) return -1;
            MB_CUDA(launch_kernel(aed_self_attn_kernel, dim3(H, B), dim3(SELF_WARPS * 32), self_smem, stream, true, 1, (const float *)qkv, K, Vc,
                                  ln_tail ? pos_b : pd, ln_tail ? 1 : 0, max_len, D, dk, att));
            if (gemm(att, D, A.so, resid(A.so_b, A.ln_cross_w, A.ln_cross_b), B, true)) return -1;
            if (!ln_tail && layer_norm(x, A.ln_cross_w, A.ln_cross_b, nullptr, xn, B, D, 0, stream, true)) return -1;
            if (gemm(xn, D, A.cq, aed_epi(OUT_F32, ACT_NONE, 1.f, A.cq_b, q, D), B, true)) return -1;
            MB_CUDA(launch_kernel(aed_cross_attn_kernel, dim3(H, B), dim3(cross_threads), cross_smem, stream, true, 1, (const float *)q, (const __half *)ckv[l].hi,
                                  (const __half *)ckv[l].lo, v_off, (const int *)d_off, (const int *)(d_off + B), max_T, D, dk, att));
            if (gemm(att, D, A.co, resid(A.co_b, A.ln_ffn_w, A.ln_ffn_b), B, true)) return -1;
            if (!ln_tail && layer_norm(x, A.ln_ffn_w, A.ln_ffn_b, nullptr, xn, B, D, 0, stream, true)) return -1;
            if (gemm(xn, D, A.ff1, aed_epi(OUT_H16, ACT_RELU, 1.f, A.ff1_b, nullptr, 0, ff, F), B, true)) return -1;
            if (gemm(ff, F, A.ff2, resid(A.ff2_b, nw, nb), B, true)) return -1;
            if (!ln_tail && layer_norm(x, nw, nb, nullptr, xn, B, D, 0, stream, true)) return -1;
        }
        // the head is evaluated at prompt positions too (its result is ignored there): one graph for all positions
        if (gemm(xn, D, aed_head, aed_epi(OUT_F32, ACT_NONE, 1.f, aed_head_b, logits, V), B, true)) return -1;
        if (ln_tail) return next(0);
        if (argmax_rows(logits, V, nullptr, B, V, best, stream, true)) return -1;
        MB_CUDA(launch_kernel(aed_select_kernel, dim3(1), dim3(((B + 31) / 32) * 32), 0, stream, true, 1, (const int *)best, eos, capn, B, st, (const int *)d_prompts,
                              max_prompt, d_tokens));
        return 0;
    };
    if (ln_tail && next(1)) return -1;                 // x and xn of position 0
    const int launches_per_position = ln_tail ? L * 8 + 2 : 1 + (2 + 3 * L) + L * 8 + 3, gemms_per_position = 6 * L + 1;   // (the contraction wrapper counts its own launches)
    (void)min_prompt;
    int n_done = 0;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int rc = 0;
    for (int p = 0; p < max_len && n_done < B && rc == 0; p++) {
        if (p == 0) {
            rc = position();                                 // eager: also sets every kernel's launch attributes
            note_launch(launches_per_position - gemms_per_position);
        } else {
            if (p == 1) {
                // positions 1.. replay one captured graph of the chained launches (no host work between the kernels of a position)
                const bool was_on = prof_on;
                prof_on = false;                             // no event records inside the capture
                if (cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
                    const int prc = position();
                    note_launch(-gemms_per_position);        // recorded, not launched
                    cudaGraph_t g = nullptr;
                    const cudaError_t e = cudaStreamEndCapture(stream, &g);
                    if (prc == 0 && e == cudaSuccess && g && cudaGraphInstantiate(&exec, g, 0) == cudaSuccess) graph = g;
                    else { if (g) cudaGraphDestroy(g); exec = nullptr; cudaGetLastError(); }
                }
                prof_on = was_on;
            }
            if (exec) {
                if (cudaGraphLaunch(exec, stream) != cudaSuccess) { set_error("aed_decode: graph launch failed"); rc = -1; }
                note_launch(launches_per_position);
            } else {
                rc = position();
                note_launch(launches_per_position - gemms_per_position);
            }
        }
        if (rc == 0 && ((p & 7) == 7 || p + 1 == max_len)) { // look at the finished count every eighth position
            MB_CUDA(cudaMemcpyAsync(&n_done, st + 6 * B, sizeof(int), cudaMemcpyDeviceToHost, stream));
            MB_CUDA(cudaStreamSynchronize(stream));
        }
    }
    if (exec) cudaGraphExecDestroy(exec);
    if (graph) cudaGraphDestroy(graph);
    if (rc) return -1;
    prof_end_span(sp);
    if (sp >= 0) prof_launches[PROF_DECODE]++;
    std::vector<int> hn(B), ht((size_t)B * capn);
    MB_CUDA(cudaMemcpyAsync(hn.data(), st + B, B * sizeof(int), cudaMemcpyDeviceToHost, stream));
    MB_CUDA(cudaMemcpyAsync(ht.data(), d_tokens, ht.size() * sizeof(int), cudaMemcpyDeviceToHost, stream));
    MB_CUDA(cudaStreamSynchronize(stream));
    if (check_status("aed_decode")) return -1;
    for (int b = 0; b < B; b++) tokens[b].assign(ht.begin() + (size_t)b * capn, ht.begin() + (size_t)b * capn + hn[b]);
    ws.off = mark;
    return 0;
}

}  // namespace mb
