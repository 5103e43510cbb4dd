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
//   head    logits[b] = head . relu(enc[b][t_b] + g[b]); a warp owns 16 rows of the
//           V (+durations) rows for all utterances and emits first-argmax candidates
//   select  one CTA per utterance merges the candidates and applies the emission
//           rule: non-blank -> emit, advance by the predicted duration (RNNT: 0),
//           blank with duration 0 -> 1, max_symbols guard (src/decoder.c:161-176)
//   lstm    (only if some utterance emitted) a row block is 4 hidden units x 4 gates of
//           [W_ih | W_hh] against [input ; previous h] of all utterances, then the cell
//           update; layers are separated by a grid sync
//   proj    g[b] = decoder_projector(h_last[b])
// The matvecs run on the warp-level tensor-core path with the utterances as the N
// dimension: weights as fp16 (hi, lo) planes (a decoded Q4_0/Q8_0 weight is exact in
// that form), activations split the same way, three MMAs per k-step, f32 accumulate —
// f32-grade like the reference's sgemv/sgemm path.
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
    chain_trigger();
    chain_wait();
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

int argmax_rows(const float *logits, int ld, const float *bias, int T, int V, int *best, cudaStream_t st, bool chain) {
    if (T <= 0) return 0;
    MB_CUDA(launch_kernel(argmax_kernel, dim3(T), dim3(256), 0, st, chain, 1, logits, ld, bias, V, best));
    return 0;
}

// ------------------------------------------------------- RNNT / TDT lock-step

// ---- tensor-core matvec for a batch of up to 16 utterances ----------------------
// out[r][b] = sum_k W[r][k] * X[b][k] with W as fp16 (hi, lo) planes streamed from L2 and
// X as fp16 (hi, lo) planes in shared memory. A warp owns 16 weight rows (the M side
// of mma.m16n8k16) and the 16 utterances are two N blocks; three MMAs per k-step
// (hi*hi, lo*hi, hi*lo) give f32-grade products. k is consumed in a permuted order
// that lets both operands be fetched with 16-byte loads: within a 32-wide chunk lane
// (g, t) holds k = 8t..8t+7 of its rows, and k-step s uses elements 4s..4s+3 of them —
// the same assignment on both operands, so the sum is unchanged.
static constexpr int XPAD = 32;                       // halves of padding per X row (bank spread)

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Accumulates chunks [c0, c1) of 32 k for rows rowA (fragment rows g) and rowB (g + 8).
// acc[nb][0..3]: rows g (0,1) and g+8 (2,3) x utterances nb*8 + 2t, +1.
__device__ __forceinline__ void rowblock_mma(const __half *__restrict__ whi, const __half *__restrict__ wlo, int ldw,
                                             int rowA, int rowB, int c0, int c1, const __half *xhi,
                                             const __half *xlo, int xs, int lane, float (&acc)[2][4]) {
    const int g = lane >> 2, t = lane & 3;
    float d0[2][4], d1[2][4];
#pragma unroll
    for (int nb = 0; nb < 2; nb++)
#pragma unroll
        for (int i = 0; i < 4; i++) { d0[nb][i] = 0.f; d1[nb][i] = 0.f; }
    const uint4 *pAh = reinterpret_cast<const uint4 *>(whi + (size_t)rowA * ldw + 8 * t);
    const uint4 *pBh = reinterpret_cast<const uint4 *>(whi + (size_t)rowB * ldw + 8 * t);
    const uint4 *pAl = reinterpret_cast<const uint4 *>(wlo + (size_t)rowA * ldw + 8 * t);
    const uint4 *pBl = reinterpret_cast<const uint4 *>(wlo + (size_t)rowB * ldw + 8 * t);
    const uint4 *x0h = reinterpret_cast<const uint4 *>(xhi + (size_t)g * xs + 8 * t);
    const uint4 *x1h = reinterpret_cast<const uint4 *>(xhi + (size_t)(g + 8) * xs + 8 * t);
    const uint4 *x0l = reinterpret_cast<const uint4 *>(xlo + (size_t)g * xs + 8 * t);
    const uint4 *x1l = reinterpret_cast<const uint4 *>(xlo + (size_t)(g + 8) * xs + 8 * t);
#pragma unroll 5
    for (int c = c0; c < c1; c++) {
        const uint4 ah = __ldg(pAh + c * 4), bh = __ldg(pBh + c * 4);      // 32 halves = 4 uint4 per chunk
        const uint4 al = __ldg(pAl + c * 4), bl = __ldg(pBl + c * 4);
        const uint4 u0h = x0h[c * 4], u1h = x1h[c * 4], u0l = x0l[c * 4], u1l = x1l[c * 4];
        // k-step 0: elements 0..3, k-step 1: elements 4..7
        mma_f16(d0[0], ah.x, bh.x, ah.y, bh.y, u0h.x, u0h.y);
        mma_f16(d0[1], ah.x, bh.x, ah.y, bh.y, u1h.x, u1h.y);
        mma_f16(d1[0], al.x, bl.x, al.y, bl.y, u0h.x, u0h.y);
        mma_f16(d1[1], al.x, bl.x, al.y, bl.y, u1h.x, u1h.y);
        mma_f16(d1[0], ah.x, bh.x, ah.y, bh.y, u0l.x, u0l.y);
        mma_f16(d1[1], ah.x, bh.x, ah.y, bh.y, u1l.x, u1l.y);
        mma_f16(d0[0], ah.z, bh.z, ah.w, bh.w, u0h.z, u0h.w);
        mma_f16(d0[1], ah.z, bh.z, ah.w, bh.w, u1h.z, u1h.w);
        mma_f16(d1[0], al.z, bl.z, al.w, bl.w, u0h.z, u0h.w);
        mma_f16(d1[1], al.z, bl.z, al.w, bl.w, u1h.z, u1h.w);
        mma_f16(d1[0], ah.z, bh.z, ah.w, bh.w, u0l.z, u0l.w);
        mma_f16(d1[1], ah.z, bh.z, ah.w, bh.w, u1l.z, u1l.w);
    }
#pragma unroll
    for (int nb = 0; nb < 2; nb++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[nb][i] = fmaf(d1[nb][i], H16_LO_INV, d0[nb][i]);
}

// Writes f32 rows [16][K] (rows >= B zero) as (hi, lo) planes into shared memory.
// Two passes — every global load of the CTA is issued before the first shared store —
// so the loads overlap instead of queueing behind stores the compiler cannot prove
// independent. value4(b, k) returns elements k..k+3 of row b.
static constexpr int STAGE_NV = 16;                   // float4 per thread: covers K <= 1024
template <typename F>
__device__ __forceinline__ void stage_x(__half *xhi, __half *xlo, int xs, int koff, int K, int B, F value4) {
    // sixteen threads per row, 16-byte columns c0, c0 + 16, ...: no division, 256 contiguous bytes per row step
    const int b = threadIdx.x >> 4, c0 = threadIdx.x & 15, k4n = K >> 2;
    float4 v[STAGE_NV];
#pragma unroll
    for (int j = 0; j < STAGE_NV; j++) {
        const int c = c0 + 16 * j;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < k4n && b < B) v[j] = value4(b, c * 4);
    }
#pragma unroll
    for (int j = 0; j < STAGE_NV; j++) {
        const int c = c0 + 16 * j;
        if (c < k4n) {
            __align__(8) __half h[4], l[4];
            split_h16(v[j].x, h[0], l[0]); split_h16(v[j].y, h[1], l[1]);
            split_h16(v[j].z, h[2], l[2]); split_h16(v[j].w, h[3], l[3]);
            *reinterpret_cast<uint2 *>(xhi + b * xs + koff + c * 4) = *reinterpret_cast<uint2 *>(h);
            *reinterpret_cast<uint2 *>(xlo + b * xs + koff + c * 4) = *reinterpret_cast<uint2 *>(l);
        }
    }
}
__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }

// Rows that already exist as fp16 (hi, lo) planes in global memory (hidden states, embedding rows) go to
// the X tile with 16-byte asynchronous copies: no registers, no conversion, one wait for all of them.
// row_hi(b) / row_lo(b) return the H halves of utterance b; columns [koff, koff + H) of the tile are written.
__device__ __forceinline__ void cp16(void *dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_wait_all() { asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory"); }
template <typename FH, typename FL>
__device__ __forceinline__ void stage_planes(__half *xhi, __half *xlo, int xs, int koff, int H, int B, FH row_hi, FL row_lo) {
    const int cpr = H >> 3;                               // 16-byte chunks per row
    for (int idx = threadIdx.x; idx < B * cpr; idx += blockDim.x) {
        const int b = idx / cpr, c = idx - b * cpr;
        cp16(xhi + b * xs + koff + 8 * c, row_hi(b) + 8 * c);
        cp16(xlo + b * xs + koff + 8 * c, row_lo(b) + 8 * c);
    }
}

struct Cand { float v; int i; };
__device__ __forceinline__ void cand_take(Cand &a, float v, int i) {
    if (v > a.v || (v == a.v && i < a.i)) { a.v = v; a.i = i; }
}

// One stacked-LSTM layer (pred_step, src/decoder.c:73-99) for all utterances. A row
// block is 4 units x 4 gates (i, f, g, o); k = [input ; previous h] is split over
// NSL warps and reduced through shared memory. Reads h[par], writes h[par^1]; c in
// place. Utterances that did not emit copy their state through.
__device__ void lstm_phase(const GreedyDev &p, int l, int par, __half *xhi, __half *xlo, float *red, int lane, int wib) {
    const int H = p.H, B = p.B, K = 2 * H, xs = K + XPAD;
    // hidden states live as fp16 (hi, lo) planes: h[parity] = [hi: L][B][H] then [lo: L][B][H] halves
    const size_t nstate = (size_t)p.L * B * H;
    const __half *hold_hi = reinterpret_cast<const __half *>(p.h[par]) + (size_t)l * B * H, *hold_lo = hold_hi + nstate;
    __half *hnew_hi = reinterpret_cast<__half *>(p.h[par ^ 1]) + (size_t)l * B * H, *hnew_lo = hnew_hi + nstate;
    float *cc = p.c + (size_t)l * B * H;
    const __half *xin_hi = l == 0 ? nullptr : reinterpret_cast<const __half *>(p.h[par ^ 1]) + (size_t)(l - 1) * B * H;
    const __half *xin_lo = l == 0 ? nullptr : xin_hi + nstate;
    constexpr int NSL = 4;
    const int nrb = H / 4, chunks = K / 32, per = (chunks + NSL - 1) / NSL;
    if (blockIdx.x * 8 < nrb * NSL) {        // a CTA without a row block to work on does not pull the activations either
        if (l == 0)
            stage_planes(xhi, xlo, xs, 0, H, B, [&](int b) { return p.emb_hi + (size_t)p.last_tok[b] * H; },
                         [&](int b) { return p.emb_lo + (size_t)p.last_tok[b] * H; });
        else
            stage_planes(xhi, xlo, xs, 0, H, B, [&](int b) { return xin_hi + (size_t)b * H; }, [&](int b) { return xin_lo + (size_t)b * H; });
        stage_planes(xhi, xlo, xs, H, H, B, [&](int b) { return hold_hi + (size_t)b * H; }, [&](int b) { return hold_lo + (size_t)b * H; });
        cp_wait_all();
    }
    __syncthreads();
    const int g = lane >> 2, t = lane & 3;
    for (int base = blockIdx.x * 8; base < nrb * NSL; base += gridDim.x * 8) {
        const int task = base + wib, rb = task / NSL, sl = task % NSL;
        const bool on = task < nrb * NSL;
        float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        // what the cell update needs besides the sums — biases, previous cell state, emission flags — is
        // fetched now, under the contraction
        float bih[4] = {0.f, 0.f, 0.f, 0.f}, bhh[4] = {0.f, 0.f, 0.f, 0.f}, cprev[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
        int em[2][2] = {{0, 0}, {0, 0}};
        if (on && sl == 0 && g < 4) {
            const int unit = rb * 4 + g;
#pragma unroll
            for (int q = 0; q < 4; q++) { bih[q] = p.b_ih[l][q * H + unit]; bhh[q] = p.b_hh[l][q * H + unit]; }
#pragma unroll
            for (int nb = 0; nb < 2; nb++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int b = nb * 8 + 2 * t + e;
                    if (b < B) { em[nb][e] = p.emit[b]; cprev[nb][e] = cc[(size_t)b * H + unit]; }
                }
        }
        if (on) {
            // fragment row lr -> gate lr/4, unit rb*4 + lr%4
            const int rowA = (g >> 2) * H + rb * 4 + (g & 3), rowB = (2 + (g >> 2)) * H + rb * 4 + (g & 3);
            const int c0 = sl * per, c1 = (sl + 1) * per < chunks ? (sl + 1) * per : chunks;
            rowblock_mma(p.wcat_hi[l], p.wcat_lo[l], K, rowA, rowB, c0, c1, xhi, xlo, xs, lane, acc);
        }
#pragma unroll
        for (int nb = 0; nb < 2; nb++)
#pragma unroll
            for (int i = 0; i < 4; i++) red[(wib * 32 + lane) * 8 + nb * 4 + i] = acc[nb][i];
        __syncthreads();
        if (on && sl == 0) {
            float z[2][4];
#pragma unroll
            for (int nb = 0; nb < 2; nb++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float s = 0.f;
                    for (int q = 0; q < NSL; q++) s += red[((wib + q) * 32 + lane) * 8 + nb * 4 + i];
                    z[nb][i] = s;
                }
            // lane g<4 holds gates i (rows g) and g (rows g+8) of unit g; lane g+4 holds f and o
#pragma unroll
            for (int nb = 0; nb < 2; nb++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const float za = z[nb][e], zb = z[nb][2 + e];
                    const float oa = __shfl_xor_sync(0xffffffffu, za, 16), ob = __shfl_xor_sync(0xffffffffu, zb, 16);
                    if (g < 4) {
                        const int unit = rb * 4 + g, b = nb * 8 + 2 * t + e;
                        if (b < B) {
                            const size_t o = (size_t)b * H + unit;
                            if (em[nb][e]) {
                                const float zi = za + bih[0] + bhh[0];
                                const float zf = oa + bih[1] + bhh[1];
                                const float zg = zb + bih[2] + bhh[2];
                                const float zo = ob + bih[3] + bhh[3];
                                const float cn = sigmoid_stable(zf) * cprev[nb][e] + sigmoid_stable(zi) * tanhf(zg);
                                cc[o] = cn;
                                __half hh, hl;
                                split_h16(sigmoid_stable(zo) * tanhf(cn), hh, hl);
                                hnew_hi[o] = hh; hnew_lo[o] = hl;
                            } else {
                                hnew_hi[o] = hold_hi[o]; hnew_lo[o] = hold_lo[o];
                            }
                        }
                    }
                }
        }
        __syncthreads();
    }
}

// g[b] = proj_b + proj_w . h_last[b] for the utterances that emitted.
__device__ void proj_phase(const GreedyDev &p, int par, bool all, __half *xhi, __half *xlo, float *red, int lane, int wib) {
    const int H = p.H, B = p.B, xs = 2 * H + XPAD;
    const size_t nstate = (size_t)p.L * B * H;
    const __half *hl_hi = reinterpret_cast<const __half *>(p.h[par]) + (size_t)(p.L - 1) * B * H, *hl_lo = hl_hi + nstate;
    constexpr int NSL = 4;
    const int nrb = (H + 15) / 16, chunks = H / 32, per = (chunks + NSL - 1) / NSL;
    if (blockIdx.x * 8 < nrb * NSL) {
        stage_planes(xhi, xlo, xs, 0, H, B, [&](int b) { return hl_hi + (size_t)b * H; }, [&](int b) { return hl_lo + (size_t)b * H; });
        cp_wait_all();
    }
    __syncthreads();
    const int g = lane >> 2, t = lane & 3;
    for (int base = blockIdx.x * 8; base < nrb * NSL; base += gridDim.x * 8) {
        const int task = base + wib, rb = task / NSL, sl = task % NSL;
        const bool on = task < nrb * NSL;
        float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        // the encoder values the epilogue adds to g are fetched now, under the contraction (-1: past the end)
        // likewise the projector bias of an utterance that emitted, or the g an utterance that did not keeps
        float ev[2][4], addv[2][4];
        bool fresh[2][4];
#pragma unroll
        for (int nb = 0; nb < 2; nb++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int r = rb * 16 + g + (i >> 1) * 8, b = nb * 8 + 2 * t + (i & 1);
                ev[nb][i] = -1.f; addv[nb][i] = 0.f; fresh[nb][i] = false;
                if (on && sl == 0 && r < H && b < B) {
                    fresh[nb][i] = all || p.emit[b] != 0;
                    addv[nb][i] = fresh[nb][i] ? p.proj_b[r] : p.g[(size_t)b * H + r];
                    const int tb = p.t[b];
                    if (tb < p.enc_len[b]) ev[nb][i] = p.enc[(size_t)(p.enc_off[b] + tb) * H + r];
                }
            }
        bool past[2][4];
#pragma unroll
        for (int nb = 0; nb < 2; nb++)
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int b = nb * 8 + 2 * t + (i & 1);
                past[nb][i] = !(on && sl == 0 && b < B && p.t[b] < p.enc_len[b]);
            }
        if (on) {
            const int rA = rb * 16 + g, rB = rA + 8;
            const int c0 = sl * per, c1 = (sl + 1) * per < chunks ? (sl + 1) * per : chunks;
            rowblock_mma(p.proj_hi, p.proj_lo, H, rA < H ? rA : H - 1, rB < H ? rB : H - 1, c0, c1, xhi, xlo, xs, lane, acc);
        }
#pragma unroll
        for (int nb = 0; nb < 2; nb++)
#pragma unroll
            for (int i = 0; i < 4; i++) red[(wib * 32 + lane) * 8 + nb * 4 + i] = acc[nb][i];
        __syncthreads();
        if (on && sl == 0) {
#pragma unroll
            for (int nb = 0; nb < 2; nb++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float s = 0.f;
                    for (int q = 0; q < NSL; q++) s += red[((wib + q) * 32 + lane) * 8 + nb * 4 + i];
                    const int r = rb * 16 + g + (i >> 1) * 8, b = nb * 8 + 2 * t + (i & 1);
                    if (r < H && b < B) {
                        // g, and with it the joint input of the coming step for this utterance's current frame
                        // (an utterance that did not emit keeps its g but may have moved to another frame)
                        const size_t o = (size_t)b * H + r;
                        float gv = addv[nb][i];
                        if (fresh[nb][i]) { gv = s + addv[nb][i]; p.g[o] = gv; }
                        const float jv = past[nb][i] ? 0.f : fmaxf(ev[nb][i] + gv, 0.f);
                        __half jh, jl;
                        split_h16(jv, jh, jl);
                        p.jx_hi[o] = jh; p.jx_lo[o] = jl;
                    }
                }
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(256, 1)
greedy_kernel(GreedyDev p) {
    cg::grid_group grid = cg::this_grid();
    extern __shared__ __align__(16) uint8_t dsm[];
    const int H = p.H, B = p.B, V = p.V, VL = p.V + p.ND;
    const int xs = 2 * H + XPAD;
    __half *xhi = reinterpret_cast<__half *>(dsm);
    __half *xlo = xhi + 16 * xs;
    float *red = reinterpret_cast<float *>(xlo + 16 * xs);          // [8 warps][32 lanes][8]
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    int par = (!p.init_state && p.par_state) ? *p.par_state : 0;   // read before the first grid sync; written after the last
    for (int i = threadIdx.x; i < 16 * xs; i += blockDim.x) { xhi[i] = __float2half_rn(0.f); xlo[i] = __float2half_rn(0.f); }
    __syncthreads();                                               // rows of absent utterances stay zero for every plane copy

    if (p.init_state) {
        // SOS = blank on a zero state (src/decoder.c:151): run the prediction net once
        if (blockIdx.x == 0 && threadIdx.x < B) { p.emit[threadIdx.x] = 1; p.last_tok[threadIdx.x] = p.blank; }
        grid.sync();
        for (int l = 0; l < p.L; l++) { lstm_phase(p, l, par, xhi, xlo, red, lane, wib); grid.sync(); }
        par ^= 1;
        proj_phase(p, par, true, xhi, xlo, red, lane, wib);
        grid.sync();
    }
    bool jx_valid = p.init_state != 0;     // the planes of relu(enc[t] + g) left by the last projector phase are current

    constexpr int NSL = 2;
    const int nrb = (VL + 15) / 16, chunks = H / 32, per = (chunks + NSL - 1) / NSL;
    __shared__ int srow[16];
    // optional phase timers (clock64 of CTA 0): head, sync, select+sync, lstm+syncs, proj+sync, steps, emit steps
    const bool timing = p.dbg != nullptr && blockIdx.x == 0 && threadIdx.x == 0;
    long long tq = timing ? clock64() : 0;
#define PHASE_MARK(slot) do { if (timing) { const long long n_ = clock64(); p.dbg[slot] += n_ - tq; tq = n_; } } while (0)
    for (int step = 0; step < p.max_steps; step++) {
        // ---- head: joint = relu(enc[t] + g) -> logits -> first-argmax candidates per row block
        // frame of every utterance first (one round trip), so that the row loads below depend on nothing
        // they have to wait for: an utterance past its end reads its last frame and is zeroed afterwards
        if (threadIdx.x < 16) {
            int row = -1;
            if (threadIdx.x < B) {
                const int tb = p.t[threadIdx.x], len = p.enc_len[threadIdx.x];
                if (tb < len) row = p.enc_off[threadIdx.x] + tb;
            }
            srow[threadIdx.x] = row;
        }
        __syncthreads();
        if (blockIdx.x * 8 < nrb * NSL && jx_valid) {
            stage_planes(xhi, xlo, xs, 0, H, B, [&](int b) { return p.jx_hi + (size_t)b * H; }, [&](int b) { return p.jx_lo + (size_t)b * H; });
            cp_wait_all();
        } else if (blockIdx.x * 8 < nrb * NSL)
        stage_x(xhi, xlo, xs, 0, H, B, [&](int b, int k) {
            const int row = srow[b];
            const float4 e = ld4(p.enc + (size_t)(row < 0 ? 0 : row) * H + k), gg = ld4(p.g + (size_t)b * H + k);
            const float z = row < 0 ? 0.f : 1.f;
            return make_float4(z * fmaxf(e.x + gg.x, 0.f), z * fmaxf(e.y + gg.y, 0.f), z * fmaxf(e.z + gg.z, 0.f), z * fmaxf(e.w + gg.w, 0.f));
        });
        __syncthreads();
        PHASE_MARK(7);
        for (int base = blockIdx.x * 8; base < nrb * NSL; base += gridDim.x * 8) {
            const int task = base + wib, rb = task / NSL, sl = task % NSL;
            const bool on = task < nrb * NSL;
            float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            const int rA = rb * 16 + g, rB = rA + 8;
            const float biasA = on && sl == 0 && rA < VL ? p.head_b[rA] : 0.f, biasB = on && sl == 0 && rB < VL ? p.head_b[rB] : 0.f;
            if (on) {
                const int c0 = sl * per, c1 = (sl + 1) * per < chunks ? (sl + 1) * per : chunks;
                rowblock_mma(p.head_hi, p.head_lo, H, rA < VL ? rA : VL - 1, rB < VL ? rB : VL - 1, c0, c1, xhi, xlo, xs, lane, acc);
            }
#pragma unroll
            for (int nb = 0; nb < 2; nb++)
#pragma unroll
                for (int i = 0; i < 4; i++) red[(wib * 32 + lane) * 8 + nb * 4 + i] = acc[nb][i];
            __syncthreads();
            if (on && sl == 0) {
#pragma unroll
                for (int nb = 0; nb < 2; nb++)
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const float va = red[(wib * 32 + lane) * 8 + nb * 4 + e] + red[((wib + 1) * 32 + lane) * 8 + nb * 4 + e] + biasA;
                        const float vb = red[(wib * 32 + lane) * 8 + nb * 4 + 2 + e] + red[((wib + 1) * 32 + lane) * 8 + nb * 4 + 2 + e] + biasB;
                        Cand tk{-3.0e38f, 0x7fffffff}, du{-3.0e38f, 0x7fffffff};
                        if (rA < V) cand_take(tk, va, rA); else if (rA < VL) cand_take(du, va, rA);
                        if (rB < V) cand_take(tk, vb, rB); else if (rB < VL) cand_take(du, vb, rB);
                        // reduce over the eight lanes that hold the other rows of this utterance
#pragma unroll
                        for (int o = 4; o < 32; o <<= 1) {
                            cand_take(tk, __shfl_xor_sync(0xffffffffu, tk.v, o), __shfl_xor_sync(0xffffffffu, tk.i, o));
                            cand_take(du, __shfl_xor_sync(0xffffffffu, du.v, o), __shfl_xor_sync(0xffffffffu, du.i, o));
                        }
                        const int b = nb * 8 + 2 * t + e;
                        if (g == 0 && b < B) {
                            p.cand_v[((size_t)b * 2 + 0) * nrb + rb] = tk.v; p.cand_i[((size_t)b * 2 + 0) * nrb + rb] = tk.i;
                            p.cand_v[((size_t)b * 2 + 1) * nrb + rb] = du.v; p.cand_i[((size_t)b * 2 + 1) * nrb + rb] = du.i;
                        }
                    }
            }
            __syncthreads();
        }
        // flags are double-buffered by step parity: a CTA that runs ahead into the next
        // step must not overwrite what a slower CTA is still reading
        int *fl = p.flags + (step & 1) * 2;
        if (blockIdx.x == 0 && threadIdx.x == 0) { fl[0] = 0; fl[1] = 1; }
        PHASE_MARK(0);
        grid.sync();
        PHASE_MARK(1);
        // ---- select: CTA b merges candidates and applies the emission rule
        if (blockIdx.x < B) {
            const int b = blockIdx.x;
            __shared__ float sv[2][8];
            __shared__ int si[2][8];
            // the utterance's state is fetched while the candidates are merged
            int tb = 0, st_len = 0, st_no = 0, st_eh = 0;
            if (threadIdx.x == 0) { tb = p.t[b]; st_len = p.enc_len[b]; st_no = p.n_out[b]; st_eh = p.emitted_here[b]; }
            Cand best[2];
            for (int kind = 0; kind < 2; kind++) {
                Cand c{-3.0e38f, 0x7fffffff};
                for (int w = threadIdx.x; w < nrb; w += blockDim.x)
                    cand_take(c, p.cand_v[((size_t)b * 2 + kind) * nrb + w], p.cand_i[((size_t)b * 2 + kind) * nrb + w]);
                best[kind] = c;
            }
#pragma unroll
            for (int kind = 0; kind < 2; kind++) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1)
                    cand_take(best[kind], __shfl_xor_sync(0xffffffffu, best[kind].v, o), __shfl_xor_sync(0xffffffffu, best[kind].i, o));
                if (lane == 0) { sv[kind][wib] = best[kind].v; si[kind][wib] = best[kind].i; }
            }
            __syncthreads();
            if (threadIdx.x == 0) {
#pragma unroll
                for (int kind = 0; kind < 2; kind++) {
                    Cand c{sv[kind][0], si[kind][0]};
#pragma unroll
                    for (int w = 1; w < 8; w++) cand_take(c, sv[kind][w], si[kind][w]);
                    best[kind] = c;
                }
                int em = 0;
                if (tb < st_len) {
                    const int k = best[0].i;
                    int dur = p.ND > 0 ? p.durations[best[1].i - V] : (k == p.blank ? 1 : 0);
                    if (k != p.blank) {
                        const int no = st_no;
                        if (no < p.cap) { p.tokens[(size_t)b * p.cap + no] = k; p.frames[(size_t)b * p.cap + no] = tb; p.n_out[b] = no + 1; }
                        em = 1;
                        p.last_tok[b] = k;
                        const int eh = st_eh + 1;
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
                if (tb < st_len) atomicExch(&fl[1], 0);
            }
        }
        grid.sync();
        PHASE_MARK(2);
        const int any_emit = *reinterpret_cast<volatile int *>(&fl[0]);
        const int all_done = *reinterpret_cast<volatile int *>(&fl[1]);
        if (timing) { p.dbg[5] += 1; p.dbg[6] += any_emit; }
        if (any_emit) {
            for (int l = 0; l < p.L; l++) { lstm_phase(p, l, par, xhi, xlo, red, lane, wib); grid.sync(); }
            PHASE_MARK(3);
            par ^= 1;
            proj_phase(p, par, false, xhi, xlo, red, lane, wib);
            grid.sync();
            PHASE_MARK(4);
        }
        jx_valid = any_emit != 0;
        if (all_done) break;
    }
#undef PHASE_MARK
    if (blockIdx.x == 0 && threadIdx.x == 0) { p.flags[4] = par; if (p.par_state) *p.par_state = par; }
}

int greedy_launch(const GreedyDev &p, cudaStream_t st, int want_blocks) {
    int dev = 0, sms = 0, coop = 0;
    MB_CUDA(cudaGetDevice(&dev));
    MB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    MB_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    if (!coop) { set_error("greedy decode: device lacks cooperative launch"); return -1; }
    const size_t smem = 2 * 16 * (size_t)(2 * p.H + XPAD) * sizeof(__half) + 8 * 32 * 8 * sizeof(float);
    if (smem > 48 * 1024)
        MB_CUDA(cudaFuncSetAttribute(greedy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int per_sm = 0;
    MB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, greedy_kernel, 256, smem));
    if (per_sm < 1) { set_error("greedy decode: kernel does not fit an SM"); return -1; }
    int blocks = want_blocks > 0 && want_blocks < sms ? want_blocks : sms;
    if (blocks < p.B) { set_error("greedy decode: batch %d exceeds SM count", p.B); return -1; }
    GreedyDev pc = p;
    void *args[] = {&pc};
    MB_CUDA(cudaLaunchCooperativeKernel((void *)greedy_kernel, dim3(blocks), dim3(256), args, smem, st));
    return 0;
}

}  // namespace mb
