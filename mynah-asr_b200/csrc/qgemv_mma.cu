// Weight-streaming small-T matmul for the ggml 32-element block formats (Q4_0, Q8_0) on the
// warp-level tensor-core path: out[T,n] = x[T,k] W^T, T <= 4 per launch.
//
// The scalar kernel (qgemv.cu) spends ~7 issue slots per weight on nibble extraction,
// int->float conversion and the FMA, which caps it far below HBM bandwidth. Here the
// stored integers become fp16 MMA fragments with ~1.5 logic instructions per weight
// (two weights per LOP3 / PRMT, `q | 0x6400` is the fp16 number 1024 + q, one HSUB2 takes
// the offset off again) and mma.sync m16n8k16 does the multiply-accumulate:
//   * M side = 16 weight rows of a warp; the 8 columns of the N side are the (hi, lo)
//     fp16 planes of up to 4 activation rows (column 2j = hi of row j, 2j+1 = lo), so one
//     MMA forms q*x_hi and q*x_lo together and a lane ends up holding both for "its"
//     activation row; K = one 32-element block = two k-steps; q is exact in fp16, hence
//     q*x is formed to f32 grade;
//   * the block's f16 scale d multiplies the block's accumulator afterwards
//     (out += d * sum_k q_k x_k), which is exactly the reference's decode w = d*q
//     (third_party/ingot/src/dequant.c:72-83,131-156) followed by an f32 dot.
// Within a block the k order is free (the same permutation is applied to the activations
// when they are staged), so the fragments are built from whole 32-bit words.
//
// Weights are re-tiled once at load into a layout in which every lane's loads are 16-byte
// vectors (same bytes per parameter as the stored blocks: 0.5625 Q4_0, 1.0625 Q8_0).
#include "kernels.h"
#include "qweight.h"

namespace mb {

static constexpr int QM_WARPS = 8;
static constexpr int QM_DEPTH = 6;        // groups of stored bytes in flight per warp
static constexpr int QM_SLOT = 1152;      // 2 x 512 B of quants + 2 x 64 B of scales

template <int BYTES>
__device__ __forceinline__ void cp_async(void *dst, const void *src) {
    if (BYTES == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(smem_u32(dst)), "l"(src), "n"(BYTES) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ------------------------------------------------------------------ re-tiling
// Q4_0: per row, per group of 4 blocks, per t in 0..3: bytes 4t..4t+3 of each of the 4 blocks.
// Q8_0: per row, per group of 2 blocks, per t in 0..3: bytes 8t..8t+7 of each of the 2 blocks.
// Scales: f16 [n][k/32].
__global__ void retile_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ qs, __half *__restrict__ ds,
                              int n, int k, int fmt) {
    const size_t nblk = (size_t)n * (k / 32);
    const size_t b = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (b >= nblk) return;
    const int bpr = k / 32;
    const size_t row = b / bpr;
    const int blk = (int)(b % bpr);
    if (fmt == FMT_GGML_Q4_0) {
        const uint8_t *p = raw + b * 18;
        ds[b] = __ushort_as_half((unsigned short)(p[0] | (p[1] << 8)));
        uint8_t *dst = qs + row * (size_t)(k / 2) + (size_t)(blk / 4) * 64 + (blk % 4) * 4;
        for (int t = 0; t < 4; t++)
            for (int i = 0; i < 4; i++) dst[t * 16 + i] = p[2 + 4 * t + i];
    } else {
        const uint8_t *p = raw + b * 34;
        ds[b] = __ushort_as_half((unsigned short)(p[0] | (p[1] << 8)));
        uint8_t *dst = qs + row * (size_t)k + (size_t)(blk / 2) * 64 + (blk % 2) * 8;
        for (int t = 0; t < 4; t++)
            for (int i = 0; i < 8; i++) dst[t * 16 + i] = p[2 + 8 * t + i];
    }
}

int qgemv_mma_retile(const QWeight &w, uint8_t *qs, __half *ds, cudaStream_t st) {
    const size_t nblk = (size_t)w.n * (w.k / 32);
    retile_kernel<<<(unsigned)((nblk + 255) / 256), 256, 0, st>>>(w.raw, qs, ds, w.n, w.k, w.fmt);
    MB_CUDA(cudaGetLastError());
    return 0;
}

// ------------------------------------------------------------------ fragments
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t hsub2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
// Q4_0 word (bytes b0..b3 of one lane's share of a block; low nibble = element 4t+i, high nibble =
// element 16+4t+i). Returns the two k-steps' fragments as fp16 pairs of q-8:
//   lo[0] = (e0, e2), lo[1] = (e1, e3) from the low nibbles, hi[0..1] likewise from the high nibbles.
__device__ __forceinline__ void q4_frag(uint32_t w, uint32_t (&lo)[2], uint32_t (&hi)[2]) {
    constexpr uint32_t M = 0x000F000Fu, E = 0x64006400u, OFF = 0x64086408u;   // 1024 + 8 in both halves
    lo[0] = hsub2((w & M) | E, OFF);
    lo[1] = hsub2(((w >> 8) & M) | E, OFF);
    hi[0] = hsub2(((w >> 4) & M) | E, OFF);
    hi[1] = hsub2(((w >> 12) & M) | E, OFF);
}
// Q8_0 word (int8 e0..e3): fp16 pairs (e0, e1) and (e2, e3).
__device__ __forceinline__ void q8_frag(uint32_t w, uint32_t (&f)[2]) {
    constexpr uint32_t E = 0x64646464u, OFF = 0x64806480u;                    // 1024 + 128
    const uint32_t u = w ^ 0x80808080u;                                        // signed -> biased unsigned
    f[0] = hsub2(__byte_perm(u, E, 0x4140), OFF);
    f[1] = hsub2(__byte_perm(u, E, 0x4342), OFF);
}

// activation slot of element e (0..31) of a block, matching the fragment order above
__device__ __forceinline__ int x_slot(int fmt, int e) {
    if (fmt == FMT_GGML_Q4_0) {
        const int s = e >> 4, t = (e & 15) >> 2, i = e & 3;
        return s * 16 + t * 4 + ((i & 1) * 2 + (i >> 1));        // (e0, e2, e1, e3)
    }
    const int t = e >> 3, j = e & 7;                             // lane t owns elements 8t..8t+7
    return (j >> 2) * 16 + t * 4 + (j & 3);
}

struct QmArgs {
    const uint8_t *qs;
    const __half *ds;
    int n, k;
    const float *x;
    int ldx;
    float *out;
    int ldo;
    const float *bias;
    int T;
};

// One warp: 16 weight rows x one K slice. KS warps of a CTA share a row tile (K split), the
// remaining factor of the 8 warps covers consecutive row tiles.
template <int FMT>
__global__ void __launch_bounds__(QM_WARPS * 32, 2)
qgemv_mma_kernel(const QmArgs a, const int ks_log2) {
    extern __shared__ __align__(16) uint8_t qm_smem[];
    __half *xh = reinterpret_cast<__half *>(qm_smem);              // [T][k] permuted, hi
    const int xs = a.k + 16;                                       // padded row: spreads the rows over banks
    __half *xl = xh + (size_t)a.T * xs;                            // lo (pre-scaled by 2^11)
    float *red = reinterpret_cast<float *>(xl + (size_t)a.T * xs);    // [8 warps][32 lanes][4]
    uint8_t *ring_base = reinterpret_cast<uint8_t *>(red + QM_WARPS * 32 * 4);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int KS = 1 << ks_log2, kslice = warp & (KS - 1), tiles_per_cta = QM_WARPS >> ks_log2;
    const int nblk = a.k / 32;

    // ---- stage the activations once: fp16 (hi, lo), block-permuted
    for (int i = threadIdx.x; i < a.T * a.k; i += blockDim.x) {
        const int row = i / a.k, e = i % a.k;
        __half h, l;
        split_h16(a.x[(size_t)row * a.ldx + e], h, l);
        const int dst = row * xs + (e & ~31) + x_slot(FMT, e & 31);
        xh[dst] = h;
        xl[dst] = l;
    }
    __syncthreads();

    constexpr int BPG = FMT == FMT_GGML_Q4_0 ? 4 : 2;             // blocks per 64-byte group
    const int ngrp = nblk / BPG;
    const int g0 = (int)((long long)ngrp * kslice / KS), g1 = (int)((long long)ngrp * (kslice + 1) / KS);
    const size_t rowq = FMT == FMT_GGML_Q4_0 ? (size_t)a.k / 2 : (size_t)a.k;
    // B column g of the MMA = plane (g & 1) of activation row g >> 1
    const bool colon = (g >> 1) < a.T;
    const __half *xcol = ((g & 1) ? xl : xh) + (size_t)(colon ? (g >> 1) : 0) * xs + t * 4;
    const int ntiles = (a.n + 15) / 16;

    for (int tile0 = blockIdx.x * tiles_per_cta; tile0 < ntiles; tile0 += gridDim.x * tiles_per_cta) {
        const int tile = tile0 + (warp >> ks_log2);
        float acc[2] = {0.f, 0.f};                                // rows g and g+8, activation row t
        if (tile < ntiles) {
            const int rA = min(tile * 16 + g, a.n - 1), rB = min(tile * 16 + g + 8, a.n - 1);
            const uint4 *qA = reinterpret_cast<const uint4 *>(a.qs + (size_t)rA * rowq) + t;
            const uint4 *qB = reinterpret_cast<const uint4 *>(a.qs + (size_t)rB * rowq) + t;
            const __half *dA = a.ds + (size_t)rA * nblk, *dB = a.ds + (size_t)rB * nblk;
            // the stored bytes go through a per-warp ring of asynchronous copies (QM_DEPTH groups in
            // flight per warp) so that HBM latency is covered without spending registers on it
            uint8_t *ring = ring_base + warp * (QM_DEPTH * QM_SLOT);
            auto issue = [&](int grp, int slot) {
                uint8_t *sl = ring + slot * QM_SLOT;
                cp_async<16>(sl + lane * 16, qA + grp * 4);
                cp_async<16>(sl + 512 + lane * 16, qB + grp * 4);
                if (t == 0) {
                    cp_async<BPG * 2>(sl + 1024 + g * 8, dA + grp * BPG);
                    cp_async<BPG * 2>(sl + 1088 + g * 8, dB + grp * BPG);
                }
            };
#pragma unroll
            for (int i = 0; i < QM_DEPTH; i++) {
                if (g0 + i < g1) issue(g0 + i, i);
                cp_async_commit();
            }
            for (int grp = g0; grp < g1; grp++) {
                const int slot = (grp - g0) % QM_DEPTH;
                const uint8_t *sl = ring + slot * QM_SLOT;
                cp_async_wait<QM_DEPTH - 1>();
                __syncwarp();
                const uint4 wa = *reinterpret_cast<const uint4 *>(sl + lane * 16);
                const uint4 wb = *reinterpret_cast<const uint4 *>(sl + 512 + lane * 16);
                const uint32_t wav[4] = {wa.x, wa.y, wa.z, wa.w}, wbv[4] = {wb.x, wb.y, wb.z, wb.w};
                float da[BPG], db[BPG];
                if (BPG == 4) {
                    const uint2 ua = *reinterpret_cast<const uint2 *>(sl + 1024 + g * 8);
                    const uint2 ub = *reinterpret_cast<const uint2 *>(sl + 1088 + g * 8);
                    const __half2 a01 = *reinterpret_cast<const __half2 *>(&ua.x), a23 = *reinterpret_cast<const __half2 *>(&ua.y);
                    const __half2 b01 = *reinterpret_cast<const __half2 *>(&ub.x), b23 = *reinterpret_cast<const __half2 *>(&ub.y);
                    da[0] = __low2float(a01); da[1] = __high2float(a01); da[2] = __low2float(a23); da[3] = __high2float(a23);
                    db[0] = __low2float(b01); db[1] = __high2float(b01); db[2] = __low2float(b23); db[3] = __high2float(b23);
                } else {
                    const __half2 a01 = *reinterpret_cast<const __half2 *>(sl + 1024 + g * 8);
                    const __half2 b01 = *reinterpret_cast<const __half2 *>(sl + 1088 + g * 8);
                    da[0] = __low2float(a01); da[1] = __high2float(a01);
                    db[0] = __low2float(b01); db[1] = __high2float(b01);
                }
#pragma unroll
                for (int b = 0; b < BPG; b++) {
                    const int blk = grp * BPG + b;
                    // activations of this block: k-step 0 at +0, k-step 1 at +16 (4 halves each)
                    uint2 x0 = make_uint2(0, 0), x1 = make_uint2(0, 0);
                    if (colon) {
                        x0 = *reinterpret_cast<const uint2 *>(xcol + blk * 32);
                        x1 = *reinterpret_cast<const uint2 *>(xcol + blk * 32 + 16);
                    }
                    float c[4] = {0.f, 0.f, 0.f, 0.f};            // (row g: hi, lo), (row g+8: hi, lo) of activation row t
                    if (FMT == FMT_GGML_Q4_0) {
                        uint32_t alo[2], ahi[2], blo[2], bhi[2];
                        q4_frag(wav[b], alo, ahi);
                        q4_frag(wbv[b], blo, bhi);
                        mma16816(c, alo[0], blo[0], alo[1], blo[1], x0.x, x0.y);
                        mma16816(c, ahi[0], bhi[0], ahi[1], bhi[1], x1.x, x1.y);
                    } else {
                        uint32_t a0[2], a1[2], b0[2], b1[2];
                        q8_frag(wav[2 * b], a0); q8_frag(wav[2 * b + 1], a1);
                        q8_frag(wbv[2 * b], b0); q8_frag(wbv[2 * b + 1], b1);
                        mma16816(c, a0[0], b0[0], a0[1], b0[1], x0.x, x0.y);
                        mma16816(c, a1[0], b1[0], a1[1], b1[1], x1.x, x1.y);
                    }
                    // out += d * (q.x_hi + 2^-11 q.x_lo)
                    acc[0] = fmaf(da[b], fmaf(c[1], H16_LO_INV, c[0]), acc[0]);
                    acc[1] = fmaf(db[b], fmaf(c[3], H16_LO_INV, c[2]), acc[1]);
                }
                __syncwarp();                                   // every lane is done with this slot
                if (grp + QM_DEPTH < g1) issue(grp + QM_DEPTH, slot);
                cp_async_commit();
            }
            cp_async_wait<0>();
        }
        if (KS > 1) {
            red[(warp * 32 + lane) * 4 + 0] = acc[0];
            red[(warp * 32 + lane) * 4 + 1] = acc[1];
            __syncthreads();
        }
        if (tile < ntiles && kslice == 0) {
#pragma unroll
            for (int i = 0; i < 2; i++) {
                float v = acc[i];
                for (int q = 1; q < KS; q++) v += red[((warp + q) * 32 + lane) * 4 + i];   // fixed order
                const int r = tile * 16 + g + i * 8;
                if (r < a.n && t < a.T) a.out[(size_t)t * a.ldo + r] = v + (a.bias ? a.bias[r] : 0.0f);
            }
        }
        if (KS > 1) __syncthreads();
    }
}

int qgemv_mma(const QWeight &w, const float *x, int ldx, float *out, int ldo, const float *bias, int T, cudaStream_t st) {
    if (!w.mma_q || !w.mma_d) { set_error("qgemv_mma: weight has no re-tiled planes"); return -1; }
    const int sms = device_sm_count();
    const int ntiles = cdiv(w.n, 16);
    int ks_log2 = 0;                      // split K over warps until the grid is full (or slices get short)
    while (ks_log2 < 3 && (ntiles << ks_log2) < sms * QM_WARPS * 2 && (w.k >> (ks_log2 + 1)) >= 512) ks_log2++;
    for (int t0 = 0; t0 < T; t0 += 4) {
        QmArgs a;
        a.qs = w.mma_q; a.ds = w.mma_d; a.n = w.n; a.k = w.k;
        a.T = T - t0 < 4 ? T - t0 : 4;
        a.x = x + (size_t)t0 * ldx; a.ldx = ldx; a.out = out + (size_t)t0 * ldo; a.ldo = ldo; a.bias = bias;
        const size_t smem = (size_t)a.T * (w.k + 16) * 4 + QM_WARPS * 32 * 4 * sizeof(float) + QM_WARPS * QM_DEPTH * QM_SLOT;
        if (smem > 200 * 1024) { set_error("qgemv_mma: T*k too large for shared memory"); return -1; }
        const int tiles_per_cta = QM_WARPS >> ks_log2;
        int blocks = cdiv(ntiles, tiles_per_cta);
        if (blocks > sms * 2) blocks = sms * 2;
        if (w.fmt == FMT_GGML_Q4_0) {
            MB_CUDA(cudaFuncSetAttribute(qgemv_mma_kernel<FMT_GGML_Q4_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            qgemv_mma_kernel<FMT_GGML_Q4_0><<<blocks, QM_WARPS * 32, smem, st>>>(a, ks_log2);
        } else {
            MB_CUDA(cudaFuncSetAttribute(qgemv_mma_kernel<FMT_GGML_Q8_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            qgemv_mma_kernel<FMT_GGML_Q8_0><<<blocks, QM_WARPS * 32, smem, st>>>(a, ks_log2);
        }
        MB_CUDA(cudaGetLastError());
    }
    return 0;
}

}  // namespace mb
