// Relative-position multi-head self-attention of the FastConformer block
// (the reference's attention / attention_banded, src/encoder.c:220-410):
//
//   s[t,j] = ((q_t + bias_u) . k_j  +  (q_t + bias_v) . rk[T-1+j-t]) / sqrt(dk)
//   p = softmax over the visible window, ctx_t = sum_j p[t,j] v_j
//
// rk = pos_emb * relative_k_proj^T is produced by the contraction kernel; the
// rel-shift bd[t, T-1+j-t] is applied in closed form (src/encoder.c:385-386), so
// neither the [T,T] scores nor the [T,2T-1] position term ever reach HBM.
//
// Tiled kernel: one CTA = 64 queries of one (segment, head), four warps of 16
// queries, key tiles of 64. K, V and the 127-row window of rk that the tile's
// diagonals touch are staged in shared memory as fp16; both score terms and P.V
// run on the warp-level tensor-core path (mma.sync m16n8k16, f32 accumulate) with
// an online softmax in f32. The position term of a warp is a 16 x 80 band whose
// skew (column c - r) is undone through a small per-warp shared buffer.
//
// The window for left >= 0 is the reference's chunked-limited one: chunks of
// right+1 frames, left/chunk chunks back (src/encoder.c:371-381).
#include "kernels.h"

namespace mb {

struct AttnDev {
    const float *q;
    int ldq;
    const __half *k, *v, *rk;        // fp16 [rows, d]
    const float *bias_u, *bias_v;
    float *ctx_f32;
    __half *ctx_hi, *ctx_lo;
    const int *seg_off, *seg_len, *rk_off;
    int d, H, left, right;
    float scaling;
};

__device__ __forceinline__ void window(const AttnDev &a, int t, int len, int &jlo, int &jhi) {
    if (a.left < 0) { jlo = 0; jhi = len; return; }
    const int chunk = a.right + 1, lc = a.left / chunk, tc = t / chunk;
    jlo = (tc - lc) * chunk; if (jlo < 0) jlo = 0;
    jhi = (tc + 1) * chunk; if (jhi > len) jhi = len;
}

// ------------------------------------------------------------------ plain kernel
// One warp per (segment, head, query). Same operand rounding as the tiled kernel
// (fp16 q+bias, k, rk, v; f32 accumulation), different summation order. Used by the
// tests as an on-device cross-check.
__global__ void __launch_bounds__(128)
attn_plain_kernel(AttnDev a, int max_len) {
    const int b = blockIdx.z, h = blockIdx.y;
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int len = a.seg_len[b];
    if (t >= len) return;
    const int off = a.seg_off[b], dk = a.d / a.H, ho = h * dk;
    const __half *rk = a.rk + (size_t)a.rk_off[b] * a.d;
    const int per = dk / 32;   // dk in {32,64,96,128}
    float qu[4], qv[4], acc[4] = {0, 0, 0, 0};
    for (int i = 0; i < per; i++) {
        const float qq = a.q[(size_t)(off + t) * a.ldq + ho + lane * per + i];
        qu[i] = __half2float(__float2half_rn(qq + a.bias_u[ho + lane * per + i]));
        qv[i] = __half2float(__float2half_rn(qq + a.bias_v[ho + lane * per + i]));
    }
    int jlo, jhi;
    window(a, t, len, jlo, jhi);
    float m = -3.0e38f, l = 0.0f;
    for (int j = jlo; j < jhi; j++) {
        const __half *kr = a.k + (size_t)(off + j) * a.d + ho + lane * per;
        const __half *pr = rk + (size_t)(len - 1 + j - t) * a.d + ho + lane * per;
        float s = 0.0f;
        for (int i = 0; i < per; i++) s += qu[i] * __half2float(kr[i]) + qv[i] * __half2float(pr[i]);
        s = warp_sum(s) * a.scaling;
        const float mn = fmaxf(m, s), corr = expf(m - mn), p = expf(s - mn);
        const float ph = __half2float(__float2half_rn(p));
        const __half *vr = a.v + (size_t)(off + j) * a.d + ho + lane * per;
        l = l * corr + p;
        for (int i = 0; i < per; i++) acc[i] = acc[i] * corr + ph * __half2float(vr[i]);
        m = mn;
    }
    const float inv = 1.0f / l;
    for (int i = 0; i < per; i++) {
        const float y = acc[i] * inv;
        const size_t o = (size_t)(off + t) * a.d + ho + lane * per + i;
        if (a.ctx_f32) a.ctx_f32[o] = y;
        if (a.ctx_hi) {
            __half hh, ll;
            split_h16(y, hh, ll);
            a.ctx_hi[o] = hh;
            if (a.ctx_lo) a.ctx_lo[o] = ll;
        }
    }
}

// ------------------------------------------------------------------ tiled kernel
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float x, float y) {
    __half2 h = __floats2half2_rn(x, y);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ void ldsm_x4(uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3, const void *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_u32(p)));
}
// 16-byte asynchronous global -> shared copy; `valid` false writes zeros without reading.
__device__ __forceinline__ void cp_async16_zfill(void *dst, const void *src, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(valid ? 16 : 0)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x2_trans(uint32_t &r0, uint32_t &r1, const void *p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(smem_u32(p)));
}

static constexpr int AT_Q = 64, AT_K = 64, AT_BDW = 80, AT_BDS = 81;

template <int DK>
__global__ void __launch_bounds__(128, 2)
attn_tiled_kernel(AttnDev a) {
    constexpr int LD = DK + 8;                       // padded fp16 row (conflict-free fragment loads)
    extern __shared__ __align__(16) uint8_t smem_at[];
    __half *Ks = reinterpret_cast<__half *>(smem_at);
    __half *Vs = Ks + AT_K * LD;
    __half *Rs = Vs + AT_K * LD;                     // 128 rows of the rk window
    float *BD = reinterpret_cast<float *>(Rs + 128 * LD);

    const int b = blockIdx.z, h = blockIdx.y, tq0 = blockIdx.x * AT_Q;
    const int len = a.seg_len[b];
    if (tq0 >= len) return;
    const int off = a.seg_off[b], ho = h * DK;
    const __half *rkg = a.rk + (size_t)a.rk_off[b] * a.d;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    float *BDw = BD + warp * 16 * AT_BDS;

    // ---- query fragments (A operand), both bias flavours, rounded to fp16 once
    uint32_t qu[DK / 16][4], qv[DK / 16][4];
    {
        const int r0 = tq0 + warp * 16 + g, r1 = r0 + 8;
        const float *q0 = a.q + (size_t)(off + r0) * a.ldq + ho;
        const float *q1 = a.q + (size_t)(off + r1) * a.ldq + ho;
#pragma unroll
        for (int ks = 0; ks < DK / 16; ks++) {
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {
                const int c = ks * 16 + hf * 8 + 2 * tq;
                const float2 u = *reinterpret_cast<const float2 *>(a.bias_u + ho + c);
                const float2 vb = *reinterpret_cast<const float2 *>(a.bias_v + ho + c);
                float2 x0 = make_float2(0.f, 0.f), x1 = make_float2(0.f, 0.f);
                if (r0 < len) x0 = *reinterpret_cast<const float2 *>(q0 + c);
                if (r1 < len) x1 = *reinterpret_cast<const float2 *>(q1 + c);
                qu[ks][hf * 2 + 0] = pack_h2(x0.x + u.x, x0.y + u.y);
                qu[ks][hf * 2 + 1] = pack_h2(x1.x + u.x, x1.y + u.y);
                qv[ks][hf * 2 + 0] = pack_h2(x0.x + vb.x, x0.y + vb.y);
                qv[ks][hf * 2 + 1] = pack_h2(x1.x + vb.x, x1.y + vb.y);
            }
        }
    }

    // rows of this lane: t0 = first, t1 = t0 + 8
    const int t0 = tq0 + warp * 16 + g, t1 = t0 + 8;
    int jlo0, jhi0, jlo1, jhi1;
    window(a, t0 < len ? t0 : len - 1, len, jlo0, jhi0);
    window(a, t1 < len ? t1 : len - 1, len, jlo1, jhi1);
    // key range the whole CTA has to visit
    int cta_lo, cta_hi, tmp;
    window(a, tq0, len, cta_lo, tmp);
    window(a, (tq0 + AT_Q - 1 < len) ? tq0 + AT_Q - 1 : len - 1, len, tmp, cta_hi);

    float o[DK / 8][4];
#pragma unroll
    for (int i = 0; i < DK / 8; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -3.0e38f, m1 = -3.0e38f, l0 = 0.f, l1 = 0.f;

    for (int j0 = (cta_lo / AT_K) * AT_K; j0 < cta_hi; j0 += AT_K) {
        __syncthreads();
        // ---- stage K and the rk window (group 0), then V (group 1), as asynchronous 16-byte copies:
        // the score terms start as soon as group 0 has landed, V arrives under them
        constexpr int CPR = DK / 8;                   // 16-byte chunks per row
        const int pbase = len - 1 + j0 - tq0 - (AT_Q - 1);
        for (int i = threadIdx.x; i < AT_K * CPR; i += 128) {
            const int r = i / CPR, c = (i % CPR) * 8;
            const bool ok = j0 + r < len;
            cp_async16_zfill(Ks + r * LD + c, a.k + (size_t)(off + (ok ? j0 + r : 0)) * a.d + ho + c, ok);
        }
        for (int i = threadIdx.x; i < 128 * CPR; i += 128) {
            const int r = i / CPR, c = (i % CPR) * 8, p = pbase + r;
            const bool ok = p >= 0 && p <= 2 * len - 2;
            cp_async16_zfill(Rs + r * LD + c, rkg + (size_t)(ok ? p : 0) * a.d + ho + c, ok);
        }
        cp_async_commit();
        for (int i = threadIdx.x; i < AT_K * CPR; i += 128) {
            const int r = i / CPR, c = (i % CPR) * 8;
            const bool ok = j0 + r < len;
            cp_async16_zfill(Vs + r * LD + c, a.v + (size_t)(off + (ok ? j0 + r : 0)) * a.d + ho + c, ok);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        // ---- content term: S = (q+u) K^T, 16 x 64 per warp
        float s[AT_K / 8][4];
#pragma unroll
        for (int nb = 0; nb < AT_K / 8; nb++) { s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f; }
        // B fragments by ldmatrix.x4: one load covers two k-steps of an 8-key block
        const int lrow = lane & 7, lcol = (lane >> 3) * 8;
#pragma unroll
        for (int ks = 0; ks < DK / 16; ks += 2) {
#pragma unroll
            for (int nb = 0; nb < AT_K / 8; nb++) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4(b0, b1, b2, b3, Ks + (nb * 8 + lrow) * LD + ks * 16 + lcol);
                mma16816(s[nb], qu[ks], b0, b1);
                mma16816(s[nb], qu[ks + 1], b2, b3);
            }
        }
        // ---- position term: band of 80 rk rows for this warp, skewed back through BDw
        const int rbase = 48 - 16 * warp;            // window row of band column 0
#pragma unroll
        for (int half = 0; half < 2; half++) {
            float bd[AT_BDW / 16][4];
#pragma unroll
            for (int nb = 0; nb < AT_BDW / 16; nb++) { bd[nb][0] = bd[nb][1] = bd[nb][2] = bd[nb][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < DK / 16; ks += 2) {
#pragma unroll
                for (int nb = 0; nb < AT_BDW / 16; nb++) {
                    const int x = (half * (AT_BDW / 16) + nb) * 8 + lrow;
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(b0, b1, b2, b3, Rs + (rbase + x) * LD + ks * 16 + lcol);
                    mma16816(bd[nb], qv[ks], b0, b1);
                    mma16816(bd[nb], qv[ks + 1], b2, b3);
                }
            }
#pragma unroll
            for (int nb = 0; nb < AT_BDW / 16; nb++) {
                const int x = (half * (AT_BDW / 16) + nb) * 8 + 2 * tq;
                BDw[g * AT_BDS + x] = bd[nb][0];
                BDw[g * AT_BDS + x + 1] = bd[nb][1];
                BDw[(g + 8) * AT_BDS + x] = bd[nb][2];
                BDw[(g + 8) * AT_BDS + x + 1] = bd[nb][3];
            }
        }
        __syncwarp();
        // ---- scores, mask, online softmax
        float mx0 = m0, mx1 = m1;
#pragma unroll
        for (int nb = 0; nb < AT_K / 8; nb++) {
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int c = nb * 8 + 2 * tq + e, j = j0 + c;
                const float v0 = (s[nb][e] + BDw[g * AT_BDS + c - g + 15]) * a.scaling;
                const float v1 = (s[nb][2 + e] + BDw[(g + 8) * AT_BDS + c - (g + 8) + 15]) * a.scaling;
                const bool ok0 = j >= jlo0 && j < jhi0, ok1 = j >= jlo1 && j < jhi1;
                s[nb][e] = ok0 ? v0 : -3.0e38f;
                s[nb][2 + e] = ok1 ? v1 : -3.0e38f;
                if (ok0) mx0 = fmaxf(mx0, v0);
                if (ok1) mx1 = fmaxf(mx1, v1);
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float c0 = expf(m0 - mx0), c1 = expf(m1 - mx1);
        m0 = mx0; m1 = mx1;
        float ps0 = 0.f, ps1 = 0.f;
        uint32_t pa[AT_K / 16][4];
#pragma unroll
        for (int nb = 0; nb < AT_K / 8; nb++) {
            float p[4];
#pragma unroll
            for (int e = 0; e < 2; e++) {
                p[e] = s[nb][e] > -1.0e38f ? expf(s[nb][e] - mx0) : 0.f;
                p[2 + e] = s[nb][2 + e] > -1.0e38f ? expf(s[nb][2 + e] - mx1) : 0.f;
            }
            ps0 += p[0] + p[1];
            ps1 += p[2] + p[3];
            pa[nb >> 1][(nb & 1) * 2 + 0] = pack_h2(p[0], p[1]);
            pa[nb >> 1][(nb & 1) * 2 + 1] = pack_h2(p[2], p[3]);
        }
        l0 = l0 * c0 + ps0;
        l1 = l1 * c1 + ps1;
#pragma unroll
        for (int i = 0; i < DK / 8; i++) { o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1; }
        // ---- O += P V  (B fragments via transposed ldmatrix on row-major V)
        cp_async_wait<0>();
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < AT_K / 16; ks++) {
#pragma unroll
            for (int nb = 0; nb < DK / 8; nb++) {
                uint32_t b0, b1;
                ldsm_x2_trans(b0, b1, Vs + (ks * 16 + (lane & 15)) * LD + nb * 8);
                mma16816(o[nb], pa[ks], b0, b1);
            }
        }
        __syncwarp();
    }
    // ---- normalise and store
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float i0 = l0 > 0.f ? 1.0f / l0 : 0.f, i1 = l1 > 0.f ? 1.0f / l1 : 0.f;
#pragma unroll
    for (int nb = 0; nb < DK / 8; nb++) {
        const int c = ho + nb * 8 + 2 * tq;
#pragma unroll
        for (int rr = 0; rr < 2; rr++) {
            const int t = rr ? t1 : t0;
            if (t >= len) continue;
            const float y0 = o[nb][rr * 2] * (rr ? i1 : i0), y1 = o[nb][rr * 2 + 1] * (rr ? i1 : i0);
            const size_t idx = (size_t)(off + t) * a.d + c;
            if (a.ctx_f32) *reinterpret_cast<float2 *>(a.ctx_f32 + idx) = make_float2(y0, y1);
            if (a.ctx_hi) {
                __half h0, lw0, h1, lw1;
                split_h16(y0, h0, lw0);
                split_h16(y1, h1, lw1);
                *reinterpret_cast<__half2 *>(a.ctx_hi + idx) = __halves2half2(h0, h1);
                if (a.ctx_lo) *reinterpret_cast<__half2 *>(a.ctx_lo + idx) = __halves2half2(lw0, lw1);
            }
        }
    }
}

template <int DK>
static int launch_tiled(const AttnDev &dv, int batch, int max_len, cudaStream_t st) {
    constexpr int LD = DK + 8;
    const int smem = (2 * AT_K + 128) * LD * 2 + 4 * 16 * AT_BDS * 4;
    static PerDevice configured = {};
    int dev = 0;
    if (configured.below((size_t)smem, &dev)) {
        MB_CUDA(cudaFuncSetAttribute(attn_tiled_kernel<DK>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        configured.record(dev, (size_t)smem);
    }
    dim3 grid(cdiv(max_len, AT_Q), dv.H, batch);
    attn_tiled_kernel<DK><<<grid, 128, smem, st>>>(dv);
    MB_CUDA(cudaGetLastError());
    return 0;
}

int attention_forward(const AttnArgs &a, int impl, cudaStream_t st) {
    if (a.batch <= 0 || a.max_len <= 0) return 0;
    const int dk = a.d / a.H;
    AttnDev dv;
    dv.q = a.q; dv.ldq = a.ldq; dv.k = a.k; dv.v = a.v; dv.rk = a.rk;
    dv.bias_u = a.bias_u; dv.bias_v = a.bias_v; dv.ctx_f32 = a.ctx_f32;
    dv.ctx_hi = a.ctx_h.hi; dv.ctx_lo = a.ctx_h.lo;
    dv.seg_off = a.seg_off; dv.seg_len = a.seg_len; dv.rk_off = a.rk_off;
    dv.d = a.d; dv.H = a.H; dv.left = a.left; dv.right = a.right;
    dv.scaling = 1.0f / sqrtf((float)dk);
    if (impl == 0 && attention_tc_eligible(a)) return attention_tc(a, st);
    if ((impl == 0 || impl == 2) && (dk == 64 || dk == 128) && (a.ldq % 2) == 0 && (a.d % 8) == 0) {
        return dk == 64 ? launch_tiled<64>(dv, a.batch, a.max_len, st) : launch_tiled<128>(dv, a.batch, a.max_len, st);
    }
    if (dk % 32 != 0 || dk > 128) { set_error("attention: head dim %d unsupported", dk); return -1; }
    dim3 grid(cdiv(a.max_len, 4), a.H, a.batch);
    attn_plain_kernel<<<grid, 128, 0, st>>>(dv, a.max_len);
    MB_CUDA(cudaGetLastError());
    return 0;
}

}  // namespace mb
