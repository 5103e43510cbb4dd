// Weight-streaming quantised matmul with the block decode fused into the tcgen05 operand
// pipeline: out[T,n] = x[T,k] W^T for T <= 8, W stored as ggml Q4_0 / Q8_0 blocks.
// The bandwidth-bound half of the reference's mynah_asr_qmat_mul (src/qmat.c:508-597).
//
// Per CTA (persistent, one per SM), 32 warps with fixed roles:
//   * warp 0, one thread: streams the stored bytes of a stage (128 weight rows x 128 k: the
//     quants and the four f16 block scales per row, laid out contiguously at load) from HBM
//     into a shared-memory ring with bulk asynchronous copies (cp.async.bulk, no multicast)
//     tracked by mbarriers — 70-90 KB in flight per SM to cover HBM latency;
//   * warps 8-23, four groups of four: group g decodes block g of every stage. A thread owns
//     one weight row, turns its 32 integers into fp16 (`q | 0x6400` is the fp16 number 1024 + q,
//     so two weights cost one LOP3/PRMT and half an HSUB2) and writes them with tcgen05.st into
//     tensor memory, where they are the A operand — the decoded weights never touch shared memory;
//   * warps 1-4, one thread each: issuer g issues the tcgen05.mma (kind::f16, M = 128 weight rows,
//     N = 16, K = 16) of block g — one thread gets an MMA out every ~45 cycles whatever its size, so
//     the small ones here need several issuers — with A from tensor memory and B from shared memory: B is the fp16 (hi, lo) planes of up to 8
//     activation rows, resident in shared memory for the CTA's K slice. Each 32-element block
//     gets its own 16 accumulator columns, because the block scale d has to multiply the block's
//     dot afterwards (w = d*q, ingot dequant.c:72-83);
//   * warps 24-31, two groups of four: read the block dots back (tcgen05.ld; thread = weight row)
//     and fold them into f32 accumulators: out += d * (q.x_hi + 2^-11 q.x_lo);
//   * every warp but the streamer's first stages its share of the activations (warps 5-7 do only that).
// Large K, or few rows, are split over CTAs (fixed K slice per CTA, so its activations are staged
// once); the slices are then summed in a fixed order by a second small kernel, so results are
// reproducible. Every mbarrier wait is bounded; a wait that runs out sets a status word and the
// kernel unwinds.
#include "kernels.h"
#include "qweight.h"

namespace mb {

static constexpr int QS_ROWS = 128;           // weight rows per tile (UMMA M)
static constexpr int QS_SK = 128;             // k per stage
static constexpr int QS_NB = 4;               // 32-element blocks per stage
static constexpr int QS_N = 16;               // UMMA N: (hi, lo) x 8 activation rows
static constexpr int QS_MAX_SLICE_ST = 32;    // stages of K per CTA slice (4096 k)
static constexpr int QS_FIRST_ISSUER = 1;     // warps 1-4: one MMA issuer per block of the stage
static constexpr int QS_FIRST_DECODE = 8, QS_DECODE_WARPS = 16;
static constexpr int QS_FIRST_SCALE = 24, QS_SCALE_WARPS = 8;
static constexpr int QS_THREADS = (QS_FIRST_SCALE + QS_SCALE_WARPS) * 32;     // 1024
static constexpr int QS_X_CHUNK = QS_N * 128;                 // 2 KB: 16 rows x 64 k of fp16
static constexpr int QS_X_STAGE = 2 * QS_X_CHUNK;             // 4 KB per stage of K
static constexpr int QS_TMEM_COLS = 256;                      // A: 2 stages x 64 columns, D: 2 stages x 64
static constexpr int QS_D_COL0 = 128;
static constexpr int QS_SCALE_BYTES = QS_NB * QS_ROWS * 2;    // 1 KB of f16 block scales per stage

__host__ __device__ constexpr int qs_quant_bytes(int fmt) { return fmt == FMT_GGML_Q4_0 ? QS_ROWS * QS_SK / 2 : QS_ROWS * QS_SK; }
__host__ __device__ constexpr int qs_stage_bytes(int fmt) { return qs_quant_bytes(fmt) + QS_SCALE_BYTES; }
__host__ __device__ constexpr int qs_raw_depth(int fmt) { return fmt == FMT_GGML_Q4_0 ? 8 : 5; }

// -------------------------------------------------------------------- re-tiling at load
// [tile][stage][ quants: [16-byte chunk c][row 0..127][16 B] | scales: [block 0..3][row 0..127] f16 ]
// Q4_0: chunk c is block c (32 nibbles); Q8_0: chunks 2b, 2b+1 are the halves of block b.
// A decode warp reads consecutive 16-byte pieces: conflict-free 128-bit shared loads.
__global__ void qs_retile_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ dst, int n, int k, int fmt) {
    const size_t b = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    const int bpr = k / 32;
    if (b >= (size_t)n * bpr) return;
    const int row = (int)(b / bpr), blk = (int)(b % bpr);
    const int tile = row / QS_ROWS, rl = row % QS_ROWS, st = blk / QS_NB, bs = blk % QS_NB;
    const int qb = fmt == FMT_GGML_Q4_0 ? 16 : 32;
    uint8_t *stage = dst + ((size_t)tile * (k / QS_SK) + st) * qs_stage_bytes(fmt);
    const uint8_t *p = raw + b * (qb + 2);
    for (int i = 0; i < qb; i++) stage[((bs * (qb / 16) + i / 16) * QS_ROWS + rl) * 16 + (i & 15)] = p[2 + i];
    uint8_t *sc = stage + qs_quant_bytes(fmt) + (bs * QS_ROWS + rl) * 2;
    sc[0] = p[0];
    sc[1] = p[1];
}

size_t qstream_tc_bytes(int fmt, int n, int k) {
    return (size_t)cdiv(n, QS_ROWS) * (k / QS_SK) * qs_stage_bytes(fmt);
}

int qstream_tc_retile(const QWeight &w, uint8_t *dst, cudaStream_t st) {
    MB_CUDA(cudaMemsetAsync(dst, 0, qstream_tc_bytes(w.fmt, w.n, w.k), st));
    const size_t nblk = (size_t)w.n * (w.k / 32);
    qs_retile_kernel<<<(unsigned)((nblk + 255) / 256), 256, 0, st>>>(w.raw, dst, w.n, w.k, w.fmt);
    MB_CUDA(cudaGetLastError());
    return 0;
}

// K slices for an [n, k] weight on a device with `sms` multiprocessors: as few as the shared
// memory allows (4096 k of activations per CTA), more when the row tiles alone would leave
// most multiprocessors idle. Depends on the shape and the device only, never on T.
static int qs_pick_nslice(int n, int k, int sms) {
    const int nst = k / QS_SK, ntiles = cdiv(n, QS_ROWS);
    int ns = cdiv(nst, QS_MAX_SLICE_ST);
    const int want = sms / ntiles, most = nst / 2 > 1 ? nst / 2 : 1;          // at least 256 k per slice
    if (want > ns) ns = want < most ? want : most;
    return ns < 1 ? 1 : ns;
}

static int qs_sm_count() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 0;
    }
    return sms > 0 ? sms : 148;
}

size_t qstream_tc_scratch_bytes(int n, int k) {
    const int ns = qs_pick_nslice(n, k, qs_sm_count());
    return ns > 1 ? (size_t)ns * 8 * n * sizeof(float) : 0;
}

// -------------------------------------------------------------------- device helpers
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ uint32_t hsub2u(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
// eight Q4_0 weights of one 32-bit word -> eight fp16 (q-8): bytes i = 0..3 hold element i in the
// low nibble and element i+16 in the high one; the result order is (e0,e2) (e1,e3) (e16,e18) (e17,e19)
__device__ __forceinline__ void q4_word(uint32_t w, uint32_t *r) {
    constexpr uint32_t M = 0x000F000Fu, E = 0x64006400u, OFF = 0x64086408u;
    r[0] = hsub2u((w & M) | E, OFF);
    r[1] = hsub2u(((w >> 8) & M) | E, OFF);
    r[2] = hsub2u(((w >> 4) & M) | E, OFF);
    r[3] = hsub2u(((w >> 12) & M) | E, OFF);
}
// four int8 -> four fp16, natural order
__device__ __forceinline__ void q8_word(uint32_t w, uint32_t *r) {
    constexpr uint32_t E = 0x64646464u, OFF = 0x64806480u;
    const uint32_t u = w ^ 0x80808080u;
    r[0] = hsub2u(__byte_perm(u, E, 0x4140), OFF);
    r[1] = hsub2u(__byte_perm(u, E, 0x4342), OFF);
}
// position (0..31) of element e of a block along the K axis of the decoded operand
__device__ __forceinline__ int qs_slot(int fmt, int e) {
    if (fmt != FMT_GGML_Q4_0) return e;
    const int c = (e & 15) >> 2, i = e & 3;
    return 8 * c + 4 * (e >> 4) + ((i & 1) * 2 + (i >> 1));
}
// D[tmem] (+)= A[tmem] * B[smem]; fp16 inputs, f32 accumulators. A: lane = row, one 32-bit
// column per two consecutive k.
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 16 registers per thread -> 32 lanes x 16 consecutive columns of tensor memory
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t *r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 32 lanes x (2 | 4 | 8 | 16) consecutive f32 columns -> registers
template <int NC>
__device__ __forceinline__ void tc_ldn(uint32_t taddr, float *v) {
    uint32_t *r = reinterpret_cast<uint32_t *>(v);
    if constexpr (NC == 2) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(taddr) : "memory");
    } else if constexpr (NC == 4) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
    } else if constexpr (NC == 8) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                     : "r"(taddr) : "memory");
    } else {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr) : "memory");
    }
}
__device__ __forceinline__ void named_bar_sync(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

struct QsArgs {
    const uint8_t *wt;          // re-tiled weights
    int n, k, T;
    const float *x;
    int ldx;
    float *dst;                 // out [T][ldo] when nslice == 1, else partial [nslice][T][n]
    int ldo;
    const float *bias;
    int nslice;                 // K slices (CTA c works on slice c % nslice)
    int max_slice_st;           // stages of the longest slice (sizes the activation tile)
    int *status;
};

// NT: activation rows read back from the accumulators (1, 2, 4 or 8; T <= NT)
template <int FMT, int NT>
__global__ void __launch_bounds__(QS_THREADS, 1)
qstream_tc_kernel(const QsArgs a) {
    constexpr int SB = qs_stage_bytes(FMT);
    constexpr int QBYTES = qs_quant_bytes(FMT);
    constexpr int DEPTH = qs_raw_depth(FMT);
    extern __shared__ uint8_t qs_smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(qs_smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *x_tile = smem;                                                // max_slice_st x 4 KB, 128-byte swizzle
    uint8_t *raw = x_tile + (size_t)a.max_slice_st * QS_X_STAGE;           // DEPTH x SB
    float *xch = reinterpret_cast<float *>(raw + DEPTH * SB);              // 2 x 8 x 128: sums of read-back group 1
    uint64_t *raw_full = reinterpret_cast<uint64_t *>(xch + 2 * 8 * QS_ROWS);
    uint64_t *raw_empty = raw_full + DEPTH;
    uint64_t *a_full = raw_empty + DEPTH;                                  // [parity][block]
    uint64_t *d_full = a_full + 2 * QS_NB;
    uint64_t *d_free = d_full + 2;
    uint64_t *x_full = d_free + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(x_full + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nst_total = a.k / QS_SK;
    const int slice = blockIdx.x % a.nslice, cta_in_slice = blockIdx.x / a.nslice;
    const int ctas_per_slice = gridDim.x / a.nslice;                       // the grid is a multiple of nslice
    const int s0 = (int)((long long)nst_total * slice / a.nslice), s1 = (int)((long long)nst_total * (slice + 1) / a.nslice);
    const int nst = s1 - s0;                                               // stages of this CTA's slice
    const int ntiles = (a.n + QS_ROWS - 1) / QS_ROWS;
    const int my_tiles = cta_in_slice < ntiles ? (ntiles - cta_in_slice + ctas_per_slice - 1) / ctas_per_slice : 0;
    const int total = my_tiles * nst;                                      // stages this CTA works through

    if (threadIdx.x == 0) {
        for (int i = 0; i < DEPTH; i++) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], QS_DECODE_WARPS + QS_SCALE_WARPS); }
        for (int i = 0; i < 2 * QS_NB; i++) mbar_init(&a_full[i], QS_DECODE_WARPS / QS_NB);
        for (int i = 0; i < 2; i++) { mbar_init(&d_full[i], QS_NB); mbar_init(&d_free[i], QS_SCALE_WARPS); }
        mbar_init(x_full, QS_THREADS / 32 - 1);
        mbar_fence_init();
    }
    if (warp == QS_FIRST_ISSUER) { tc_alloc(tmem_slot, QS_TMEM_COLS); tc_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // ---- activations of this slice: fp16 (hi, lo) rows 2j, 2j+1, K-major, 128-byte swizzle, each
    // block's k in the order the decode produces. Rows past 2T stay as they are: their accumulator
    // columns are never written out. Every warp but the streamer's takes (row, stage) units of 128 k,
    // two units = eight loads per lane in flight at a time.
    if (warp != 0) {
        const int units = a.T * nst, slot = qs_slot(FMT, lane);
        const float *xs = a.x + (size_t)s0 * QS_SK;
        for (int u0 = warp - 1; u0 < units; u0 += 2 * (QS_THREADS / 32 - 1)) {
            float v[2][4];
#pragma unroll
            for (int uu = 0; uu < 2; uu++) {
                const int u = u0 + uu * (QS_THREADS / 32 - 1);
                const int j = u / nst, st = u - j * nst;
#pragma unroll
                for (int i = 0; i < 4; i++) v[uu][i] = u < units ? __ldg(xs + (size_t)j * a.ldx + st * QS_SK + lane + 32 * i) : 0.f;
            }
#pragma unroll
            for (int uu = 0; uu < 2; uu++) {
                const int u = u0 + uu * (QS_THREADS / 32 - 1);
                if (u >= units) break;
                const int j = u / nst, st = u - j * nst;
                const int r0 = 2 * j, r1 = 2 * j + 1;
#pragma unroll
                for (int i = 0; i < 4; i++) {            // k = 128 st + 32 i + lane: 64-k chunk 2 st + (i >> 1), block i & 1 of it
                    __half h, l;
                    split_h16(v[uu][i], h, l);
                    const int pos = (i & 1) * 32 + slot, c16 = pos >> 3;
                    uint8_t *base = x_tile + (2 * st + (i >> 1)) * QS_X_CHUNK + (pos & 7) * 2;
                    *reinterpret_cast<__half *>(base + r0 * 128 + ((c16 ^ (r0 & 7)) << 4)) = h;
                    *reinterpret_cast<__half *>(base + r1 * 128 + ((c16 ^ (r1 & 7)) << 4)) = l;
                }
            }
        }
        fence_async_smem();                              // generic-proxy stores -> visible to the tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(x_full);
    }

    if (warp == 0) {
        if (lane == 0) {
            // ---------------------------------------------------------- byte streamer
            int rs = 0, it = 0;
            uint32_t rph = 0;
            bool ok = true;
            for (int ti = 0; ti < my_tiles && ok; ti++) {
                const uint8_t *src = a.wt + ((size_t)(cta_in_slice + ti * ctas_per_slice) * nst_total + s0) * SB;
                for (int st = 0; st < nst; st++) {
                    if (it >= DEPTH && !mbar_wait(&raw_empty[rs], rph ^ 1)) { ok = false; break; }
                    mbar_expect_tx(&raw_full[rs], SB);
                    bulk_load(raw + rs * SB, src + (size_t)st * SB, SB, &raw_full[rs]);
                    it++;
                    if (++rs == DEPTH) { rs = 0; rph ^= 1; }
                }
            }
            if (!ok) atomicExch(a.status, ST_TIMEOUT_PRODUCER);
            // every copy this thread started has to land before the CTA may exit
            for (int j = it > DEPTH ? it - DEPTH : 0; j < it; j++) mbar_wait(&raw_full[j % DEPTH], (uint32_t)((j / DEPTH) & 1));
        }
    } else if (warp >= QS_FIRST_ISSUER && warp < QS_FIRST_ISSUER + QS_NB) {
        if (lane == 0 && total > 0) {
            // ---------------------------------------------------------- MMA issuer of block b
            const int b = warp - QS_FIRST_ISSUER;
            bool ok = mbar_wait(x_full, 0);
            const uint64_t bdesc0 = umma_desc_sw128(smem_u32(x_tile));
            constexpr uint32_t idesc = umma_idesc_f16(QS_ROWS, QS_N);
            int st = 0;
            for (int it = 0; it < total && ok; it++) {
                const int par = it & 1;
                const uint32_t uph = (uint32_t)((it >> 1) & 1);
                if (!mbar_wait(&a_full[par * QS_NB + b], uph)) { ok = false; break; }
                if (it >= 2 && !mbar_wait(&d_free[par], uph ^ 1)) { ok = false; break; }
                tc_fence_after();
                const uint64_t bd = bdesc0 + (uint64_t)((st * QS_X_STAGE + (b >> 1) * QS_X_CHUNK + (b & 1) * 64) >> 4);
                const uint32_t acol = tmem_base + par * 64 + b * 16, dcol = tmem_base + QS_D_COL0 + par * 64 + b * 16;
                tc_mma_f16_ts(dcol, acol, bd, idesc, 0);
                tc_mma_f16_ts(dcol, acol + 8, bd + 2, idesc, 1);
                tc_commit(&d_full[par]);
                if (++st == nst) st = 0;
            }
            if (!ok) atomicExch(a.status, ST_TIMEOUT_MMA);
        }
    } else if (warp >= QS_FIRST_DECODE && warp < QS_FIRST_DECODE + QS_DECODE_WARPS) {
        // ---------------------------------------------------------------- decode warps
        const int g = (warp - QS_FIRST_DECODE) >> 2;         // block of the stage this group decodes
        const int row = (warp & 3) * 32 + lane;              // weight row = TMEM lane (quarter warp % 4)
        const uint32_t tdst = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + g * 16;
        int rs = 0;
        uint32_t rph = 0;
        for (int it = 0; it < total; it++) {
            const int par = it & 1;
            const uint32_t uph = (uint32_t)((it >> 1) & 1);
            bool ok = mbar_wait(&raw_full[rs], rph);
            if (ok && it >= 2) ok = mbar_wait(&d_full[par], uph ^ 1);      // MMAs of stage it-2 are done with this A region
            if (!__all_sync(0xffffffffu, ok)) { if (lane == 0) atomicExch(a.status, ST_TIMEOUT_PRODUCER); break; }
            tc_fence_after();
            const uint8_t *src = raw + rs * SB;
            uint32_t r[16];
            if (FMT == FMT_GGML_Q4_0) {
                const uint4 q = *reinterpret_cast<const uint4 *>(src + (g * QS_ROWS + row) * 16);
                q4_word(q.x, r); q4_word(q.y, r + 4); q4_word(q.z, r + 8); q4_word(q.w, r + 12);
            } else {
                const uint4 q0 = *reinterpret_cast<const uint4 *>(src + ((2 * g) * QS_ROWS + row) * 16);
                const uint4 q1 = *reinterpret_cast<const uint4 *>(src + ((2 * g + 1) * QS_ROWS + row) * 16);
                q8_word(q0.x, r); q8_word(q0.y, r + 2); q8_word(q0.z, r + 4); q8_word(q0.w, r + 6);
                q8_word(q1.x, r + 8); q8_word(q1.y, r + 10); q8_word(q1.z, r + 12); q8_word(q1.w, r + 14);
            }
            tc_st16(tdst + par * 64, r);
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&a_full[par * QS_NB + g]); mbar_arrive(&raw_empty[rs]); }
            if (++rs == DEPTH) { rs = 0; rph ^= 1; }
        }
    } else if (warp >= QS_FIRST_SCALE) {
        // ---------------------------------------------------------------- read-back warps
        const int h = (warp - QS_FIRST_SCALE) >> 2;          // this group folds blocks 2h, 2h+1 of every stage
        const int row = (warp & 3) * 32 + lane;
        const uint32_t tsrc = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + QS_D_COL0 + (2 * h) * 16;
        int rs = 0, it = 0;
        uint32_t rph = 0;
        bool ok = true;
        for (int ti = 0; ti < my_tiles; ti++) {
            float ah[NT], al[NT];
#pragma unroll
            for (int j = 0; j < NT; j++) ah[j] = al[j] = 0.f;
            for (int st = 0; st < nst; st++, it++) {
                const int par = it & 1;
                const uint32_t uph = (uint32_t)((it >> 1) & 1);
                if (ok) {
                    bool w = mbar_wait(&d_full[par], uph);
                    if (w) w = mbar_wait(&raw_full[rs], rph);              // completed long ago; orders the scale reads
                    if (!__all_sync(0xffffffffu, w)) { ok = false; if (lane == 0) atomicExch(a.status, ST_TIMEOUT_EPILOGUE); }
                }
                if (ok) {
                    tc_fence_after();
                    float v0[2 * NT], v1[2 * NT];
                    tc_ldn<2 * NT>(tsrc + par * 64, v0);
                    tc_ldn<2 * NT>(tsrc + par * 64 + 16, v1);
                    const __half *dp = reinterpret_cast<const __half *>(raw + rs * SB + QBYTES) + (2 * h) * QS_ROWS + row;
                    const float d0 = __half2float(dp[0]), d1 = __half2float(dp[QS_ROWS]);
                    tc_wait_ld();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) { mbar_arrive(&d_free[par]); mbar_arrive(&raw_empty[rs]); }
#pragma unroll
                    for (int j = 0; j < NT; j++) {
                        ah[j] = fmaf(d0, v0[2 * j], ah[j]);
                        al[j] = fmaf(d0, v0[2 * j + 1], al[j]);
                        ah[j] = fmaf(d1, v1[2 * j], ah[j]);
                        al[j] = fmaf(d1, v1[2 * j + 1], al[j]);
                    }
                }
                if (++rs == DEPTH) { rs = 0; rph ^= 1; }
            }
            // group 1 hands its sums to group 0 (fixed order: blocks 0,1 of every stage, then blocks 2,3)
            float *xb = xch + (ti & 1) * (8 * QS_ROWS);
            if (h == 1) {
#pragma unroll
                for (int j = 0; j < NT; j++) xb[j * QS_ROWS + row] = fmaf(al[j], H16_LO_INV, ah[j]);
            }
            named_bar_sync(1, QS_SCALE_WARPS * 32);
            const int r = (cta_in_slice + ti * ctas_per_slice) * QS_ROWS + row;
            if (h == 0 && ok && r < a.n) {
#pragma unroll
                for (int j = 0; j < NT; j++) {
                    if (j < a.T) {
                        const float v = fmaf(al[j], H16_LO_INV, ah[j]) + xb[j * QS_ROWS + row];
                        if (a.nslice == 1) a.dst[(size_t)j * a.ldo + r] = v + (a.bias ? a.bias[r] : 0.f);
                        else a.dst[((size_t)slice * a.T + j) * a.n + r] = v;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == QS_FIRST_ISSUER) tc_dealloc(tmem_base, QS_TMEM_COLS);
}

// out[j][r] = bias[r] + sum over slices (ascending) of partial[s][j][r]
__global__ void qs_reduce_kernel(const float *__restrict__ partial, float *__restrict__ out, int ldo, const float *__restrict__ bias,
                                 int n, int T, int nslice) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x, j = blockIdx.y;
    if (r >= n) return;
    float v = 0.f;
    for (int s = 0; s < nslice; s++) v += partial[((size_t)s * T + j) * n + r];
    out[(size_t)j * ldo + r] = v + (bias ? bias[r] : 0.f);
}

static size_t qs_smem_bytes(int fmt, int max_slice_st) {
    return 1024 + (size_t)max_slice_st * QS_X_STAGE + (size_t)qs_raw_depth(fmt) * qs_stage_bytes(fmt) + 2 * 8 * QS_ROWS * sizeof(float) +
           (2 * qs_raw_depth(fmt) + 2 * QS_NB + 5) * 8 + 16;
}

template <int FMT, int NT>
static int qs_launch(const QsArgs &a, int grid, size_t smem, cudaStream_t st) {
    static size_t configured = 0;                // largest dynamic shared memory size requested so far
    if (smem > configured) {
        MB_CUDA(cudaFuncSetAttribute(qstream_tc_kernel<FMT, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    qstream_tc_kernel<FMT, NT><<<grid, QS_THREADS, smem, st>>>(a);
    MB_CUDA(cudaGetLastError());
    return 0;
}

// Partial sums of the K slices go through w.tc_scratch (qstream_tc_scratch_bytes(n, k) bytes, allocated
// with the weight): calls on one weight must not overlap in time.
int qstream_tc(const QWeight &w, const float *x, int ldx, float *out, int ldo, const float *bias, int T, int *status,
               cudaStream_t st) {
    float *scratch = w.tc_scratch;
    if (!w.tc_q) { set_error("qstream_tc: weight has no streaming layout"); return -1; }
    if (T < 1 || T > 8) { set_error("qstream_tc: T=%d outside 1..8", T); return -1; }
    const int sms = qs_sm_count();
    const int nst_total = w.k / QS_SK;
    const int nslice = qs_pick_nslice(w.n, w.k, sms);
    if (nslice > 1 && !scratch) { set_error("qstream_tc: [%d,%d] needs a partial-sum buffer", w.n, w.k); return -1; }
    const int ntiles = cdiv(w.n, QS_ROWS);
    int grid = ntiles * nslice < sms ? ntiles * nslice : sms;
    grid -= grid % nslice;                       // same number of CTAs on every slice
    if (grid < nslice) grid = nslice;
    QsArgs a;
    a.wt = w.tc_q; a.n = w.n; a.k = w.k; a.T = T; a.x = x; a.ldx = ldx; a.ldo = ldo; a.bias = bias;
    a.nslice = nslice; a.max_slice_st = cdiv(nst_total, nslice); a.status = status;
    a.dst = nslice == 1 ? out : scratch;
    const size_t smem = qs_smem_bytes(w.fmt, a.max_slice_st);
    const int nt = T <= 1 ? 1 : T <= 2 ? 2 : T <= 4 ? 4 : 8;
    int rc;
    if (w.fmt == FMT_GGML_Q4_0)
        rc = nt == 1 ? qs_launch<FMT_GGML_Q4_0, 1>(a, grid, smem, st) : nt == 2 ? qs_launch<FMT_GGML_Q4_0, 2>(a, grid, smem, st)
           : nt == 4 ? qs_launch<FMT_GGML_Q4_0, 4>(a, grid, smem, st) : qs_launch<FMT_GGML_Q4_0, 8>(a, grid, smem, st);
    else
        rc = nt == 1 ? qs_launch<FMT_GGML_Q8_0, 1>(a, grid, smem, st) : nt == 2 ? qs_launch<FMT_GGML_Q8_0, 2>(a, grid, smem, st)
           : nt == 4 ? qs_launch<FMT_GGML_Q8_0, 4>(a, grid, smem, st) : qs_launch<FMT_GGML_Q8_0, 8>(a, grid, smem, st);
    if (rc) return rc;
    if (nslice > 1) {
        qs_reduce_kernel<<<dim3(cdiv(w.n, 256), T), 256, 0, st>>>(scratch, out, ldo, bias, w.n, T, nslice);
        MB_CUDA(cudaGetLastError());
    }
    return 0;
}

}  // namespace mb
