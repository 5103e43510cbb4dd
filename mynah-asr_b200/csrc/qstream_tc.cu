// Weight-streaming quantised matmul on the tcgen05 integer tensor path:
// out[T,n] = x[T,k] W^T for T <= 8, W stored as ggml Q4_0 / Q8_0 / Q4_K blocks.
// The bandwidth-bound half of the reference's mynah_asr_qmat_mul (src/qmat.c:508-597).
//
// Arithmetic. A stored block is 32 integers q and an f16 scale d (w = d*q, ingot dequant.c:72-83).
// Each 32-element block of an activation row is written as 2^e * (p0 + p1/2^7 + p2/2^14 + p3/2^21)
// with four int8 planes p and a power-of-two block scale, so every step of the split is exact and
// the row is reproduced to 2^-28 of the block's largest element. The tensor core then forms the
// exact int32 dots q.p0 .. q.p3 of every (weight row, block), and a thread folds them in f32:
// out += d * 2^e * (v0 + v1/2^7 + v2/2^14 + v3/2^21). No product is ever rounded before that fold.
// Q4_K (256-element super-blocks, w = d*sc*q - dmin*m per 32-element sub-block with 6-bit sc, m;
// ingot dequant.c:131-156): the dots are taken with the unsigned nibbles, the fold uses d*sc and the
// offset term dmin*m times the block's activation sum.
//
// Per CTA (persistent, one per SM), 32 warps with fixed roles:
//   * warps 0 and 5-7, one thread each: stream the stored bytes of every fourth stage (128 weight
//     rows x 128 k: the quants and the four f16 block scales per row, laid out contiguously at
//     load) from HBM into a shared-memory ring (4 or 8 stages deep) with bulk asynchronous copies
//     (cp.async.bulk, one CTA each) tracked by mbarriers — 36-136 KB in flight per SM to cover HBM
//     latency. One thread needs ~400 cycles per copy it starts, more than a stage may take;
//   * warps 8-23, four groups of four: group g handles the stages g, g+4, ... A thread owns one
//     weight row and moves its 32 integers into tensor memory with tcgen05.st, where they are the
//     A operand: Q8_0 bytes go as they are, a Q4_0 word becomes two words of (q-8)*16 with three
//     logic instructions; the row's four block scales follow into two more columns. The weights
//     never pass through shared memory a second time and the ring slot is free again at once;
//   * warps 1-4, one thread each: an issuer takes every fourth stage and issues its four
//     tcgen05.mma (kind::i8, M = 128 weight rows, N = 16 or 32 plane rows, K = 32, one per block) —
//     one thread gets an MMA out every ~45 cycles whatever its size, so the small ones here need
//     several issuers. B is the int8 planes of the activations, resident in shared memory for the
//     CTA's K slice. Each block has its own accumulator columns, because d and 2^e multiply the
//     block's dots afterwards;
//   * warps 24-31, two groups of four: read the block dots and scales back (tcgen05.ld; thread =
//     weight row) and fold them into f32 accumulators;
//   * every warp but the streamers' first splits its share of the activations into planes.
// Large K, or few rows, are split over CTAs (fixed K slice per CTA, so its activations are staged
// once); the slices are then summed in a fixed order by a second small kernel, so results are
// reproducible and a row's result does not depend on T. Every mbarrier wait is bounded; a wait
// that runs out sets a status word and the kernel unwinds.
#include "kernels.h"
#include "qweight.h"

namespace mb {

static constexpr int QS_ROWS = 128;           // weight rows per tile (UMMA M)
static constexpr int QS_SK = 128;             // k per stage
static constexpr int QS_NB = 4;               // 32-element blocks per stage
static constexpr int QS_PLANES = 4;           // int8 planes per activation row
static constexpr int QS_MAX_SLICE_ST = 32;    // stages of K per CTA slice (4096 k)
static constexpr int QS_STREAMERS = 4;        // warps 0, 5, 6, 7
static constexpr int QS_FIRST_ISSUER = 1;     // warps 1-4: MMA issuers
static constexpr int QS_FIRST_DECODE = 8, QS_DECODE_WARPS = 16;
static constexpr int QS_FIRST_SCALE = 24, QS_SCALE_WARPS = 8;
static constexpr int QS_THREADS = (QS_FIRST_SCALE + QS_SCALE_WARPS) * 32;     // 1024
static constexpr int QS_A_COLS = 8;                           // tensor-memory columns of one decoded block (32 int8)
static constexpr int QS_TMEM_COLS = 512;
static constexpr int QS_SC_COL0 = 384;                        // eight 4-column slots: a row's scale record of the stage
static constexpr int QS_SC_SLOTS = 8;
static constexpr int QS_SC_COLS = 4;

// per row and stage: Q4_0 / Q8_0 four f16 block scales (8 bytes); Q4_K f16 d, f16 dmin, sc[4], m[4] (12 bytes)
__host__ __device__ constexpr int qs_scale_rec(int fmt) { return fmt == FMT_GGML_Q4_K ? 12 : 8; }
__host__ __device__ constexpr int qs_quant_bytes(int fmt) { return fmt == FMT_GGML_Q8_0 ? QS_ROWS * QS_SK : QS_ROWS * QS_SK / 2; }
__host__ __device__ constexpr int qs_stage_bytes(int fmt) { return qs_quant_bytes(fmt) + QS_ROWS * qs_scale_rec(fmt); }
// stored-byte stages in flight (a power of two) beside 4096 k of activation planes (64 KB for up to
// 4 rows, 128 KB for 8): 72 / 36 KB of Q4_0, 136 / 68 KB of Q8_0 (16 stages of Q4_0 measured no faster)
__host__ __device__ constexpr int qs_raw_depth(int fmt, int nt) { return 8 / (nt == 8 ? 2 : 1); }

// 6-bit scale / min j of a Q4_K super-block (get_scale_min_k4, ingot dequant.c:120-129)
__host__ __device__ inline void qs_k4_scale_min(const uint8_t *sc, int j, int *s, int *m) {
    if (j < 4) { *s = sc[j] & 63; *m = sc[j + 4] & 63; }
    else { *s = (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4); *m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
}

// -------------------------------------------------------------------- re-tiling at load
// [tile][stage][ quants: [16-byte chunk c][row 0..127][16 B] | scales: [row 0..127][block 0..3] f16 ]
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
    uint8_t *sc = stage + qs_quant_bytes(fmt) + (rl * QS_NB + bs) * 2;
    sc[0] = p[0];
    sc[1] = p[1];
}

// Q4_K: one thread per (row, super-block) fills the two stages the super-block spans. A stage holds the 64
// quant bytes of its two 64-element groups A, B as four 16-byte chunks (bytes 0-15 and 16-31 of A, then of B;
// low nibbles of a group's 32 bytes are its first sub-block, high nibbles its second) and the record
// d, dmin, sc[4], m[4] of the stage's four sub-blocks.
__global__ void qs_retile_q4k_kernel(const uint8_t *__restrict__ raw, uint8_t *__restrict__ dst, int n, int k) {
    const size_t sbi = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    const int spr = k / 256;
    if (sbi >= (size_t)n * spr) return;
    const int row = (int)(sbi / spr), sb = (int)(sbi % spr);
    const int tile = row / QS_ROWS, rl = row % QS_ROWS;
    const uint8_t *p = raw + sbi * 144;                   // d, dmin (f16), scales[12], qs[128]
    for (int half = 0; half < 2; half++) {
        uint8_t *stage = dst + ((size_t)tile * (k / QS_SK) + 2 * sb + half) * qs_stage_bytes(FMT_GGML_Q4_K);
        for (int i = 0; i < 64; i++) stage[((i / 16) * QS_ROWS + rl) * 16 + (i & 15)] = p[16 + 64 * half + i];
        uint8_t *rec = stage + qs_quant_bytes(FMT_GGML_Q4_K) + rl * 12;
        rec[0] = p[0]; rec[1] = p[1]; rec[2] = p[2]; rec[3] = p[3];
        for (int b = 0; b < 4; b++) {
            int sc, m;
            qs_k4_scale_min(p + 4, 4 * half + b, &sc, &m);
            rec[4 + b] = (uint8_t)sc; rec[8 + b] = (uint8_t)m;
        }
    }
}

size_t qstream_tc_bytes(int fmt, int n, int k) {
    return (size_t)cdiv(n, QS_ROWS) * (k / QS_SK) * qs_stage_bytes(fmt);
}

int qstream_tc_retile(const QWeight &w, uint8_t *dst, cudaStream_t st) {
    MB_CUDA(cudaMemsetAsync(dst, 0, qstream_tc_bytes(w.fmt, w.n, w.k), st));
    const size_t nblk = (size_t)w.n * (w.k / 32);
    if (w.fmt == FMT_GGML_Q4_K)
        qs_retile_q4k_kernel<<<(unsigned)((nblk / 8 + 255) / 256), 256, 0, st>>>(w.raw, dst, w.n, w.k);
    else
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
    return device_sm_count();
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
// D[tmem] (+)= A[tmem] * B[smem]; int8 inputs, int32 accumulators. A: lane = row, one 32-bit
// column per four consecutive k.
__device__ __forceinline__ void tc_mma_i8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// instruction descriptor: D s32, A s8 (or u8), B s8, both K-major, M x N
__host__ __device__ constexpr uint32_t qs_idesc_i8(int M, int N, bool a_unsigned) {
    return (2u << 4) | ((a_unsigned ? 0u : 1u) << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// 8 registers per thread -> 32 lanes x 8 consecutive columns of tensor memory
__device__ __forceinline__ void tc_st8(uint32_t taddr, const uint32_t *r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tc_st4(uint32_t taddr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r0), "r"(r1), "r"(r2), "r"(r3) : "memory");
}
__device__ __forceinline__ void tc_ld4u(uint32_t taddr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(taddr) : "memory");
}
// 32 registers per thread -> 32 lanes x 32 consecutive columns of tensor memory
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t *r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 32 lanes x (4 | 8 | 16 | 32) consecutive 32-bit columns -> registers
template <int NC>
__device__ __forceinline__ void tc_ldn(uint32_t taddr, int *r) {
    if constexpr (NC == 4) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
    } else if constexpr (NC == 8) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                     : "r"(taddr) : "memory");
    } else if constexpr (NC == 16) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
            : "r"(taddr) : "memory");
    } else {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
              "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
              "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
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

// NT: activation rows the accumulators are read back for (1, 2, 4 or 8; T <= NT). The MMA's N is
// the 4 NT plane rows, padded to 16.
template <int FMT, int NT>
__global__ void __launch_bounds__(QS_THREADS, 1)
qstream_tc_kernel(const QsArgs a) {
    constexpr int SB = qs_stage_bytes(FMT);
    constexpr int QBYTES = qs_quant_bytes(FMT);
    constexpr int DEPTH = qs_raw_depth(FMT, NT);
    constexpr int N = NT <= 4 ? 16 : 32;                    // plane rows of the B operand (row 4j+p: plane p of activation row j)
    constexpr int NCOL = QS_PLANES * NT;                    // accumulator columns that carry data
    constexpr int XT = N * 128;                             // bytes of planes per stage: N rows x 128 k of int8, 128-byte swizzle
    constexpr int DST = QS_NB * N;                          // accumulator columns per stage
    // Q4_0 with one activation row: the decode warps are the bound, so the nibbles go to the tensor core
    // unsigned (q*16, one logic operation less per word) and the read-back warps, which have time to spare
    // there, subtract 8*16 times the block's plane sums from the int32 dots — the same integers as the
    // signed form gives (measured: 4.5 % faster at one row, 9 % slower at two)
    constexpr bool U4 = FMT == FMT_GGML_Q4_0 && NT == 1;
    // Stages in tensor memory: AP of decoded weights, one per decode group, and DP of accumulators.
    // Every barrier below is waited on by threads that lag it by at most one phase: a decode group
    // comes back to its own A slot, a read-back group to its own accumulator slots.
    constexpr int AP = QS_DECODE_WARPS / 4;                 // 4
    constexpr int DP = NT <= 4 ? 4 : 2;
    constexpr int AST = QS_NB * QS_A_COLS;                  // A columns per stage
    constexpr int D_COL0 = AP * AST;                        // accumulators start after the A stages (AP * AST + DP * DST <= 512)
    extern __shared__ uint8_t qs_smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(qs_smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *x_tile = smem;                                                // max_slice_st x XT
    uint8_t *raw = x_tile + (size_t)a.max_slice_st * XT;                   // DEPTH x SB
    float *xch = reinterpret_cast<float *>(raw + DEPTH * SB);              // 2 x 8 x 128: sums of read-back group 1
    float *sxs = xch + 2 * 8 * QS_ROWS;                                    // [stage][block][NT] activation block scales 2^e
    float *sxsum = sxs + (size_t)a.max_slice_st * QS_NB * NT;              // Q4_K: [stage][block][NT] sums of the activations
    int *psum = reinterpret_cast<int *>(sxsum + (FMT == FMT_GGML_Q4_K ? (size_t)a.max_slice_st * QS_NB * NT : 0));   // U4: [stage][block][NT][plane] 128 x plane sums
    uint64_t *raw_full = reinterpret_cast<uint64_t *>(psum + (U4 ? (size_t)a.max_slice_st * QS_NB * NT * QS_PLANES : 0));
    uint64_t *raw_empty = raw_full + DEPTH;
    uint64_t *a_full = raw_empty + DEPTH;
    uint64_t *a_free = a_full + AP;                                        // used when DP != AP; else d_full says the same
    uint64_t *d_full = a_free + AP;
    uint64_t *d_free = d_full + DP;
    uint64_t *x_full = d_free + DP;
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
        for (int i = 0; i < DEPTH; i++) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], 4); }   // the four warps of one decode group
        for (int i = 0; i < AP; i++) { mbar_init(&a_full[i], 4); mbar_init(&a_free[i], 1); }
        for (int i = 0; i < DP; i++) { mbar_init(&d_full[i], 1); mbar_init(&d_free[i], 4); }
        mbar_init(x_full, QS_THREADS / 32 - QS_STREAMERS);
        mbar_fence_init();
    }
    if (warp == QS_FIRST_ISSUER) { tc_alloc(tmem_slot, QS_TMEM_COLS); tc_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 || (warp > QS_FIRST_ISSUER + 3 && warp < QS_FIRST_DECODE)) {
        if (lane == 0) {
            // ---------------------------------------------------------- byte streamer of the stages s, s+4, ...
            // (DEPTH is a multiple of 4, so a streamer keeps to its own ring slots)
            const int s = warp == 0 ? 0 : warp - QS_FIRST_ISSUER - 3;
            int ti = s / nst, st = s - ti * nst, it = s;
            bool ok = true;
            for (; it < total; it += QS_STREAMERS) {
                const int rs = it & (DEPTH - 1);
                if (it >= DEPTH && !mbar_wait(&raw_empty[rs], (uint32_t)(((it / DEPTH) & 1) ^ 1))) { ok = false; break; }
                mbar_expect_tx(&raw_full[rs], SB);
                bulk_load(raw + rs * SB, a.wt + ((size_t)(cta_in_slice + ti * ctas_per_slice) * nst_total + s0 + st) * SB, SB, &raw_full[rs]);
                st += QS_STREAMERS;
                while (st >= nst) { st -= nst; ti++; }
            }
            if (!ok) atomicExch(a.status, ST_TIMEOUT_PRODUCER);
            // every copy this thread started has to land before the CTA may exit
            for (int j = it - QS_STREAMERS; j >= s && j >= it - DEPTH; j -= QS_STREAMERS) mbar_wait(&raw_full[j & (DEPTH - 1)], (uint32_t)((j / DEPTH) & 1));
        }
    } else {
        // ---- every other warp first splits its share of this slice's activations into int8 planes
        // (units of one row x one stage; eight loads per lane in flight). Block b of a row:
        // 2^e with |x| * 2^-e < 64 for the block's largest |x|, then four exact rounding steps.
        // Plane rows past 4T stay as they are: their accumulator columns are never written out.
        const int units = a.T * nst;
        const float *xs = a.x + (size_t)s0 * QS_SK;
        constexpr int NW = QS_THREADS / 32 - QS_STREAMERS;
        for (int u0 = warp < QS_FIRST_DECODE ? warp - 1 : warp - QS_STREAMERS; u0 < units; u0 += 2 * NW) {
            float v[2][4];
#pragma unroll
            for (int uu = 0; uu < 2; uu++) {
                const int u = u0 + uu * NW;
                const int j = u / nst, st = u - j * nst;
#pragma unroll
                for (int b = 0; b < 4; b++) v[uu][b] = u < units ? __ldg(xs + (size_t)j * a.ldx + st * QS_SK + 32 * b + lane) : 0.f;
            }
#pragma unroll
            for (int uu = 0; uu < 2; uu++) {
                const int u = u0 + uu * NW;
                if (u >= units) break;
                const int j = u / nst, st = u - j * nst;
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    const float m = warp_max(fabsf(v[uu][b]));
                    int eb = (__float_as_int(m) >> 23) - 132;                // floor(log2 m) - 5
                    eb = eb < -100 ? -100 : eb;
                    const float sinv = m > 0.f ? __int_as_float((127 - eb) << 23) : 0.f;
                    float r = v[uu][b] * sinv;
                    const int kpos = 32 * b + lane;
#pragma unroll
                    for (int p = 0; p < QS_PLANES; p++) {
                        const float pl = rintf(r);
                        r = (r - pl) * 128.f;
                        const int row = QS_PLANES * j + p;
                        *reinterpret_cast<int8_t *>(x_tile + st * XT + row * 128 + (((kpos >> 4) ^ (row & 7)) << 4) + (kpos & 15)) = (int8_t)(int)pl;
                        if (U4) {
                            const int ps = __reduce_add_sync(0xffffffffu, (int)pl);
                            if (lane == 0) psum[((st * QS_NB + b) * NT + j) * QS_PLANES + p] = ps * 128;
                        }
                    }
                    if (lane == 0) sxs[(st * QS_NB + b) * NT + j] = m > 0.f ? __int_as_float((127 + eb) << 23) : 0.f;
                    if (FMT == FMT_GGML_Q4_K) {
                        const float sum = warp_sum(v[uu][b]);
                        if (lane == 0) sxsum[(st * QS_NB + b) * NT + j] = sum;
                    }
                }
            }
        }
        fence_async_smem();                              // generic-proxy stores -> visible to the tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(x_full);

        if (warp >= QS_FIRST_ISSUER && warp < QS_FIRST_ISSUER + DP) {
            if (lane == 0 && total > 0) {
                // ------------------------------------------------------ MMA issuer of the stages i, i+DP, ...
                // (an issuer returns to its own accumulator slot, and to an A slot only after the decode
                // group that fills it has been there, so no barrier is ever more than a phase ahead)
                const int i = warp - QS_FIRST_ISSUER;
                bool ok = mbar_wait(x_full, 0);
                const uint64_t bdesc0 = umma_desc_sw128(smem_u32(x_tile));
                constexpr uint32_t idesc = qs_idesc_i8(QS_ROWS, N, FMT == FMT_GGML_Q4_K || U4);
                int st = i % nst;
                for (int it = i; it < total && ok; it += DP) {
                    const int as = it & (AP - 1);
                    if (!mbar_wait(&a_full[as], (uint32_t)((it / AP) & 1))) { ok = false; break; }
                    if (it >= DP && !mbar_wait(&d_free[i], (uint32_t)(((it / DP) & 1) ^ 1))) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t bd = bdesc0 + (uint64_t)((st * XT) >> 4);
#pragma unroll
                    for (int b = 0; b < QS_NB; b++)
                        tc_mma_i8_ts(tmem_base + D_COL0 + i * DST + b * N, tmem_base + (as * QS_NB + b) * QS_A_COLS, bd + (uint64_t)(2 * b), idesc, 0);
                    if (DP != AP) tc_commit(&a_free[as]);
                    tc_commit(&d_full[i]);
                    st += DP;
                    while (st >= nst) st -= nst;
                }
                if (!ok) atomicExch(a.status, ST_TIMEOUT_MMA);
            }
        } else if (warp >= QS_FIRST_DECODE && warp < QS_FIRST_DECODE + QS_DECODE_WARPS) {
            // ------------------------------------------------------------ decode warps
            // Group g takes the stages it = g, g+4, ...: the wait - load - store - wait::st chain of
            // one stage is several hundred cycles long, so four stages are in flight in four groups.
            const int g = (warp - QS_FIRST_DECODE) >> 2;
            const int row = (warp & 3) * 32 + lane;              // weight row = TMEM lane (quarter warp % 4)
            const uint32_t tdst = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
            for (int it = g; it < total; it += AP) {
                const int rs = it & (DEPTH - 1);
                if (!__all_sync(0xffffffffu, mbar_wait(&raw_full[rs], (uint32_t)((it / DEPTH) & 1)))) { if (lane == 0) atomicExch(a.status, ST_TIMEOUT_PRODUCER); break; }
                const uint8_t *src = raw + rs * SB + row * 16;
                uint32_t r[QS_NB * QS_A_COLS];
                if (FMT == FMT_GGML_Q4_0) {
                    // byte i of a block holds element i (low nibble) and element i+16 (high nibble):
                    // (q-8)*16 as a signed byte is the nibble in the high half with its top bit flipped
                    // (U4: left unflipped, q*16 unsigned)
                    constexpr uint32_t HM = 0xF0F0F0F0u, FL = U4 ? 0u : 0x80808080u;
#pragma unroll
                    for (int b = 0; b < QS_NB; b++) {
                        const uint4 q = *reinterpret_cast<const uint4 *>(src + b * QS_ROWS * 16);
                        uint32_t *rb = r + b * QS_A_COLS;
                        rb[0] = ((q.x << 4) & HM) ^ FL; rb[1] = ((q.y << 4) & HM) ^ FL; rb[2] = ((q.z << 4) & HM) ^ FL; rb[3] = ((q.w << 4) & HM) ^ FL;
                        rb[4] = (q.x & HM) ^ FL; rb[5] = (q.y & HM) ^ FL; rb[6] = (q.z & HM) ^ FL; rb[7] = (q.w & HM) ^ FL;
                    }
                } else if (FMT == FMT_GGML_Q4_K) {
                    // 32 quant bytes hold two sub-blocks: low nibbles of byte i = element i of the first, high
                    // nibbles = element i of the second; unsigned q*16 in the high half of a byte
                    constexpr uint32_t HM = 0xF0F0F0F0u;
#pragma unroll
                    for (int gq = 0; gq < 2; gq++) {
                        const uint4 q0 = *reinterpret_cast<const uint4 *>(src + (2 * gq) * QS_ROWS * 16);
                        const uint4 q1 = *reinterpret_cast<const uint4 *>(src + (2 * gq + 1) * QS_ROWS * 16);
                        uint32_t *lo = r + (2 * gq) * QS_A_COLS, *hi = lo + QS_A_COLS;
                        lo[0] = (q0.x << 4) & HM; lo[1] = (q0.y << 4) & HM; lo[2] = (q0.z << 4) & HM; lo[3] = (q0.w << 4) & HM;
                        lo[4] = (q1.x << 4) & HM; lo[5] = (q1.y << 4) & HM; lo[6] = (q1.z << 4) & HM; lo[7] = (q1.w << 4) & HM;
                        hi[0] = q0.x & HM; hi[1] = q0.y & HM; hi[2] = q0.z & HM; hi[3] = q0.w & HM;
                        hi[4] = q1.x & HM; hi[5] = q1.y & HM; hi[6] = q1.z & HM; hi[7] = q1.w & HM;
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 2 * QS_NB; c++) {
                        const uint4 q = *reinterpret_cast<const uint4 *>(src + c * QS_ROWS * 16);
                        r[4 * c] = q.x; r[4 * c + 1] = q.y; r[4 * c + 2] = q.z; r[4 * c + 3] = q.w;
                    }
                }
                // the row's scale record of this stage (8 or 12 bytes)
                const uint32_t *recp = reinterpret_cast<const uint32_t *>(raw + rs * SB + QBYTES + row * qs_scale_rec(FMT));
                const uint32_t rec0 = recp[0], rec1 = recp[1], rec2 = FMT == FMT_GGML_Q4_K ? recp[2] : 0u;
                // only now is A slot g needed: the MMAs of stage it-AP, its last user, must be done
                // (the loads and the unpacking above are off the slot's critical path)
                if (it >= AP && !__all_sync(0xffffffffu, mbar_wait(DP == AP ? &d_full[g] : &a_free[g], (uint32_t)(((it / AP) & 1) ^ 1)))) {
                    if (lane == 0) atomicExch(a.status, ST_TIMEOUT_PRODUCER);
                    break;
                }
                tc_fence_after();
                tc_st32(tdst + g * AST, r);
                tc_st4(tdst + QS_SC_COL0 + (it & (QS_SC_SLOTS - 1)) * QS_SC_COLS, rec0, rec1, rec2, 0u);   // slot it-8 was read before the MMAs of it-4 could start
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) { mbar_arrive(&a_full[g]); mbar_arrive(&raw_empty[rs]); }
            }
        } else if (warp >= QS_FIRST_SCALE) {
            // ------------------------------------------------------------ read-back warps
            // Group h folds the stages with it % 2 == h (two stages in flight); at the end of a row
            // tile group 1 hands its sums to group 0.
            const int h = (warp - QS_FIRST_SCALE) >> 2;
            const int row = (warp & 3) * 32 + lane;
            const uint32_t tsrc = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + D_COL0;
            constexpr float DQ = FMT == FMT_GGML_Q8_0 ? 1.f : 0.0625f;     // 4-bit weights sit in tensor memory times 16
            constexpr float P7 = 0.0078125f;                              // 2^-7 between planes
            constexpr int BPL = NCOL <= 8 ? 4 : NCOL == 16 ? 2 : 1;        // blocks read back per tcgen05.wait::ld
            int it = 0;
            bool ok = __all_sync(0xffffffffu, mbar_wait(x_full, 0));   // the block scales 2^e are in place
            if (!ok && lane == 0) atomicExch(a.status, ST_TIMEOUT_EPILOGUE);
            for (int ti = 0; ti < my_tiles; ti++) {
                float acc[NT];
#pragma unroll
                for (int j = 0; j < NT; j++) acc[j] = 0.f;
                const int it_end = it + nst;
                int st = (it & 1) != h;                      // this group's first stage of the tile
                for (it += st; it < it_end; it += 2, st += 2) {
                    const int par = it & (DP - 1);
                    const uint32_t uph = (uint32_t)((it / DP) & 1);
                    if (ok && !__all_sync(0xffffffffu, mbar_wait(&d_full[par], uph))) { ok = false; if (lane == 0) atomicExch(a.status, ST_TIMEOUT_EPILOGUE); }
                    if (!ok) continue;
                    tc_fence_after();
                    uint32_t sc0, sc1, sc2, sc3;             // the row's scale record, left by the decode warps
                    tc_ld4u(tsrc - D_COL0 + QS_SC_COL0 + (it & (QS_SC_SLOTS - 1)) * QS_SC_COLS, sc0, sc1, sc2, sc3);
                    float d[QS_NB], dm[QS_NB];
#pragma unroll
                    for (int b0 = 0; b0 < QS_NB; b0 += BPL) {
                        int v[BPL][NCOL];
#pragma unroll
                        for (int bb = 0; bb < BPL; bb++) tc_ldn<NCOL>(tsrc + par * DST + (b0 + bb) * N, v[bb]);
                        tc_wait_ld();
                        if (b0 == 0) {
                            const __half2 h01 = *reinterpret_cast<const __half2 *>(&sc0), h23 = *reinterpret_cast<const __half2 *>(&sc1);
                            if (FMT == FMT_GGML_Q4_K) {      // record: d, dmin | sc[4] | m[4]; w = (d sc) q - (dmin m)
                                const float dd = __low2float(h01) * DQ, dmin = __high2float(h01);
#pragma unroll
                                for (int b = 0; b < QS_NB; b++) {
                                    d[b] = dd * (float)((sc1 >> (8 * b)) & 0xFFu);
                                    dm[b] = dmin * (float)((sc2 >> (8 * b)) & 0xFFu);
                                }
                            } else {
                                d[0] = __low2float(h01) * DQ; d[1] = __high2float(h01) * DQ; d[2] = __low2float(h23) * DQ; d[3] = __high2float(h23) * DQ;
                            }
                        }
                        if (b0 + BPL == QS_NB) {             // the whole stage is in registers: its accumulators may be reused
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&d_free[par]);
                        }
                        float ds[BPL][NT];
#pragma unroll
                        for (int bb = 0; bb < BPL; bb++) {
                            const float *sp = sxs + (st * QS_NB + b0 + bb) * NT;
#pragma unroll
                            for (int j = 0; j < NT; j++) ds[bb][j] = d[b0 + bb] * sp[j];
                        }
#pragma unroll
                        for (int bb = 0; bb < BPL; bb++)
#pragma unroll
                            for (int j = 0; j < NT; j++) {
                                if (U4) {
                                    const int4 ps = *reinterpret_cast<const int4 *>(psum + ((st * QS_NB + b0 + bb) * NT + j) * QS_PLANES);
                                    v[bb][4 * j] -= ps.x; v[bb][4 * j + 1] -= ps.y; v[bb][4 * j + 2] -= ps.z; v[bb][4 * j + 3] -= ps.w;
                                }
                                const float f = fmaf(fmaf(fmaf((float)v[bb][4 * j + 3], P7, (float)v[bb][4 * j + 2]), P7, (float)v[bb][4 * j + 1]), P7,
                                                     (float)v[bb][4 * j]);
                                acc[j] = fmaf(ds[bb][j], f, acc[j]);
                                if (FMT == FMT_GGML_Q4_K) acc[j] = fmaf(-dm[b0 + bb], sxsum[(st * QS_NB + b0 + bb) * NT + j], acc[j]);
                            }
                    }
                }
                it = it_end;
                // group 1 hands its sums to group 0
                float *xb = xch + (ti & 1) * (8 * QS_ROWS);
                if (h == 1) {
#pragma unroll
                    for (int j = 0; j < NT; j++) xb[j * QS_ROWS + row] = acc[j];
                }
                named_bar_sync(1, QS_SCALE_WARPS * 32);
                const int r = (cta_in_slice + ti * ctas_per_slice) * QS_ROWS + row;
                if (h == 0 && ok && r < a.n) {
#pragma unroll
                    for (int j = 0; j < NT; j++) {
                        if (j < a.T) {
                            const float v = acc[j] + xb[j * QS_ROWS + row];
                            if (a.nslice == 1) a.dst[(size_t)j * a.ldo + r] = v + (a.bias ? a.bias[r] : 0.f);
                            else a.dst[((size_t)slice * a.T + j) * a.n + r] = v;
                        }
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

static size_t qs_smem_bytes(int fmt, int nt, int max_slice_st) {
    const int nrows = nt <= 4 ? 16 : 32;
    return 1024 + (size_t)max_slice_st * nrows * 128 + (size_t)qs_raw_depth(fmt, nt) * qs_stage_bytes(fmt) + 2 * 8 * QS_ROWS * sizeof(float) +
           (size_t)max_slice_st * QS_NB * nt * sizeof(float) * (fmt == FMT_GGML_Q4_K ? 2 : fmt == FMT_GGML_Q4_0 && nt == 1 ? 1 + QS_PLANES : 1) + (2 * qs_raw_depth(fmt, nt) + 4 * 4 + 1) * 8 + 16;
}

template <int FMT, int NT>
static int qs_launch(const QsArgs &a, int grid, cudaStream_t st) {
    static PerDevice configured = {};            // largest dynamic shared memory size requested so far, per device
    const size_t smem = qs_smem_bytes(FMT, NT, a.max_slice_st);
    int dev = 0;
    if (configured.below(smem, &dev)) {
        MB_CUDA(cudaFuncSetAttribute(qstream_tc_kernel<FMT, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured.record(dev, smem);
    }
    qstream_tc_kernel<FMT, NT><<<grid, QS_THREADS, smem, st>>>(a);
    MB_CUDA(cudaGetLastError());
    return 0;
}

// Partial sums of the K slices go through w.tc_scratch (qstream_tc_scratch_bytes(n, k) bytes, allocated
// with the weight): calls on one weight must not overlap in time. Activations must be finite.
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
    const int nt = T <= 1 ? 1 : T <= 2 ? 2 : T <= 4 ? 4 : 8;
    int rc;
    if (w.fmt == FMT_GGML_Q4_0)
        rc = nt == 1 ? qs_launch<FMT_GGML_Q4_0, 1>(a, grid, st) : nt == 2 ? qs_launch<FMT_GGML_Q4_0, 2>(a, grid, st)
           : nt == 4 ? qs_launch<FMT_GGML_Q4_0, 4>(a, grid, st) : qs_launch<FMT_GGML_Q4_0, 8>(a, grid, st);
    else if (w.fmt == FMT_GGML_Q4_K)
        rc = nt == 1 ? qs_launch<FMT_GGML_Q4_K, 1>(a, grid, st) : nt == 2 ? qs_launch<FMT_GGML_Q4_K, 2>(a, grid, st)
           : nt == 4 ? qs_launch<FMT_GGML_Q4_K, 4>(a, grid, st) : qs_launch<FMT_GGML_Q4_K, 8>(a, grid, st);
    else
        rc = nt == 1 ? qs_launch<FMT_GGML_Q8_0, 1>(a, grid, st) : nt == 2 ? qs_launch<FMT_GGML_Q8_0, 2>(a, grid, st)
           : nt == 4 ? qs_launch<FMT_GGML_Q8_0, 4>(a, grid, st) : qs_launch<FMT_GGML_Q8_0, 8>(a, grid, st);
    if (rc) return rc;
    if (nslice > 1) {
        qs_reduce_kernel<<<dim3(cdiv(w.n, 256), T), 256, 0, st>>>(scratch, out, ldo, bias, w.n, T, nslice);
        MB_CUDA(cudaGetLastError());
    }
    return 0;
}

}  // namespace mb
