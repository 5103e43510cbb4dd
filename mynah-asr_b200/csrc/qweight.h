// A weight matrix [n, k] (PyTorch linear layout) resident in HBM — the device
// counterpart of the reference's mynah_asr_qmat (src/qmat.h:39-47).
#pragma once
#include "common.cuh"

namespace mb {

struct QWeight {
    int fmt = 0;                // FMT_* (kernels.h)
    int n = 0, k = 0;
    uint8_t *raw = nullptr;     // stored blocks exactly as given (padded by 64 bytes); small-M kernels stream these
    size_t raw_bytes = 0;
    float *scales = nullptr;    // native formats: [n] or [n, k/32]
    __half *hi = nullptr;       // decoded operand planes [n, k] for the tensor-core contraction
    __half *lo = nullptr;
    float *f32 = nullptr;       // decoded f32 copy (only where a kernel wants f32 weights)
    float *bias = nullptr;      // optional [n]
    uint8_t *mma_q = nullptr;   // Q4_0 / Q8_0 quants re-tiled for the tensor-core small-T kernel (qgemv_mma.cu)
    __half *mma_d = nullptr;    // their block scales [n, k/32]
    uint8_t *tc_q = nullptr;    // Q4_0 / Q8_0 stages re-tiled for the tcgen05 streaming kernel (qstream_tc.cu)
    float *tc_scratch = nullptr;  // its K-slice partial sums, when the shape is split over K
};

// What a kernel launcher needs from an opaque mynah_b200_qmat handle.
struct QmatView {
    const QWeight *w;
    cudaStream_t stream;
};
QmatView qmat_view(const void *handle);

}  // namespace mb
