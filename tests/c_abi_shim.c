/* The reference-side binding of the existing CUDA hook (src/backend.c:23-26, 74-78), as a C11
 * translation unit: proves that include/mynah_b200.h is plain C and that the library links from C.
 * Built and run by tests/test_abi.py; it makes no compute call unless a device is present. */
#include <stdio.h>

#include "mynah_b200.h"

int mynah_asr_cuda_available(void) { return mynah_b200_available(); }

int mynah_asr_cuda_gemm_wt(const float *x, const float *w, float *out, int T, int n, int k) {
    return mynah_b200_gemm_wt(x, w, out, T, n, k);      /* 0 ok, -1: the caller falls back to its CPU path */
}

int main(void) {
    mynah_b200_config cfg;
    mynah_b200_config_default(&cfg);
    if (cfg.n_fft != 512 || cfg.hop_length != 160 || cfg.strict != 1) return 2;
    if (!mynah_asr_cuda_available()) {
        float x[64] = {0}, w[64] = {0}, out[1];
        if (mynah_asr_cuda_gemm_wt(x, w, out, 1, 1, 64) != -1) return 3;    /* no device: must refuse, not compute */
        printf("no device: %s\n", mynah_b200_last_error());
        return 0;
    }
    printf("device present\n");
    return 0;
}
