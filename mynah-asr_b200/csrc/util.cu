// Error string plumbing shared by every translation unit.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace mb {
static thread_local char g_err[512] = "";
void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
const char *last_error() { return g_err; }

bool PerDevice::below(size_t want, int *dev) const {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= MB_MAX_DEVICES) { *dev = -1; return true; }
    *dev = d;
    return __atomic_load_n(&v[d], __ATOMIC_ACQUIRE) < want;
}
void PerDevice::record(int dev, size_t want) {
    // racing threads configure the same attribute with the same or a larger value; keep the maximum
    if (dev < 0 || dev >= MB_MAX_DEVICES) return;
    size_t cur = __atomic_load_n(&v[dev], __ATOMIC_ACQUIRE);
    while (cur < want && !__atomic_compare_exchange_n(&v[dev], &cur, want, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE)) {}
}
int device_sm_count() {
    static PerDevice sms = {};
    int dev = 0;
    if (!sms.below(1, &dev)) return (int)sms.v[dev];
    int n = 0;
    if (dev < 0 || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    sms.record(dev, (size_t)n);
    return n;
}
}  // namespace mb
