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
}  // namespace mb
