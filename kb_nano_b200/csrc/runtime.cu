// Error string, launch counter and device queries shared by every entry point.
#include <atomic>
#include <stdarg.h>

#include "common.cuh"

namespace kbn {

static thread_local char g_err[512] = "";
std::atomic<int64_t> g_launches{0};

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace kbn

extern "C" {

int kbn_version(void) { return 1; }
const char* kbn_last_error(void) { return kbn::g_err; }
int64_t kbn_launch_count(void) { return kbn::g_launches.load(); }

}  // extern "C"
