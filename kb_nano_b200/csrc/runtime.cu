// Error string, launch counter and device queries shared by every entry point.
#include <atomic>
#include <stdarg.h>

#include "common.cuh"

namespace kbn {
int gemm_status_ptr(int32_t** out);
}

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

__device__ int32_t g_gemm_status = 0;

int gemm_status_ptr(int32_t** out) {
    KBN_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(out), g_gemm_status));
    return KBN_OK;
}

}  // namespace kbn

extern "C" {

int kbn_version(void) { return 1; }
const char* kbn_last_error(void) { return kbn::g_err; }
int64_t kbn_launch_count(void) { return kbn::g_launches.load(); }

int kbn_gemm_status(int32_t* host_out, kbn_stream_t stream) {
    using namespace kbn;
    KBN_REQUIRE(host_out, KBN_ERR_ARG, "kbn_gemm_status: null pointer");
    KBN_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    KBN_CUDA(cudaMemcpyFromSymbol(host_out, g_gemm_status, sizeof(int32_t)));
    return KBN_OK;
}

}  // extern "C"
