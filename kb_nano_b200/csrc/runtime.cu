// Error string, launch counter and device queries shared by every entry point.
#include <atomic>
#include <stdarg.h>

#include "gemm_common.cuh"

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


// The word's device address, looked up once per device (the same value whichever host thread stores it first).
int gemm_status_ptr(int32_t** out) {
    static std::atomic<int32_t*> cached[64];
    int dev = 0;
    KBN_CUDA(cudaGetDevice(&dev));
    KBN_REQUIRE(dev >= 0 && dev < 64, KBN_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    int32_t* p = cached[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        KBN_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_gemm_status));
        cached[dev].store(p, std::memory_order_release);
    }
    *out = p;
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

int kbn_gemm_clear_status(kbn_stream_t stream) {
    using namespace kbn;
    int32_t* p = nullptr;
    int rc = gemm_status_ptr(&p);
    if (rc != KBN_OK) return rc;
    KBN_CUDA(cudaMemsetAsync(p, 0, sizeof(int32_t), static_cast<cudaStream_t>(stream)));
    return KBN_OK;
}


}  // extern "C"
