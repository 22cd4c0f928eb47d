// Shared host/device helpers for the kbn FP8 library (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "../../include/kbn_fp8.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "kbn_fp8 is written for sm_100a only"
#endif

namespace kbn {

// ---- error reporting -----------------------------------------------------------------------
void set_error(const char* fmt, ...);   // thread-local message returned by kbn_last_error()

#define KBN_REQUIRE(cond, code, ...)            \
    do {                                        \
        if (!(cond)) {                          \
            ::kbn::set_error(__VA_ARGS__);      \
            return (code);                      \
        }                                       \
    } while (0)

#define KBN_CUDA(call)                                                                        \
    do {                                                                                      \
        cudaError_t e__ = (call);                                                             \
        if (e__ != cudaSuccess) {                                                             \
            ::kbn::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), __FILE__, \
                             __LINE__);                                                       \
            return KBN_ERR_CUDA;                                                              \
        }                                                                                     \
    } while (0)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int sm_count();   // SMs of the current device (cached per device)

extern std::atomic<int64_t> g_launches;   // kernels launched by this library (kbn_launch_count)
static inline void count_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// Checks the launch that was just enqueued.
#define KBN_CHECK_LAUNCH()                                                                    \
    do {                                                                                      \
        cudaError_t e__ = cudaGetLastError();                                                 \
        if (e__ != cudaSuccess) {                                                             \
            ::kbn::set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(e__),     \
                             __FILE__, __LINE__);                                             \
            return KBN_ERR_CUDA;                                                              \
        }                                                                                     \
        ::kbn::count_launch();                                                                \
    } while (0)

// ---- device helpers --------------------------------------------------------------------------
#ifdef __CUDACC__

// Launch with programmatic stream serialisation: the grid may be scheduled while the kernel before it in the stream
// is still running (if that kernel allows it, else when it has ended).  The kernel must call pdl_prologue_done() before
// it reads anything that kernel may have written and before its own first global write.
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Lets the next kernel of the stream be scheduled under this one, then waits until the kernel before this one has
// ended and its writes are visible.  What a kernel does before this call must not depend on that kernel.
__device__ __forceinline__ void pdl_prologue_done() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ uint32_t abs_bf16x2(uint32_t a) { return a & 0x7fff7fffu; }

__device__ __forceinline__ uint32_t max_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Per half: the larger of |a| and |b| with the sign of a*b -- absmax chains need no separate abs until the end.
__device__ __forceinline__ uint32_t absmax_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// {hi, lo} fp32 -> packed bf16x2, round-to-nearest-even
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

// two fp32 -> two e4m3 bytes (lo in bits 0-7), round-to-nearest-even, saturating to +-448
__device__ __forceinline__ uint32_t pack_e4m3x2(float lo, float hi) {
    uint16_t d;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(d) : "f"(hi), "f"(lo));
    return d;
}

// Power-of-two scale 2^ceil(log2(a/448)) of a positive normal fp32 `a`, by exponent arithmetic:
// a = m*2^k with m in [1,2); a/448 = (m/1.75)*2^(k-8), so the ceiling is k-8, plus one when
// m > 1.75.  Returns the biased exponent field of the scale (scale bits = field << 23).
__device__ __forceinline__ uint32_t ue8m0_scale_field(float a) {
    uint32_t b = __float_as_uint(a);
    return (b >> 23) - 8u + ((b & 0x7fffffu) > 0x600000u ? 1u : 0u);
}

#endif  // __CUDACC__

}  // namespace kbn
