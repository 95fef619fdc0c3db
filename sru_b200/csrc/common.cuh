// Shared device/host helpers of the sru_b200 library (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/sru_b200.h"

namespace srub {

// ---------------------------------------------------------------------------------------
// Host-side error plumbing (thread-local message, no exceptions across the C ABI)
// ---------------------------------------------------------------------------------------
int set_error(int code, const char *fmt, ...);
int *device_error_flag();  // device int, set non-zero by a kernel whose bounded wait gave up
int ensure_context();      // binds the device's primary context to this thread if it has none; 0 or SRU_ERR_CUDA

// Tuning / diagnostic options (sru_b200_set_option).  Each starts from the environment variable
// SRU_B200_<NAME IN CAPITALS>, read ONCE per process on first use; a negative value means "not set,
// let the library choose".
enum Option {
    OPT_FWD_V, OPT_BWD_V, OPT_SCAN_THREADS, OPT_FWD_THREADS, OPT_BWD_THREADS, OPT_SCAN_SS, OPT_SCAN_STAGES,
    OPT_FORCE_GENERIC, OPT_FWD_SPLIT, OPT_GEMM_KSPLIT, OPT_GEMM_2SM, OPT_GEMM_EPI_WARPS, OPT_GEMM_DYNAMIC,
    OPT_GEMM_RASTER, OPT_GEMM_TMA_STORE, OPT_COUNT
};
int option(Option o, int dflt);   // the option's value, or dflt when it is not set

// Which scan kernel family the calling thread's most recent scan launch used (sru_b200_last_scan_kernel).
enum { SCAN_KERNEL_NONE = 0, SCAN_KERNEL_PIPELINED = 1, SCAN_KERNEL_GENERIC = 2, SCAN_KERNEL_SPLIT = 3 };
void note_scan_kernel(int which);

#define SRUB_CUDA_CHECK(expr)                                                              \
    do {                                                                                   \
        cudaError_t err__ = (expr);                                                        \
        if (err__ != cudaSuccess)                                                          \
            return ::srub::set_error(SRU_ERR_CUDA, "%s failed: %s", #expr,                 \
                                     cudaGetErrorString(err__));                           \
    } while (0)

static inline size_t dtype_size(int dt) {
    switch (dt) {
        case SRU_F32: return 4;
        case SRU_F16: return 2;
        case SRU_BF16: return 2;
        case SRU_F64: return 8;
    }
    return 0;
}

// ---------------------------------------------------------------------------------------
// Storage <-> compute conversions
// ---------------------------------------------------------------------------------------
template <typename T> struct Cvt;
template <> struct Cvt<float> {
    __device__ __forceinline__ static float to_f(float v) { return v; }
    __device__ __forceinline__ static float from_f(float v) { return v; }
};
template <> struct Cvt<double> {
    __device__ __forceinline__ static double to_f(double v) { return v; }
    __device__ __forceinline__ static double from_f(double v) { return v; }
};
template <> struct Cvt<__half> {
    __device__ __forceinline__ static float to_f(__half v) { return __half2float(v); }
    __device__ __forceinline__ static __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct Cvt<__nv_bfloat16> {
    __device__ __forceinline__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ __forceinline__ static __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// N elements of T moved as one unit with the widest vector access its size allows (<= 16 B).
template <int BYTES> struct PackAlign {
    static constexpr int value = (BYTES % 16 == 0) ? 16 : (BYTES % 8 == 0) ? 8 : (BYTES % 4 == 0) ? 4 : 2;
};
template <typename T, int N> struct alignas(PackAlign<sizeof(T) * N>::value) Pack {
    T v[N];
};

// ---------------------------------------------------------------------------------------
// PTX: mbarrier + bulk asynchronous copy (TMA engine, untiled form)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
// One probe of the barrier.  The thread is suspended by the hardware until the phase completes or about a
// microsecond has passed (the hint), so a warp that waits costs its scheduler a probe per microsecond, not a spin.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(1000u)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Wait for the barrier phase with the given parity, for at most ~2 s.  Returns false
// on timeout; the caller records the failure and leaves its loop instead of hanging.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 128; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > 2000000000ull) return false;
    }
}
// global -> this CTA's shared memory, completion counted in bytes on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst_smem, const void *src, uint32_t bytes,
                                              uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

// ---------------------------------------------------------------------------------------
// Fast sigmoid pieces: sigma(z) = 1 / (1 + 2^(-z*log2(e)))
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
constexpr float kNegLog2e = -1.4426950408889634f;

}  // namespace srub
