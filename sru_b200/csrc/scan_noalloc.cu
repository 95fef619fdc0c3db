// Backward scan for callers that are not allowed to allocate device memory.
//
// sru_b200_scan_backward needs a few megabytes of scratch (the per-row-tile partial sums of
// grad_weight_c / grad_bias that a second small kernel adds up) and asks its caller for it.
// Some callers cannot provide any: code running inside a region where cudaMalloc is forbidden
// or would deadlock (a stream-ordered section whose allocator is frozen, a real-time inference
// loop with a fixed memory plan, a plugin host that hands out no allocator at all).  For them
// this file keeps the scratch in a fixed array that is part of the library image: every GPU
// that loads the library holds kNoAllocScratchBytes of it until the process exits.
//
// The array's name is only a host-side handle, not a device address, so the entry point looks
// the address up with cudaGetSymbolAddress, once per device, with that device current.  That
// first call on a device is the set-up call; make it before starting any stream capture.
#include "common.cuh"

namespace srub {
namespace {

constexpr size_t kNoAllocScratchBytes = 8u << 20;  // 8 MiB per device

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// Device address of the scratch array on the current device, resolved on first use there.
int noalloc_scratch(void **out) {
    static void *addr[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_error(SRU_ERR_CUDA, "cudaGetDevice failed: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return set_error(SRU_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    if (!addr[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p)
            return set_error(SRU_ERR_CUDA, "cudaGetSymbolAddress(scratch) failed: %s", cudaGetErrorString(e));
        addr[dev] = p;
    }
    *out = addr[dev];
    return 0;
}

}  // namespace
}  // namespace srub

using namespace srub;

extern "C" size_t sru_b200_scan_backward_noalloc_max_bytes(void) { return kNoAllocScratchBytes; }

extern "C" int sru_b200_scan_backward_noalloc(
    void *grad_u, void *grad_x, void *grad_wc, void *grad_bias, void *grad_init, const void *u, const void *x,
    const void *weight_c, const void *bias, const void *c_init, const void *mask_c, const uint8_t *mask_pad,
    const void *c_hist, const void *grad_h, const void *grad_last, int64_t length, int64_t batch, int64_t hidden,
    int dirs, int k, int activation_type, int skip_type, int is_custom, double scale_x, int dtype, int c_dtype,
    void *stream) {
    const size_t need = sru_b200_scan_backward_workspace_bytes(length, batch, hidden, dirs, k, dtype);
    if (need > kNoAllocScratchBytes)
        return set_error(SRU_ERR_WORKSPACE,
                         "problem needs %zu bytes of scratch but the built-in scratch holds %zu "
                         "(batch*dirs*hidden must stay below %zu); use sru_b200_scan_backward with a caller workspace",
                         need, (size_t)kNoAllocScratchBytes,
                         (size_t)(kNoAllocScratchBytes / (4 * (dtype == SRU_F64 ? sizeof(double) : sizeof(float)))) + 1);
    void *scratch = nullptr;
    const int rc = noalloc_scratch(&scratch);
    if (rc) return rc;
    // Nothing in the scratch has to start at zero: each launch overwrites every partial it later
    // reads.  The same kernels as sru_b200_scan_backward run, with the built-in array as workspace.
    return sru_b200_scan_backward(grad_u, grad_x, grad_wc, grad_bias, grad_init, u, x, weight_c, bias, c_init,
                                  mask_c, mask_pad, c_hist, grad_h, grad_last, length, batch, hidden, dirs, k,
                                  activation_type, skip_type, is_custom, scale_x, dtype, c_dtype, scratch,
                                  kNoAllocScratchBytes, stream);
}
