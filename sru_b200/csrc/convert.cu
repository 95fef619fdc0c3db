// Element type conversion between the 16-bit storage types and float32, 16 bytes per thread and access.
//
// Where it is used: the module returns h in the type the reference returns (float32 for a float32 input under
// 16-bit autocast, sru/ops.py:116-127) while the layers hand 16-bit h to each other; the last layer's h is widened
// once, and its gradient narrowed once.  The framework's converting copy reaches about a quarter of the HBM bandwidth
// on these sizes (2.1 G elements); this kernel is bound by it.
#include <algorithm>

#include "common.cuh"

namespace srub {

template <typename TI, typename TO>
__global__ void __launch_bounds__(256) convert_kernel(TO *__restrict__ dst, const TI *__restrict__ src, int64_t n8) {
    // n8 groups of 8 elements; the tail (n % 8) is done by convert_tail_kernel.  Four groups per thread and iteration,
    // all loads first: 64-128 bytes in flight per thread keep HBM busy with the few resident waves of this grid.
    constexpr int U = 4;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < n8; i0 += stride * U) {
        Pack<TI, 8> in[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = i0 + u * stride;
            if (i < n8) in[u] = *reinterpret_cast<const Pack<TI, 8> *>(src + i * 8);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = i0 + u * stride;
            if (i < n8) {
                Pack<TO, 8> out;
#pragma unroll
                for (int j = 0; j < 8; ++j) out.v[j] = Cvt<TO>::from_f(Cvt<TI>::to_f(in[u].v[j]));
                *reinterpret_cast<Pack<TO, 8> *>(dst + i * 8) = out;
            }
        }
    }
}

template <typename TI, typename TO>
__global__ void convert_tail_kernel(TO *__restrict__ dst, const TI *__restrict__ src, int64_t first, int64_t n) {
    const int64_t i = first + threadIdx.x;
    if (i < n) dst[i] = Cvt<TO>::from_f(Cvt<TI>::to_f(src[i]));
}

template <typename TI, typename TO>
static int launch_convert(void *dst, const void *src, int64_t n, cudaStream_t st) {
    const int64_t n8 = n / 8;
    if (n8 > 0) {
        const int64_t want = (n8 + 256 * 4 - 1) / (256 * 4);
        const unsigned blocks = (unsigned)std::min<int64_t>(want, 148 * 16);     // grid-stride: a few resident waves of a B200
        convert_kernel<TI, TO><<<blocks, 256, 0, st>>>(static_cast<TO *>(dst), static_cast<const TI *>(src), n8);
    }
    if (n8 * 8 < n) convert_tail_kernel<TI, TO><<<1, 8, 0, st>>>(static_cast<TO *>(dst), static_cast<const TI *>(src), n8 * 8, n);
    SRUB_CUDA_CHECK(cudaGetLastError());
    return 0;
}

}  // namespace srub

extern "C" int sru_b200_convert(void *dst, const void *src, int64_t n, int src_dtype, int dst_dtype, void *stream) {
    using namespace srub;
    if (n < 0 || (n > 0 && (!dst || !src))) return set_error(SRU_ERR_BAD_ARG, "convert: null pointer or negative count");
    if (n == 0) return 0;
    if ((reinterpret_cast<uintptr_t>(dst) & 15u) || (reinterpret_cast<uintptr_t>(src) & 15u))
        return set_error(SRU_ERR_BAD_ARG, "convert: pointers must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (src_dtype == SRU_BF16 && dst_dtype == SRU_F32) return launch_convert<__nv_bfloat16, float>(dst, src, n, st);
    if (src_dtype == SRU_F16 && dst_dtype == SRU_F32) return launch_convert<__half, float>(dst, src, n, st);
    if (src_dtype == SRU_F32 && dst_dtype == SRU_BF16) return launch_convert<float, __nv_bfloat16>(dst, src, n, st);
    if (src_dtype == SRU_F32 && dst_dtype == SRU_F16) return launch_convert<float, __half>(dst, src, n, st);
    return set_error(SRU_ERR_UNSUPPORTED, "convert: %d -> %d (one side must be float32, the other bf16 or fp16)", src_dtype,
                     dst_dtype);
}
