// float32 contraction on the 16-bit tensor cores by operand splitting (sm_100a).
//
// tcgen05 has no full-precision float32 form (kind::tf32 keeps 10 mantissa bits), so a float32 projection would have
// to leave the tensor cores.  Instead each float32 operand is written as the sum of three bfloat16 numbers,
//     a = a1 + a2 + a3,   a1 = bf16(a), a2 = bf16(a - a1), a3 = bf16(a - a1 - a2)        (8 + 8 + 8 mantissa bits),
// and the product is assembled from the six partial products whose weight is at least 2^-16 of the leading one:
//     a*b ~ a1 b1 + a1 b2 + a2 b1 + a1 b3 + a3 b1 + a2 b2            (what is dropped is below 2^-24 relative).
// All six run as ONE bf16 GEMM with fp32 accumulation in tensor memory: the reduction dimension is made six times
// as long, op(A') = [A1 A1 A2 A1 A3 A2] and op(B') = [B1; B2; B1; B3; B1; B2] stacked along K.  A small kernel
// writes the stacked 16-bit operands into the caller's workspace; the contraction itself is the tcgen05 GEMM of
// gemm_tcgen05.cu with its fp32 epilogue.  Cost: six times the bf16 work and 3x the operands' bytes as scratch -
// still several times faster than a float32 FMA GEMM, and no library kernel on the path.
#include <algorithm>

#include "common.cuh"

namespace srub {
namespace {

// which of the three pieces goes into slab s of the stacked operand
__constant__ int kPieceA[6] = {0, 0, 1, 0, 2, 1};
__constant__ int kPieceB[6] = {0, 1, 0, 2, 0, 1};

__device__ __forceinline__ void split3(float v, __nv_bfloat16 (&p)[3]) {
    p[0] = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(p[0]);
    p[1] = __float2bfloat16_rn(r1);
    p[2] = __float2bfloat16_rn(r1 - __bfloat162float(p[1]));
}

// src (rows, cols) float32, row pitch ld.  along_cols: dst (rows, 6*cols), slab s occupies columns [s*cols, (s+1)*cols);
// otherwise dst (6*rows, cols), slab s occupies rows [s*rows, (s+1)*rows).  is_b selects the piece table.
__global__ void split_stack_kernel(const float *__restrict__ src, __nv_bfloat16 *__restrict__ dst, int64_t rows,
                                   int64_t cols, int64_t ld, int along_cols, int is_b) {
    const int64_t n = rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / cols, c = i - r * cols;
        __nv_bfloat16 p[3];
        split3(src[r * ld + c], p);
#pragma unroll
        for (int s = 0; s < 6; ++s) {
            const int piece = is_b ? kPieceB[s] : kPieceA[s];
            const __nv_bfloat16 v = piece == 0 ? p[0] : (piece == 1 ? p[1] : p[2]);
            if (along_cols) dst[r * (6 * cols) + s * cols + c] = v;
            else dst[(s * rows + r) * cols + c] = v;
        }
    }
}

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace
}  // namespace srub

using namespace srub;

extern "C" size_t sru_b200_gemm_f32_workspace_bytes(int64_t m, int64_t n, int64_t k_dim) {
    if (m <= 0 || n <= 0 || k_dim <= 0) return 0;
    const size_t a = align256((size_t)6 * m * k_dim * 2), b = align256((size_t)6 * k_dim * n * 2);
    return a + b + align256(sru_b200_gemm_workspace_bytes(m, n, 6 * k_dim, 0));
}

extern "C" int sru_b200_gemm_f32(float *c, const float *a, const float *b, const float *col_bias, int64_t m, int64_t n,
                                 int64_t k_dim, int64_t lda, int64_t ldb, int64_t ldc, int trans_a, int trans_b,
                                 int accumulate, void *workspace, size_t workspace_bytes, void *stream) {
    if (m < 0 || n < 0 || k_dim < 1) return set_error(SRU_ERR_BAD_ARG, "bad gemm sizes");
    if (m == 0 || n == 0) return 0;
    if (!c || !a || !b) return set_error(SRU_ERR_BAD_ARG, "gemm pointers must not be null");
    if (m % 8 || n % 8 || k_dim % 8 || ldc % 8)
        return set_error(SRU_ERR_UNSUPPORTED, "float32 gemm: M, N, K and ldc must be multiples of 8");
    const size_t need = sru_b200_gemm_f32_workspace_bytes(m, n, k_dim);
    if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return set_error(SRU_ERR_WORKSPACE, "float32 gemm: 256-byte aligned workspace of %zu bytes needed, %zu given", need,
                         workspace_bytes);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    __nv_bfloat16 *a6 = reinterpret_cast<__nv_bfloat16 *>(ws);
    const size_t a_bytes = align256((size_t)6 * m * k_dim * 2), b_bytes = align256((size_t)6 * k_dim * n * 2);
    __nv_bfloat16 *b6 = reinterpret_cast<__nv_bfloat16 *>(ws + a_bytes);
    void *inner_ws = ws + a_bytes + b_bytes;
    const size_t inner_bytes = workspace_bytes - a_bytes - b_bytes;
    // op(A) is M x K: stored (M, K) -> stack along its columns; stored (K, M) (trans_a) -> stack along its rows
    {
        const int64_t rows = trans_a ? k_dim : m, cols = trans_a ? m : k_dim;
        const unsigned blocks = (unsigned)std::min<int64_t>((rows * cols + 255) / 256, 148 * 16);
        split_stack_kernel<<<blocks, 256, 0, st>>>(a, a6, rows, cols, lda, trans_a ? 0 : 1, 0);
        SRUB_CUDA_CHECK(cudaGetLastError());
    }
    // op(B) is K x N: stored (K, N) -> stack along its rows; stored (N, K) (trans_b) -> stack along its columns
    {
        const int64_t rows = trans_b ? n : k_dim, cols = trans_b ? k_dim : n;
        const unsigned blocks = (unsigned)std::min<int64_t>((rows * cols + 255) / 256, 148 * 16);
        split_stack_kernel<<<blocks, 256, 0, st>>>(b, b6, rows, cols, ldb, trans_b ? 1 : 0, 1);
        SRUB_CUDA_CHECK(cudaGetLastError());
    }
    const int64_t lda6 = trans_a ? m : 6 * k_dim, ldb6 = trans_b ? 6 * k_dim : n;
    return sru_b200_gemm_ws(c, a6, b6, col_bias, m, n, 6 * k_dim, lda6, ldb6, ldc, trans_a, trans_b, SRU_BF16, SRU_F32,
                            accumulate, inner_ws, inner_bytes, stream);
}
