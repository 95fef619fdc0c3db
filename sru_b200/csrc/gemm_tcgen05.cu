// placeholder, replaced by the tcgen05 GEMM
#include "common.cuh"
extern "C" int sru_b200_gemm(void *c, const void *a, const void *b, const float *col_bias, int64_t m,
                             int64_t n, int64_t k_dim, int64_t lda, int64_t ldb, int64_t ldc, int trans_a,
                             int trans_b, int ab_dtype, int c_dtype, int accumulate, void *stream) {
    return srub::set_error(SRU_ERR_UNSUPPORTED, "gemm not built yet");
}
