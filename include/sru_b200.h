/*
 * sru_b200 -- C ABI of the B200 (sm_100a) SRU hot path: the light-recurrence scan
 * (forward / backward) and the projection GEMM U = x * W.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless said
 * otherwise; every call is asynchronous on the given CUDA stream (a cudaStream_t
 * passed as void*).  Return value: 0 on success, a negative SRU_ERR_* code
 * otherwise; sru_b200_last_error() gives the message of the calling thread's last
 * failure.  No exception crosses this boundary and there is no CPU fallback.
 *
 * Tensor layouts are the reference's (asappresearch/sru v2.6.0):
 *   u, grad_u      (L, B, dirs, d, k)   gate index innermost
 *                  (sru/csrc/sru_cuda_kernel.cu:54,218; sru/ops.py:176)
 *   x, h, grad_h, grad_x, c_hist   (L, B, dirs*d)
 *   weight_c, bias, grad_weight_c, grad_bias   (2, dirs, d)
 *                  (sru_cuda_kernel.cu:47-51,212-216; ops.py:183-185)
 *   custom V / its gradient (is_custom != 0)   (L, B, dirs, d, 2)
 *   c_init, mask_c, c_last, grad_last, grad_init   (B, dirs*d)
 *   mask_pad       (L, B) bytes, non-zero = padded position
 *                  (sru_cuda_kernel.cu:56,61)
 *
 * Element types.  `dtype` is the storage type of the large per-time-step tensors
 * (u, x, h, grad_h, grad_u, grad_x, custom V); `c_dtype` is the storage type of
 * c_hist (the same as dtype, or SRU_F32).  The small per-column tensors
 * (weight_c when not custom, bias, c_init, mask_c, c_last, grad_last,
 * grad_weight_c when not custom, grad_bias, grad_init) are float, or double when
 * dtype == SRU_F64.  Arithmetic is float (double for SRU_F64).
 */
#ifndef SRU_B200_H_
#define SRU_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { SRU_F32 = 0, SRU_F16 = 1, SRU_BF16 = 2, SRU_F64 = 3 };

enum {
    SRU_OK = 0,
    SRU_ERR_BAD_ARG = -1,      /* null pointer, bad size, unknown enum value        */
    SRU_ERR_UNSUPPORTED = -2,  /* combination not implemented (message says which)  */
    SRU_ERR_WORKSPACE = -3,    /* workspace missing or too small                    */
    SRU_ERR_CUDA = -4,         /* a CUDA runtime / driver call failed               */
    SRU_ERR_DEVICE = -5        /* a kernel reported a timed-out wait (see below)    */
};

/* Library version, major*10000 + minor*100 + patch. */
int sru_b200_version(void);

/* Message of the calling thread's most recent failure ("" if none). */
const char *sru_b200_last_error(void);

/*
 * Synchronises `stream` and returns SRU_ERR_DEVICE if any kernel since the last
 * call gave up a bounded wait (an mbarrier that never completed); the flag is
 * cleared.  Kernels never spin without a limit, so a lost copy shows up here as
 * an error code instead of a hang.
 */
int sru_b200_check_device_error(void *stream);

/*
 * Tuning and diagnostic options.  No counterpart in the reference (its launch configuration is fixed,
 * sru/csrc/sru_cuda_kernel.cu:841-846).  Every option starts "not set" (the library chooses) or from
 * the environment variable SRU_B200_<NAME IN CAPITALS>, which is read once per process; afterwards only
 * these calls change it.  A negative value un-sets an option.  Process-wide, not per stream.
 *   fwd_v, bwd_v                       columns per thread of the pipelined scans (1, 2, 4)
 *   scan_threads, fwd_threads, bwd_threads   consumer threads per CTA (32..128)
 *   scan_ss, scan_stages               time steps per ring stage, ring depth
 *   force_generic                      1: always the one-thread-per-column kernels
 *   fwd_split                          forward scan with the state chain and the output arithmetic on
 *                                      separate warps: 1 always (where the shape allows), 0 never
 *   gemm_ksplit, gemm_2sm, gemm_epi_warps    K slabs, pair kernel on/off, epilogue warps (4 or 8)
 *   gemm_raster                        tile order of the persistent GEMM grid: 1 consecutive tiles run down M,
 *                                      0 along N (default: whichever re-reads the smaller operand)
 *   gemm_tma_store                     16-bit output of the pair GEMM through tiled bulk stores from shared memory
 *                                      (1) or warp stores (0); default: bulk stores for K <= 512
 *   gemm_dynamic                       1: the pair GEMM hands out its tiles dynamically (needs the
 *                                      workspace form of the call); for products that share the GPU with
 *                                      a collective
 * Unknown names give SRU_ERR_BAD_ARG.  sru_b200_get_option returns the value, or -1 when not set.
 */
int sru_b200_set_option(const char *name, int value);
int sru_b200_get_option(const char *name);

/*
 * Which kernel family served the calling thread's most recent scan call (forward or backward):
 * 0 none yet / the call failed before a launch, 1 pipelined (TMA ring, registers across time),
 * 2 generic (one thread per column: custom V, tanh, odd hidden sizes, unaligned pointers, fp64),
 * 3 pipelined with split roles (forward, few columns).  No counterpart in the reference.
 */
int sru_b200_last_scan_kernel(void);

/*
 * Forward scan.  Replaces the four forward launchers of the reference,
 * sru_cuda_forward_simple / sru_cuda_bi_forward_simple / sru_cuda_forward /
 * sru_cuda_bi_forward (sru/csrc/sru_cuda_kernel.cu:827-860, :911-944, :995-1036,
 * :1039-1080), and the glue around them in sru/cuda_functional.py:38-153:
 * x*scale_x (:73-78) is applied in the kernel, and last_hidden (:146-152) is
 * written to c_last by the kernel.
 *
 *   h        out, every element written (0 at padded positions)
 *   c_hist   out, may be NULL (inference: the backward pass is not needed)
 *   c_last   out, may be NULL; final state per column: c[L-1] for direction 0,
 *            c[0] for direction 1
 *   x        used only when skip_type == 1 (may be NULL otherwise)
 *   bias     may be NULL: the bias has already been added to u by the producer
 *   c_init   may be NULL (zeros); mask_c, mask_pad may be NULL
 *   dirs     1 or 2; k 3 or 4; activation_type 0 (identity) or 1 (tanh)
 *   skip_type 0 none, 1 x (k == 3), 2 u[...,3] (k == 4)
 *   scale_x  multiplies x when skip_type == 1 (pass 1.0 for none)
 */
int sru_b200_scan_forward(
    void *h, void *c_hist, void *c_last,
    const void *u, const void *x, const void *weight_c, const void *bias,
    const void *c_init, const void *mask_c, const uint8_t *mask_pad,
    int64_t length, int64_t batch, int64_t hidden, int dirs, int k,
    int activation_type, int skip_type, int is_custom, double scale_x,
    int dtype, int c_dtype, void *stream);

/*
 * Bytes of scratch the backward scan needs for the same problem (partials of the
 * batch reduction of grad_weight_c / grad_bias).  Never more than
 * 32 * batch * dirs * hidden bytes.
 */
size_t sru_b200_scan_backward_workspace_bytes(
    int64_t length, int64_t batch, int64_t hidden, int dirs, int k, int dtype);

/*
 * Backward scan.  Replaces sru_cuda_backward_simple / sru_cuda_bi_backward_simple /
 * sru_cuda_backward / sru_cuda_bi_backward (sru_cuda_kernel.cu:863-908, :947-992,
 * :1083-1136, :1139-1192) and the host tail of sru/cuda_functional.py:253-260:
 * grad_x is multiplied by scale_x in the kernel and grad_weight_c / grad_bias are
 * reduced over the batch on the device, deterministically (fixed summation order,
 * no atomics), into (2, dirs, d).
 *
 *   grad_u     out, every element written (0 at padded positions)
 *   grad_x     out when skip_type == 1 (NULL otherwise)
 *   grad_wc    out: (2, dirs, d), or the per-step (L, B, dirs, d, 2) when is_custom
 *   grad_bias  out (2, dirs, d);  grad_init out (B, dirs*d)
 *   c_hist     the forward's saved states; grad_last may be NULL (zeros)
 *   workspace  device scratch of at least ..._workspace_bytes(); contents are
 *              undefined afterwards; calls sharing one workspace must be
 *              stream-ordered
 */
int sru_b200_scan_backward(
    void *grad_u, void *grad_x, void *grad_wc, void *grad_bias, void *grad_init,
    const void *u, const void *x, const void *weight_c, const void *bias,
    const void *c_init, const void *mask_c, const uint8_t *mask_pad,
    const void *c_hist, const void *grad_h, const void *grad_last,
    int64_t length, int64_t batch, int64_t hidden, int dirs, int k,
    int activation_type, int skip_type, int is_custom, double scale_x,
    int dtype, int c_dtype, void *workspace, size_t workspace_bytes, void *stream);

/*
 * Backward scan that allocates nothing and takes no workspace argument.  It has no
 * counterpart in the reference (whose operators allocate their outputs and scratch
 * themselves); it exists for hosts that must not, or cannot, allocate device memory
 * around the call: a serving loop with a fixed memory plan, a plugin sandbox without
 * an allocator, a section of a stream in which allocation calls are forbidden.
 *
 * Arguments, results and kernels are those of sru_b200_scan_backward; the scratch is a
 * fixed array inside the library, sru_b200_scan_backward_noalloc_max_bytes() bytes
 * (8 MiB) on every GPU that has loaded the library, held until the process exits.
 *
 *   - Limit: the problem must satisfy
 *       sru_b200_scan_backward_workspace_bytes(...) <= ..._noalloc_max_bytes(),
 *     i.e. batch * dirs * hidden <= 524288 (262144 for SRU_F64); larger problems get
 *     SRU_ERR_WORKSPACE and a message naming both sizes.
 *   - The first call on each device resolves the array's device address (that device
 *     must be current).  Make that first call before any stream capture begins.
 *   - All calls on a device share the one array.  Nothing in it needs clearing between
 *     calls, but two calls whose kernels overlap on the GPU (different streams without
 *     an ordering between them) race on it: keep calls on one device stream-ordered.
 *   - No cudaMalloc, no allocating library routine; inputs and outputs are still the caller's.
 *     One exception to "no runtime memory call at all": on a host thread that has no CUDA context
 *     bound yet, the library binds the device's primary context with cudaFree(NULL), which frees
 *     nothing and allocates nothing; a thread that already has a context (any thread that has made
 *     a runtime call on this device) never reaches it.
 */
size_t sru_b200_scan_backward_noalloc_max_bytes(void);

int sru_b200_scan_backward_noalloc(
    void *grad_u, void *grad_x, void *grad_wc, void *grad_bias, void *grad_init,
    const void *u, const void *x, const void *weight_c, const void *bias,
    const void *c_init, const void *mask_c, const uint8_t *mask_pad,
    const void *c_hist, const void *grad_h, const void *grad_last,
    int64_t length, int64_t batch, int64_t hidden, int dirs, int k,
    int activation_type, int skip_type, int is_custom, double scale_x,
    int dtype, int c_dtype, void *stream);

/*
 * Dense contraction on the tcgen05 tensor cores, the replacement for the three
 * library GEMMs around the scan: U = x * W of SRUCell.compute_U
 * (sru/modules.py:363-378) and, in backward, grad_x = grad_U * W^T and
 * grad_W = x^T * grad_U that autograd derives from it.
 *
 *   C[M,N] (row-major, leading dimension ldc) = op(A) * op(B) (+ col_bias)
 *   op(A) is M x K: A stored row-major (M,K) when trans_a == 0, or (K,M) when 1
 *   op(B) is K x N: B stored row-major (K,N) when trans_b == 0, or (N,K) when 1
 *   ab_dtype  SRU_BF16 or SRU_F16 (fp32 accumulation in tensor memory)
 *   c_dtype   SRU_BF16, SRU_F16 or SRU_F32
 *   col_bias  float[N] added to every row in the epilogue, or NULL.  With the gate
 *             bias of the SRU scattered to the gate-innermost columns
 *             ((dir*d+j)*k+1 -> bias[0,dir,j], (dir*d+j)*k+2 -> bias[1,dir,j])
 *             this folds `bias` into U, and the scan is then called with bias=NULL.
 *   accumulate  non-zero: C += result (C read in the epilogue)
 * Leading dimensions are in elements and must make every row start 16-byte aligned.
 */
int sru_b200_gemm(
    void *c, const void *a, const void *b, const float *col_bias,
    int64_t m, int64_t n, int64_t k_dim,
    int64_t lda, int64_t ldb, int64_t ldc,
    int trans_a, int trans_b, int ab_dtype, int c_dtype, int accumulate, void *stream);

/*
 * Lays the layer's gate bias out as the col_bias vector of the projection above, so that the GEMM's
 * epilogue adds it to U and the scan runs with bias = NULL.  `bias` is the layer's parameter, float
 * (2, width) with width = dirs * d (sru/modules.py:150; index map sru_cuda_kernel.cu:47-51);
 * `col_bias` receives float[width * k]: bias[0][j] at column j*k + 1, bias[1][j] at column j*k + 2, zeros
 * at the candidate column j*k and (k = 4) the highway column j*k + 3.  grad_bias still comes from the
 * backward scan (the column sums of grad_U at those columns are what it accumulates, :148,:156).
 */
int sru_b200_gate_bias_columns(float *col_bias, const float *bias, int64_t width, int k, void *stream);

/*
 * dst[i] = (dst type) src[i] for n elements, between float32 and one of the 16-bit types (either direction; round to
 * nearest even when narrowing).  Pointers 16-byte aligned.  Stands in for the framework's converting copy where the
 * module widens the last layer's 16-bit h to the float32 the reference returns (sru/ops.py:116-127) and narrows its
 * gradient; no counterpart in the reference's extension.
 */
int sru_b200_convert(void *dst, const void *src, int64_t n, int src_dtype, int dst_dtype, void *stream);

/*
 * The same contraction with caller-provided scratch.  Products whose output tiles alone
 * cannot fill the GPU but whose reduction is long (the weight gradient x^T grad_U:
 * M = input width, K = length * batch) are cut into K slabs whose fp32 partial results go to
 * `workspace` and are summed by a second small kernel.  With the option gemm_dynamic the pair
 * kernel also keeps its tile counter and mailboxes there.  sru_b200_gemm_workspace_bytes()
 * says how much scratch the call wants (0: none); with a NULL or smaller workspace
 * the call behaves exactly like sru_b200_gemm.  Calls that share one workspace must be stream-ordered.  Same library-GEMM counterpart in the
 * reference as sru_b200_gemm (sru/modules.py:363-378 and its autograd).
 */
size_t sru_b200_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k_dim, int has_bias);

int sru_b200_gemm_ws(
    void *c, const void *a, const void *b, const float *col_bias,
    int64_t m, int64_t n, int64_t k_dim,
    int64_t lda, int64_t ldb, int64_t ldc,
    int trans_a, int trans_b, int ab_dtype, int c_dtype, int accumulate,
    void *workspace, size_t workspace_bytes, void *stream);

/*
 * The same contraction for float32 operands and a float32 result, still on the 16-bit tensor cores: each operand
 * is split into three bfloat16 pieces and the six significant partial products are accumulated in fp32 by ONE
 * bf16 GEMM over a six-fold reduction length (error about 2^-24 relative per product, i.e. float32 level).  This
 * is what SRUCell.compute_U's `x.mm(weight)` (sru/modules.py:363-378) is for float32 tensors, where the reference
 * calls the library's float32 GEMM.  M, N, K and ldc must be multiples of 8; `workspace` (256-byte aligned,
 * ..._f32_workspace_bytes() bytes: three times the operands' size plus the inner product's own scratch) holds the
 * stacked 16-bit operands.  Leading dimensions lda / ldb are those of the float32 matrices, in elements.
 */
size_t sru_b200_gemm_f32_workspace_bytes(int64_t m, int64_t n, int64_t k_dim);

int sru_b200_gemm_f32(
    float *c, const float *a, const float *b, const float *col_bias,
    int64_t m, int64_t n, int64_t k_dim,
    int64_t lda, int64_t ldb, int64_t ldc,
    int trans_a, int trans_b, int accumulate,
    void *workspace, size_t workspace_bytes, void *stream);

/*
 * Layer normalisation over the last dimension: the nn.LayerNorm an SRU layer applies to its input
 * (sru/modules.py:252-253) or to its output (:278-279; constructed at :155-160 with the default
 * eps 1e-5 and an affine weight and bias).  In the reference this is a library operator (ATen's
 * layer_norm); its published definition is
 *
 *   y[r, :] = (x[r, :] - mean_r) * rstd_r * gamma + beta,     rstd_r = 1 / sqrt(var_r + eps),
 *
 * mean_r and the biased variance var_r taken over the n elements of row r.
 *
 *   x (rows, n)   SRU_F32, SRU_F16 or SRU_BF16, rows contiguous
 *   y (rows, n)   x's type; or SRU_F16 / SRU_BF16 with fp32 x, which writes the normalised rows
 *                 directly in the type the projection GEMM consumes (one rounding, as casting an
 *                 fp32 result would)
 *   gamma, beta   float[n], either may be NULL (ones / zeros)
 *   mean, rstd    float[rows], out; needed by the backward pass, either may be NULL
 *   n             a multiple of 8 (16-bit x) or 4 (fp32 x), at most 4096: other row lengths get
 *                 SRU_ERR_UNSUPPORTED
 */
int sru_b200_layer_norm_forward(
    void *y, float *mean, float *rstd, const void *x, const float *gamma, const float *beta,
    int64_t rows, int64_t n, double eps, int x_dtype, int y_dtype, void *stream);

/* Scratch of the backward pass: per-CTA column sums, at most 4 * (number of SMs) * 2 * n floats. */
size_t sru_b200_layer_norm_backward_workspace_bytes(int64_t rows, int64_t n);

/*
 * Backward of the above (what autograd derives for nn.LayerNorm in the reference):
 *   dx = (dy*gamma - mean_n(dy*gamma) - xhat * mean_n(dy*gamma*xhat)) * rstd,  xhat = (x - mean) * rstd
 *   dgamma = sum over rows of dy * xhat,   dbeta = sum over rows of dy
 * dy has y's type, dx has x's type; dgamma / dbeta are float[n] and either may be NULL.  The column
 * sums are formed in a fixed order (no atomics): repeated calls give identical bits.
 */
int sru_b200_layer_norm_backward(
    void *dx, float *dgamma, float *dbeta, const void *dy, const void *x,
    const float *mean, const float *rstd, const float *gamma,
    int64_t rows, int64_t n, int x_dtype, int y_dtype,
    void *workspace, size_t workspace_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SRU_B200_H_ */
