// extern "C" entry points of libsru_b200.so (declared in include/sru_b200.h): argument
// validation, dispatch between the pipelined and the generic scan kernels, error plumbing.
#include <atomic>
#include <cctype>
#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "scan.cuh"

namespace srub {

static thread_local char tl_error[512] = "";

int set_error(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
    va_end(ap);
    return code;
}

// ---- options: environment defaults read once, then changed only through sru_b200_set_option ----
static const char *const kOptionNames[OPT_COUNT] = {
    "fwd_v", "bwd_v", "scan_threads", "fwd_threads", "bwd_threads", "scan_ss", "scan_stages",
    "force_generic", "fwd_split", "gemm_ksplit", "gemm_2sm", "gemm_epi_warps", "gemm_dynamic", "gemm_raster", "gemm_tma_store"};
static std::atomic<int> g_options[OPT_COUNT];
static std::once_flag g_options_once;

static void load_option_defaults() {
    for (int i = 0; i < OPT_COUNT; ++i) {
        std::string env = "SRU_B200_";
        for (const char *c = kOptionNames[i]; *c; ++c) env.push_back((char)toupper((unsigned char)*c));
        const char *e = getenv(env.c_str());
        g_options[i].store((e && *e) ? atoi(e) : -1);
    }
}

int option(Option o, int dflt) {
    std::call_once(g_options_once, load_option_defaults);
    const int v = g_options[o].load(std::memory_order_relaxed);
    return v < 0 ? dflt : v;
}

static int find_option(const char *name) {
    if (!name) return -1;
    for (int i = 0; i < OPT_COUNT; ++i)
        if (strcmp(name, kOptionNames[i]) == 0) return i;
    return -1;
}

static thread_local int tl_scan_kernel = SCAN_KERNEL_NONE;
void note_scan_kernel(int which) { tl_scan_kernel = which; }

__device__ int g_device_error = 0;

int *device_error_flag() {
    // one address per device; looked up on first use with that device current
    static int *cache[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!cache[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_error) != cudaSuccess) return nullptr;
        cache[dev] = static_cast<int *>(p);
    }
    return cache[dev];
}

// Driver entry points (the tensor-map encoder) need the device's primary context current on the calling
// thread.  A thread that has only inherited a device ordinal (an autograd worker, for instance) gets it
// bound by a no-op runtime call; a thread that already has a context makes no runtime call at all, so that
// the launchers stay legal inside a stream capture.
int ensure_context() {
    typedef CUresult (*GetCurrent)(CUcontext *);
    static GetCurrent get_current = nullptr;
    if (!get_current) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            get_current = reinterpret_cast<GetCurrent>(ptr);
    }
    CUcontext ctx = nullptr;
    if (get_current && get_current(&ctx) == CUDA_SUCCESS && ctx != nullptr) return 0;
    SRUB_CUDA_CHECK(cudaFree(nullptr));
    return 0;
}

static int check_common(int64_t L, int64_t B, int64_t d, int dirs, int k, int act, int skip,
                        int dtype, int c_dtype) {
    if (L < 0 || B < 0 || d < 1) return set_error(SRU_ERR_BAD_ARG, "bad sizes L=%lld B=%lld d=%lld",
                                                  (long long)L, (long long)B, (long long)d);
    if (d * dirs > 0x7fffffff / 8) return set_error(SRU_ERR_BAD_ARG, "hidden size too large");
    if (dirs != 1 && dirs != 2) return set_error(SRU_ERR_BAD_ARG, "dirs must be 1 or 2, got %d", dirs);
    if (k != 3 && k != 4) return set_error(SRU_ERR_BAD_ARG, "k must be 3 or 4, got %d", k);
    if (act != 0 && act != 1) return set_error(SRU_ERR_BAD_ARG, "activation_type must be 0 or 1, got %d", act);
    if (skip < 0 || skip > 2) return set_error(SRU_ERR_BAD_ARG, "skip_type must be 0, 1 or 2, got %d", skip);
    if (skip == 1 && k != 3) return set_error(SRU_ERR_BAD_ARG, "skip_type 1 needs k == 3");
    if (skip == 2 && k != 4) return set_error(SRU_ERR_BAD_ARG, "skip_type 2 needs k == 4");
    if (dtype < SRU_F32 || dtype > SRU_F64) return set_error(SRU_ERR_BAD_ARG, "unknown dtype %d", dtype);
    if (c_dtype != dtype && !(c_dtype == SRU_F32 && (dtype == SRU_F16 || dtype == SRU_BF16)))
        return set_error(SRU_ERR_BAD_ARG, "c_dtype %d not allowed with dtype %d", c_dtype, dtype);
    return 0;
}

}  // namespace srub

using namespace srub;

extern "C" {

int sru_b200_version(void) { return 200; }

int sru_b200_set_option(const char *name, int value) {
    const int i = find_option(name);
    if (i < 0) return set_error(SRU_ERR_BAD_ARG, "unknown option '%s'", name ? name : "(null)");
    std::call_once(g_options_once, load_option_defaults);
    g_options[i].store(value < 0 ? -1 : value);
    return 0;
}

int sru_b200_get_option(const char *name) {
    const int i = find_option(name);
    if (i < 0) return set_error(SRU_ERR_BAD_ARG, "unknown option '%s'", name ? name : "(null)");
    return option(static_cast<Option>(i), -1);
}

int sru_b200_last_scan_kernel(void) { return tl_scan_kernel; }

const char *sru_b200_last_error(void) { return tl_error; }

int sru_b200_check_device_error(void *stream) {
    int *flag = device_error_flag();
    if (!flag) return set_error(SRU_ERR_CUDA, "device error flag unavailable");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int v = 0;
    SRUB_CUDA_CHECK(cudaMemcpyAsync(&v, flag, sizeof(int), cudaMemcpyDeviceToHost, st));
    SRUB_CUDA_CHECK(cudaStreamSynchronize(st));
    if (v != 0) {
        SRUB_CUDA_CHECK(cudaMemsetAsync(flag, 0, sizeof(int), st));
        SRUB_CUDA_CHECK(cudaStreamSynchronize(st));
        return set_error(SRU_ERR_DEVICE, "a kernel gave up a bounded wait (site %d)", v);
    }
    return 0;
}

int sru_b200_scan_forward(void *h, void *c_hist, void *c_last, const void *u, const void *x,
                          const void *weight_c, const void *bias, const void *c_init,
                          const void *mask_c, const uint8_t *mask_pad, int64_t length, int64_t batch,
                          int64_t hidden, int dirs, int k, int activation_type, int skip_type,
                          int is_custom, double scale_x, int dtype, int c_dtype, void *stream) {
    int rc = check_common(length, batch, hidden, dirs, k, activation_type, skip_type, dtype, c_dtype);
    if (rc) return rc;
    if (length == 0 || batch == 0) return 0;
    if (!h || !u || !weight_c) return set_error(SRU_ERR_BAD_ARG, "h, u and weight_c must not be null");
    if (skip_type == 1 && !x) return set_error(SRU_ERR_BAD_ARG, "skip_type 1 needs x");
    ScanArgs a;
    memset(&a, 0, sizeof(a));
    a.h = h; a.c_hist = c_hist; a.c_last = c_last;
    a.u = u; a.x = x; a.weight_c = weight_c; a.bias = bias; a.c_init = c_init;
    a.mask_c = mask_c; a.mask_pad = mask_pad;
    a.L = length; a.B = batch; a.d = (int)hidden; a.dirs = dirs; a.k = k;
    a.activation_type = activation_type; a.skip_type = skip_type; a.is_custom = is_custom ? 1 : 0;
    a.scale_x = scale_x; a.dtype = dtype; a.c_dtype = c_dtype;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    note_scan_kernel(SCAN_KERNEL_NONE);
    rc = launch_scan_pipelined(a, false, st);   // notes which of its kernel families took the call
    if (rc != 0) return rc < 0 ? rc : 0;
    note_scan_kernel(SCAN_KERNEL_GENERIC);
    return launch_scan_generic(a, false, st);
}

size_t sru_b200_scan_backward_workspace_bytes(int64_t length, int64_t batch, int64_t hidden, int dirs,
                                              int k, int dtype) {
    (void)length; (void)k;
    if (batch < 0 || hidden < 0 || dirs < 1) return 0;
    const size_t per = (dtype == SRU_F64) ? sizeof(double) : sizeof(float);
    return (size_t)batch * 4 * (size_t)hidden * dirs * per;
}

int sru_b200_scan_backward(void *grad_u, void *grad_x, void *grad_wc, void *grad_bias, void *grad_init,
                           const void *u, const void *x, const void *weight_c, const void *bias,
                           const void *c_init, const void *mask_c, const uint8_t *mask_pad,
                           const void *c_hist, const void *grad_h, const void *grad_last,
                           int64_t length, int64_t batch, int64_t hidden, int dirs, int k,
                           int activation_type, int skip_type, int is_custom, double scale_x, int dtype,
                           int c_dtype, void *workspace, size_t workspace_bytes, void *stream) {
    int rc = check_common(length, batch, hidden, dirs, k, activation_type, skip_type, dtype, c_dtype);
    if (rc) return rc;
    if (length == 0 || batch == 0) return 0;
    if (!grad_u || !grad_wc || !grad_bias || !grad_init || !u || !weight_c || !c_hist || !grad_h)
        return set_error(SRU_ERR_BAD_ARG, "a required pointer is null");
    if (skip_type == 1 && (!x || !grad_x)) return set_error(SRU_ERR_BAD_ARG, "skip_type 1 needs x and grad_x");
    const size_t need = sru_b200_scan_backward_workspace_bytes(length, batch, hidden, dirs, k, dtype);
    if (!workspace || workspace_bytes < need)
        return set_error(SRU_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    ScanArgs a;
    memset(&a, 0, sizeof(a));
    a.grad_u = grad_u; a.grad_x = grad_x; a.grad_wc = grad_wc; a.grad_bias = grad_bias; a.grad_init = grad_init;
    a.u = u; a.x = x; a.weight_c = weight_c; a.bias = bias; a.c_init = c_init;
    a.mask_c = mask_c; a.mask_pad = mask_pad; a.c_hist = const_cast<void *>(c_hist);
    a.grad_h = grad_h; a.grad_last = grad_last; a.workspace = workspace;
    a.L = length; a.B = batch; a.d = (int)hidden; a.dirs = dirs; a.k = k;
    a.activation_type = activation_type; a.skip_type = skip_type; a.is_custom = is_custom ? 1 : 0;
    a.scale_x = scale_x; a.dtype = dtype; a.c_dtype = c_dtype;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    note_scan_kernel(SCAN_KERNEL_NONE);
    rc = launch_scan_pipelined(a, true, st);
    if (rc != 0) return rc < 0 ? rc : 0;
    note_scan_kernel(SCAN_KERNEL_GENERIC);
    return launch_scan_generic(a, true, st);
}

}  // extern "C"
