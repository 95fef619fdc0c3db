// Generic scan kernels: one thread per (batch, direction, hidden) column, direct global
// accesses, every option of the operator (k = 3/4, all skip types, tanh, custom per-step
// V, any hidden size, any alignment, fp64).  They serve the shapes the pipelined kernels
// do not take (odd hidden sizes, custom V, tanh) and are the simplest statement of the
// arithmetic on the device.  64-bit indexing throughout.
//
// Arithmetic follows the reference kernels sru/csrc/sru_cuda_kernel.cu:378-445 (forward),
// :447-578 (backward) and their bidirectional forms :580-665, :667-822; the direction is a
// property of the column (dir = (col % D) / d) instead of a second set of kernels.
#include "scan.cuh"

namespace srub {

template <typename CT> __device__ __forceinline__ CT sigmoid_exact(CT z);
template <> __device__ __forceinline__ float sigmoid_exact<float>(float z) {
    return 1.f / (1.f + expf(-z));
}
template <> __device__ __forceinline__ double sigmoid_exact<double>(double z) {
    return 1.0 / (1.0 + exp(-z));
}
// g = sigmoid(z) together with 1 - g, each with full relative accuracy.  (1 - g) taken from the rounded g
// loses every digit g shares with 1: a gate of 0.9993 leaves the difference with a relative error of
// 1e-4 in fp32, and the backward pass multiplies gradients by it.  With a = exp(-|z|), r = 1/(1+a):
// the larger of the two is r and the smaller a*r, exactly complementary.
template <typename CT> __device__ __forceinline__ CT exp_neg_abs(CT z);
template <> __device__ __forceinline__ float exp_neg_abs<float>(float z) { return expf(-fabsf(z)); }
template <> __device__ __forceinline__ double exp_neg_abs<double>(double z) { return exp(-fabs(z)); }
template <typename CT> __device__ __forceinline__ CT sigmoid_pair(CT z, CT *one_minus) {
    const CT a = exp_neg_abs<CT>(z);
    const CT r = (CT)1 / ((CT)1 + a), q = a * r;
    *one_minus = (z >= (CT)0) ? q : r;
    return (z >= (CT)0) ? r : q;
}
template <typename CT> __device__ __forceinline__ CT tanh_exact(CT z);
template <> __device__ __forceinline__ float tanh_exact<float>(float z) { return tanhf(z); }
template <> __device__ __forceinline__ double tanh_exact<double>(double z) { return tanh(z); }

template <typename T, typename TC, typename CT>
__global__ void __launch_bounds__(128) scan_fwd_generic(ScanArgs a) {
    const int64_t D = (int64_t)a.d * a.dirs;
    const int64_t ncols = a.B * D;
    const int64_t col = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= ncols) return;
    const int64_t b = col / D, dj = col % D;
    const int dir = (int)(dj / a.d);
    const int k = a.k;
    const T *u = (const T *)a.u;
    const T *x = (const T *)a.x;
    const T *vcus = (const T *)a.weight_c;       // custom V, storage dtype
    const CT *wc = (const CT *)a.weight_c;       // (2, D), compute dtype
    const CT *bias = (const CT *)a.bias;
    T *h = (T *)a.h;
    TC *ch = (TC *)a.c_hist;
    const CT b1 = bias ? bias[dj] : (CT)0, b2 = bias ? bias[D + dj] : (CT)0;
    const CT m = a.mask_c ? ((const CT *)a.mask_c)[col] : (CT)1;
    CT cur = a.c_init ? ((const CT *)a.c_init)[col] : (CT)0;
    CT wc1 = 0, wc2 = 0;
    if (!a.is_custom) { wc1 = wc[dj]; wc2 = wc[D + dj]; }
    const CT scale = (CT)a.scale_x;

    for (int64_t n = 0; n < a.L; ++n) {
        const int64_t t = dir ? (a.L - 1 - n) : n;
        const int64_t row = t * a.B + b;
        const int64_t o = row * D + dj;
        if (!a.mask_pad || !a.mask_pad[row]) {
            const T *up = u + o * k;
            const CT u0 = Cvt<T>::to_f(up[0]), u1 = Cvt<T>::to_f(up[1]), u2 = Cvt<T>::to_f(up[2]);
            if (a.is_custom) { wc1 = Cvt<T>::to_f(vcus[o * 2]); wc2 = Cvt<T>::to_f(vcus[o * 2 + 1]); }
            const CT xv = (a.skip_type == 0) ? (CT)0
                        : (a.skip_type == 1) ? (CT)Cvt<T>::to_f(x[o]) * scale
                                             : (CT)Cvt<T>::to_f(up[3]);
            const CT g1 = sigmoid_exact<CT>(u1 + wc1 * cur + b1);
            const CT g2 = sigmoid_exact<CT>(u2 + wc2 * cur + b2);
            cur = (cur - u0) * g1 + u0;
            const CT act = a.activation_type ? tanh_exact<CT>(cur) : cur;
            const CT hv = a.skip_type ? ((act - xv) * m * g2 + xv) : (act * m * g2);
            h[o] = Cvt<T>::from_f(hv);
        } else {
            h[o] = Cvt<T>::from_f((CT)0);
        }
        if (ch) ch[o] = Cvt<TC>::from_f(cur);
    }
    if (a.c_last) ((CT *)a.c_last)[col] = cur;
}

template <typename T, typename TC, typename CT>
__global__ void __launch_bounds__(128) scan_bwd_generic(ScanArgs a) {
    const int64_t D = (int64_t)a.d * a.dirs;
    const int64_t ncols = a.B * D;
    const int64_t col = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (col >= ncols) return;
    const int64_t b = col / D, dj = col % D;
    const int dir = (int)(dj / a.d);
    const int k = a.k;
    const T *u = (const T *)a.u;
    const T *x = (const T *)a.x;
    const T *vcus = (const T *)a.weight_c;
    const CT *wc = (const CT *)a.weight_c;
    const CT *bias = (const CT *)a.bias;
    const TC *ch = (const TC *)a.c_hist;
    const T *gh_p = (const T *)a.grad_h;
    T *gu = (T *)a.grad_u;
    T *gx = (T *)a.grad_x;
    T *gv = (T *)a.grad_wc;  // custom: per-step gradient of V
    const CT b1 = bias ? bias[dj] : (CT)0, b2 = bias ? bias[D + dj] : (CT)0;
    const CT m = a.mask_c ? ((const CT *)a.mask_c)[col] : (CT)1;
    const CT c0 = a.c_init ? ((const CT *)a.c_init)[col] : (CT)0;
    CT wc1 = 0, wc2 = 0;
    if (!a.is_custom) { wc1 = wc[dj]; wc2 = wc[D + dj]; }
    const CT scale = (CT)a.scale_x;
    CT gwc1 = 0, gwc2 = 0, gb1 = 0, gb2 = 0;
    CT cur = a.grad_last ? ((const CT *)a.grad_last)[col] : (CT)0;

    for (int64_t n = a.L - 1; n >= 0; --n) {
        const int64_t t = dir ? (a.L - 1 - n) : n;
        const int64_t row = t * a.B + b;
        const int64_t o = row * D + dj;
        T *gup = gu + o * k;
        if (!a.mask_pad || !a.mask_pad[row]) {
            const int64_t tp = dir ? (t + 1) : (t - 1);
            const CT cp = (n > 0) ? (CT)Cvt<TC>::to_f(ch[(tp * a.B + b) * D + dj]) : c0;
            const T *up = u + o * k;
            const CT u0 = Cvt<T>::to_f(up[0]), u1 = Cvt<T>::to_f(up[1]), u2 = Cvt<T>::to_f(up[2]);
            if (a.is_custom) { wc1 = Cvt<T>::to_f(vcus[o * 2]); wc2 = Cvt<T>::to_f(vcus[o * 2 + 1]); }
            const CT xv = (a.skip_type == 0) ? (CT)0
                        : (a.skip_type == 1) ? (CT)Cvt<T>::to_f(x[o]) * scale
                                             : (CT)Cvt<T>::to_f(up[3]);
            const CT gh = Cvt<T>::to_f(gh_p[o]);
            CT omg1, omg2;   // 1 - g1, 1 - g2
            const CT g1 = sigmoid_pair<CT>(u1 + wc1 * cp + b1, &omg1);
            const CT g2 = sigmoid_pair<CT>(u2 + wc2 * cp + b2, &omg2);
            const CT cv = Cvt<TC>::to_f(ch[o]);
            const CT act = a.activation_type ? tanh_exact<CT>(cv) : cv;
            const CT dact = a.activation_type ? ((CT)1 - act * act) : (CT)1;

            const CT gg2 = gh * (act - xv) * m * (g2 * omg2);
            const CT gc = gh * m * (g2 * dact) + cur;
            const CT gg1 = gc * (cp - u0) * (g1 * omg1);
            gb1 += gg1; gb2 += gg2;
            gwc1 += gg1 * cp; gwc2 += gg2 * cp;
            if (a.is_custom) {
                gv[o * 2] = Cvt<T>::from_f(gg1 * cp);
                gv[o * 2 + 1] = Cvt<T>::from_f(gg2 * cp);
            }
            cur = gc * g1 + gg1 * wc1 + gg2 * wc2;
            gup[0] = Cvt<T>::from_f(gc * omg1);
            gup[1] = Cvt<T>::from_f(gg1);
            gup[2] = Cvt<T>::from_f(gg2);
            const CT gxv = gh * ((CT)1 - g2 * m);
            if (k == 4) gup[3] = Cvt<T>::from_f(a.skip_type == 2 ? gxv : (CT)0);
            if (a.skip_type == 1) gx[o] = Cvt<T>::from_f(gxv * scale);
        } else {
            for (int g = 0; g < k; ++g) gup[g] = Cvt<T>::from_f((CT)0);
            if (a.skip_type == 1) gx[o] = Cvt<T>::from_f((CT)0);
            if (a.is_custom) { gv[o * 2] = Cvt<T>::from_f((CT)0); gv[o * 2 + 1] = Cvt<T>::from_f((CT)0); }
        }
    }
    // per-column partials, layout [row tile = b][4][D]; reduced by reduce_partials
    CT *part = (CT *)a.workspace + (b * 4) * D + dj;
    part[0] = gwc1; part[D] = gwc2; part[2 * D] = gb1; part[3 * D] = gb2;
    ((CT *)a.grad_init)[col] = cur;
}

// out[g][dj] = sum over row tiles r of part[r][g][dj].  A CTA of 256 threads owns 32 columns: thread (slice, column)
// adds every 8th tile with four independent accumulators (a serial sum waits for each load in turn), then the
// eight slices are combined in a fixed order: deterministic for a given tile count.
template <typename CT>
__global__ void __launch_bounds__(256)
reduce_partials(const CT *__restrict__ part, CT *__restrict__ grad_wc,
                CT *__restrict__ grad_bias, int64_t ntiles, int64_t D, int write_wc) {
    __shared__ CT sm[8][32];
    const int cx = threadIdx.x & 31, slice = threadIdx.x >> 5;
    const int64_t i = (int64_t)blockIdx.x * 32 + cx;  // over 4*D
    const int64_t w = 4 * D;
    CT a0 = 0, a1 = 0, a2 = 0, a3 = 0;
    if (i < w) {
        int64_t r = slice;
        for (; r + 24 < ntiles; r += 32) {
            a0 += part[r * w + i];
            a1 += part[(r + 8) * w + i];
            a2 += part[(r + 16) * w + i];
            a3 += part[(r + 24) * w + i];
        }
        for (; r < ntiles; r += 8) a0 += part[r * w + i];
    }
    sm[slice][cx] = (a0 + a1) + (a2 + a3);
    __syncthreads();
    if (slice == 0 && i < w) {
        CT s = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) s += sm[k][cx];
        if (i < 2 * D) {
            if (write_wc) grad_wc[i] = s;
        } else {
            grad_bias[i - 2 * D] = s;
        }
    }
}

template <typename CT>
int launch_reduce_partials(const void *part, void *grad_wc, void *grad_bias, int64_t ntiles,
                           int64_t D, int write_wc, cudaStream_t st) {
    const int64_t blocks = (4 * D + 31) / 32;
    reduce_partials<CT><<<(unsigned)blocks, 256, 0, st>>>((const CT *)part, (CT *)grad_wc,
                                                         (CT *)grad_bias, ntiles, D, write_wc);
    SRUB_CUDA_CHECK(cudaGetLastError());
    return 0;
}
template int launch_reduce_partials<float>(const void *, void *, void *, int64_t, int64_t, int, cudaStream_t);
template int launch_reduce_partials<double>(const void *, void *, void *, int64_t, int64_t, int, cudaStream_t);

template <typename T, typename TC, typename CT>
static int launch_generic_t(const ScanArgs &a, bool backward, cudaStream_t st) {
    const int64_t ncols = a.B * a.d * a.dirs;
    const int threads = 128;
    const int64_t blocks = (ncols + threads - 1) / threads;
    if (blocks > 0x7fffffff) return set_error(SRU_ERR_BAD_ARG, "too many columns");
    if (!backward) {
        scan_fwd_generic<T, TC, CT><<<(unsigned)blocks, threads, 0, st>>>(a);
    } else {
        scan_bwd_generic<T, TC, CT><<<(unsigned)blocks, threads, 0, st>>>(a);
    }
    SRUB_CUDA_CHECK(cudaGetLastError());
    if (backward)
        return launch_reduce_partials<CT>(a.workspace, a.grad_wc, a.grad_bias, a.B,
                                          (int64_t)a.d * a.dirs, a.is_custom ? 0 : 1, st);
    return 0;
}

int launch_scan_generic(const ScanArgs &a, bool backward, cudaStream_t st) {
    const int dt = a.dtype, ct = a.c_dtype;
    if (dt == SRU_F64 && ct == SRU_F64) return launch_generic_t<double, double, double>(a, backward, st);
    if (dt == SRU_F32 && ct == SRU_F32) return launch_generic_t<float, float, float>(a, backward, st);
    if (dt == SRU_F16 && ct == SRU_F16) return launch_generic_t<__half, __half, float>(a, backward, st);
    if (dt == SRU_F16 && ct == SRU_F32) return launch_generic_t<__half, float, float>(a, backward, st);
    if (dt == SRU_BF16 && ct == SRU_BF16) return launch_generic_t<__nv_bfloat16, __nv_bfloat16, float>(a, backward, st);
    if (dt == SRU_BF16 && ct == SRU_F32) return launch_generic_t<__nv_bfloat16, float, float>(a, backward, st);
    return set_error(SRU_ERR_UNSUPPORTED, "dtype %d with c_dtype %d", dt, ct);
}

}  // namespace srub
