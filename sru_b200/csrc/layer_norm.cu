// Layer normalisation over the last dimension, forward and backward: the nn.LayerNorm that the SRU layer
// applies to its input (pre-norm) or to its output (post-norm), sru/modules.py:252-253 and :278-279.
//
//   y = (x - mean) * rstd * gamma + beta,   mean / biased variance over the n elements of a row,
//   rstd = 1 / sqrt(var + eps)
//   dx = (dy*gamma - mean_n(dy*gamma) - xhat * mean_n(dy*gamma*xhat)) * rstd,   xhat = (x - mean) * rstd
//   dgamma = sum_rows dy * xhat,   dbeta = sum_rows dy
//
// Both kernels are bound by HBM traffic: forward reads x and writes y once (the output may be written
// directly in the 16-bit type the following GEMM consumes), backward reads dy and x and writes dx once.
// A row is held in registers by 1, 2 or 4 warps (up to 32 elements per thread, 16-byte accesses); the
// column sums of the backward are kept per thread across all rows a CTA visits, combined per CTA in a
// fixed order and finished by a second small kernel: no atomics, results do not depend on scheduling.
#include <algorithm>
#include <type_traits>

#include "common.cuh"

namespace srub {
namespace {

constexpr int kLnThreads = 128;   // 4 warps per CTA
constexpr int kLnElems = 32;      // elements of a row per thread, at most

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum of `v` over the WPR warps that share a row (fixed order).  Every thread of the CTA calls this the
// same number of times; `red` is float[2][4][2] in shared memory and `parity` alternates between calls.
template <int WPR>
__device__ __forceinline__ void row_sum2(float &a, float &b, float (*red)[4][2], int &parity, int warp, int lane) {
    a = warp_sum(a);
    b = warp_sum(b);
    if (WPR > 1) {
        if (lane == 0) { red[parity][warp][0] = a; red[parity][warp][1] = b; }
        __syncthreads();
        const int w0 = (warp / WPR) * WPR;
        a = 0.f; b = 0.f;
#pragma unroll
        for (int w = 0; w < WPR; ++w) { a += red[parity][w0 + w][0]; b += red[parity][w0 + w][1]; }
        parity ^= 1;
    }
}

// VE consecutive elements of T as they come from memory: 32-bit words, unpacked to float on use (explicit
// bit operations, so that the register cost of a packed row is exactly its size).
template <typename T, int VE> struct Words {
    static constexpr int NW = VE * (int)sizeof(T) / 4;
    uint32_t w[NW];
    __device__ __forceinline__ void load(const T *p) {
        if constexpr (NW == 4) {
            const uint4 v = *reinterpret_cast<const uint4 *>(p);
            w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
        } else {
            static_assert(NW == 2, "8 or 16 bytes per vector");
            const uint2 v = *reinterpret_cast<const uint2 *>(p);
            w[0] = v.x; w[1] = v.y;
        }
    }
    __device__ __forceinline__ void unpack(float (&out)[VE]) const {
        if constexpr (sizeof(T) == 4) {
#pragma unroll
            for (int j = 0; j < VE; ++j) out[j] = __uint_as_float(w[j]);
        } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
#pragma unroll
            for (int k = 0; k < NW; ++k) {
                out[2 * k] = __uint_as_float(w[k] << 16);
                out[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
            }
        } else {
#pragma unroll
            for (int k = 0; k < NW; ++k) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[k]));
                out[2 * k] = f.x;
                out[2 * k + 1] = f.y;
            }
        }
    }
};

template <typename T, int VE> struct RowVec {
    // loads / stores VE consecutive elements (16 bytes of the narrower of the two types involved)
    static __device__ __forceinline__ void load(float (&out)[VE], const T *p) {
        const Pack<T, VE> v = *reinterpret_cast<const Pack<T, VE> *>(p);
#pragma unroll
        for (int j = 0; j < VE; ++j) out[j] = Cvt<T>::to_f(v.v[j]);
    }
    static __device__ __forceinline__ void store(T *p, const float (&in)[VE]) {
        Pack<T, VE> v;
#pragma unroll
        for (int j = 0; j < VE; ++j) v.v[j] = Cvt<T>::from_f(in[j]);
        *reinterpret_cast<Pack<T, VE> *>(p) = v;
    }
};

// TI: type of x (and dx); TO: type of y (and dy); WPR: warps per row
template <typename TI, typename TO, int WPR>
__global__ void __launch_bounds__(kLnThreads, 3)
ln_fwd_kernel(TO *__restrict__ y, float *__restrict__ mean_out, float *__restrict__ rstd_out,
              const TI *__restrict__ x, const float *__restrict__ gamma, const float *__restrict__ beta,
              int64_t rows, int n, float eps) {
    constexpr int VE = 16 / sizeof(TI), NV = kLnElems / VE, RPC = 4 / WPR;
    __shared__ float red[2][4][2];
    extern __shared__ __align__(16) float dyn[];   // gamma[n], beta[n]
    float *gsm = dyn, *bsm = dyn + n;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = warp / WPR, wir = warp % WPR;
    const int nvec = n / VE;
    const float inv_n = 1.f / (float)n;
    int parity = 0;

    for (int c = threadIdx.x; c < n; c += kLnThreads) {
        gsm[c] = gamma ? gamma[c] : 1.f;
        bsm[c] = beta ? beta[c] : 0.f;
    }
    __syncthreads();

    struct Raw { Words<TI, VE> x[NV]; bool valid; };
    // rows are fetched one iteration ahead (two register buffers used in turn)
    auto load = [&](Raw &r, int64_t base) {
        const int64_t row = base + group;
        r.valid = row < rows;
        if (r.valid) {
            const TI *xr = x + row * n;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int v = wir * 32 + lane + i * 32 * WPR;
                if (v < nvec) r.x[i].load(xr + v * VE);
            }
        }
    };
    auto process = [&](const Raw &r, int64_t base) {
        const int64_t row = base + group;
        float val[NV][VE];
        float s = 0.f, unused = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int v = wir * 32 + lane + i * 32 * WPR;
            if (r.valid && v < nvec) {
                r.x[i].unpack(val[i]);
            } else {
#pragma unroll
                for (int j = 0; j < VE; ++j) val[i][j] = 0.f;
            }
#pragma unroll
            for (int j = 0; j < VE; ++j) s += val[i][j];
        }
        row_sum2<WPR>(s, unused, red, parity, warp, lane);
        const float mean = s * inv_n;
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int v = wir * 32 + lane + i * 32 * WPR;
            if (v < nvec) {
#pragma unroll
                for (int j = 0; j < VE; ++j) { const float d = val[i][j] - mean; q = fmaf(d, d, q); }
            }
        }
        row_sum2<WPR>(q, unused, red, parity, warp, lane);
        const float rstd = 1.f / sqrtf(q * inv_n + eps);
        const float nmr = -mean * rstd;
        TO *yr = y + row * n;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int v = wir * 32 + lane + i * 32 * WPR;
            if (r.valid && v < nvec) {
                float gv[VE], bv[VE], o[VE];
#pragma unroll
                for (int j = 0; j < VE; j += 4) {
                    *reinterpret_cast<float4 *>(&gv[j]) = *reinterpret_cast<const float4 *>(gsm + v * VE + j);
                    *reinterpret_cast<float4 *>(&bv[j]) = *reinterpret_cast<const float4 *>(bsm + v * VE + j);
                }
#pragma unroll
                for (int j = 0; j < VE; ++j) o[j] = fmaf(fmaf(val[i][j], rstd, nmr), gv[j], bv[j]);
                RowVec<TO, VE>::store(yr + v * VE, o);
            }
        }
        if (r.valid && wir == 0 && lane == 0) {
            if (mean_out) mean_out[row] = mean;
            if (rstd_out) rstd_out[row] = rstd;
        }
    };

    const int64_t stride = (int64_t)gridDim.x * RPC;
    int64_t base = (int64_t)blockIdx.x * RPC;
    if constexpr (sizeof(TI) == 2) {
        // 16-bit rows are half the bytes: two rows ahead (three buffers in turn) to keep as much in flight
        Raw A, B, C;
        if (base < rows) load(A, base);
        if (base + stride < rows) load(B, base + stride);
        while (base < rows) {
            if (base + 2 * stride < rows) load(C, base + 2 * stride);
            process(A, base);
            base += stride;
            if (base >= rows) break;
            if (base + 2 * stride < rows) load(A, base + 2 * stride);
            process(B, base);
            base += stride;
            if (base >= rows) break;
            if (base + 2 * stride < rows) load(B, base + 2 * stride);
            process(C, base);
            base += stride;
        }
    } else {
        Raw A, B;
        if (base < rows) load(A, base);
        while (base < rows) {
            if (base + stride < rows) load(B, base + stride);
            process(A, base);
            base += stride;
            if (base >= rows) break;
            if (base + stride < rows) load(A, base + stride);
            process(B, base);
            base += stride;
        }
    }
}

// One row's share of a thread as it comes from memory (packed), plus the row's statistics.
template <typename TI, typename TO, int VE, int NV> struct LnRawRow {
    Words<TI, VE> x[NV];
    Words<TO, VE> d[NV];
    float mu, rs;
    bool valid;
};

template <typename TI, typename TO, int WPR>
__global__ void __launch_bounds__(kLnThreads, sizeof(TI) == 2 ? 3 : 2)
ln_bwd_kernel(TI *__restrict__ dx, float *__restrict__ part, const TO *__restrict__ dy,
              const TI *__restrict__ x, const float *__restrict__ mean, const float *__restrict__ rstd,
              const float *__restrict__ gamma, int64_t rows, int n) {
    constexpr int VE = 16 / sizeof(TI), NV = kLnElems / VE, RPC = 4 / WPR;
    using Raw = LnRawRow<TI, TO, VE, NV>;
    __shared__ float red[2][4][2];
    extern __shared__ __align__(16) float dyn[];   // gamma[n], then the CTA's column sums [2][n]
    float *gsm = dyn, *colsum = dyn + n;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = warp / WPR, wir = warp % WPR;
    const int nvec = n / VE;
    const float inv_n = 1.f / (float)n;
    int parity = 0;

    for (int c = threadIdx.x; c < n; c += kLnThreads) gsm[c] = gamma ? gamma[c] : 1.f;
    __syncthreads();

    float dg[NV][VE], db[NV][VE];
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int j = 0; j < VE; ++j) { dg[i][j] = 0.f; db[i][j] = 0.f; }

    // Rows are fetched one iteration ahead (two register buffers used in turn), so that the loads of the
    // next row are in flight while this one is reduced and written.
    auto load = [&](Raw &r, int64_t base) {
        const int64_t row = base + group;
        r.valid = row < rows;
        r.mu = 0.f; r.rs = 0.f;
        if (r.valid) {
            r.mu = mean[row]; r.rs = rstd[row];
            const TI *xr = x + row * n;
            const TO *dyr = dy + row * n;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int v = wir * 32 + lane + i * 32 * WPR;
                if (v < nvec) {
                    r.x[i].load(xr + v * VE);
                    r.d[i].load(dyr + v * VE);
                }
            }
        }
    };
    auto process = [&](const Raw &r, int64_t base) {
        const int64_t row = base + group;
        const float nmr = -r.mu * r.rs;       // xhat = x * rs + nmr
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int v = wir * 32 + lane + i * 32 * WPR;
            if (r.valid && v < nvec) {
                float gv[VE], xv[VE], dvv[VE];
#pragma unroll
                for (int j = 0; j < VE; j += 4)
                    *reinterpret_cast<float4 *>(&gv[j]) = *reinterpret_cast<const float4 *>(gsm + v * VE + j);
                r.x[i].unpack(xv);
                r.d[i].unpack(dvv);
#pragma unroll
                for (int j = 0; j < VE; ++j) {
                    const float xh = fmaf(xv[j], r.rs, nmr);
                    const float dv = dvv[j];
                    const float t = dv * gv[j];
                    s1 += t;
                    s2 = fmaf(t, xh, s2);
                    dg[i][j] = fmaf(dv, xh, dg[i][j]);
                    db[i][j] += dv;
                }
            }
        }
        row_sum2<WPR>(s1, s2, red, parity, warp, lane);
        // dx = rs*(dy*g - c1 - xhat*c2) = rs*(dy*g) + kx*x + k0
        const float c1 = s1 * inv_n, c2 = s2 * inv_n;
        const float kx = -r.rs * r.rs * c2;
        const float k0 = -r.rs * (c1 + nmr * c2);
        TI *dxr = dx + row * n;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int v = wir * 32 + lane + i * 32 * WPR;
            if (r.valid && v < nvec) {
                float gv[VE], o[VE], xv[VE], dvv[VE];
#pragma unroll
                for (int j = 0; j < VE; j += 4)
                    *reinterpret_cast<float4 *>(&gv[j]) = *reinterpret_cast<const float4 *>(gsm + v * VE + j);
                r.x[i].unpack(xv);
                r.d[i].unpack(dvv);
#pragma unroll
                for (int j = 0; j < VE; ++j) o[j] = fmaf(dvv[j] * gv[j], r.rs, fmaf(kx, xv[j], k0));
                RowVec<TI, VE>::store(dxr + v * VE, o);
            }
        }
    };

    const int64_t stride = (int64_t)gridDim.x * RPC;
    int64_t base = (int64_t)blockIdx.x * RPC;
    Raw A, B;
    if (base < rows) load(A, base);
    while (base < rows) {
        if (base + stride < rows) load(B, base + stride);
        process(A, base);
        base += stride;
        if (base >= rows) break;
        if (base + stride < rows) load(A, base + stride);
        process(B, base);
        base += stride;
    }

    // column sums of this CTA: the row groups add theirs one after the other (fixed order)
#pragma unroll 1
    for (int gsel = 0; gsel < RPC; ++gsel) {
        if (group == gsel) {
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const int v = wir * 32 + lane + i * 32 * WPR;
                if (v < nvec) {
#pragma unroll
                    for (int j = 0; j < VE; ++j) {
                        const int c = v * VE + j;
                        if (gsel == 0) { colsum[c] = dg[i][j]; colsum[n + c] = db[i][j]; }
                        else { colsum[c] += dg[i][j]; colsum[n + c] += db[i][j]; }
                    }
                }
            }
        }
        __syncthreads();
    }
    float *out = part + (size_t)blockIdx.x * 2 * n;
    for (int c = threadIdx.x; c < 2 * n; c += kLnThreads) out[c] = colsum[c];
}

// dgamma[c] / dbeta[c] = sum over the CTAs' column sums.  A CTA of 256 threads owns 32 columns: thread (slice, column)
// adds every 8th partial with four independent accumulators (the loads of a serial sum would each wait for the one
// before: 444 partials took 35 us that way), then the eight slices are combined in a fixed order.
__global__ void __launch_bounds__(256)
ln_reduce_kernel(const float *__restrict__ part, int nparts, int n,
                 float *__restrict__ dgamma, float *__restrict__ dbeta) {
    __shared__ float sm[8][32];
    const int cx = threadIdx.x & 31, slice = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + cx;
    const size_t w = (size_t)2 * n;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    if (c < 2 * n) {
        int p = slice;
        for (; p + 24 < nparts; p += 32) {
            a0 += part[(size_t)p * w + c];
            a1 += part[(size_t)(p + 8) * w + c];
            a2 += part[(size_t)(p + 16) * w + c];
            a3 += part[(size_t)(p + 24) * w + c];
        }
        for (; p < nparts; p += 8) a0 += part[(size_t)p * w + c];
    }
    sm[slice][cx] = (a0 + a1) + (a2 + a3);
    __syncthreads();
    if (slice == 0 && c < 2 * n) {
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) s += sm[k][cx];
        if (c < n) { if (dgamma) dgamma[c] = s; }
        else if (dbeta) dbeta[c - n] = s;
    }
}

int sm_count() {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
        return n;
    return 148;
}

// warps per row for a row of n elements of a type with VE elements per 16 bytes; 0: not supported
int warps_per_row(int64_t n, int ve) {
    if (n < 1 || n % ve != 0) return 0;
    for (int wpr = 1; wpr <= 4; wpr *= 2)
        if ((int64_t)wpr * 32 * kLnElems >= n) return wpr;
    return 0;
}

constexpr int kLnMaxBwdCtasPerSm = 4;   // the backward holds ~190 registers per thread: never more than this resident

template <typename K> int bwd_blocks(K kernel, int64_t rows, int n, int wpr) {
    const int rpc = 4 / wpr;
    const int64_t want = (rows + rpc - 1) / rpc;
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, kLnThreads, (size_t)3 * n * sizeof(float)) != cudaSuccess || occ < 1)
        occ = 1;
    occ = std::min(occ, kLnMaxBwdCtasPerSm);
    return (int)std::min<int64_t>(want, (int64_t)sm_count() * occ);   // one resident wave: every CTA keeps column sums
}

template <typename TI, typename TO, int WPR>
int ln_forward_w(void *y, float *mean, float *rstd, const void *x, const float *gamma, const float *beta,
                 int64_t rows, int n, float eps, cudaStream_t st) {
    auto kernel = ln_fwd_kernel<TI, TO, WPR>;
    const size_t smem = (size_t)2 * n * sizeof(float);
    constexpr int rpc = 4 / WPR;
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, kLnThreads, smem) != cudaSuccess || occ < 1) occ = 1;
    // one resident wave that walks the rows: gamma and beta are staged in shared memory once per CTA
    const int blocks = (int)std::min<int64_t>((rows + rpc - 1) / rpc, (int64_t)sm_count() * occ);
    kernel<<<blocks, kLnThreads, smem, st>>>((TO *)y, mean, rstd, (const TI *)x, gamma, beta, rows, n, eps);
    SRUB_CUDA_CHECK(cudaGetLastError());
    return 0;
}

template <typename TI, typename TO>
int ln_forward_t(void *y, float *mean, float *rstd, const void *x, const float *gamma, const float *beta,
                 int64_t rows, int n, float eps, int wpr, cudaStream_t st) {
    switch (wpr) {
        case 1: return ln_forward_w<TI, TO, 1>(y, mean, rstd, x, gamma, beta, rows, n, eps, st);
        case 2: return ln_forward_w<TI, TO, 2>(y, mean, rstd, x, gamma, beta, rows, n, eps, st);
        default: return ln_forward_w<TI, TO, 4>(y, mean, rstd, x, gamma, beta, rows, n, eps, st);
    }
}

template <typename TI, typename TO, int WPR>
int ln_backward_w(void *dx, void *workspace, size_t workspace_bytes, const void *dy, const void *x, const float *mean,
                  const float *rstd, const float *gamma, int64_t rows, int n, int *nparts, cudaStream_t st) {
    auto kernel = ln_bwd_kernel<TI, TO, WPR>;
    const size_t smem = (size_t)3 * n * sizeof(float);
    if (smem > 40 * 1024)   // beyond the default limit once the static part is added; cheap, and per device
        SRUB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int blocks = bwd_blocks(kernel, rows, n, WPR);
    const size_t need = (size_t)blocks * 2 * (size_t)n * sizeof(float);
    if (!workspace || workspace_bytes < need)
        return set_error(SRU_ERR_WORKSPACE, "layer-norm backward needs %zu bytes of workspace, got %zu", need, workspace_bytes);
    kernel<<<blocks, kLnThreads, smem, st>>>((TI *)dx, (float *)workspace, (const TO *)dy,
                                                                     (const TI *)x, mean, rstd, gamma, rows, n);
    SRUB_CUDA_CHECK(cudaGetLastError());
    *nparts = blocks;
    return 0;
}

template <typename TI, typename TO>
int ln_backward_t(void *dx, void *workspace, size_t workspace_bytes, const void *dy, const void *x, const float *mean,
                  const float *rstd, const float *gamma, int64_t rows, int n, int wpr, int *nparts, cudaStream_t st) {
    switch (wpr) {
        case 1: return ln_backward_w<TI, TO, 1>(dx, workspace, workspace_bytes, dy, x, mean, rstd, gamma, rows, n, nparts, st);
        case 2: return ln_backward_w<TI, TO, 2>(dx, workspace, workspace_bytes, dy, x, mean, rstd, gamma, rows, n, nparts, st);
        default: return ln_backward_w<TI, TO, 4>(dx, workspace, workspace_bytes, dy, x, mean, rstd, gamma, rows, n, nparts, st);
    }
}

int check_ln(int64_t rows, int64_t n, int x_dtype, int y_dtype, int *wpr) {
    if (rows < 0 || n < 1) return set_error(SRU_ERR_BAD_ARG, "bad sizes rows=%lld n=%lld", (long long)rows, (long long)n);
    const bool x16 = (x_dtype == SRU_F16 || x_dtype == SRU_BF16);
    if (!(x_dtype == SRU_F32 || x16)) return set_error(SRU_ERR_BAD_ARG, "x_dtype must be fp32, fp16 or bf16");
    if (!(y_dtype == x_dtype || (x_dtype == SRU_F32 && (y_dtype == SRU_F16 || y_dtype == SRU_BF16))))
        return set_error(SRU_ERR_UNSUPPORTED, "y_dtype %d with x_dtype %d: y must have x's type, or be 16-bit with fp32 x",
                         y_dtype, x_dtype);
    *wpr = warps_per_row(n, x16 ? 8 : 4);
    if (*wpr == 0)
        return set_error(SRU_ERR_UNSUPPORTED, "row length %lld: must be a multiple of %d and at most %d",
                         (long long)n, x16 ? 8 : 4, 4 * 32 * kLnElems);
    return 0;
}

}  // namespace
}  // namespace srub

using namespace srub;

extern "C" {

int sru_b200_layer_norm_forward(void *y, float *mean, float *rstd, const void *x, const float *gamma,
                                const float *beta, int64_t rows, int64_t n, double eps, int x_dtype,
                                int y_dtype, void *stream) {
    int wpr = 0;
    if (int rc = check_ln(rows, n, x_dtype, y_dtype, &wpr)) return rc;
    if (rows == 0) return 0;
    if (!y || !x) return set_error(SRU_ERR_BAD_ARG, "y and x must not be NULL");
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u)
        return set_error(SRU_ERR_BAD_ARG, "x and y must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const float e = (float)eps;
    const int ni = (int)n;
    if (x_dtype == SRU_F32 && y_dtype == SRU_F32) return ln_forward_t<float, float>(y, mean, rstd, x, gamma, beta, rows, ni, e, wpr, st);
    if (x_dtype == SRU_F32 && y_dtype == SRU_BF16) return ln_forward_t<float, __nv_bfloat16>(y, mean, rstd, x, gamma, beta, rows, ni, e, wpr, st);
    if (x_dtype == SRU_F32 && y_dtype == SRU_F16) return ln_forward_t<float, __half>(y, mean, rstd, x, gamma, beta, rows, ni, e, wpr, st);
    if (x_dtype == SRU_BF16) return ln_forward_t<__nv_bfloat16, __nv_bfloat16>(y, mean, rstd, x, gamma, beta, rows, ni, e, wpr, st);
    return ln_forward_t<__half, __half>(y, mean, rstd, x, gamma, beta, rows, ni, e, wpr, st);
}

size_t sru_b200_layer_norm_backward_workspace_bytes(int64_t rows, int64_t n) {
    if (rows < 1 || n < 1) return 0;
    // one set of column sums (dgamma, dbeta) per CTA of the one resident wave
    const int64_t blocks = std::min<int64_t>(rows, (int64_t)sm_count() * kLnMaxBwdCtasPerSm);
    return (size_t)blocks * 2 * (size_t)n * sizeof(float);
}

int sru_b200_layer_norm_backward(void *dx, float *dgamma, float *dbeta, const void *dy, const void *x,
                                 const float *mean, const float *rstd, const float *gamma, int64_t rows,
                                 int64_t n, int x_dtype, int y_dtype, void *workspace, size_t workspace_bytes,
                                 void *stream) {
    int wpr = 0;
    if (int rc = check_ln(rows, n, x_dtype, y_dtype, &wpr)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows == 0) {
        if (dgamma) SRUB_CUDA_CHECK(cudaMemsetAsync(dgamma, 0, (size_t)n * sizeof(float), st));
        if (dbeta) SRUB_CUDA_CHECK(cudaMemsetAsync(dbeta, 0, (size_t)n * sizeof(float), st));
        return 0;
    }
    if (!dx || !dy || !x || !mean || !rstd) return set_error(SRU_ERR_BAD_ARG, "dx, dy, x, mean and rstd must not be NULL");
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx)) & 15u)
        return set_error(SRU_ERR_BAD_ARG, "x, dy and dx must be 16-byte aligned");
    const int ni = (int)n;
    int rc, nparts = 0;
    if (x_dtype == SRU_F32 && y_dtype == SRU_F32) rc = ln_backward_t<float, float>(dx, workspace, workspace_bytes, dy, x, mean, rstd, gamma, rows, ni, wpr, &nparts, st);
    else if (x_dtype == SRU_F32 && y_dtype == SRU_BF16) rc = ln_backward_t<float, __nv_bfloat16>(dx, workspace, workspace_bytes, dy, x, mean, rstd, gamma, rows, ni, wpr, &nparts, st);
    else if (x_dtype == SRU_F32 && y_dtype == SRU_F16) rc = ln_backward_t<float, __half>(dx, workspace, workspace_bytes, dy, x, mean, rstd, gamma, rows, ni, wpr, &nparts, st);
    else if (x_dtype == SRU_BF16) rc = ln_backward_t<__nv_bfloat16, __nv_bfloat16>(dx, workspace, workspace_bytes, dy, x, mean, rstd, gamma, rows, ni, wpr, &nparts, st);
    else rc = ln_backward_t<__half, __half>(dx, workspace, workspace_bytes, dy, x, mean, rstd, gamma, rows, ni, wpr, &nparts, st);
    if (rc) return rc;
    if (dgamma || dbeta) {
        ln_reduce_kernel<<<(2 * ni + 31) / 32, 256, 0, st>>>(static_cast<const float *>(workspace), nparts, ni, dgamma, dbeta);
        SRUB_CUDA_CHECK(cudaGetLastError());
    }
    return 0;
}

}  // extern "C"
