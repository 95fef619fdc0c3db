// Pipelined scan kernels for sm_100a.
//
// Work decomposition.  A CTA owns a tile of BR batch rows x HW hidden units of ONE
// direction; each consumer thread owns V adjacent hidden units of one row and keeps their
// state (c, or dL/dc and the four parameter-gradient accumulators) in registers for the
// whole sequence.  Time is the only sequential axis.
//
// Memory pipeline.  The per-step inputs of the tile (the gate pre-activations U, the
// highway input x, and for backward c[t-1] and grad_h) are contiguous slabs of HW*k (or
// HW) elements per row.  One extra warp, the producer, streams them kTS time steps at a
// time into a ring of NS shared-memory stages with untiled bulk asynchronous copies
// (cp.async.bulk, completion counted on an mbarrier per stage); consumers wait on the
// stage's "full" barrier, read their 4..48-byte slices with vector shared loads, and
// release the stage through its "empty" barrier.  The depth in time of the ring, not the
// number of resident threads, provides the bytes in flight that HBM needs.  Outputs go
// straight from registers to global memory with V*sizeof(T)-byte stores that are
// contiguous across the warp.
//
// Every wait is bounded (mbar_wait_bounded); on a timeout the thread raises the device
// error flag, stops processing and falls through to the end of the kernel.
//
// Arithmetic (same as the reference kernels sru/csrc/sru_cuda_kernel.cu:60-78 forward,
// :130-176 backward, with the direction taken from the tile instead of col % 2d):
//   g1 = s(u1 + wc1*c' + b1), g2 = s(u2 + wc2*c' + b2), c = (c' - u0)*g1 + u0,
//   h = (c - x')*m*g2 + x',  x' = x*scale_x (k=3) | u3 (k=4) | 0,
// where s(z) = 1/(1 + 2^(-z*log2 e)) is evaluated with ex2.approx / rcp.approx and the
// -log2 e factor is folded into wc and b once per column.
#include "scan.cuh"

namespace srub {

constexpr int kTS = 4;            // time steps per pipeline stage
constexpr int kBarBytes = 256;    // room for 2 * 16 mbarriers at the start of shared memory
constexpr int kMaxStages = 16;

struct PipeArgs {
    ScanArgs a;
    TileCfg c;
    int *err;
};

// Gate evaluation.  ACC (fp32 storage): the reference's own expression 1/(1+expf(-z)) with
// full-precision expf and IEEE division, so fp32 results stay within 1e-5 of an fp32 CPU run
// over long sequences.  !ACC (16-bit storage): -log2(e) folded into wc and b once per column,
// then ex2.approx + rcp.approx (two MUFU operations per gate).
template <bool ACC> struct Gate {
    static __device__ __forceinline__ float fold(float v) { return ACC ? v : v * kNegLog2e; }
    // multiplies (gg1*wc1f + gg2*wc2f) back to (gg1*wc1 + gg2*wc2)
    static constexpr float kUnfold = ACC ? 1.f : -0.6931471805599453f;
    static __device__ __forceinline__ float eval(float c, float wcf, float u, float bf) {
        if (ACC) {
            const float z = fmaf(wcf, c, u) + bf;
            return 1.f / (1.f + expf(-z));
        } else {
            return rcp_approx(1.f + ex2_approx(fmaf(c, wcf, fmaf(u, kNegLog2e, bf))));
        }
    }
};

template <typename T, typename TC, int V, int K>
__global__ void __launch_bounds__(160) scan_fwd_pipe(const PipeArgs p) {
    extern __shared__ __align__(128) uint8_t smem[];
    using G = Gate<sizeof(T) == 4>;
    const ScanArgs &a = p.a;
    const int HW = p.c.hw, BR = p.c.br, TPR = p.c.tpr, NS = p.c.nstages;
    const int tid = threadIdx.x;
    const int nthr_c = blockDim.x - 32;
    const int lane = tid & 31;
    const bool has_x = (K == 3) && (a.skip_type == 1);
    const int64_t D = (int64_t)a.d * a.dirs;
    const int ht = blockIdx.x % p.c.nht, rt = blockIdx.x / p.c.nht;
    const int64_t dj0 = (int64_t)ht * HW;
    const int dir = (int)(dj0 / a.d);
    const int64_t b0 = (int64_t)rt * BR;
    const int nrows = (int)min((int64_t)BR, a.B - b0);
    const int64_t L = a.L;
    const int nst = (int)((L + kTS - 1) / kTS);

    const uint32_t bar_full = smem_u32(smem);
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;
    const uint32_t u_slab = (uint32_t)HW * K * sizeof(T);   // bytes per (step,row)
    const uint32_t x_slab = has_x ? (uint32_t)HW * sizeof(T) : 0;
    const uint32_t u_region = kTS * BR * u_slab;
    const uint32_t stage_bytes = u_region + kTS * BR * x_slab;
    uint8_t *stage0 = smem + kBarBytes;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, nthr_c / 32);
        }
        fence_mbar_init();
    }
    __syncthreads();

    if (tid >= nthr_c) {
        // ------------------------------ producer warp ------------------------------
        const T *u = (const T *)a.u;
        const T *x = (const T *)a.x;
        const int ntens = has_x ? 2 : 1;
        for (int it = 0; it < nst; ++it) {
            const int s = it % NS;
            if (it >= NS) {
                if (!mbar_wait_bounded(bar_empty + 8 * s, ((it / NS) - 1) & 1)) {
                    if (lane == 0) atomicExch(p.err, 1);
                    break;
                }
            }
            const int64_t n0 = (int64_t)it * kTS;
            const int steps = (int)min((int64_t)kTS, L - n0);
            if (lane == 0)
                mbar_arrive_expect_tx(bar_full + 8 * s, (uint32_t)steps * nrows * (u_slab + x_slab));
            __syncwarp();
            const uint32_t sbase = smem_u32(stage0 + (size_t)s * stage_bytes);
            const int ncopies = steps * nrows * ntens;
            for (int idx = lane; idx < ncopies; idx += 32) {
                const int which = idx % ntens;
                const int rr = (idx / ntens) % nrows;
                const int ts = idx / (ntens * nrows);
                const int64_t n = n0 + ts;
                const int64_t t = dir ? (L - 1 - n) : n;
                const int64_t o = ((t * a.B + b0 + rr) * D + dj0);
                if (which == 0)
                    bulk_copy_g2s(sbase + (ts * BR + rr) * u_slab, u + o * K, u_slab, bar_full + 8 * s);
                else
                    bulk_copy_g2s(sbase + u_region + (ts * BR + rr) * x_slab, x + o, x_slab,
                                  bar_full + 8 * s);
            }
        }
        return;
    }

    // -------------------------------- consumers --------------------------------
    const int r = tid / TPR;
    const int hc = (tid - r * TPR) * V;
    const bool active = (tid < BR * TPR) && (r < nrows);
    const int64_t b = b0 + (active ? r : 0);
    const int64_t col = b * D + dj0 + hc;
    const bool has_pad = a.mask_pad != nullptr;

    float c[V], wc1n[V], wc2n[V], b1n[V], b2n[V], mk[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
        c[i] = 0.f; wc1n[i] = 0.f; wc2n[i] = 0.f; b1n[i] = 0.f; b2n[i] = 0.f; mk[i] = 1.f;
    }
    if (active) {
        const float *wc = (const float *)a.weight_c;
        const float *bias = (const float *)a.bias;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const int64_t dj = dj0 + hc + i;
            wc1n[i] = G::fold(wc[dj]);
            wc2n[i] = G::fold(wc[D + dj]);
            if (bias) { b1n[i] = G::fold(bias[dj]); b2n[i] = G::fold(bias[D + dj]); }
            if (a.mask_c) mk[i] = ((const float *)a.mask_c)[col + i];
            if (a.c_init) c[i] = ((const float *)a.c_init)[col + i];
        }
    }
    const float scale = (float)a.scale_x;
    // Running pointers: one add per time step instead of rebuilding (t*B + b)*D + ... each step.
    const int64_t t_first = dir ? (L - 1) : 0;
    const int64_t ostep = dir ? -(a.B * D) : (a.B * D);
    T *hp = (T *)a.h + (t_first * a.B + b) * D + dj0 + hc;
    const bool has_hist = a.c_hist != nullptr;
    TC *cp = (TC *)a.c_hist + (has_hist ? (t_first * a.B + b) * D + dj0 + hc : 0);
    const int64_t pstep = dir ? -a.B : a.B;
    const uint8_t *pp = has_pad ? a.mask_pad + t_first * a.B + b : nullptr;
    const uint32_t su = BR * u_slab, sx = BR * x_slab;
    const uint32_t u_off = r * u_slab + hc * K * sizeof(T);
    const uint32_t x_off = u_region + r * x_slab + hc * sizeof(T);

    // pad flags of scan steps n_first .. n_first+kTS-1, one bit each; fetched two stages ahead
    auto load_pad = [&](int64_t n_first) -> uint32_t {
        uint32_t bits = 0;
        if (has_pad && active) {
            const uint8_t *q = pp + n_first * pstep;
#pragma unroll
            for (int ts = 0; ts < kTS; ++ts)
                if (n_first + ts < L) bits |= (q[ts * pstep] ? 1u : 0u) << ts;
        }
        return bits;
    };
    uint32_t pad0 = load_pad(0), pad1 = load_pad(kTS);

    int s = 0;
    uint32_t ph = 0;
    for (int it = 0; it < nst; ++it) {
        if (!mbar_wait_bounded(bar_full + 8 * s, ph)) {
            atomicExch(p.err, 2);
            break;
        }
        const uint32_t pad_cur = pad0;
        pad0 = pad1;
        pad1 = load_pad((int64_t)(it + 2) * kTS);
        const uint8_t *sb = stage0 + (size_t)s * stage_bytes;
        const int steps = (int)min((int64_t)kTS, L - (int64_t)it * kTS);
        if (active) {
#pragma unroll
            for (int ts = 0; ts < kTS; ++ts) {
                if (ts < steps) {
                    Pack<T, V> ho;
                    if (!((pad_cur >> ts) & 1u)) {
                        const Pack<T, V * K> up = *reinterpret_cast<const Pack<T, V * K> *>(sb + u_off + ts * su);
                        Pack<T, V> xp;
                        if (has_x) xp = *reinterpret_cast<const Pack<T, V> *>(sb + x_off + ts * sx);
#pragma unroll
                        for (int i = 0; i < V; ++i) {
                            const float u0 = Cvt<T>::to_f(up.v[i * K + 0]);
                            const float u1 = Cvt<T>::to_f(up.v[i * K + 1]);
                            const float u2 = Cvt<T>::to_f(up.v[i * K + 2]);
                            float xv = 0.f;
                            if (K == 4) xv = Cvt<T>::to_f(up.v[i * K + K - 1]);
                            else if (has_x) xv = Cvt<T>::to_f(xp.v[i]) * scale;
                            const float g1 = G::eval(c[i], wc1n[i], u1, b1n[i]);
                            const float g2 = G::eval(c[i], wc2n[i], u2, b2n[i]);
                            c[i] = fmaf(c[i] - u0, g1, u0);
                            ho.v[i] = Cvt<T>::from_f(fmaf((c[i] - xv) * mk[i], g2, xv));
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < V; ++i) ho.v[i] = Cvt<T>::from_f(0.f);
                    }
                    *reinterpret_cast<Pack<T, V> *>(hp) = ho;
                    hp += ostep;
                    if (has_hist) {
                        Pack<TC, V> co;
#pragma unroll
                        for (int i = 0; i < V; ++i) co.v[i] = Cvt<TC>::from_f(c[i]);
                        *reinterpret_cast<Pack<TC, V> *>(cp) = co;
                        cp += ostep;
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * s);
        if (++s == NS) { s = 0; ph ^= 1; }
    }
    if (a.c_last && active) {
        Pack<float, V> cl;
#pragma unroll
        for (int i = 0; i < V; ++i) cl.v[i] = c[i];
        *reinterpret_cast<Pack<float, V> *>((float *)a.c_last + col) = cl;
    }
}

// Backward: scan step m = 0 .. L-1 visits n = L-1-m (the forward's scan order reversed).
//   gg2 = gh*(c - x')*m*g2(1-g2); gc = gh*m*g2 + cur; gg1 = gc*(c' - u0)*g1(1-g1)
//   grad_u = [gc(1-g1), gg1, gg2 (, gh(1-g2 m))]; grad_x = gh(1-g2 m)*scale_x
//   cur <- gc*g1 + gg1*wc1 + gg2*wc2; accumulators gb1 += gg1, gb2 += gg2,
//   gwc1 += gg1*c', gwc2 += gg2*c'.   c (this step's state) is recomputed from c'.
template <typename T, typename TC, int V, int K>
__global__ void __launch_bounds__(160) scan_bwd_pipe(const PipeArgs p) {
    extern __shared__ __align__(128) uint8_t smem[];
    using G = Gate<sizeof(T) == 4>;
    const ScanArgs &a = p.a;
    const int HW = p.c.hw, BR = p.c.br, TPR = p.c.tpr, NS = p.c.nstages;
    const int tid = threadIdx.x;
    const int nthr_c = blockDim.x - 32;
    const int lane = tid & 31;
    const bool has_x = (K == 3) && (a.skip_type == 1);
    const int64_t D = (int64_t)a.d * a.dirs;
    const int ht = blockIdx.x % p.c.nht, rt = blockIdx.x / p.c.nht;
    const int64_t dj0 = (int64_t)ht * HW;
    const int dir = (int)(dj0 / a.d);
    const int64_t b0 = (int64_t)rt * BR;
    const int nrows = (int)min((int64_t)BR, a.B - b0);
    const int64_t L = a.L;
    const int nst = (int)((L + kTS - 1) / kTS);

    const uint32_t bar_full = smem_u32(smem);
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;
    const uint32_t u_slab = (uint32_t)HW * K * sizeof(T);
    const uint32_t x_slab = has_x ? (uint32_t)HW * sizeof(T) : 0;
    const uint32_t c_slab = (uint32_t)HW * sizeof(TC);
    const uint32_t g_slab = (uint32_t)HW * sizeof(T);
    const uint32_t u_region = kTS * BR * u_slab;
    const uint32_t x_region = kTS * BR * x_slab;
    const uint32_t c_region = kTS * BR * c_slab;
    const uint32_t stage_bytes = u_region + x_region + c_region + kTS * BR * g_slab;
    uint8_t *stage0 = smem + kBarBytes;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, nthr_c / 32);
        }
        fence_mbar_init();
    }
    __syncthreads();

    const int r = tid / TPR;
    const int hc = (tid - r * TPR) * V;
    const bool active = (tid < nthr_c) && (tid < BR * TPR) && (r < nrows);
    float gwc1[V], gwc2[V], gb1[V], gb2[V];
#pragma unroll
    for (int i = 0; i < V; ++i) { gwc1[i] = 0.f; gwc2[i] = 0.f; gb1[i] = 0.f; gb2[i] = 0.f; }

    if (tid >= nthr_c) {
        // ------------------------------ producer warp ------------------------------
        const T *u = (const T *)a.u;
        const T *x = (const T *)a.x;
        const TC *chp = (const TC *)a.c_hist;
        const T *gh = (const T *)a.grad_h;
        const int ntens = has_x ? 4 : 3;
        for (int it = 0; it < nst; ++it) {
            const int s = it % NS;
            if (it >= NS) {
                if (!mbar_wait_bounded(bar_empty + 8 * s, ((it / NS) - 1) & 1)) {
                    if (lane == 0) atomicExch(p.err, 3);
                    break;
                }
            }
            const int64_t m0 = (int64_t)it * kTS;
            const int steps = (int)min((int64_t)kTS, L - m0);
            // the step with n == 0 (m == L-1) has no c[t-1] slab: c_init is used instead
            const bool has_first = (m0 + steps == L);
            if (lane == 0) {
                uint32_t bytes = (uint32_t)steps * nrows * (u_slab + x_slab + c_slab + g_slab);
                if (has_first) bytes -= (uint32_t)nrows * c_slab;
                mbar_arrive_expect_tx(bar_full + 8 * s, bytes);
            }
            __syncwarp();
            const uint32_t sbase = smem_u32(stage0 + (size_t)s * stage_bytes);
            const int ncopies = steps * nrows * ntens;
            for (int idx = lane; idx < ncopies; idx += 32) {
                const int which = idx % ntens;
                const int rr = (idx / ntens) % nrows;
                const int ts = idx / (ntens * nrows);
                const int64_t n = L - 1 - (m0 + ts);
                const int64_t t = dir ? (L - 1 - n) : n;
                const int64_t o = ((t * a.B + b0 + rr) * D + dj0);
                const uint32_t bar = bar_full + 8 * s;
                if (which == 0) {
                    bulk_copy_g2s(sbase + (ts * BR + rr) * u_slab, u + o * K, u_slab, bar);
                } else if (which == 1) {
                    bulk_copy_g2s(sbase + u_region + x_region + c_region + (ts * BR + rr) * g_slab,
                                  gh + o, g_slab, bar);
                } else if (which == 2) {
                    if (n > 0) {
                        const int64_t tp = dir ? (t + 1) : (t - 1);
                        const int64_t op = ((tp * a.B + b0 + rr) * D + dj0);
                        bulk_copy_g2s(sbase + u_region + x_region + (ts * BR + rr) * c_slab, chp + op,
                                      c_slab, bar);
                    }
                } else {
                    bulk_copy_g2s(sbase + u_region + (ts * BR + rr) * x_slab, x + o, x_slab, bar);
                }
            }
        }
    } else {
        // -------------------------------- consumers --------------------------------
        const int64_t b = b0 + (active ? r : 0);
        const int64_t col = b * D + dj0 + hc;
        const bool has_pad = a.mask_pad != nullptr;
        float cur[V], wc1n[V], wc2n[V], b1n[V], b2n[V], mk[V], c0[V];
#pragma unroll
        for (int i = 0; i < V; ++i) {
            cur[i] = 0.f; wc1n[i] = 0.f; wc2n[i] = 0.f; b1n[i] = 0.f; b2n[i] = 0.f; mk[i] = 1.f; c0[i] = 0.f;
        }
        if (active) {
            const float *wc = (const float *)a.weight_c;
            const float *bias = (const float *)a.bias;
#pragma unroll
            for (int i = 0; i < V; ++i) {
                const int64_t dj = dj0 + hc + i;
                wc1n[i] = G::fold(wc[dj]);
                wc2n[i] = G::fold(wc[D + dj]);
                if (bias) { b1n[i] = G::fold(bias[dj]); b2n[i] = G::fold(bias[D + dj]); }
                if (a.mask_c) mk[i] = ((const float *)a.mask_c)[col + i];
                if (a.c_init) c0[i] = ((const float *)a.c_init)[col + i];
                if (a.grad_last) cur[i] = ((const float *)a.grad_last)[col + i];
            }
        }
        const float scale = (float)a.scale_x;
        // Backward step m visits the forward's scan step n = L-1-m, i.e. time t = dir ? m : L-1-m.
        const int64_t t_first = dir ? 0 : (L - 1);
        const int64_t ostep = dir ? (a.B * D) : -(a.B * D);
        const int64_t o_first = (t_first * a.B + b) * D + dj0 + hc;
        T *gup = (T *)a.grad_u + o_first * K;
        T *gxp = (T *)a.grad_x + (has_x ? o_first : 0);
        const int64_t pstep = dir ? a.B : -a.B;
        const uint8_t *pp = has_pad ? a.mask_pad + t_first * a.B + b : nullptr;
        const uint32_t su = BR * u_slab, sx = BR * x_slab, sc = BR * c_slab, sg = BR * g_slab;
        const uint32_t u_off = r * u_slab + hc * K * sizeof(T);
        const uint32_t x_off = u_region + r * x_slab + hc * sizeof(T);
        const uint32_t c_off = u_region + x_region + r * c_slab + hc * sizeof(TC);
        const uint32_t g_off = u_region + x_region + c_region + r * g_slab + hc * sizeof(T);

        auto load_pad = [&](int64_t m_first) -> uint32_t {
            uint32_t bits = 0;
            if (has_pad && active) {
                const uint8_t *q = pp + m_first * pstep;
#pragma unroll
                for (int ts = 0; ts < kTS; ++ts)
                    if (m_first + ts < L) bits |= (q[ts * pstep] ? 1u : 0u) << ts;
            }
            return bits;
        };
        uint32_t pad0 = load_pad(0), pad1 = load_pad(kTS);

        int s = 0;
        uint32_t ph = 0;
        for (int it = 0; it < nst; ++it) {
            if (!mbar_wait_bounded(bar_full + 8 * s, ph)) {
                atomicExch(p.err, 4);
                break;
            }
            const uint32_t pad_cur = pad0;
            pad0 = pad1;
            pad1 = load_pad((int64_t)(it + 2) * kTS);
            const uint8_t *sb = stage0 + (size_t)s * stage_bytes;
            const int64_t left = L - (int64_t)it * kTS;   // steps left including this stage
            const int steps = (int)min((int64_t)kTS, left);
            if (active) {
#pragma unroll
                for (int ts = 0; ts < kTS; ++ts) {
                    if (ts < steps) {
                        Pack<T, V * K> guo;
                        Pack<T, V> gxo;
                        if (!((pad_cur >> ts) & 1u)) {
                            const bool at_start = (ts == left - 1);   // n == 0: the state before it is c_init
                            const Pack<T, V * K> up = *reinterpret_cast<const Pack<T, V * K> *>(sb + u_off + ts * su);
                            const Pack<T, V> ghp = *reinterpret_cast<const Pack<T, V> *>(sb + g_off + ts * sg);
                            Pack<T, V> xp;
                            if (has_x) xp = *reinterpret_cast<const Pack<T, V> *>(sb + x_off + ts * sx);
                            Pack<TC, V> cpp;
                            if (!at_start) cpp = *reinterpret_cast<const Pack<TC, V> *>(sb + c_off + ts * sc);
#pragma unroll
                            for (int i = 0; i < V; ++i) {
                                const float u0 = Cvt<T>::to_f(up.v[i * K + 0]);
                                const float u1 = Cvt<T>::to_f(up.v[i * K + 1]);
                                const float u2 = Cvt<T>::to_f(up.v[i * K + 2]);
                                float xv = 0.f;
                                if (K == 4) xv = Cvt<T>::to_f(up.v[i * K + K - 1]);
                                else if (has_x) xv = Cvt<T>::to_f(xp.v[i]) * scale;
                                const float cp = at_start ? c0[i] : Cvt<TC>::to_f(cpp.v[i]);
                                const float gh = Cvt<T>::to_f(ghp.v[i]);
                                const float g1 = G::eval(cp, wc1n[i], u1, b1n[i]);
                                const float g2 = G::eval(cp, wc2n[i], u2, b2n[i]);
                                const float dc = cp - u0;
                                const float cv = fmaf(dc, g1, u0);
                                const float ghm = gh * mk[i];
                                const float gg2 = ghm * (cv - xv) * (g2 - g2 * g2);
                                const float gc = fmaf(ghm, g2, cur[i]);
                                const float gg1 = gc * dc * (g1 - g1 * g1);
                                gb1[i] += gg1;
                                gb2[i] += gg2;
                                gwc1[i] = fmaf(gg1, cp, gwc1[i]);
                                gwc2[i] = fmaf(gg2, cp, gwc2[i]);
                                cur[i] = fmaf(gc, g1, G::kUnfold * fmaf(gg1, wc1n[i], gg2 * wc2n[i]));
                                const float gxv = fmaf(-ghm, g2, gh);
                                guo.v[i * K + 0] = Cvt<T>::from_f(fmaf(-gc, g1, gc));
                                guo.v[i * K + 1] = Cvt<T>::from_f(gg1);
                                guo.v[i * K + 2] = Cvt<T>::from_f(gg2);
                                if (K == 4) guo.v[i * K + K - 1] = Cvt<T>::from_f(gxv);
                                gxo.v[i] = Cvt<T>::from_f(gxv * scale);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < V * K; ++i) guo.v[i] = Cvt<T>::from_f(0.f);
#pragma unroll
                            for (int i = 0; i < V; ++i) gxo.v[i] = Cvt<T>::from_f(0.f);
                        }
                        *reinterpret_cast<Pack<T, V * K> *>(gup) = guo;
                        gup += ostep * K;
                        if (has_x) {
                            *reinterpret_cast<Pack<T, V> *>(gxp) = gxo;
                            gxp += ostep;
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * s);
            if (++s == NS) { s = 0; ph ^= 1; }
        }
        if (active) {
            Pack<float, V> gi;
#pragma unroll
            for (int i = 0; i < V; ++i) gi.v[i] = cur[i];
            *reinterpret_cast<Pack<float, V> *>((float *)a.grad_init + col) = gi;
        }
    }

    // ---- batch reduction of the parameter gradients over the tile's rows ----
    __syncthreads();  // all stages consumed; the ring is reused as red[BR][4][HW]
    float *red = reinterpret_cast<float *>(stage0);
    if (tid < nthr_c && tid < BR * TPR) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const size_t base = (size_t)r * 4 * HW + hc + i;
            red[base] = active ? gwc1[i] : 0.f;
            red[base + HW] = active ? gwc2[i] : 0.f;
            red[base + 2 * HW] = active ? gb1[i] : 0.f;
            red[base + 3 * HW] = active ? gb2[i] : 0.f;
        }
    }
    __syncthreads();
    float *part = (float *)a.workspace + (size_t)rt * 4 * D + dj0;
    for (int idx = tid; idx < 4 * HW; idx += blockDim.x) {
        const int g = idx / HW, j = idx - g * HW;
        float sum = 0.f;
        for (int rr = 0; rr < nrows; ++rr) sum += red[(size_t)rr * 4 * HW + idx];
        part[(size_t)g * D + j] = sum;
    }
}

// ---------------------------------------------------------------------------------------
// Host side: tile selection and dispatch
// ---------------------------------------------------------------------------------------
static int g_num_sms = 0;
static int num_sms() {
    if (g_num_sms == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            g_num_sms = n;
        else
            g_num_sms = 148;
    }
    return g_num_sms;
}

static int env_int(const char *name, int dflt) {
    const char *e = getenv(name);
    return (e && *e) ? atoi(e) : dflt;
}

// Chooses V, the tile and the ring.  Returns false when the shape is not eligible.
static bool choose_tile(int64_t L, int64_t B, int64_t d, int dirs, int k, int skip_type, int dtype,
                        int c_dtype, bool backward, TileCfg *out) {
    const int s = (int)dtype_size(dtype);
    if (dtype == SRU_F64 || s == 0) return false;
    const int granule = 16 / s;  // elements per 16 bytes
    if (d % granule != 0 || L < 1 || B < 1) return false;
    const int64_t D = d * dirs, ncols = B * D;
    const int sms = num_sms();
    const int vmax = granule, vmin = (s == 2) ? 2 : 1;
    // Columns per thread.  Measured on B200: with three or more warps per SM available, V = 4
    // amortises the per-step overhead best (V = 8 costs registers and occupancy for nothing);
    // smaller problems are bound by per-step latency and want as many warps as possible.
    int v = (ncols / (32 * 4) >= (int64_t)sms * 3 && vmax >= 4) ? 4 : vmin;
    v = env_int(backward ? "SRU_B200_BWD_V" : "SRU_B200_FWD_V", v);
    if (v < vmin || v > vmax || (v & (v - 1))) return false;
    // consumer threads per CTA: two warps, one when that is needed to give every SM a CTA
    int ntc = (ncols / ((int64_t)v * 64) >= (int64_t)sms) ? 64 : 32;
    ntc = env_int("SRU_B200_SCAN_THREADS", ntc);
    if (ntc < 32 || ntc > 128 || ntc % 32) return false;
    // hidden width of the tile: largest divisor of d, multiple of the granule, <= v*ntc
    int hw = 0;
    for (int64_t cand = (int64_t)v * ntc; cand >= granule; cand -= granule) {
        if (d % cand == 0) { hw = (int)cand; break; }
    }
    if (hw == 0) return false;
    const int tpr = hw / v;
    int br = (int)std::min<int64_t>(B, std::max(1, ntc / tpr));
    const int cthreads = ((br * tpr + 31) / 32) * 32;
    if (cthreads > 128) return false;
    const bool has_x = (k == 3 && skip_type == 1);
    const int sc = (int)dtype_size(c_dtype);
    size_t per_row_step = (size_t)hw * (k * s + (has_x ? s : 0));
    if (backward) per_row_step += (size_t)hw * (sc + s);
    const size_t stage_bytes = (size_t)kTS * br * per_row_step;
    // ring: about 72 KB per CTA slot, shared by the CTAs expected on one SM
    const int64_t nctas = ((B + br - 1) / br) * (D / hw);
    int cta_per_sm = (int)std::min<int64_t>(std::max<int64_t>(1, (nctas + sms - 1) / sms), 2048 / (cthreads + 32));
    size_t ring = std::min<size_t>(200 * 1024 / cta_per_sm, 96 * 1024);
    int ns = (int)(ring / stage_bytes);
    ns = std::max(2, std::min(ns, kMaxStages));
    ns = env_int("SRU_B200_SCAN_STAGES", ns);
    ns = std::max(2, std::min(ns, kMaxStages));
    size_t smem = kBarBytes + (size_t)ns * stage_bytes;
    if (backward) smem = std::max(smem, kBarBytes + (size_t)br * 4 * hw * sizeof(float));
    if (smem > 227 * 1024) {
        ns = (int)((227 * 1024 - kBarBytes) / stage_bytes);
        if (ns < 2) return false;
        smem = kBarBytes + (size_t)ns * stage_bytes;
    }
    out->hw = hw; out->br = br; out->tpr = tpr;
    out->nht = (int)(D / hw); out->nrt = (int)((B + br - 1) / br);
    out->nstages = ns; out->v = v; out->threads = cthreads + 32; out->smem = smem;
    return nctas <= 0x7fffffff;
}

static bool pipelined_eligible(const ScanArgs &a) {
    if (a.is_custom || a.activation_type != 0) return false;
    if (a.k == 3 && a.skip_type == 2) return false;
    if (a.k == 4 && a.skip_type != 2) return false;
    if (a.dtype == SRU_F64) return false;
    if (env_int("SRU_B200_FORCE_GENERIC", 0)) return false;
    return true;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

size_t pipelined_workspace_bytes(int64_t L, int64_t B, int64_t d, int dirs, int k, int dtype) {
    (void)L; (void)k; (void)dtype;
    return (size_t)B * 4 * d * dirs * sizeof(float);  // upper bound: one row per tile
}

template <typename T, typename TC, int V, int K>
static int launch_t(const PipeArgs &p, bool backward, cudaStream_t st) {
    auto fwd = scan_fwd_pipe<T, TC, V, K>;
    auto bwd = scan_bwd_pipe<T, TC, V, K>;
    const void *fn = backward ? (const void *)bwd : (const void *)fwd;
    if (p.c.smem > 48 * 1024)
        SRUB_CUDA_CHECK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.c.smem));
    const unsigned grid = (unsigned)((int64_t)p.c.nht * p.c.nrt);
    if (backward) bwd<<<grid, p.c.threads, p.c.smem, st>>>(p);
    else fwd<<<grid, p.c.threads, p.c.smem, st>>>(p);
    SRUB_CUDA_CHECK(cudaGetLastError());
    return 1;
}

template <typename T, typename TC, int K>
static int launch_v(const PipeArgs &p, bool backward, cudaStream_t st) {
    constexpr int s = sizeof(T);
    switch (p.c.v) {
        case 1: if constexpr (s == 4) return launch_t<T, TC, 1, K>(p, backward, st); break;
        case 2: return launch_t<T, TC, 2, K>(p, backward, st);
        case 4: return launch_t<T, TC, 4, K>(p, backward, st);
        case 8: if constexpr (s == 2) return launch_t<T, TC, 8, K>(p, backward, st); break;
    }
    return set_error(SRU_ERR_UNSUPPORTED, "columns per thread %d", p.c.v);
}

template <typename T, typename TC>
static int launch_k(const PipeArgs &p, bool backward, cudaStream_t st) {
    return p.a.k == 3 ? launch_v<T, TC, 3>(p, backward, st) : launch_v<T, TC, 4>(p, backward, st);
}

int launch_scan_pipelined(const ScanArgs &a, bool backward, cudaStream_t st) {
    if (!pipelined_eligible(a)) return 0;
    PipeArgs p;
    p.a = a;
    if (!choose_tile(a.L, a.B, a.d, a.dirs, a.k, a.skip_type, a.dtype, a.c_dtype, backward, &p.c)) return 0;
    // bulk copies need 16-byte aligned sources; packed stores need V*sizeof(T) alignment
    const void *ptrs[] = {a.u, a.x, a.h, a.c_hist, a.grad_h, a.grad_u, a.grad_x, a.c_last, a.c_init,
                          a.grad_last, a.grad_init, a.mask_c};
    for (const void *q : ptrs)
        if (q && !aligned16(q)) return 0;
    p.err = device_error_flag();
    if (!p.err) return set_error(SRU_ERR_CUDA, "device error flag unavailable");
    const int dt = a.dtype, ct = a.c_dtype;
    int rc;
    if (dt == SRU_F32 && ct == SRU_F32) rc = launch_k<float, float>(p, backward, st);
    else if (dt == SRU_F16 && ct == SRU_F16) rc = launch_k<__half, __half>(p, backward, st);
    else if (dt == SRU_F16 && ct == SRU_F32) rc = launch_k<__half, float>(p, backward, st);
    else if (dt == SRU_BF16 && ct == SRU_BF16) rc = launch_k<__nv_bfloat16, __nv_bfloat16>(p, backward, st);
    else if (dt == SRU_BF16 && ct == SRU_F32) rc = launch_k<__nv_bfloat16, float>(p, backward, st);
    else return set_error(SRU_ERR_UNSUPPORTED, "dtype %d with c_dtype %d", dt, ct);
    if (rc < 0) return rc;
    if (backward) {
        const int r2 = launch_reduce_partials<float>(a.workspace, a.grad_wc, a.grad_bias, p.c.nrt,
                                                     (int64_t)a.d * a.dirs, 1, st);
        if (r2 < 0) return r2;
    }
    return 1;
}

}  // namespace srub
