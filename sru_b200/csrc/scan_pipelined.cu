// Pipelined scan kernels for sm_100a.
//
// Work decomposition.  A CTA owns a tile of BR batch rows x HW hidden units of ONE
// direction; each consumer thread owns V adjacent hidden units of one row and keeps their
// state (c, or dL/dc and the four parameter-gradient accumulators) in registers for the
// whole sequence.  Time is the only sequential axis.
//
// Memory pipeline.  Every streamed tensor (the gate pre-activations U, the highway input x,
// and for backward c[t-1] and grad_h) is described to the TMA engine by a 3-D tensor map
// (row bytes, batch, time).  One elected producer thread per CTA issues ONE
// cp.async.bulk.tensor request per tensor and ring stage: a box of SS time steps x BR rows x
// the tile's hidden slice, landing in one of NS shared-memory stages and completing on that
// stage's "full" mbarrier.  (Per-row untiled bulk copies were measured first: each costs the
// issuing warp ~100 cycles, which capped small tiles at ~1 TB/s; a box request moves 4-16x
// the bytes per instruction.)  Consumers wait on the stage's "full" barrier, read their
// 4..48-byte slices with vector shared loads, and release the stage through its "empty"
// barrier.  The depth in time of the ring, not the number of resident threads, provides the
// bytes in flight that HBM needs.  Boxes that stick out of the tensor in time or batch are
// zero-filled by the hardware.  Outputs go straight from registers to global memory with
// V*sizeof(T)-byte stores that are contiguous across the warp.
//
// Latency.  Small problems leave about one warp per SM sub-partition, so what bounds them is
// the dependent-instruction latency of one time step.  The body of a 4-step block is therefore
// branch-free (padding and the c_init boundary are selects, the options are template
// parameters) and unrolled, which lets the scheduler overlap the loads, conversions and output
// arithmetic of neighbouring steps with the one chain that is truly serial: c' -> gate -> c.
//
// Every wait is bounded (mbar_wait_bounded); on a timeout the thread raises the device
// error flag, stops processing and falls through to the end of the kernel.
//
// Arithmetic (same as the reference kernels sru/csrc/sru_cuda_kernel.cu:60-78 forward,
// :130-176 backward, with the direction taken from the tile instead of col % 2d):
//   g1 = s(u1 + wc1*c' + b1), g2 = s(u2 + wc2*c' + b2), c = (c' - u0)*g1 + u0,
//   h = (c - x')*m*g2 + x',  x' = x*scale_x (k=3) | u3 (k=4).
#include <cudaTypedefs.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "scan_pipe_common.cuh"

namespace srub {

template <typename T, typename TC, int V, int K>
__global__ void __launch_bounds__(160) scan_fwd_pipe(const __grid_constant__ ScanMaps maps, const PipeArgs p) {
    extern __shared__ __align__(128) uint8_t smem[];
    using G = GateFor<T>;
    const ScanArgs &a = p.a;
    const int HW = p.c.hw, BR = p.c.br, TPR = p.c.tpr, NS = p.c.nstages, SS = p.c.ss;
    const int tid = threadIdx.x;
    const int nthr_c = blockDim.x - 32;
    const int lane = tid & 31;
    constexpr bool has_x = (K == 3);   // k = 3 without a highway term is served by the generic kernel
    const int64_t D = (int64_t)a.d * a.dirs;
    const int ht = blockIdx.x % p.c.nht, rt = blockIdx.x / p.c.nht;
    const int64_t dj0 = (int64_t)ht * HW;
    const int dir = (int)(dj0 / a.d);
    const bool asc = (dir == 0);        // this tile walks time upwards
    const int64_t b0 = (int64_t)rt * BR;
    const int nrows = (int)min((int64_t)BR, a.B - b0);
    const int64_t L = a.L;
    const int nst = (int)((L + SS - 1) / SS);

    const uint32_t bar_full = smem_u32(smem);
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;
    const uint32_t u_slab = (uint32_t)HW * K * sizeof(T);   // bytes per (step,row)
    const uint32_t x_slab = has_x ? (uint32_t)HW * sizeof(T) : 0;
    const uint32_t u_region = align128(SS * BR * u_slab);
    const uint32_t x_region = align128(SS * BR * x_slab);
    const bool has_pad = a.mask_pad != nullptr;
    const uint32_t pad_region = has_pad ? align128(SS * BR) : 0;   // flags [row][step of the stage], one byte each
    const uint32_t stage_bytes = u_region + x_region + pad_region;
    uint8_t *stage0 = smem + kBarBytes;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(bar_full + 8 * s, a.mask_pad ? 2 : 1);   // the copies' arrive, and the pad flags'
            mbar_init(bar_empty + 8 * s, nthr_c / 32);
        }
        fence_mbar_init();
    }
    __syncthreads();

    if (tid >= nthr_c) {
        // ------------------- producer warp: lane 0 issues the copies, all lanes stage the pad flags -------------------
        const int xu = (int)(dj0 * K * sizeof(T) / 8), xx = (int)(dj0 * sizeof(T) / 8);
        PadStager pads(a.mask_pad, a.B, L, b0, BR, SS, lane);
        // ascending tiles take times [it*SS, it*SS+SS); descending ones the mirrored window,
        // which may start below 0 (the box is zero-filled there, the flags read as "not padded")
        auto first_time = [&](int it) { return asc ? it * SS : (int)(L - (int64_t)(it + 1) * SS); };
        if (has_pad) pads.fetch(first_time(0));
        int s = 0;
        uint32_t ph = 1;   // the first pass over the ring finds every stage free
        for (int it = 0; it < nst; ++it) {
            int ok = (lane == 0) ? (int)mbar_wait_bounded(bar_empty + 8 * s, ph) : 1;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { if (lane == 0) atomicExch(p.err, 1); break; }
            const uint32_t bar = bar_full + 8 * s;
            const uint32_t sbase = smem_u32(stage0) + (uint32_t)s * stage_bytes;
            if (lane == 0) {
                const int t0 = first_time(it);
                mbar_arrive_expect_tx(bar, (uint32_t)SS * BR * (u_slab + x_slab));
                tma_load_3d(sbase, &maps.u, bar, xu, (int)b0, t0);
                if (has_x) tma_load_3d(sbase + u_region, &maps.x, bar, xx, (int)b0, t0);
            }
            if (has_pad) {
                // this stage's flags were read from global memory one stage ago; the next stage's are
                // requested now and not looked at until the next trip, so their latency stays off every path
                pads.store(sbase + u_region + x_region);
                if (it + 1 < nst) pads.fetch(first_time(it + 1));
                __syncwarp();
                if (lane == 0) mbar_arrive(bar);   // second arrival: releases all lanes' flag writes to the consumers
            }
            if (++s == NS) { s = 0; ph ^= 1; }
        }
        return;
    }

    // -------------------------------- consumers --------------------------------
    const int r = tid / TPR;
    const int hc = (tid - r * TPR) * V;
    const bool active = (tid < BR * TPR) && (r < nrows);
    const int64_t b = b0 + (active ? r : 0);
    const int64_t col = b * D + dj0 + hc;
    const bool has_hist = a.c_hist != nullptr;

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
    const int64_t t_first = asc ? 0 : (L - 1);
    const int64_t ostep = asc ? (a.B * D) : -(a.B * D);
    T *hp = (T *)a.h + (t_first * a.B + b) * D + dj0 + hc;
    TC *cp = (TC *)a.c_hist + (has_hist ? (t_first * a.B + b) * D + dj0 + hc : 0);
    const int su = BR * (int)u_slab, sx = BR * (int)x_slab;      // bytes between time slabs of a stage
    const uint32_t u_off = r * u_slab + hc * K * sizeof(T);
    const uint32_t x_off = u_region + r * x_slab + hc * sizeof(T);
    const uint32_t pad_off = u_region + x_region + r * SS;       // this row's flags of the stage

    // A step's packs are loaded at the step.  Requesting them one step ahead (a software pipeline of depth one)
    // was measured on B200: timed alone at full clocks it gained 4-8 % for two and four columns per thread, but inside
    // the power-capped training step (SM clock ~1.2-1.35 GHz) the 50 extra registers cost more in resident warps than
    // the earlier loads gained (2048-wide layer, L = 1000, batch 256: 16.8 ms -> 19.4-21.1 ms per step), and one
    // column per thread lost 30 % everywhere.  Not done.
    const int dsu = asc ? su : -su, dsx = asc ? sx : -sx;   // bytes to the next step's slab in scan order
    // (the packed two-columns-per-instruction arithmetic of the backward kernel was measured here too: no gain, the
    // forward pass is not issue-bound: 16.0 vs 16.3-16.5 ms per step of the 12-layer benchmark)

    // One block of kTS steps.  ub / xb point at this thread's slice in the slab of the block's first step.
    auto block = [&](uint32_t ub, uint32_t xb, uint32_t pad_bits, int steps, auto pad_c, auto hist_c, auto full_c) {
        constexpr bool PAD = decltype(pad_c)::value, HIST = decltype(hist_c)::value, FULL = decltype(full_c)::value;
#pragma unroll
        for (int ts = 0; ts < kTS; ++ts) {
            if (!FULL && ts >= steps) break;
            const bool pad = PAD && ((pad_bits >> (8 * ts)) & 0xffu);
            const Pack<T, V * K> up = lds_pack<Pack<T, V * K>>(ub + ts * dsu);
            Pack<T, V> xp;
            if (has_x) xp = lds_pack<Pack<T, V>>(xb + ts * dsx);
            float hv[V];
            {
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    const float u0 = Cvt<T>::to_f(up.v[i * K + 0]);
                    const float u1 = Cvt<T>::to_f(up.v[i * K + 1]);
                    const float u2 = Cvt<T>::to_f(up.v[i * K + 2]);
                    const float xv = (K == 4) ? Cvt<T>::to_f(up.v[i * K + K - 1]) : Cvt<T>::to_f(xp.v[i]) * scale;
                    const float g1 = G::eval(c[i], wc1n[i], u1, b1n[i]);
                    const float g2 = G::eval(c[i], wc2n[i], u2, b2n[i]);
                    const float cn = fmaf(c[i] - u0, g1, u0);
                    const float hn = fmaf((cn - xv) * mk[i], g2, xv);
                    c[i] = pad ? c[i] : cn;
                    hv[i] = pad ? 0.f : hn;
                }
            }
            Pack<T, V> ho;
            pack_from_float(ho, hv);
            *reinterpret_cast<Pack<T, V> *>(hp) = ho;
            hp += ostep;
            if (HIST) {
                Pack<TC, V> co;
                pack_from_float(co, c);
                *reinterpret_cast<Pack<TC, V> *>(cp) = co;
                cp += ostep;
            }
        }
    };

    auto run = [&](auto pad_c, auto hist_c) {
        constexpr bool PADF = decltype(pad_c)::value;
        int s = 0;
        uint32_t ph = 0;
        int64_t n = 0;   // scan step of the next block
        for (int it = 0; it < nst; ++it) {
            if (!mbar_wait_bounded(bar_full + 8 * s, ph)) {
                atomicExch(p.err, 2);
                break;
            }
            const uint32_t sb = order_after_wait(smem_u32(stage0) + (uint32_t)s * stage_bytes);
            for (int q = 0; q < SS && n < L; q += kTS, n += kTS) {
                if (active) {
                    // the block's four flags, byte ts = scan step ts of the block
                    const uint32_t pad_cur = PADF ? pad_word(sb + pad_off, q, SS, asc) : 0u;
                    const int slab = asc ? q : (SS - 1 - q);
                    const uint32_t ub = sb + u_off + slab * su, xb = sb + x_off + slab * sx;
                    const int64_t left = L - n;
                    if (left >= kTS) block(ub, xb, pad_cur, kTS, pad_c, hist_c, BoolC<true>{});
                    else block(ub, xb, pad_cur, (int)left, pad_c, hist_c, BoolC<false>{});
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * s);
            if (++s == NS) { s = 0; ph ^= 1; }
        }
    };
    if (has_pad) {
        if (has_hist) run(BoolC<true>{}, BoolC<true>{}); else run(BoolC<true>{}, BoolC<false>{});
    } else {
        if (has_hist) run(BoolC<false>{}, BoolC<true>{}); else run(BoolC<false>{}, BoolC<false>{});
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
__global__ void __launch_bounds__(160) scan_bwd_pipe(const __grid_constant__ ScanMaps maps, const PipeArgs p) {
    extern __shared__ __align__(128) uint8_t smem[];
    using G = GateFor<T>;
    const ScanArgs &a = p.a;
    const int HW = p.c.hw, BR = p.c.br, TPR = p.c.tpr, NS = p.c.nstages, SS = p.c.ss;
    const int tid = threadIdx.x;
    const int nthr_c = blockDim.x - 32;
    const int lane = tid & 31;
    constexpr bool has_x = (K == 3);
    const int64_t D = (int64_t)a.d * a.dirs;
    const int ht = blockIdx.x % p.c.nht, rt = blockIdx.x / p.c.nht;
    const int64_t dj0 = (int64_t)ht * HW;
    const int dir = (int)(dj0 / a.d);
    const bool asc = (dir == 1);        // the backward walk of a reverse-direction tile goes up in time
    const int64_t b0 = (int64_t)rt * BR;
    const int nrows = (int)min((int64_t)BR, a.B - b0);
    const int64_t L = a.L;
    const int nst = (int)((L + SS - 1) / SS);

    const uint32_t bar_full = smem_u32(smem);
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;
    const uint32_t u_slab = (uint32_t)HW * K * sizeof(T);
    const uint32_t x_slab = has_x ? (uint32_t)HW * sizeof(T) : 0;
    const uint32_t c_slab = (uint32_t)HW * sizeof(TC);
    const uint32_t g_slab = (uint32_t)HW * sizeof(T);
    const uint32_t u_region = align128(SS * BR * u_slab);
    const uint32_t x_region = align128(SS * BR * x_slab);
    const uint32_t c_region = align128(SS * BR * c_slab);
    const uint32_t g_region = align128(SS * BR * g_slab);
    const bool has_pad = a.mask_pad != nullptr;
    const uint32_t pad_region = has_pad ? align128(SS * BR) : 0;   // flags [row][step of the stage], one byte each
    const uint32_t in_region = u_region + x_region + c_region + g_region;
    const uint32_t stage_bytes = in_region + pad_region;
    uint8_t *stage0 = smem + kBarBytes;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(bar_full + 8 * s, a.mask_pad ? 2 : 1);   // the copies' arrive, and the pad flags'
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
        // ------------------- producer warp: lane 0 issues the copies, all lanes stage the pad flags -------------------
        const int xu = (int)(dj0 * K * sizeof(T) / 8), xx = (int)(dj0 * sizeof(T) / 8);
        const int xc = (int)(dj0 * sizeof(TC) / 8);
        PadStager pads(a.mask_pad, a.B, L, b0, BR, SS, lane);
        auto first_time = [&](int it) { return asc ? it * SS : (int)(L - (int64_t)(it + 1) * SS); };
        if (has_pad) pads.fetch(first_time(0));
        int s = 0;
        uint32_t ph = 1;
        for (int it = 0; it < nst; ++it) {
            int ok = (lane == 0) ? (int)mbar_wait_bounded(bar_empty + 8 * s, ph) : 1;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { if (lane == 0) atomicExch(p.err, 3); break; }
            const uint32_t bar = bar_full + 8 * s;
            const uint32_t sbase = smem_u32(stage0) + (uint32_t)s * stage_bytes;
            if (lane == 0) {
                const int t0 = first_time(it);
                mbar_arrive_expect_tx(bar, (uint32_t)SS * BR * (u_slab + x_slab + c_slab + g_slab));
                tma_load_3d(sbase, &maps.u, bar, xu, (int)b0, t0);
                if (has_x) tma_load_3d(sbase + u_region, &maps.x, bar, xx, (int)b0, t0);
                // the state BEFORE each step: one time step further along this walk (out-of-range rows,
                // i.e. the predecessor of the sequence start, are zero-filled and replaced by c_init)
                tma_load_3d(sbase + u_region + x_region, &maps.c, bar, xc, (int)b0, asc ? t0 + 1 : t0 - 1);
                tma_load_3d(sbase + u_region + x_region + c_region, &maps.g, bar, xx, (int)b0, t0);
            }
            if (has_pad) {
                pads.store(sbase + in_region);
                if (it + 1 < nst) pads.fetch(first_time(it + 1));
                __syncwarp();
                if (lane == 0) mbar_arrive(bar);   // second arrival: releases all lanes' flag writes to the consumers
            }
            if (++s == NS) { s = 0; ph ^= 1; }
        }
    } else {
        // -------------------------------- consumers --------------------------------
        const int64_t b = b0 + (active ? r : 0);
        const int64_t col = b * D + dj0 + hc;
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
        const int64_t t_first = asc ? 0 : (L - 1);
        const int64_t ostep = asc ? (a.B * D) : -(a.B * D);
        const int64_t o_first = (t_first * a.B + b) * D + dj0 + hc;
        T *gup = (T *)a.grad_u + o_first * K;
        T *gxp = (T *)a.grad_x + (has_x ? o_first : 0);
        const int su = BR * (int)u_slab, sx = BR * (int)x_slab, sc = BR * (int)c_slab, sg = BR * (int)g_slab;
        const uint32_t u_off = r * u_slab + hc * K * sizeof(T);
        const uint32_t x_off = u_region + r * x_slab + hc * sizeof(T);
        const uint32_t c_off = u_region + x_region + r * c_slab + hc * sizeof(TC);
        const uint32_t g_off = u_region + x_region + c_region + r * g_slab + hc * sizeof(T);
        const uint32_t pad_off = in_region + r * SS;                 // this row's flags of the stage

        // (packs are loaded at the step: see the forward kernel for why not one step ahead; the backward lost a resident
        // CTA per SM to the 40 extra registers and 30 % of its throughput)
        const int dsu = asc ? su : -su, dsx = asc ? sx : -sx, dsc = asc ? sc : -sc, dsg = asc ? sg : -sg;
        // 16-bit storage (tanh gates): a thread's columns are processed in PAIRS with the packed float32 instructions
        // of f32x2.cuh.  Measured inside the 12-layer training step, both builds on one box: 26.5-27.0 -> 24.6-24.7 ms
        // per step (0.78-0.80 -> 0.86 of the HBM peak at an SM clock of 1.2-1.35 GHz, where the kernel is issue-bound).
        constexpr bool kPairs = (sizeof(T) == 2) && (V % 2 == 0);

        // One block of kTS steps; ub / xb / cb / gb point at this thread's slices in the slab of the block's first step.
        // LAST marks the final block (ragged, and holding the step whose predecessor state is c_init); all other
        // blocks are full and branch-free.
        auto block = [&](uint32_t ub, uint32_t xb, uint32_t cb, uint32_t gb, uint32_t pad_bits, int steps, auto pad_c,
                         auto last_c) {
            constexpr bool PAD = decltype(pad_c)::value, LAST = decltype(last_c)::value;
#pragma unroll
            for (int ts = 0; ts < kTS; ++ts) {
                if (LAST && ts >= steps) break;
                const bool pad = PAD && ((pad_bits >> (8 * ts)) & 0xffu);
                const bool at_start = LAST && (ts == steps - 1);
                const Pack<T, V * K> up = lds_pack<Pack<T, V * K>>(ub + ts * dsu);
                const Pack<T, V> ghp = lds_pack<Pack<T, V>>(gb + ts * dsg);
                Pack<T, V> xp;
                if (has_x) xp = lds_pack<Pack<T, V>>(xb + ts * dsx);
                const Pack<TC, V> cpp = lds_pack<Pack<TC, V>>(cb + ts * dsc);
                float guv[V * K], gxv_[V];
                if constexpr (kPairs) {
                    // two columns per instruction (f32x2.cuh).  Same formulas as the scalar form below; 1 - g is formed
                    // explicitly (the packed instructions take no negated operand), which moves a rounding or two but
                    // nothing a 16-bit output can show.
                    const F2 half = f2_splat(0.5f), one = f2_splat(1.f), scale2 = f2_splat(scale), unfold = f2_splat(G::kUnfold);
#pragma unroll
                    for (int i = 0; i < V; i += 2) {
                        const F2 u0 = f2_make(Cvt<T>::to_f(up.v[i * K + 0]), Cvt<T>::to_f(up.v[(i + 1) * K + 0]));
                        const F2 u1 = f2_make(Cvt<T>::to_f(up.v[i * K + 1]), Cvt<T>::to_f(up.v[(i + 1) * K + 1]));
                        const F2 u2 = f2_make(Cvt<T>::to_f(up.v[i * K + 2]), Cvt<T>::to_f(up.v[(i + 1) * K + 2]));
                        F2 xv;
                        if (K == 4) xv = f2_make(Cvt<T>::to_f(up.v[i * K + K - 1]), Cvt<T>::to_f(up.v[(i + 1) * K + K - 1]));
                        else xv = f2_mul(f2_make(Cvt<T>::to_f(xp.v[i]), Cvt<T>::to_f(xp.v[i + 1])), scale2);
                        const F2 cprev = at_start ? f2_make(c0[i], c0[i + 1])
                                                  : f2_make(Cvt<TC>::to_f(cpp.v[i]), Cvt<TC>::to_f(cpp.v[i + 1]));
                        const F2 gh = f2_make(Cvt<T>::to_f(ghp.v[i]), Cvt<T>::to_f(ghp.v[i + 1]));
                        const F2 wc1p = f2_make(wc1n[i], wc1n[i + 1]), wc2p = f2_make(wc2n[i], wc2n[i + 1]);
                        const F2 g1 = gate2_pair(cprev, wc1p, u1, f2_make(b1n[i], b1n[i + 1]), half);
                        const F2 g2 = gate2_pair(cprev, wc2p, u2, f2_make(b2n[i], b2n[i + 1]), half);
                        const F2 dc = f2_sub(cprev, u0);
                        const F2 cv = f2_fma(dc, g1, u0);
                        const F2 ghm = f2_mul(gh, f2_make(mk[i], mk[i + 1]));
                        const F2 curp = f2_make(cur[i], cur[i + 1]);
                        const F2 gc = f2_fma(ghm, g2, curp);
                        const F2 omg1 = f2_sub(one, g1), omg2 = f2_sub(one, g2);
                        F2 gg2 = f2_mul(f2_mul(ghm, f2_sub(cv, xv)), f2_mul(g2, omg2));
                        F2 gg1 = f2_mul(f2_mul(gc, dc), f2_mul(g1, omg1));
                        F2 gu0 = f2_mul(gc, omg1);
                        F2 gxv = f2_sub(gh, f2_mul(ghm, g2));
                        const F2 curn = f2_fma(gc, g1, f2_mul(unfold, f2_fma(gg1, wc1p, f2_mul(gg2, wc2p))));
                        if (PAD) {
                            const F2 zero = f2_splat(0.f);
                            gg1 = f2_select(pad, zero, gg1); gg2 = f2_select(pad, zero, gg2);
                            gu0 = f2_select(pad, zero, gu0); gxv = f2_select(pad, zero, gxv);
                        }
                        float a0, a1;
                        f2_split(f2_select(pad, curp, curn), a0, a1);
                        cur[i] = a0; cur[i + 1] = a1;
                        f2_split(f2_add(f2_make(gb1[i], gb1[i + 1]), gg1), a0, a1);
                        gb1[i] = a0; gb1[i + 1] = a1;
                        f2_split(f2_add(f2_make(gb2[i], gb2[i + 1]), gg2), a0, a1);
                        gb2[i] = a0; gb2[i + 1] = a1;
                        f2_split(f2_fma(gg1, cprev, f2_make(gwc1[i], gwc1[i + 1])), a0, a1);
                        gwc1[i] = a0; gwc1[i + 1] = a1;
                        f2_split(f2_fma(gg2, cprev, f2_make(gwc2[i], gwc2[i + 1])), a0, a1);
                        gwc2[i] = a0; gwc2[i + 1] = a1;
                        f2_split(gu0, guv[i * K + 0], guv[(i + 1) * K + 0]);
                        f2_split(gg1, guv[i * K + 1], guv[(i + 1) * K + 1]);
                        f2_split(gg2, guv[i * K + 2], guv[(i + 1) * K + 2]);
                        if (K == 4) f2_split(gxv, guv[i * K + K - 1], guv[(i + 1) * K + K - 1]);
                        f2_split(f2_mul(gxv, scale2), gxv_[i], gxv_[i + 1]);
                    }
                } else {
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    const float u0 = Cvt<T>::to_f(up.v[i * K + 0]);
                    const float u1 = Cvt<T>::to_f(up.v[i * K + 1]);
                    const float u2 = Cvt<T>::to_f(up.v[i * K + 2]);
                    const float xv = (K == 4) ? Cvt<T>::to_f(up.v[i * K + K - 1]) : Cvt<T>::to_f(xp.v[i]) * scale;
                    const float cprev = at_start ? c0[i] : Cvt<TC>::to_f(cpp.v[i]);
                    const float gh = Cvt<T>::to_f(ghp.v[i]);
                    float omg1, omg2;   // 1 - g1, 1 - g2 (fp32 storage only)
                    const float g1 = G::eval_pair(cprev, wc1n[i], u1, b1n[i], &omg1);
                    const float g2 = G::eval_pair(cprev, wc2n[i], u2, b2n[i], &omg2);
                    const float dc = cprev - u0;
                    const float cv = fmaf(dc, g1, u0);
                    const float ghm = gh * mk[i];
                    const float gc = fmaf(ghm, g2, cur[i]);
                    // g(1-g) and gc(1-g1): from the exact complement for fp32 storage, one fused
                    // multiply-add each for 16-bit storage (whose rounding hides the difference)
                    const float dg1 = G::kPair ? g1 * omg1 : fmaf(-g1, g1, g1);
                    const float dg2 = G::kPair ? g2 * omg2 : fmaf(-g2, g2, g2);
                    float gg2 = ghm * (cv - xv) * dg2;
                    float gg1 = gc * dc * dg1;
                    float gu0 = G::kPair ? gc * omg1 : fmaf(-gc, g1, gc);
                    float gxv = fmaf(-ghm, g2, gh);
                    const float curn = fmaf(gc, g1, G::kUnfold * fmaf(gg1, wc1n[i], gg2 * wc2n[i]));
                    if (PAD) {
                        gg1 = pad ? 0.f : gg1; gg2 = pad ? 0.f : gg2; gu0 = pad ? 0.f : gu0; gxv = pad ? 0.f : gxv;
                    }
                    cur[i] = pad ? cur[i] : curn;
                    gb1[i] += gg1;
                    gb2[i] += gg2;
                    gwc1[i] = fmaf(gg1, cprev, gwc1[i]);
                    gwc2[i] = fmaf(gg2, cprev, gwc2[i]);
                    guv[i * K + 0] = gu0;
                    guv[i * K + 1] = gg1;
                    guv[i * K + 2] = gg2;
                    if (K == 4) guv[i * K + K - 1] = gxv;
                    gxv_[i] = gxv * scale;
                }
                }
                Pack<T, V * K> guo;
                pack_from_float(guo, guv);
                *reinterpret_cast<Pack<T, V * K> *>(gup) = guo;
                gup += ostep * K;
                if (has_x) {
                    Pack<T, V> gxo;
                    pack_from_float(gxo, gxv_);
                    *reinterpret_cast<Pack<T, V> *>(gxp) = gxo;
                    gxp += ostep;
                }
            }
        };

        auto run = [&](auto pad_c) {
            constexpr bool PADF = decltype(pad_c)::value;
            int s = 0;
            uint32_t ph = 0;
            int64_t m = 0;   // backward step of the next block
            for (int it = 0; it < nst; ++it) {
                if (!mbar_wait_bounded(bar_full + 8 * s, ph)) {
                    atomicExch(p.err, 4);
                    break;
                }
                const uint32_t sb = order_after_wait(smem_u32(stage0) + (uint32_t)s * stage_bytes);
                for (int q = 0; q < SS && m < L; q += kTS, m += kTS) {
                    if (active) {
                        const uint32_t pad_cur = PADF ? pad_word(sb + pad_off, q, SS, asc) : 0u;
                        const int slab = asc ? q : (SS - 1 - q);
                        const uint32_t ub = sb + u_off + slab * su, xb = sb + x_off + slab * sx;
                        const uint32_t cb = sb + c_off + slab * sc, gb = sb + g_off + slab * sg;
                        const int64_t left = L - m;   // steps left including this block
                        if (left > kTS) block(ub, xb, cb, gb, pad_cur, kTS, pad_c, BoolC<false>{});
                        else block(ub, xb, cb, gb, pad_cur, (int)left, pad_c, BoolC<true>{});
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_empty + 8 * s);
                if (++s == NS) { s = 0; ph ^= 1; }
            }
        };
        if (has_pad) run(BoolC<true>{}); else run(BoolC<false>{});

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
// Host side: tile selection, tensor maps and dispatch
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

static PFN_cuTensorMapEncodeTiled_v12000 scan_encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
    }
    return fn;
}

// 3-D map over a (L, B, row) tensor whose rows are row_bytes long, in 8-byte elements:
// dims (row_bytes/8, B, L), box (box_bytes/8, br, ss), no swizzle, out-of-range reads give zeros.
static int make_scan_map(CUtensorMap *map, const void *base, int64_t row_bytes, int64_t B, int64_t L,
                         int64_t box_bytes, int br, int ss) {
    auto fn = scan_encode_fn();
    if (!fn) return set_error(SRU_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
    cuuint64_t dims[3] = {(cuuint64_t)(row_bytes / 8), (cuuint64_t)B, (cuuint64_t)L};
    cuuint64_t strides[2] = {(cuuint64_t)row_bytes, (cuuint64_t)(row_bytes * B)};
    cuuint32_t box[3] = {(cuuint32_t)(box_bytes / 8), (cuuint32_t)br, (cuuint32_t)ss};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(SRU_ERR_CUDA, "cuTensorMapEncodeTiled (scan) failed with %d", (int)r);
    return 0;
}

// Chooses V, the tile and the ring.  Returns false when the shape is not eligible.
// split: geometry for the split-role forward kernel (scan_split.cu): at most two columns per thread, a second
// set of consumer warps, and a float per column-step of shared memory in every stage for the states.
static bool choose_tile(int64_t L, int64_t B, int64_t d, int dirs, int k, int skip_type, int dtype,
                        int c_dtype, bool backward, bool has_pad, bool split, TileCfg *out) {
    const int s = (int)dtype_size(dtype);
    if (dtype == SRU_F64 || s == 0) return false;
    const int granule = 16 / s;  // elements per 16 bytes
    if (d % granule != 0 || L < 1 || B < 1 || L > 0x7fffff00 || B > 0x7fffffff) return false;
    const int64_t D = d * dirs, ncols = B * D;
    const int sms = num_sms();
    const int vmax = 4, vmin = 1;
    // Columns per thread (V) and consumer threads per CTA, from sweeps on B200 keyed by w = warps of
    // columns per SM.  Plenty of warps: V = 4 (8 bytes of every tensor per thread and step) amortises
    // the per-step overhead best.  Few warps: each warp is alone on its scheduler and bound by the
    // latency of its own instruction stream, so narrower threads (more warps) win, down to V = 1.
    // The backward, with twice the reads per step, moves to fatter CTAs earlier; fp32 columns carry
    // twice the bytes, so their V is about half.  V = 8 never won anywhere.
    const int64_t w = ncols / (32 * (int64_t)sms);
    int v, ntc;
    if (s == 2) {
        if (!backward) {
            if (w >= 20) { v = 4; ntc = (w >= 40 && w < 80) ? 128 : 64; }
            else if (w >= 10) { v = has_pad ? 2 : 4; ntc = has_pad ? 64 : 128; }
            else if (w >= 5) { v = 1; ntc = 64; }
            else { v = 1; ntc = 128; }
        } else {
            if (w >= 80) { v = 4; ntc = 64; }
            else if (w >= 40) { v = 2; ntc = 128; }
            else if (w >= 20) { v = 4; ntc = 128; }
            else if (w >= 10) { v = has_pad ? 2 : 4; ntc = has_pad ? 64 : 128; }
            else { v = 1; ntc = 64; }
        }
    } else {
        if (!backward) { v = (w >= 20) ? 2 : 1; ntc = 128; }
        else if (w >= 80) { v = 2; ntc = 64; }
        else if (w >= 20) { v = 4; ntc = 64; }
        else { v = 2; ntc = 128; }
    }
    while (ntc > 32 && ncols / ((int64_t)v * ntc) < (int64_t)sms / 2) ntc /= 2;   // tiny problems: spread over the SMs
    if (split) {
        // measured on B200 (16-bit storage): one column per thread and two chain warps per CTA below ten column-warps
        // per SM (16 K columns: 0.65 of the HBM peak against 0.43 for the one-role kernel), two columns and four chain
        // warps from there on (64 K columns: 0.73-0.86 against 0.67-0.72)
        if (w < 10) { v = 1; ntc = 64; } else { v = 2; ntc = 128; }
    }
    v = option(backward ? OPT_BWD_V : OPT_FWD_V, v);
    if (v < vmin || v > (split ? 2 : vmax) || (v & (v - 1))) return false;
    ntc = option(OPT_SCAN_THREADS, ntc);
    ntc = option(backward ? OPT_BWD_THREADS : OPT_FWD_THREADS, ntc);
    if (ntc < 32 || ntc > 128 || ntc % 32) return false;
    // hidden width of the tile: largest divisor of d, multiple of the granule, <= v*ntc, and with a
    // U slab of at most 2048 bytes (256 eight-byte elements, the widest box the tensor map takes)
    int hw = 0;
    for (int64_t cand = (int64_t)v * ntc; cand >= granule; cand -= granule) {
        if (d % cand == 0 && cand * k * s <= 2048) { hw = (int)cand; break; }
    }
    if (hw == 0) return false;
    const int tpr = hw / v;
    int br = (int)std::min<int64_t>(B, std::max(1, ntc / tpr));
    if (has_pad) br = std::min(br, 32 * kPadPerLane / kTS);   // the producer warp stages rows x steps <= 256 flags
    const int cthreads = ((br * tpr + 31) / 32) * 32;
    if (cthreads > 128) return false;
    const bool has_x = (k == 3 && skip_type == 1);
    const int sc = (int)dtype_size(c_dtype);
    size_t per_row_step = (size_t)hw * (k * s + (has_x ? s : 0));
    if (backward) per_row_step += (size_t)hw * (sc + s);
    if (split) per_row_step += (size_t)hw * sizeof(float);
    const int cta_threads = (split ? 2 : 1) * cthreads + 32;
    const size_t bar_bytes = split ? kSplitBarBytes : kBarBytes;
    // time steps per stage: one request should carry about 16 KB (fewer barrier round trips per
    // step), as long as three stages still fit the CTA's share of shared memory
    const int64_t nctas0 = ((B + br - 1) / br) * (D / hw);
    const int cps0 = (int)std::min<int64_t>(std::max<int64_t>(1, (nctas0 + sms - 1) / sms), 2048 / cta_threads);
    const size_t ring0 = std::min<size_t>(200 * 1024 / cps0, 96 * 1024);
    int ss = kTS;
    while (ss < 32 && (size_t)ss * br * per_row_step < 16 * 1024 && (size_t)(2 * ss) * br * per_row_step * 3 <= ring0) ss *= 2;
    ss = option(OPT_SCAN_SS, ss);
    if (ss < kTS || ss > 64 || ss % kTS) return false;
    while (has_pad && br * ss > 32 * kPadPerLane) ss -= kTS;
    auto stage_size = [&](int steps) {
        size_t t = align128((uint32_t)(steps * br * hw * k * s)) + align128((uint32_t)(has_x ? steps * br * hw * s : 0));
        if (backward) t += align128((uint32_t)(steps * br * hw * sc)) + align128((uint32_t)(steps * br * hw * s));
        if (split) t += align128((uint32_t)(steps * br * hw * sizeof(float)));
        if (has_pad) t += align128((uint32_t)(steps * br));
        return t;
    };
    // forced or derived, a stage length that leaves no room for two stages is shortened rather than refused
    while (ss > kTS && bar_bytes + 2 * stage_size(ss) > 227 * 1024) ss -= kTS;
    const size_t stage_bytes = stage_size(ss);
    // ring: shared by the CTAs expected on one SM
    const int64_t nctas = ((B + br - 1) / br) * (D / hw);
    int cta_per_sm = (int)std::min<int64_t>(std::max<int64_t>(1, (nctas + sms - 1) / sms), 2048 / cta_threads);
    size_t ring = std::min<size_t>(200 * 1024 / cta_per_sm, 96 * 1024);
    int ns = (int)(ring / stage_bytes);
    ns = std::max(2, std::min(ns, kMaxStages));
    ns = option(OPT_SCAN_STAGES, ns);
    ns = std::max(2, std::min(ns, kMaxStages));
    size_t smem = bar_bytes + (size_t)ns * stage_bytes;
    if (backward) smem = std::max(smem, bar_bytes + (size_t)br * 4 * hw * sizeof(float));
    if (smem > 227 * 1024) {
        ns = (int)((227 * 1024 - bar_bytes) / stage_bytes);
        if (ns < 2) return false;
        smem = bar_bytes + (size_t)ns * stage_bytes;
    }
    out->hw = hw; out->br = br; out->tpr = tpr;
    out->nht = (int)(D / hw); out->nrt = (int)((B + br - 1) / br);
    out->nstages = ns; out->ss = ss; out->v = v;
    out->threads = cta_threads; out->smem = smem;
    return nctas <= 0x7fffffff;
}

static bool pipelined_eligible(const ScanArgs &a) {
    if (a.is_custom || a.activation_type != 0) return false;
    if (a.k == 3 && a.skip_type != 1) return false;   // k = 3 without a highway term: generic kernel
    if (a.k == 4 && a.skip_type != 2) return false;
    if (a.dtype == SRU_F64) return false;
    if (option(OPT_FORCE_GENERIC, 0)) return false;
    return true;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

size_t pipelined_workspace_bytes(int64_t L, int64_t B, int64_t d, int dirs, int k, int dtype) {
    (void)L; (void)k; (void)dtype;
    return (size_t)B * 4 * d * dirs * sizeof(float);  // upper bound: one row per tile
}

template <typename T, typename TC, int V, int K>
static int launch_t(const ScanMaps &maps, const PipeArgs &p, bool backward, cudaStream_t st) {
    auto fwd = scan_fwd_pipe<T, TC, V, K>;
    auto bwd = scan_bwd_pipe<T, TC, V, K>;
    // the opt-in to more than 48 KB of dynamic shared memory is made once per kernel instance and device
    static bool opted[2][64] = {{false}};
    int dev = 0;
    SRUB_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return set_error(SRU_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    if (!opted[backward ? 1 : 0][dev]) {
        const void *fn = backward ? (const void *)bwd : (const void *)fwd;
        SRUB_CUDA_CHECK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        opted[backward ? 1 : 0][dev] = true;
    }
    const unsigned grid = (unsigned)((int64_t)p.c.nht * p.c.nrt);
    if (backward) bwd<<<grid, p.c.threads, p.c.smem, st>>>(maps, p);
    else fwd<<<grid, p.c.threads, p.c.smem, st>>>(maps, p);
    SRUB_CUDA_CHECK(cudaGetLastError());
    return 1;
}

template <typename T, typename TC, int K>
static int launch_v(const ScanMaps &maps, const PipeArgs &p, bool backward, cudaStream_t st) {
    switch (p.c.v) {
        case 1: return launch_t<T, TC, 1, K>(maps, p, backward, st);
        case 2: return launch_t<T, TC, 2, K>(maps, p, backward, st);
        case 4: return launch_t<T, TC, 4, K>(maps, p, backward, st);
    }
    return set_error(SRU_ERR_UNSUPPORTED, "columns per thread %d", p.c.v);
}

template <typename T, typename TC>
static int launch_k(const ScanMaps &maps, const PipeArgs &p, bool backward, cudaStream_t st) {
    return p.a.k == 3 ? launch_v<T, TC, 3>(maps, p, backward, st) : launch_v<T, TC, 4>(maps, p, backward, st);
}

int launch_scan_pipelined(const ScanArgs &a, bool backward, cudaStream_t st) {
    if (!pipelined_eligible(a)) return 0;
    // tensor maps need 16-byte aligned bases; packed stores need V*sizeof(T) alignment
    const void *ptrs[] = {a.u, a.x, a.h, a.c_hist, a.grad_h, a.grad_u, a.grad_x, a.c_last, a.c_init,
                          a.grad_last, a.grad_init, a.mask_c};
    for (const void *q : ptrs)
        if (q && !aligned16(q)) return 0;
    int *err = device_error_flag();
    if (!err) return set_error(SRU_ERR_CUDA, "device error flag unavailable");
    PipeArgs p;
    p.a = a;
    // Forward problems with few column-warps per SM go to the split-role kernel (option fwd_split: 1 always where
    // the shape allows, 0 never).
    bool split = false;
    if (!backward) {
        const int forced = option(OPT_FWD_SPLIT, -1);
        const int64_t w = a.B * (int64_t)a.d * a.dirs / (32 * (int64_t)num_sms());
        // By default (measured inside the benchmark steps, both kernels on one box): 16-bit storage, k = 3, and either
        // fewer than ten column-warps per SM (16 K columns: 0.62 of the HBM peak against 0.42 for the one-role kernel)
        // or fewer than twenty without a pad mask (64 K columns, 2048 wide: 0.86 against 0.70).  With a pad mask at
        // 64 K columns the one-role kernel is ahead (0.81 against 0.66), with more warps it hides its latencies by
        // itself (0.74 against 0.47 at 28 warps), and the k = 4 form was slower at every size.
        split = forced < 0 ? (a.k == 3 && dtype_size(a.dtype) == 2 && (w < 10 || (w < 20 && a.mask_pad == nullptr)))
                           : (forced != 0);
        if (split && !choose_tile(a.L, a.B, a.d, a.dirs, a.k, a.skip_type, a.dtype, a.c_dtype, false,
                                  a.mask_pad != nullptr, true, &p.c))
            split = false;
    }
    if (!split && !choose_tile(a.L, a.B, a.d, a.dirs, a.k, a.skip_type, a.dtype, a.c_dtype, backward,
                               a.mask_pad != nullptr, false, &p.c))
        return 0;
    p.err = err;

    // the tensor-map encoder is a driver entry point: this thread needs the primary context
    if (int rc = ensure_context()) return rc;
    const int64_t s = (int64_t)dtype_size(a.dtype), sc = (int64_t)dtype_size(a.c_dtype);
    const int64_t D = (int64_t)a.d * a.dirs;
    ScanMaps maps;
    memset(&maps, 0, sizeof(maps));
    int rc = make_scan_map(&maps.u, a.u, D * a.k * s, a.B, a.L, (int64_t)p.c.hw * a.k * s, p.c.br, p.c.ss);
    if (rc) return rc;
    if (a.k == 3) {
        rc = make_scan_map(&maps.x, a.x, D * s, a.B, a.L, (int64_t)p.c.hw * s, p.c.br, p.c.ss);
        if (rc) return rc;
    }
    if (backward) {
        rc = make_scan_map(&maps.c, a.c_hist, D * sc, a.B, a.L, (int64_t)p.c.hw * sc, p.c.br, p.c.ss);
        if (rc) return rc;
        rc = make_scan_map(&maps.g, a.grad_h, D * s, a.B, a.L, (int64_t)p.c.hw * s, p.c.br, p.c.ss);
        if (rc) return rc;
    }

    if (split) {
        rc = launch_scan_split(maps, p, st);
        if (rc < 0) return rc;
        note_scan_kernel(SCAN_KERNEL_SPLIT);
        return 1;
    }
    const int dt = a.dtype, ct = a.c_dtype;
    if (dt == SRU_F32 && ct == SRU_F32) rc = launch_k<float, float>(maps, p, backward, st);
    else if (dt == SRU_F16 && ct == SRU_F16) rc = launch_k<__half, __half>(maps, p, backward, st);
    else if (dt == SRU_F16 && ct == SRU_F32) rc = launch_k<__half, float>(maps, p, backward, st);
    else if (dt == SRU_BF16 && ct == SRU_BF16) rc = launch_k<__nv_bfloat16, __nv_bfloat16>(maps, p, backward, st);
    else if (dt == SRU_BF16 && ct == SRU_F32) rc = launch_k<__nv_bfloat16, float>(maps, p, backward, st);
    else return set_error(SRU_ERR_UNSUPPORTED, "dtype %d with c_dtype %d", dt, ct);
    if (rc < 0) return rc;
    if (backward) {
        const int r2 = launch_reduce_partials<float>(a.workspace, a.grad_wc, a.grad_bias, p.c.nrt,
                                                     (int64_t)a.d * a.dirs, 1, st);
        if (r2 < 0) return r2;
    }
    note_scan_kernel(SCAN_KERNEL_PIPELINED);
    return 1;
}

}  // namespace srub
