// Forward scan with split roles, for problems with few columns (sm_100a).
//
// The pipelined forward kernel (scan_pipelined.cu) gives each column to one thread that does everything
// for a time step.  Only a small part of that work is truly serial in time:
//
//     g1 = s(u1 + wc1*c' + b1),   c = (c' - u0)*g1 + u0                      (the state chain)
//
// while the reset gate, the output, its conversion and the stores need c' and c but feed nothing back:
//
//     g2 = s(u2 + wc2*c' + b2),   h = (c - x')*m*g2 + x'                      (the output work)
//
// With many columns per SM the scheduler hides one warp's dependent chain behind other warps.  With few
// (long-sequence inference at small batch: 16 K columns are 3.5 warps per SM, less than one per scheduler)
// a warp is alone, and its step costs the chain's latency PLUS the issue slots of everything else in the
// same instruction stream.  Here a column belongs to a PAIR of threads in two different warps:
//
//   chain warps     read u0, u1 from the stage, advance c, and leave c_t (fp32) in a per-stage buffer in
//                   shared memory -- about a dozen instructions around a ~30-cycle dependent chain;
//   follower warps  one stage behind, read u2 (u3), x, the flags and the c_t of the whole stage, and do the
//                   reset gate, the output arithmetic and all global stores (h, the state history);
//   producer warp   as in the pipelined kernel: one TMA box per tensor and stage, pad flags staged one
//                   stage ahead.
//
// Both roles are written block-wise over kTS = 4 time steps: a block's loads and conversions first, then the
// arithmetic of the four steps side by side (the follower's steps are independent of each other; the chain's are
// serial only through c), then the block's stores.  A warp that issues in order thus has four independent
// instruction streams to overlap, instead of one step's dependent latency after the other.  The states travel
// from chain to follower as one 16-byte vector per column and block.
//
// Synchronisation per ring stage: full[s] (TMA bytes + pad flags -> chain and follower), cready[s][w]
// (chain warp w -> follower warp w: the stage's c values are in shared memory), empty[s] (followers ->
// producer).  The chain never waits for a follower directly; it runs ahead by up to the ring depth.
// Every wait is bounded; a timeout raises the device error flag and the thread drains to the end.
//
// Arithmetic, tile geometry, tensor maps and outputs are those of scan_fwd_pipe; results are bit-identical
// to it (same operations in the same order per column).
#include <cudaTypedefs.h>

#include "scan_pipe_common.cuh"

namespace srub {

constexpr int kSplitMaxChainWarps = 4;

template <typename T, typename TC, int V, int K>
__global__ void __launch_bounds__(288) scan_fwd_split(const __grid_constant__ ScanMaps maps, const PipeArgs p) {
    extern __shared__ __align__(128) uint8_t smem[];
    using G = GateFor<T>;
    const ScanArgs &a = p.a;
    const int HW = p.c.hw, BR = p.c.br, TPR = p.c.tpr, NS = p.c.nstages, SS = p.c.ss;
    const int tid = threadIdx.x;
    const int nthr_c = (blockDim.x - 32) / 2;      // chain threads = follower threads
    const int nwarp_c = nthr_c / 32;
    const int lane = tid & 31;
    constexpr bool has_x = (K == 3);
    const int64_t D = (int64_t)a.d * a.dirs;
    const int ht = blockIdx.x % p.c.nht, rt = blockIdx.x / p.c.nht;
    const int64_t dj0 = (int64_t)ht * HW;
    const int dir = (int)(dj0 / a.d);
    const bool asc = (dir == 0);
    const int64_t b0 = (int64_t)rt * BR;
    const int nrows = (int)min((int64_t)BR, a.B - b0);
    const int64_t L = a.L;
    const int nst = (int)((L + SS - 1) / SS);

    // barriers: full[16] | empty[16] | cready[16][4]
    const uint32_t bar_full = smem_u32(smem);
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;
    const uint32_t bar_cready = bar_empty + 8 * kMaxStages;
    const uint32_t u_slab = (uint32_t)HW * K * sizeof(T);
    const uint32_t x_slab = has_x ? (uint32_t)HW * sizeof(T) : 0;
    const uint32_t c_slab = (uint32_t)HW * sizeof(float);
    const uint32_t u_region = align128(SS * BR * u_slab);
    const uint32_t x_region = align128(SS * BR * x_slab);
    const uint32_t c_region = align128(SS * BR * c_slab);
    const bool has_pad = a.mask_pad != nullptr;
    const uint32_t pad_region = has_pad ? align128(SS * BR) : 0;
    const uint32_t stage_bytes = u_region + x_region + c_region + pad_region;
    uint8_t *stage0 = smem + kSplitBarBytes;

    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(bar_full + 8 * s, has_pad ? 2 : 1);
            mbar_init(bar_empty + 8 * s, nwarp_c);
            for (int w = 0; w < kSplitMaxChainWarps; ++w) mbar_init(bar_cready + 8 * (s * kSplitMaxChainWarps + w), 1);
        }
        fence_mbar_init();
    }
    __syncthreads();

    if (tid >= 2 * nthr_c) {
        // ------------------------------------ producer warp ------------------------------------
        const int xu = (int)(dj0 * K * sizeof(T) / 8), xx = (int)(dj0 * sizeof(T) / 8);
        PadStager pads(a.mask_pad, a.B, L, b0, BR, SS, lane);
        auto first_time = [&](int it) { return asc ? it * SS : (int)(L - (int64_t)(it + 1) * SS); };
        if (has_pad) pads.fetch(first_time(0));
        int s = 0;
        uint32_t ph = 1;
        for (int it = 0; it < nst; ++it) {
            int ok = (lane == 0) ? (int)mbar_wait_bounded(bar_empty + 8 * s, ph) : 1;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { if (lane == 0) atomicExch(p.err, 5); break; }
            const uint32_t bar = bar_full + 8 * s;
            const uint32_t sbase = smem_u32(stage0) + (uint32_t)s * stage_bytes;
            if (lane == 0) {
                const int t0 = first_time(it);
                mbar_arrive_expect_tx(bar, (uint32_t)SS * BR * (u_slab + x_slab));
                tma_load_3d(sbase, &maps.u, bar, xu, (int)b0, t0);
                if (has_x) tma_load_3d(sbase + u_region, &maps.x, bar, xx, (int)b0, t0);
            }
            if (has_pad) {
                pads.store(sbase + u_region + x_region + c_region);
                if (it + 1 < nst) pads.fetch(first_time(it + 1));
                __syncwarp();
                if (lane == 0) mbar_arrive(bar);
            }
            if (++s == NS) { s = 0; ph ^= 1; }
        }
        return;
    }

    const bool chain = tid < nthr_c;
    const int ct = chain ? tid : tid - nthr_c;     // index of the column owner within its role
    const int cw = ct >> 5;                        // warp pair
    const int r = ct / TPR;
    const int hc = (ct - r * TPR) * V;
    const bool active = (ct < BR * TPR) && (r < nrows);
    const int64_t b = b0 + (active ? r : 0);
    // threads without a column (tile edge, rows past the batch) run the same instruction stream on the first
    // column's slots of the stage and store nothing, so that the loops need no per-thread branch
    const int ro = active ? r : 0, ho_ = active ? hc : 0;
    const int64_t col = b * D + dj0 + hc;
    const int su = BR * (int)u_slab, sx = BR * (int)x_slab;      // bytes between time slabs
    const int sc4 = BR * (int)c_slab * kTS;                      // bytes between blocks of four steps in the state buffer
    const uint32_t u_off = ro * u_slab + ho_ * K * sizeof(T);
    const uint32_t x_off = u_region + ro * x_slab + ho_ * sizeof(T);
    const uint32_t c_off = u_region + x_region + (ro * HW + ho_) * kTS * sizeof(float);   // [block][row][column][step]
    const uint32_t pad_off = u_region + x_region + c_region + ro * SS;

    float c[V];
#pragma unroll
    for (int i = 0; i < V; ++i) c[i] = (active && a.c_init) ? ((const float *)a.c_init)[col + i] : 0.f;

    if (chain) {
        // ------------------------------------ chain warps ------------------------------------
        float wc1n[V], b1n[V];
#pragma unroll
        for (int i = 0; i < V; ++i) {
            wc1n[i] = 0.f; b1n[i] = 0.f;
            if (active) {
                const int64_t dj = dj0 + hc + i;
                wc1n[i] = G::fold(((const float *)a.weight_c)[dj]);
                if (a.bias) b1n[i] = G::fold(((const float *)a.bias)[dj]);
            }
        }
        // Running shared-memory addresses: `ua` points at this thread's group in the slab of the block's first step,
        // the next step's slab is dsu bytes further in scan order (negative for tiles that walk time downwards).
        const int dsu = asc ? su : -su;
        const uint32_t first_u = u_off + (asc ? 0u : (uint32_t)((SS - 1) * su));
        const uint32_t first_p = pad_off + (asc ? 0u : (uint32_t)(SS - kTS));
        const int dpa = asc ? kTS : -kTS;
        // one step of the chain for all V columns; returns nothing, updates c
        auto step = [&](uint32_t ua, bool pad, float (&cs)[V][kTS], int ts) {
#pragma unroll
            for (int i = 0; i < V; ++i) {
                // u0 and u1 come first in the gate-innermost group of a column (single-element loads: a group starts
                // on an element boundary only)
                const float u0 = Cvt<T>::to_f(lds_pack<Pack<T, 1>>(ua + i * K * sizeof(T)).v[0]);
                const float u1 = Cvt<T>::to_f(lds_pack<Pack<T, 1>>(ua + i * K * sizeof(T) + sizeof(T)).v[0]);
                const float g1 = G::eval(c[i], wc1n[i], u1, b1n[i]);
                const float cn = fmaf(c[i] - u0, g1, u0);
                c[i] = pad ? c[i] : cn;
                cs[i][ts] = c[i];
            }
        };
        auto run = [&](auto pad_c) {
            constexpr bool PADF = decltype(pad_c)::value;
            int s = 0;
            uint32_t ph = 0;
            int64_t n = 0;
            for (int it = 0; it < nst; ++it) {
                if (!mbar_wait_bounded(bar_full + 8 * s, ph)) { atomicExch(p.err, 6); break; }
                const uint32_t sb = order_after_wait(smem_u32(stage0) + (uint32_t)s * stage_bytes);
                const int steps_here = (int)min((int64_t)SS, L - n);
                const int nfull = steps_here / kTS, rem = steps_here - nfull * kTS;
                uint32_t ua = sb + first_u, ca = sb + c_off, pa = sb + first_p;
#pragma unroll 1
                for (int blk = 0; blk < nfull; ++blk) {
                    uint32_t pad_bits = 0u;
                    if (PADF) {
                        asm("ld.shared.u32 %0, [%1];" : "=r"(pad_bits) : "r"(pa));
                        if (!asc) pad_bits = __byte_perm(pad_bits, 0, 0x0123);
                    }
                    float cs[V][kTS];
#pragma unroll
                    for (int ts = 0; ts < kTS; ++ts) step(ua + ts * dsu, PADF && ((pad_bits >> (8 * ts)) & 0xffu), cs, ts);
                    if (active) {
#pragma unroll
                        for (int i = 0; i < V; ++i)
                            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(ca + i * 16), "f"(cs[i][0]),
                                         "f"(cs[i][1]), "f"(cs[i][2]), "f"(cs[i][3]) : "memory");
                    }
                    ua += kTS * dsu; ca += sc4; pa += dpa;
                }
                if (rem > 0) {      // the sequence's last, short block
                    uint32_t pad_bits = 0u;
                    if (PADF) {
                        asm("ld.shared.u32 %0, [%1];" : "=r"(pad_bits) : "r"(pa));
                        if (!asc) pad_bits = __byte_perm(pad_bits, 0, 0x0123);
                    }
                    float cs[V][kTS];
#pragma unroll
                    for (int ts = 0; ts < kTS; ++ts) {
#pragma unroll
                        for (int i = 0; i < V; ++i) cs[i][ts] = 0.f;
                    }
#pragma unroll
                    for (int ts = 0; ts < kTS - 1; ++ts)
                        if (ts < rem) step(ua + ts * dsu, PADF && ((pad_bits >> (8 * ts)) & 0xffu), cs, ts);
                    if (active) {
#pragma unroll
                        for (int i = 0; i < V; ++i)
                            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(ca + i * 16), "f"(cs[i][0]),
                                         "f"(cs[i][1]), "f"(cs[i][2]), "f"(cs[i][3]) : "memory");
                    }
                }
                n += steps_here;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_cready + 8 * (s * kSplitMaxChainWarps + cw));
                if (++s == NS) { s = 0; ph ^= 1; }
            }
        };
        if (has_pad) run(BoolC<true>{}); else run(BoolC<false>{});
        if (a.c_last && active) {
            Pack<float, V> cl;
#pragma unroll
            for (int i = 0; i < V; ++i) cl.v[i] = c[i];
            *reinterpret_cast<Pack<float, V> *>((float *)a.c_last + col) = cl;
        }
        return;
    }

    // -------------------------------------- follower warps --------------------------------------
    float wc2n[V], b2n[V], mk[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
        wc2n[i] = 0.f; b2n[i] = 0.f; mk[i] = 1.f;
        if (active) {
            const int64_t dj = dj0 + hc + i;
            wc2n[i] = G::fold(((const float *)a.weight_c)[D + dj]);
            if (a.bias) b2n[i] = G::fold(((const float *)a.bias)[D + dj]);
            if (a.mask_c) mk[i] = ((const float *)a.mask_c)[col + i];
        }
    }
    const float scale = (float)a.scale_x;
    const bool has_hist = a.c_hist != nullptr;
    const int64_t t_first = asc ? 0 : (L - 1);
    const int64_t ostep = asc ? (a.B * D) : -(a.B * D);
    T *hp = (T *)a.h + (t_first * a.B + b) * D + dj0 + hc;
    TC *cp = (TC *)a.c_hist + (has_hist ? (t_first * a.B + b) * D + dj0 + hc : 0);

    const int dsu = asc ? su : -su, dsx = asc ? sx : -sx;
    const uint32_t first_u = u_off + (asc ? 0u : (uint32_t)((SS - 1) * su));
    const uint32_t first_x = x_off + (asc ? 0u : (uint32_t)((SS - 1) * sx));
    const uint32_t first_p = pad_off + (asc ? 0u : (uint32_t)(SS - kTS));
    const int dpa = asc ? kTS : -kTS;
    // One block: `nsteps` (4, or fewer in the sequence's last block) steps side by side.  The reset gate of a step sees
    // the state before it: the previous step's entry of the chain's vector, or the carry from the previous block.
    auto block = [&](uint32_t ua, uint32_t xa, uint32_t ca, uint32_t pad_bits, int nsteps, auto pad_c, auto hist_c,
                     auto full_c) {
        constexpr bool PADF = decltype(pad_c)::value, HIST = decltype(hist_c)::value, FULL = decltype(full_c)::value;
        float cn[V][kTS];
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const Pack<float, 4> cv = lds_pack<Pack<float, 4>>(ca + i * 16);
#pragma unroll
            for (int ts = 0; ts < kTS; ++ts) cn[i][ts] = cv.v[ts];
        }
        float hv[kTS][V];
#pragma unroll
        for (int ts = 0; ts < kTS; ++ts) {
            const bool pad = PADF && ((pad_bits >> (8 * ts)) & 0xffu);
            Pack<T, V> xp;
            if (has_x) xp = lds_pack<Pack<T, V>>(xa + ts * dsx);
#pragma unroll
            for (int i = 0; i < V; ++i) {
                const uint32_t ug = ua + ts * dsu + i * K * sizeof(T);
                const float u2 = Cvt<T>::to_f(lds_pack<Pack<T, 1>>(ug + 2 * sizeof(T)).v[0]);
                float xv;
                if (K == 4) xv = Cvt<T>::to_f(lds_pack<Pack<T, 1>>(ug + 3 * sizeof(T)).v[0]);
                else xv = Cvt<T>::to_f(xp.v[i]) * scale;
                const float cprev = (ts == 0) ? c[i] : cn[i][ts - 1];
                const float g2 = G::eval(cprev, wc2n[i], u2, b2n[i]);
                const float hn = fmaf((cn[i][ts] - xv) * mk[i], g2, xv);
                hv[ts][i] = pad ? 0.f : hn;
            }
        }
#pragma unroll
        for (int i = 0; i < V; ++i) c[i] = cn[i][kTS - 1];
        if (active) {
#pragma unroll
            for (int ts = 0; ts < kTS; ++ts) {
                if (FULL || ts < nsteps) {
                    Pack<T, V> ho;
                    pack_from_float(ho, hv[ts]);
                    stg_pack(hp + ts * ostep, ho);
                    if (HIST) {
                        float cc[V];
#pragma unroll
                        for (int i = 0; i < V; ++i) cc[i] = cn[i][ts];
                        Pack<TC, V> co;
                        pack_from_float(co, cc);
                        stg_pack(cp + ts * ostep, co);
                    }
                }
            }
        }
        hp += kTS * ostep;
        if (HIST) cp += kTS * ostep;
    };
    auto run = [&](auto pad_c, auto hist_c) {
        constexpr bool PADF = decltype(pad_c)::value;
        int s = 0;
        uint32_t ph = 0;
        int64_t n = 0;
        for (int it = 0; it < nst; ++it) {
            // the chain's arrival implies the stage's copies have landed; waiting on full[s] as well makes this
            // thread an observer of the copies' own completion (it has long completed: one probe)
            if (!mbar_wait_bounded(bar_cready + 8 * (s * kSplitMaxChainWarps + cw), ph) ||
                !mbar_wait_bounded(bar_full + 8 * s, ph)) {
                atomicExch(p.err, 7);
                break;
            }
            const uint32_t sb = order_after_wait(smem_u32(stage0) + (uint32_t)s * stage_bytes);
            const int steps_here = (int)min((int64_t)SS, L - n);
            const int nfull = steps_here / kTS, rem = steps_here - nfull * kTS;
            uint32_t ua = sb + first_u, xa = sb + first_x, ca = sb + c_off, pa = sb + first_p;
#pragma unroll 1
            for (int blk = 0; blk < nfull; ++blk) {
                uint32_t pad_bits = 0u;
                if (PADF) {
                    asm("ld.shared.u32 %0, [%1];" : "=r"(pad_bits) : "r"(pa));
                    if (!asc) pad_bits = __byte_perm(pad_bits, 0, 0x0123);
                }
                block(ua, xa, ca, pad_bits, kTS, pad_c, hist_c, BoolC<true>{});
                ua += kTS * dsu; xa += kTS * dsx; ca += sc4; pa += dpa;
            }
            if (rem > 0) {
                uint32_t pad_bits = 0u;
                if (PADF) {
                    asm("ld.shared.u32 %0, [%1];" : "=r"(pad_bits) : "r"(pa));
                    if (!asc) pad_bits = __byte_perm(pad_bits, 0, 0x0123);
                }
                block(ua, xa, ca, pad_bits, rem, pad_c, hist_c, BoolC<false>{});
            }
            n += steps_here;
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
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
template <typename T, typename TC, int V, int K>
static int launch_split_t(const ScanMaps &maps, const PipeArgs &p, cudaStream_t st) {
    auto fn = scan_fwd_split<T, TC, V, K>;
    static bool opted[64] = {false};
    int dev = 0;
    SRUB_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return set_error(SRU_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
    if (!opted[dev]) {
        SRUB_CUDA_CHECK(cudaFuncSetAttribute((const void *)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        opted[dev] = true;
    }
    const unsigned grid = (unsigned)((int64_t)p.c.nht * p.c.nrt);
    fn<<<grid, p.c.threads, p.c.smem, st>>>(maps, p);
    SRUB_CUDA_CHECK(cudaGetLastError());
    return 1;
}

template <typename T, typename TC>
static int launch_split_vk(const ScanMaps &maps, const PipeArgs &p, cudaStream_t st) {
    const int v = p.c.v, k = p.a.k;
    if (v == 1 && k == 3) return launch_split_t<T, TC, 1, 3>(maps, p, st);
    if (v == 1 && k == 4) return launch_split_t<T, TC, 1, 4>(maps, p, st);
    if (v == 2 && k == 3) return launch_split_t<T, TC, 2, 3>(maps, p, st);
    if (v == 2 && k == 4) return launch_split_t<T, TC, 2, 4>(maps, p, st);
    return set_error(SRU_ERR_UNSUPPORTED, "split forward scan: %d columns per thread", v);
}

int launch_scan_split(const ScanMaps &maps, const PipeArgs &p, cudaStream_t st) {
    const int dt = p.a.dtype, ct = p.a.c_dtype;
    if (dt == SRU_F32 && ct == SRU_F32) return launch_split_vk<float, float>(maps, p, st);
    if (dt == SRU_F16 && ct == SRU_F16) return launch_split_vk<__half, __half>(maps, p, st);
    if (dt == SRU_F16 && ct == SRU_F32) return launch_split_vk<__half, float>(maps, p, st);
    if (dt == SRU_BF16 && ct == SRU_BF16) return launch_split_vk<__nv_bfloat16, __nv_bfloat16>(maps, p, st);
    if (dt == SRU_BF16 && ct == SRU_F32) return launch_split_vk<__nv_bfloat16, float>(maps, p, st);
    return set_error(SRU_ERR_UNSUPPORTED, "dtype %d with c_dtype %d", dt, ct);
}

}  // namespace srub
