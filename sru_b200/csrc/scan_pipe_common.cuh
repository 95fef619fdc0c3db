// Pieces shared by the pipelined scan kernels: pipeline constants, the kernel argument block,
// gate evaluation, packed conversions and the producer's copy-slot bookkeeping.
#pragma once
#include <cuda.h>

#include <type_traits>

#include "f32x2.cuh"
#include "scan.cuh"

namespace srub {

constexpr int kTS = 4;            // time steps per pipeline stage
constexpr int kBarBytes = 256;    // room for 2 * 16 mbarriers at the start of shared memory
constexpr int kMaxStages = 16;
constexpr int kSplitBarBytes = 768;  // split-role forward: full[16], empty[16], chain-ready[16][4]

struct PipeArgs {
    ScanArgs a;
    TileCfg c;
    int *err;
};

__device__ __forceinline__ float tanh_approx(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Gate evaluation s(u + wc*c + b).
//  MODE 0 (fp32 storage): the reference's own expression 1/(1+expf(-z)) with full-precision
//         expf and IEEE division, so fp32 results stay within 1e-5 of an fp32 CPU run.
//  MODE 1: -log2(e) folded into wc and b once per column, ex2.approx + rcp.approx.
//  MODE 2 (16-bit storage): s(z) = 0.5*tanh(z/2) + 0.5 with 1/2 folded into wc and b and one
//         tanh.approx per gate: half the special-function work and the shortest serial chain
//         (fma -> tanh -> fma).  Its absolute error (about 3e-4) is below bf16 / fp16 output
//         rounding and inside the 2e-2 bar of the 16-bit modes.
template <int MODE> struct Gate {
    static __device__ __forceinline__ float fold(float v) {
        return MODE == 0 ? v : (MODE == 1 ? v * kNegLog2e : v * 0.5f);
    }
    // multiplies (gg1*wc1f + gg2*wc2f) back to (gg1*wc1 + gg2*wc2)
    static constexpr float kUnfold = MODE == 0 ? 1.f : (MODE == 1 ? -0.6931471805599453f : 2.f);
    static __device__ __forceinline__ float eval(float c, float wcf, float u, float bf) {
        if (MODE == 0) {
            const float z = fmaf(wcf, c, u) + bf;
            return 1.f / (1.f + expf(-z));
        } else if (MODE == 1) {
            return rcp_approx(1.f + ex2_approx(fmaf(c, wcf, fmaf(u, kNegLog2e, bf))));
        } else {
            return fmaf(tanh_approx(fmaf(c, wcf, fmaf(u, 0.5f, bf))), 0.5f, 0.5f);
        }
    }
    // The gate and its complement 1 - g for the backward pass.  fp32 storage: both with full relative
    // accuracy (1 - g from the rounded g loses the digits g shares with 1; gradients are multiplied by it):
    // with a = exp(-|z|), r = 1/(1+a), the larger of the two is r and the smaller a*r.
    static __device__ __forceinline__ float eval_pair(float c, float wcf, float u, float bf, float *one_minus) {
        if (MODE == 0) {
            const float z = fmaf(wcf, c, u) + bf;
            const float a = expf(-fabsf(z));
            const float r = 1.f / (1.f + a), q = a * r;
            *one_minus = (z >= 0.f) ? q : r;
            return (z >= 0.f) ? r : q;
        } else {
            *one_minus = 0.f;   // not used: see kPair
            return eval(c, wcf, u, bf);
        }
    }
    static constexpr bool kPair = (MODE == 0);   // eval_pair delivers the complement
};
template <typename T> using GateFor = Gate<sizeof(T) == 4 ? 0 : 2>;

// The 16-bit-storage gate (MODE 2) on a pair of columns: 0.5 * tanh(c * wcf + (u * 0.5 + bf)) + 0.5 with the same
// four roundings per lane as Gate<2>::eval.
__device__ __forceinline__ F2 gate2_pair(F2 c, F2 wcf, F2 u, F2 bf, F2 half) {
    float lo, hi;
    f2_split(f2_fma(c, wcf, f2_fma(u, half, bf)), lo, hi);
    return f2_fma(f2_make(tanh_approx(lo), tanh_approx(hi)), half, half);
}

// float[N] -> Pack<T,N>, two values per conversion instruction for the 16-bit types.
template <typename T, int N> __device__ __forceinline__ void pack_from_float(Pack<T, N> &out, const float (&v)[N]) {
#pragma unroll
    for (int i = 0; i < N; ++i) out.v[i] = Cvt<T>::from_f(v[i]);
}
template <int N> __device__ __forceinline__ void pack_from_float(Pack<__nv_bfloat16, N> &out, const float (&v)[N]) {
    if constexpr (N % 2 == 0) {
#pragma unroll
        for (int i = 0; i < N; i += 2)
            *reinterpret_cast<__nv_bfloat162 *>(&out.v[i]) = __floats2bfloat162_rn(v[i], v[i + 1]);
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) out.v[i] = __float2bfloat16_rn(v[i]);
    }
}
template <int N> __device__ __forceinline__ void pack_from_float(Pack<__half, N> &out, const float (&v)[N]) {
    if constexpr (N % 2 == 0) {
#pragma unroll
        for (int i = 0; i < N; i += 2) *reinterpret_cast<__half2 *>(&out.v[i]) = __floats2half2_rn(v[i], v[i + 1]);
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) out.v[i] = __float2half_rn(v[i]);
    }
}

// Tensor maps of the streamed tensors (3-D: row bytes / 8, batch, time), built on the host per launch.
struct ScanMaps {
    CUtensorMap u, x, c, g;   // U (and grad-independent inputs): x, saved states c, grad_h
};

// One TMA request: a box of (inner bytes/8) x rows x time steps into this CTA's shared memory.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// Split-role forward kernel (scan_split.cu): launched by launch_scan_pipelined with the maps and tile it prepared.
int launch_scan_split(const ScanMaps &maps, const PipeArgs &p, cudaStream_t st);

__host__ __device__ __forceinline__ uint32_t align128(uint32_t v) { return (v + 127u) & ~127u; }

template <bool B> using BoolC = std::integral_constant<bool, B>;

// Reads a Pack from shared memory with explicit shared-space loads.  A read through a generic pointer is
// tracked like a global load (long scoreboard) and may not be moved across the global stores of the step
// before it; ld.shared is neither, which is what lets a lone warp overlap one step's reads with the
// previous step's dependent chain.  The asm is not volatile, so that the compiler too may move it over
// stores; what keeps it behind the mbarrier wait that guards the data is its address: the caller passes
// the stage base through order_after_wait() right after the wait.
__device__ __forceinline__ uint32_t order_after_wait(uint32_t addr) {
    asm volatile("" : "+r"(addr) : : "memory");
    return addr;
}
template <typename P> __device__ __forceinline__ P lds_pack(uint32_t addr) {
    constexpr int A = alignof(P), NB = sizeof(P);
    P out;
    if constexpr (A == 16) {
        uint4 *o = reinterpret_cast<uint4 *>(&out);
#pragma unroll
        for (int i = 0; i < NB / 16; ++i)
            asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(o[i].x), "=r"(o[i].y), "=r"(o[i].z), "=r"(o[i].w) : "r"(addr + 16 * i));
    } else if constexpr (A == 8) {
        uint2 *o = reinterpret_cast<uint2 *>(&out);
#pragma unroll
        for (int i = 0; i < NB / 8; ++i)
            asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(o[i].x), "=r"(o[i].y) : "r"(addr + 8 * i));
    } else if constexpr (A == 4) {
        uint32_t *o = reinterpret_cast<uint32_t *>(&out);
#pragma unroll
        for (int i = 0; i < NB / 4; ++i) asm("ld.shared.u32 %0, [%1];" : "=r"(o[i]) : "r"(addr + 4 * i));
    } else {
        uint16_t *o = reinterpret_cast<uint16_t *>(&out);
#pragma unroll
        for (int i = 0; i < NB / 2; ++i) asm("ld.shared.u16 %0, [%1];" : "=h"(o[i]) : "r"(addr + 2 * i));
    }
    return out;
}

// Writes a Pack to global memory with an explicit global-space store: ld.shared and st.global cannot alias, so the
// shared-memory loads of a later block may be scheduled above the stores of an earlier one (the split-role kernel's
// follower warps, which work block by block, rely on it; measured on the one-role kernels it made no difference).
template <typename P> __device__ __forceinline__ void stg_pack(void *gptr, const P &v) {
    const size_t a = __cvta_generic_to_global(gptr);
    constexpr int A = alignof(P), NB = sizeof(P);
    if constexpr (A == 16) {
        const uint4 *s = reinterpret_cast<const uint4 *>(&v);
#pragma unroll
        for (int i = 0; i < NB / 16; ++i)
            asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(a + 16 * i), "r"(s[i].x), "r"(s[i].y), "r"(s[i].z), "r"(s[i].w));
    } else if constexpr (A == 8) {
        const uint2 *s = reinterpret_cast<const uint2 *>(&v);
#pragma unroll
        for (int i = 0; i < NB / 8; ++i) asm volatile("st.global.v2.u32 [%0], {%1, %2};" ::"l"(a + 8 * i), "r"(s[i].x), "r"(s[i].y));
    } else if constexpr (A == 4) {
        const uint32_t *s = reinterpret_cast<const uint32_t *>(&v);
#pragma unroll
        for (int i = 0; i < NB / 4; ++i) asm volatile("st.global.u32 [%0], %1;" ::"l"(a + 4 * i), "r"(s[i]));
    } else {
        const uint16_t *s = reinterpret_cast<const uint16_t *>(&v);
#pragma unroll
        for (int i = 0; i < NB / 2; ++i) asm volatile("st.global.u16 [%0], %1;" ::"l"(a + 2 * i), "h"(s[i]));
    }
}

// ---------------------------------------------------------------------------------------
// Pad flags.  mask_pad is (L, B) bytes; a consumer needs one flag per step of its row.  Read from
// global memory by the consumer itself, each flag's latency lands in a warp that has nothing else to
// run while it waits, which halves the throughput of small problems.  Instead the 32 lanes of the
// producer warp read the flags of a whole stage (rows x steps) one stage ahead, keep them in
// registers across the wait for the stage to drain, and write them into the stage as [row][step]
// bytes before the stage's full barrier is armed; consumers then take four steps' flags with one
// shared-memory word.
// ---------------------------------------------------------------------------------------
constexpr int kPadPerLane = 8;                 // flags per lane and stage: rows x steps <= 256
struct PadStager {
    const uint8_t *mask;
    int64_t B, L, b0;
    int nflags, ss, lane;
    uint32_t v[kPadPerLane];
    __device__ __forceinline__ PadStager(const uint8_t *mask_, int64_t B_, int64_t L_, int64_t b0_, int br, int ss_, int lane_)
        : mask(mask_), B(B_), L(L_), b0(b0_), nflags(br * ss_), ss(ss_), lane(lane_) {}
    // requests the flags of the stage whose first time step is t0 (steps outside [0, L) and rows
    // past the batch read as 0)
    __device__ __forceinline__ void fetch(int t0) {
#pragma unroll
        for (int j = 0; j < kPadPerLane; ++j) {
            const int e = lane + 32 * j;
            const int rr = e / ss, st = e - rr * ss;
            const int64_t t = (int64_t)t0 + st;
            v[j] = 0;
            if (e < nflags && t >= 0 && t < L && b0 + rr < B) v[j] = mask[t * B + b0 + rr];
        }
    }
    __device__ __forceinline__ void store(uint32_t dst) const {
#pragma unroll
        for (int j = 0; j < kPadPerLane; ++j) {
            const int e = lane + 32 * j;
            if (e < nflags) {
                const uint16_t f = (uint16_t)(v[j] ? 1 : 0);
                asm volatile("st.shared.u8 [%0], %1;" : : "r"(dst + e), "h"(f) : "memory");
            }
        }
    }
};

// Flags of the four steps of the block that starts q steps into the stage: byte ts belongs to scan
// step ts.  row_flags is the shared address of this row's ss flags, stored in time order; a
// descending tile walks them from the end, so its word is byte-reversed.
__device__ __forceinline__ uint32_t pad_word(uint32_t row_flags, int q, int ss, bool asc) {
    uint32_t w;
    asm("ld.shared.u32 %0, [%1];" : "=r"(w) : "r"(row_flags + (asc ? q : ss - kTS - q)));
    return asc ? w : __byte_perm(w, 0, 0x0123);
}


}  // namespace srub
