// Dense 16-bit GEMM on the 5th-generation tensor cores (tcgen05) for sm_100a.
//
//   C[M,N] = op(A)[M,K] * op(B)[K,N] (+ col_bias[N]) (+ C),   fp32 accumulation in tensor memory.
//
// Two kernels share the pipeline below: a pair kernel (two SMs per 256x256 tile, cta_group::2,
// described further down; used whenever there are enough tiles to fill the GPU) and the
// single-CTA kernel described here (128x256 tiles; small problems).
//
// One persistent CTA per SM, 192 threads, warp-specialised:
//   warp 0     TMA producer: cp.async.bulk.tensor loads of 128B-swizzled A / B tiles into a
//              4-stage shared-memory ring, completion counted on "full" mbarriers;
//   warp 1     allocates tensor memory (512 columns = two 128x256 fp32 accumulators) and, with
//              one elected thread, issues tcgen05.mma (M=128, N=256, K=16 per instruction,
//              operands read straight from shared memory through matrix descriptors);
//              tcgen05.commit releases ring stages and publishes finished accumulators;
//   warps 2-5  epilogue: tcgen05.ld of the accumulator quarter each warp may address
//              (TMEM lanes 32*(warp%4)..), bias / accumulate, conversion, 16-byte stores.
// The two accumulators alternate between tiles, so the epilogue of tile i overlaps the MMAs
// of tile i+1.  Tile order keeps N fastest, so the CTAs that run concurrently share A row
// blocks and the whole B operand through L2.
//
// Operand layouts.  Both operands may be "K-major" (reduction index contiguous in memory) or
// "MN-major" (the M / N index contiguous); the three products of the SRU layer need
//   forward  U = x W           A K-major,  B MN-major
//   dgrad    gx = gU W^T       A K-major,  B K-major
//   wgrad    gW = x^T gU       A MN-major, B MN-major
// and none of them needs a transposed copy.  Shared-memory tiles are the canonical 128-byte
// swizzled layouts: K-major [rows][64 elements], 8-row groups 1024 B apart; MN-major slabs of
// [64 k-rows][64 elements], 8-row groups 1024 B apart, successive 64-element chunks of the
// M / N extent 8192 B apart.  Every load is issued by one CTA for its own shared memory.
//
// Every mbarrier wait is bounded; a wait that gives up raises the device error flag and the
// CTA drains to its teardown, where tensor memory is released.
#include <cudaTypedefs.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace srub {

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kAStage = BM * BK * 2;   // 16 KB
constexpr int kBStage = BN * BK * 2;   // 32 KB
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kSmemBytes = kStages * (kAStage + kBStage) + 1024 /*align*/ + 256 /*barriers*/;

struct GemmArgs {
    void *c;
    const float *bias;
    int64_t M, N, K, ldc;
    int c_dtype, accumulate;
    int a_mn, b_mn;   // 1: MN-major operand
    uint32_t idesc;
    int tiles_m, tiles_n;
    int raster_m;       // 1: consecutive tiles walk down M (column-major over the tile grid), 0: along N
    int ksplit, kbps;   // split-K: partial products over kbps k-blocks each go to slab sp of an fp32 workspace
    // Dynamic tile order (pair kernel): word 0 is the next-unit counter, then kSchedRing mailbox words per CTA pair.
    // NULL: static order (unit = pair, pair + pairs, ...).
    unsigned long long *sched;
    int epi_warps;      // pair kernel instance: 8 or 4 epilogue warps per CTA (host side only)
    int c_tma;          // pair kernel: 16-bit output leaves shared memory through tiled bulk stores (map_c is valid)
    int *err;
};

// ---- dynamic tile order ---------------------------------------------------------------------------------
// With a static order every CTA pair owns a fixed share of the tiles, so the product lasts as long as its slowest
// pair: when another kernel (a gradient all-reduce running next to backward) holds a few SMs for a while, the pairs
// on those SMs start late and everyone waits for them.  Here the leader CTA's producer thread takes the next unit
// from a global counter and posts it to the pair's mailbox ring; the other roles of both CTAs (the peer's producer,
// the MMA thread, the epilogue warps) read it there.  A mailbox word is (iteration << 32 | unit), so a stale word
// never matches; the ring (16 words) cannot be overrun because the barriers of the pipeline already keep the roles
// within a few tiles of each other (shared-memory stages, two accumulators) and the poster runs two units ahead.  The host fills counter and mailboxes with 0xFF bytes before the launch: the counter
// then yields 0, 1, 2, ... as old value + 1, and no mailbox matches iteration 0.
constexpr int kSchedRing = 16;
constexpr int kSchedMaxPairs = 128;
constexpr int kSchedWords = 1 + kSchedMaxPairs * kSchedRing;

__device__ __forceinline__ unsigned int sched_take(const GemmArgs &g) {
    return atomicAdd(reinterpret_cast<unsigned int *>(g.sched), 1u) + 1u;
}
__device__ __forceinline__ int sched_post(const GemmArgs &g, int pair, int it, unsigned int u, int nunits) {
    const int unit = (u < (unsigned int)nunits) ? (int)u : -1;
    const unsigned long long v = ((unsigned long long)(unsigned int)it << 32) | (unsigned int)unit;
    unsigned long long *slot = g.sched + 1 + pair * kSchedRing + (it % kSchedRing);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(slot), "l"(v) : "memory");   // the word is the whole message
    return unit;
}
__device__ __forceinline__ int sched_post_next(const GemmArgs &g, int pair, int it, int nunits) {
    const unsigned int u = atomicAdd(reinterpret_cast<unsigned int *>(g.sched), 1u) + 1u;
    const int unit = (u < (unsigned int)nunits) ? (int)u : -1;
    const unsigned long long v = ((unsigned long long)(unsigned int)it << 32) | (unsigned int)unit;
    unsigned long long *slot = g.sched + 1 + pair * kSchedRing + (it % kSchedRing);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(slot), "l"(v) : "memory");   // the word is the whole message
    return unit;
}
// false in *ok: the word did not arrive within ~2 s (the caller raises the device error flag and leaves)
__device__ __forceinline__ int sched_read(const GemmArgs &g, int pair, int it, bool *ok) {
    const unsigned long long *slot = g.sched + 1 + pair * kSchedRing + (it % kSchedRing);
    const uint64_t t0 = global_timer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i) {
            unsigned long long v;
            asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(slot) : "memory");
            if ((unsigned int)(v >> 32) == (unsigned int)it) return (int)(unsigned int)v;
            if (i > 8) __nanosleep(64);
        }
        if (global_timer_ns() - t0 > 2000000000ull) { *ok = false; return -1; }
    }
}
// A role that reads its units from the mailbox.  The word of the NEXT iteration is requested while the current unit
// is being worked on (the poster is two units ahead, so it is normally there), which keeps the global-memory
// latency of the mailbox out of the per-tile critical path; only the value itself is communicated, so the
// accesses are relaxed.  Without a mailbox (g.sched == NULL) the order is static: pair, pair + pairs, ...
struct UnitReader {
    unsigned long long next_word;
    __device__ __forceinline__ static unsigned long long peek(const GemmArgs &g, int pair, int it) {
        unsigned long long v;
        const unsigned long long *slot = g.sched + 1 + pair * kSchedRing + (it % kSchedRing);
        asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(slot) : "memory");
        return v;
    }
    __device__ __forceinline__ void init(const GemmArgs &g, int pair) {
        next_word = g.sched ? peek(g, pair, 0) : 0ull;
    }
    __device__ __forceinline__ int get(const GemmArgs &g, int pair, int npairs, int nunits, int it, bool *ok) {
        if (!g.sched) {
            const int unit = pair + it * npairs;
            return unit < nunits ? unit : -1;
        }
        const unsigned long long w = next_word;
        const int unit = ((unsigned int)(w >> 32) == (unsigned int)it) ? (int)(unsigned int)w
                                                                       : sched_read(g, pair, it, ok);
        if (*ok && unit >= 0) next_word = peek(g, pair, it + 1);
        return unit;
    }
};

// One work unit of the persistent loop: a tile (or a K slab of one) and where its result goes.
struct GemmUnit {
    int tile, kb0, kb1;
    int sp;      // slab index of a split reduction (result row offset sp * M in the workspace)
};
// Units are numbered slab-major: all tiles of K slab 0, then all tiles of slab 1, ...  CTAs that run at the same
// time then work on the same K range of neighbouring tiles and share their operand blocks through L2 (numbered
// tile-major, concurrent units sit at different K offsets of one tile and nothing is shared: measured 20 % slower
// on the 2048 x 6144 x 256 000 weight gradient, which became bound by HBM).
__device__ __forceinline__ GemmUnit decode_unit(const GemmArgs &g, int unit, int nkb) {
    GemmUnit u;
    const int ntiles = g.tiles_m * g.tiles_n;
    u.sp = unit / ntiles;
    u.tile = unit - u.sp * ntiles;
    u.kb0 = u.sp * g.kbps;
    u.kb1 = min(nkb, u.kb0 + g.kbps);
    return u;
}
// Tile number -> block coordinates.  Which way consecutive tiles run decides what the concurrently running CTAs
// share: along N they share a few row blocks of A and sweep all of B once per round of the persistent grid; along
// M the other way round.  The host picks the direction that re-reads the SMALLER operand.
__device__ __forceinline__ void tile_coords(const GemmArgs &g, int tile, int *mb, int *nb) {
    if (g.raster_m) { *nb = tile / g.tiles_m; *mb = tile - *nb * g.tiles_m; }
    else { *mb = tile / g.tiles_n; *nb = tile - *mb * g.tiles_n; }
}

// ---- PTX wrappers -----------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
// Tiled bulk store: a box of this CTA's shared memory (128-byte swizzled, as the map says) to global memory; rows and
// columns of the box that lie outside the tensor are not written.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

template <typename TO> __device__ __forceinline__ void store8(TO *dst, const float *v);
template <> __device__ __forceinline__ void store8<float>(float *dst, const float *v) {
    reinterpret_cast<float4 *>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4 *>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16 *dst, const float *v) {
    uint4 o;
    __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]), p1 = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4], v[5]), p3 = __floats2bfloat162_rn(v[6], v[7]);
    o.x = *reinterpret_cast<uint32_t *>(&p0); o.y = *reinterpret_cast<uint32_t *>(&p1);
    o.z = *reinterpret_cast<uint32_t *>(&p2); o.w = *reinterpret_cast<uint32_t *>(&p3);
    *reinterpret_cast<uint4 *>(dst) = o;
}
template <> __device__ __forceinline__ void store8<__half>(__half *dst, const float *v) {
    uint4 o;
    __half2 p0 = __floats2half2_rn(v[0], v[1]), p1 = __floats2half2_rn(v[2], v[3]);
    __half2 p2 = __floats2half2_rn(v[4], v[5]), p3 = __floats2half2_rn(v[6], v[7]);
    o.x = *reinterpret_cast<uint32_t *>(&p0); o.y = *reinterpret_cast<uint32_t *>(&p1);
    o.z = *reinterpret_cast<uint32_t *>(&p2); o.w = *reinterpret_cast<uint32_t *>(&p3);
    *reinterpret_cast<uint4 *>(dst) = o;
}

// Eight values of C as one 16-byte load (rows and column groups of C are 16-byte aligned: ldc and the column offsets
// are multiples of 8 elements), unpacked to float.
template <typename TO> struct C8 { uint4 q; };
template <> struct C8<float> { float4 a, b; };
template <typename TO> __device__ __forceinline__ C8<TO> load8(const TO *src) {
    C8<TO> c;
    c.q = *reinterpret_cast<const uint4 *>(src);
    return c;
}
template <> __device__ __forceinline__ C8<float> load8<float>(const float *src) {
    C8<float> c;
    c.a = reinterpret_cast<const float4 *>(src)[0];
    c.b = reinterpret_cast<const float4 *>(src)[1];
    return c;
}
template <typename TO> __device__ __forceinline__ void add8(float *v, const C8<TO> &c) {
    const TO *e = reinterpret_cast<const TO *>(&c.q);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] += Cvt<TO>::to_f(e[j]);
}
template <> __device__ __forceinline__ void add8<float>(float *v, const C8<float> &c) {
    v[0] += c.a.x; v[1] += c.a.y; v[2] += c.a.z; v[3] += c.a.w;
    v[4] += c.b.x; v[5] += c.b.y; v[6] += c.b.z; v[7] += c.b.w;
}

// Epilogue of one 32-column chunk of one row: bias, optional accumulate, convert, store.
template <typename TO>
__device__ __forceinline__ void epilogue_chunk(const GemmArgs &g, const uint32_t (&r)[32], int64_t row, int64_t col0) {
    TO *crow = reinterpret_cast<TO *>(g.c) + row * g.ldc + col0;
#pragma unroll
    for (int j0 = 0; j0 < 32; j0 += 8) {
        if (col0 + j0 >= g.N) break;  // N is a multiple of 8
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[j0 + j]);
        if (g.bias) {
            const float4 b0 = *reinterpret_cast<const float4 *>(g.bias + col0 + j0);
            const float4 b1 = *reinterpret_cast<const float4 *>(g.bias + col0 + j0 + 4);
            v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
            v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
        }
        if (g.accumulate) add8<TO>(v, load8<TO>(crow + j0));
        store8<TO>(crow + j0, v);
    }
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: the 128B swizzle pattern repeats every 1024 bytes of shared address
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem + kStages * kAStage;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kStages * (kAStage + kBStage));
    const uint32_t bar_full = smem_u32(bars);             // [kStages]
    const uint32_t bar_empty = bar_full + 8 * kStages;    // [kStages]
    const uint32_t bar_tfull = bar_empty + 8 * kStages;   // [2]
    const uint32_t bar_tempty = bar_tfull + 16;           // [2]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kStages + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nunits = g.tiles_m * g.tiles_n * g.ksplit;   // work units: (tile, k-split)
    const int nkb = (int)((g.K + BK - 1) / BK);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(bar_tfull + 8 * i, 1); mbar_init(bar_tempty + 8 * i, 4); }
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int unit = blockIdx.x; unit < nunits && ok; unit += gridDim.x) {
                const GemmUnit u = decode_unit(g, unit, nkb);
                const int kb0 = u.kb0, kb1 = u.kb1;
                int mb, nb;
                tile_coords(g, u.tile, &mb, &nb);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait_bounded(bar_empty + 8 * stage, phase ^ 1)) { atomicExch(g.err, 11); ok = false; break; }
                    const uint32_t full = bar_full + 8 * stage;
                    mbar_arrive_expect_tx(full, kAStage + kBStage);
                    const uint32_t sa = smem_u32(smem_a + stage * kAStage);
                    const uint32_t sb = smem_u32(smem_b + stage * kBStage);
                    if (!g.a_mn) {
                        tma_load_2d(sa, &map_a, full, kb * BK, mb * BM);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j)
                            tma_load_2d(sa + j * 8192, &map_a, full, mb * BM + j * 64, kb * BK);
                    }
                    if (!g.b_mn) {
                        tma_load_2d(sb, &map_b, full, kb * BK, nb * BN);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_2d(sb + j * 8192, &map_b, full, nb * BN + j * 64, kb * BK);
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------- MMA issuer --------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int it = 0;
            // per-K16 advance of the descriptor start address: 32 B inside a K-major row,
            // two 8-row groups (2048 B) in an MN-major slab
            const uint32_t a_step = g.a_mn ? 2048u : 32u, b_step = g.b_mn ? 2048u : 32u;
            const uint32_t a_lbo = g.a_mn ? 8192u : 16u, b_lbo = g.b_mn ? 8192u : 16u;
            for (int unit = blockIdx.x; unit < nunits && ok; unit += gridDim.x, ++it) {
                const GemmUnit u = decode_unit(g, unit, nkb);
                const int kb0 = u.kb0, kb1 = u.kb1;
                const int acc = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!mbar_wait_bounded(bar_tempty + 8 * acc, acc_phase ^ 1)) { atomicExch(g.err, 12); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait_bounded(bar_full + 8 * stage, phase)) { atomicExch(g.err, 13); ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem_a + stage * kAStage);
                    const uint32_t sb = smem_u32(smem_b + stage * kBStage);
#pragma unroll
                    for (int k16 = 0; k16 < BK / 16; ++k16) {
                        const uint64_t ad = make_desc(sa + k16 * a_step, a_lbo, 1024);
                        const uint64_t bd = make_desc(sb + k16 * b_step, b_lbo, 1024);
                        tc_mma(d_tmem, ad, bd, g.idesc, ((kb - kb0) | k16) ? 1u : 0u);
                    }
                    tc_commit(bar_empty + 8 * stage);   // stage reusable once these MMAs have read it
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
                if (ok) tc_commit(bar_tfull + 8 * acc);  // accumulator complete
            }
        }
    } else {
        // --------------------------------- epilogue ---------------------------------
        const int q = warp & 3;  // TMEM lane quarter this warp may address
        int it = 0;
        for (int unit = blockIdx.x; unit < nunits; unit += gridDim.x, ++it) {
            const GemmUnit u = decode_unit(g, unit, nkb);
            const int sp = u.sp;
            int mb, nb;
            tile_coords(g, u.tile, &mb, &nb);
            const int acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            if (!mbar_wait_bounded(bar_tfull + 8 * acc, acc_phase)) { if (lane == 0) atomicExch(g.err, 14); break; }
            tc_fence_after();
            const int64_t row = (int64_t)mb * BM + q * 32 + lane;
            const int64_t col_base = (int64_t)nb * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                const int64_t col0 = col_base + c * 32;
                if (col0 >= g.N) break;
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + c * 32, r);
                tmem_ld_wait();
                if (row < g.M) {
                    if (g.c_dtype == SRU_BF16) epilogue_chunk<__nv_bfloat16>(g, r, row, col0);
                    else if (g.c_dtype == SRU_F16) epilogue_chunk<__half>(g, r, row, col0);
                    else epilogue_chunk<float>(g, r, row + (int64_t)sp * g.M, col0);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
        }
    }

    // -------------------------------- teardown --------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// =========================================================================================
// Two-SM variant (cta_group::2).  A cluster of two CTAs on neighbouring SMs computes a
// 256 x 256 tile: each CTA loads its own 128 rows of A and its own 128-column half of B into
// its shared memory, the leader CTA (cluster rank 0) issues tcgen05.mma.cta_group::2 with
// M = 256, and each SM's tensor core reads only half of the B operand from its own shared
// memory - the single-CTA kernel above is limited by that shared-memory read traffic (12 KB per
// 64 tensor cycles).  Each CTA's tensor memory holds the accumulator rows of its own 128 rows.
//   full[s]      lives in the leader; both CTAs' TMA requests complete on it (the .cta_group::2
//                form of the load addresses the leader's barrier), the leader's producer
//                announces the bytes of both.
//   empty[s], tmem_full[a]   one per CTA; tcgen05.commit from the leader arrives on both.
//   tmem_empty[a] lives in the leader; the four epilogue warps of each CTA arrive on it (the
//                peer's through its cluster-mapped address).
// No load is shared between CTAs: every TMA request lands in the shared memory of the CTA that
// issued it.
constexpr int kStages2 = 5;
constexpr int kAStage2 = 128 * BK * 2;   // 16 KB: this CTA's 128 rows of A
constexpr int kBStage2 = 128 * BK * 2;   // 16 KB: this CTA's 128 columns of B
// Eight epilogue warps per CTA: TMEM lanes 32q..32q+31 (rows) can only be read by warps with warp % 4 == q, so the two
// warps of a quarter share its 32 rows and take one 128-column half of the tile each.  With short reductions
// (K = 512: 8 k-blocks per tile) the epilogue of a tile, not its MMAs, sets the pace; eight warps halve it.
constexpr int kEpiWarps2 = 8;
constexpr int kThreads2 = 64 + 32 * kEpiWarps2;
constexpr int kStgRow = 128 * 2;               // staged output row: 128 16-bit columns, 16-byte chunks XOR-swizzled by row
constexpr int kStgWarp = 32 * kStgRow;         // per epilogue warp; 1024-byte aligned (two 32 x 128-byte store boxes)
constexpr int kBarBytes2 = 1024;               // barriers + the tensor-memory slot, padded to the staging alignment
constexpr int kSmemBytes2 = kStages2 * (kAStage2 + kBStage2) + 1024 + kBarBytes2 + kEpiWarps2 * kStgWarp;
static_assert(kSmemBytes2 <= 227 * 1024, "pair kernel shared memory");

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load of the pair form: data into THIS CTA's shared memory, completion bytes on the barrier
// at the same offset in the leader CTA (rank bit of the barrier address cleared).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar & 0xFEFFFFFFu), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t slot_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {   // arrives on `bar` in both CTAs
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"((uint16_t)3)
        : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}

// Epilogue of one warp's 32 rows x 256 columns for 16-bit outputs, staged through shared memory:
// tcgen05.ld hands each thread one ROW (32 columns at a time); written straight to global memory
// that is 32 different 128-byte lines per store instruction.  Instead the converted values go to a
// per-warp buffer row by row and are read back so that half a warp covers 256 contiguous bytes of
// one output row: every store instruction then writes two full 256-byte row segments.
//
// With a tensor map of C (map_c != nullptr) the second half goes away: the buffer is laid out as two boxes of 32 rows x
// 128 bytes in the 128-byte swizzle of the map (chunk j of row r at chunk j ^ (r & 7): conflict-free for the row-wise
// writes as well) and one lane hands both boxes to the TMA engine, which also clips rows beyond M and columns beyond N.
// The warp goes straight back to the accumulator; before it writes the buffer again it waits until the engine has read it.
template <typename TO, bool ACC>
__device__ __forceinline__ void epilogue_staged(const GemmArgs &g, uint32_t tmem_warp, int64_t row0, int64_t col_base,
                                                uint8_t *stg, int lane, int h, const CUtensorMap *map_c) {
    const int64_t row = row0 + lane;
    {
        const int64_t colh = col_base + h * 128;
        if (colh >= g.N) return;
        // the chunk's 32 bias values are requested BEFORE the wait for the accumulator load, so that their latency
        // hides behind it (all lanes read the same addresses: one broadcast transaction per request)
        auto load_bias = [&](int64_t col0, float4 (&bv)[8]) {
            if (g.bias) {
#pragma unroll
                for (int q4 = 0; q4 < 8; ++q4)
                    bv[q4] = (col0 + q4 * 4 < g.N) ? __ldg(reinterpret_cast<const float4 *>(g.bias + col0) + q4)
                                                   : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        };
        // when accumulating, the chunk's values of C are requested before the wait for the accumulator as well: one
        // 16-byte load per eight columns of this lane's row
        auto load_c = [&](int64_t col0, C8<TO> (&cv)[ACC ? 4 : 1]) {
            if (ACC && row < g.M) {
                const TO *crow = reinterpret_cast<const TO *>(g.c) + row * g.ldc + col0;
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (col0 + q * 8 < g.N) cv[q] = load8<TO>(crow + q * 8);
            }
        };
        // one chunk of 32 accumulator columns: bias, accumulate, convert, stage
        auto stage_chunk = [&](int c, int64_t col0, const uint32_t (&r)[32], const float4 (&bv)[8], const C8<TO> (&cv)[ACC ? 4 : 1]) {
#pragma unroll
            for (int j0 = 0; j0 < 32; j0 += 8) {
                float v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[j0 + j]);
                if (col0 + j0 < g.N) {
                    if (g.bias) {
                        const float4 b0 = bv[j0 / 4], b1 = bv[j0 / 4 + 1];
                        v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
                        v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
                    }
                    if constexpr (ACC) { if (row < g.M) add8<TO>(v, cv[j0 >> 3]); }
                }
                const int chunk = c * 4 + (j0 >> 3);      // 16-byte chunk of this lane's 256-byte row
                if (map_c)
                    store8<TO>(reinterpret_cast<TO *>(stg + (chunk >> 3) * 4096 + lane * 128 + (((chunk & 7) ^ (lane & 7)) << 4)), v);
                else
                    store8<TO>(reinterpret_cast<TO *>(stg + lane * kStgRow + ((chunk ^ (lane & 15)) << 4)), v);
            }
        };
        if (map_c) {
            if (lane == 0) bulk_wait_read_all();
            __syncwarp();
        }
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
            const int64_t col0 = colh + c * 32;
            if (col0 >= g.N) break;
            float4 bv[8];
            load_bias(col0, bv);
            C8<TO> cv[ACC ? 4 : 1];
            if constexpr (ACC) load_c(col0, cv);
            uint32_t r[32];
            tmem_ld32(tmem_warp + h * 128 + c * 32, r);
            tmem_ld_wait();
            stage_chunk(c, col0, r, bv, cv);
        }
        if (map_c) {
            fence_proxy_async();      // the generic-proxy writes above become visible to the bulk copy engine
            __syncwarp();
            if (lane == 0 && row0 < g.M) {
                tma_store_2d(map_c, smem_u32(stg), (int)colh, (int)row0);
                if (colh + 64 < g.N) tma_store_2d(map_c, smem_u32(stg) + 4096, (int)colh + 64, (int)row0);
                bulk_commit();
            }
            return;
        }
        __syncwarp();
        const int sub = lane >> 4, seg = lane & 15;          // two rows per pass, 16 x 16 bytes per row
        const int64_t col = colh + seg * 8;
#pragma unroll 4
        for (int rr = 0; rr < 32; rr += 2) {
            const int rl = rr + sub;
            if (row0 + rl < g.M && col < g.N) {
                const uint4 val = *reinterpret_cast<const uint4 *>(stg + rl * kStgRow + ((seg ^ (rl & 15)) << 4));
                *reinterpret_cast<uint4 *>(reinterpret_cast<TO *>(g.c) + (row0 + rl) * g.ldc + col) = val;
            }
        }
        __syncwarp();
    }
}

// EW: working epilogue warps per CTA, 4 (192 threads) or 8 (320 threads).  ACC: the 16-bit epilogue adds onto C (the
// dgrad product); a compile-time choice so that the other products do not carry the registers of the values of C.
template <int EW, bool ACC>
__global__ void __launch_bounds__(64 + 32 * EW, 1)
gemm_tcgen05_2sm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const __grid_constant__ CUtensorMap map_c, const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *smem_a = smem;
    uint8_t *smem_b = smem + kStages2 * kAStage2;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kStages2 * (kAStage2 + kBStage2));
    const uint32_t bar_full = smem_u32(bars);              // [kStages2]  (used in the leader)
    const uint32_t bar_empty = bar_full + 8 * kStages2;    // [kStages2]  (one per CTA)
    const uint32_t bar_tfull = bar_empty + 8 * kStages2;   // [2]         (one per CTA)
    const uint32_t bar_tempty = bar_tfull + 16;            // [2]         (used in the leader)
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kStages2 + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();               // 0 = leader
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int ntiles_all = g.tiles_m * g.tiles_n;
    // work units: (256 x 256 tile, K slab)
    const int nunits = ntiles_all * g.ksplit;
    const int nkb = (int)((g.K + BK - 1) / BK);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages2; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(bar_tfull + 8 * i, 1); mbar_init(bar_tempty + 8 * i, 2 * EW); }
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc2(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish2();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();     // both CTAs' barriers exist before anything signals across the pair
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------- TMA producer (both CTAs) -------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            // The leader's producer posts units two iterations ahead: the counter's round trip and the time until
            // the peer sees the mailbox stay behind a whole tile of loads.
            const bool poster = g.sched != nullptr && rank == 0;
            int ahead1 = -1;            // unit of iteration it + 1 (poster only)
            int cur = -1;
            if (poster) {
                cur = sched_post_next(g, pair, 0, nunits);
                ahead1 = sched_post_next(g, pair, 1, nunits);
            }
            UnitReader reader;
            if (!poster) reader.init(g, pair);
            for (int it = 0; ok; ++it) {
                unsigned int ticket = 0;
                if (poster) {
                    ticket = sched_take(g);                       // for iteration it + 2; looked at after the loads
                } else {
                    cur = reader.get(g, pair, npairs, nunits, it, &ok);
                    if (!ok) { atomicExch(g.err, 25); break; }
                }
                const int unit = cur;
                if (unit < 0) break;
                const GemmUnit u = decode_unit(g, unit, nkb);
                const int kb0 = u.kb0, kb1 = u.kb1;
                int mb, nb;
                tile_coords(g, u.tile, &mb, &nb);
                const int m0 = mb * 256 + (int)rank * 128;      // this CTA's rows of A
                const int n0 = nb * BN + (int)rank * 128;       // this CTA's columns of B
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait_bounded(bar_empty + 8 * stage, phase ^ 1)) { atomicExch(g.err, 21); ok = false; break; }
                    const uint32_t full = bar_full + 8 * stage;
                    if (rank == 0) mbar_arrive_expect_tx(full, 2 * (kAStage2 + kBStage2));
                    const uint32_t sa = smem_u32(smem_a + stage * kAStage2);
                    const uint32_t sb = smem_u32(smem_b + stage * kBStage2);
                    if (!g.a_mn) {
                        tma_load_2d_pair(sa, &map_a, full, kb * BK, m0);
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; ++j) tma_load_2d_pair(sa + j * 8192, &map_a, full, m0 + j * 64, kb * BK);
                    }
                    if (!g.b_mn) {
                        tma_load_2d_pair(sb, &map_b, full, kb * BK, n0);
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; ++j) tma_load_2d_pair(sb + j * 8192, &map_b, full, n0 + j * 64, kb * BK);
                    }
                    if (++stage == kStages2) { stage = 0; phase ^= 1; }
                }
                if (poster) {
                    cur = ahead1;
                    ahead1 = sched_post(g, pair, it + 2, ticket, nunits);
                }
            }
        }
    }
    else if (warp == 1) {
        // ------------------------------ MMA issuer (leader CTA only) ------------------------------
        if (lane == 0 && rank == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const uint32_t a_step = g.a_mn ? 2048u : 32u, b_step = g.b_mn ? 2048u : 32u;
            const uint32_t a_lbo = g.a_mn ? 8192u : 16u, b_lbo = g.b_mn ? 8192u : 16u;
            UnitReader reader;
            reader.init(g, pair);
            for (int it = 0; ok; ++it) {
                const int unit = reader.get(g, pair, npairs, nunits, it, &ok);
                if (!ok) { atomicExch(g.err, 26); break; }
                if (unit < 0) break;
                const GemmUnit u = decode_unit(g, unit, nkb);
                const int kb0 = u.kb0, kb1 = u.kb1;
                const int acc = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!mbar_wait_bounded(bar_tempty + 8 * acc, acc_phase ^ 1)) { atomicExch(g.err, 22); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait_bounded(bar_full + 8 * stage, phase)) { atomicExch(g.err, 23); ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem_a + stage * kAStage2);
                    const uint32_t sb = smem_u32(smem_b + stage * kBStage2);
#pragma unroll
                    for (int k16 = 0; k16 < BK / 16; ++k16) {
                        const uint64_t ad = make_desc(sa + k16 * a_step, a_lbo, 1024);
                        const uint64_t bd = make_desc(sb + k16 * b_step, b_lbo, 1024);
                        tc_mma_pair(d_tmem, ad, bd, g.idesc, ((kb - kb0) | k16) ? 1u : 0u);
                    }
                    tc_commit_pair(bar_empty + 8 * stage);    // frees the stage in both CTAs
                    if (++stage == kStages2) { stage = 0; phase ^= 1; }
                }
                if (ok) tc_commit_pair(bar_tfull + 8 * acc);   // accumulators complete in both CTAs
            }
        }
    } else {
        // ------------------------------ epilogue (both CTAs, own rows) ------------------------------
        // Eight warps (EW = 8) when the reduction is short and the epilogue sets the pace; with long reductions four,
        // each doing both column halves: eight put two busy warps on the scheduler of the MMA-issuing thread and the
        // tensor pipe loses 7 % (ncu: 92 % -> 85 % active on the K = 2048 forward product).
        const int q = warp & 3;                 // TMEM lane quarter = 32 rows of the CTA's 128
        const int h_first = (EW == 8) ? ((warp - 2) >> 2) : 0;   // 128-column halves this warp converts
        const int h_last = (EW == 8) ? h_first : 1;
        const uint32_t tempty_leader = map_to_cta(bar_tempty, 0);
        uint8_t *stg = smem + kStages2 * (kAStage2 + kBStage2) + kBarBytes2 + (warp - 2) * kStgWarp;
        bool ok = true;
        UnitReader reader;
        reader.init(g, pair);
        for (int it = 0; ; ++it) {
            // every lane reads the mailbox itself (same word: one broadcast access)
            const int unit = reader.get(g, pair, npairs, nunits, it, &ok);
            if (!ok) { if (lane == 0) atomicExch(g.err, 27); break; }
            if (unit < 0) break;
            const GemmUnit u = decode_unit(g, unit, nkb);
            const int sp = u.sp;
            int mb, nb;
            tile_coords(g, u.tile, &mb, &nb);
            const int acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            if (!mbar_wait_bounded(bar_tfull + 8 * acc, acc_phase)) { if (lane == 0) atomicExch(g.err, 24); break; }
            tc_fence_after();
            const int64_t row0 = (int64_t)mb * 256 + rank * 128 + q * 32;
            const int64_t row = row0 + lane;
            const int64_t col_base = (int64_t)nb * BN;
            const uint32_t tmem_warp = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
            if (g.c_dtype == SRU_BF16) {
                for (int h = h_first; h <= h_last; ++h)
                    epilogue_staged<__nv_bfloat16, ACC>(g, tmem_warp, row0, col_base, stg, lane, h, g.c_tma ? &map_c : nullptr);
            } else if (g.c_dtype == SRU_F16) {
                for (int h = h_first; h <= h_last; ++h)
                    epilogue_staged<__half, ACC>(g, tmem_warp, row0, col_base, stg, lane, h, g.c_tma ? &map_c : nullptr);
            } else {
#pragma unroll 1
                for (int c = h_first * 4; c < h_last * 4 + 4; ++c) {
                    const int64_t col0 = col_base + c * 32;
                    if (col0 >= g.N) break;
                    uint32_t r[32];
                    tmem_ld32(tmem_warp + c * 32, r);
                    tmem_ld_wait();
                    if (row < g.M) epilogue_chunk<float>(g, r, row + (int64_t)sp * g.M, col0);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_leader + 8 * acc);
        }
        if (g.c_tma && lane == 0) bulk_wait_all();     // this warp's stores have left shared memory and are complete
    }

    // -------------------------------- teardown --------------------------------
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();     // neither CTA leaves while its pair may still signal its barriers
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc2(tmem_base, kTmemCols);
    }
}

// Split-K tail: C = sum over slabs of the fp32 partial products (+ C when accumulating), converted.
template <typename TO>
__global__ void splitk_reduce(const float *__restrict__ ws, int nsplit, int64_t M, int64_t N, TO *__restrict__ c,
                              int64_t ldc, int accumulate) {
    const int64_t n4 = N / 4;   // N is a multiple of 8
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < M * n4; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / n4, col = (i - row * n4) * 4;
        float4 acc = *reinterpret_cast<const float4 *>(ws + row * N + col);
        for (int sp = 1; sp < nsplit; ++sp) {
            const float4 v = *reinterpret_cast<const float4 *>(ws + ((int64_t)sp * M + row) * N + col);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        // four elements of C as one access (ldc and col are multiples of 4 elements, C is 16-byte aligned)
        using P4 = Pack<TO, 4>;
        P4 *o = reinterpret_cast<P4 *>(c + row * ldc + col);
        if (accumulate) {
            const P4 old = *o;
            acc.x += Cvt<TO>::to_f(old.v[0]); acc.y += Cvt<TO>::to_f(old.v[1]);
            acc.z += Cvt<TO>::to_f(old.v[2]); acc.w += Cvt<TO>::to_f(old.v[3]);
        }
        P4 out;
        out.v[0] = Cvt<TO>::from_f(acc.x); out.v[1] = Cvt<TO>::from_f(acc.y);
        out.v[2] = Cvt<TO>::from_f(acc.z); out.v[3] = Cvt<TO>::from_f(acc.w);
        *o = out;
    }
}

// How many K slabs to cut a product into.  Two situations, both with a long reduction:
//  * the tiles alone leave most of the persistent grid idle (2 * tiles <= workers: the first layer's weight
//    gradient, 120 x 8192 over K = 256 000): slabs fill the grid, up to 3x faster;
//  * the tiles make a few rounds of the grid with a badly filled last one (192 tiles on 74 pairs are 2.6 rounds of
//    work done in 3: the 2048 x 6144 x 256 000 weight gradient): slabs make the rounds shorter and the last one
//    fuller.  Units are numbered slab-major (decode_unit), which keeps the L2 sharing of the unsplit order.
// Many rounds lose little to the last one and are left alone.
int choose_ksplit(int64_t tiles, int workers, int nkb) {
    const int forced = option(OPT_GEMM_KSPLIT, 0);
    if (forced > 0) return std::min(forced, 16);
    if (nkb < 64) return 1;
    auto fill = [&](int s) {
        const int64_t units = tiles * s;
        return (double)units / (double)(((units + workers - 1) / workers) * workers);
    };
    if (2 * tiles <= (int64_t)workers) {
        int best = 1;
        double best_eff = 0.0;
        for (int s = 1; s <= 8; ++s) {
            if (nkb / s < 16) break;
            if (fill(s) > best_eff + 0.04) { best_eff = fill(s); best = s; }
        }
        return best;
    }
    if (tiles > 6 * (int64_t)workers || fill(1) >= 0.93) return 1;
    int best = 1;
    double best_eff = fill(1);
    for (int s = 2; s <= 6; ++s) {
        if (nkb / s < 64) break;
        if (fill(s) >= 0.95) return s;                       // the smallest split that fills the rounds
        if (fill(s) > best_eff + 0.04) { best_eff = fill(s); best = s; }
    }
    return best;
}

// ---- host side --------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    }
    return fn;
}

// 2-D tensor map over a row-major matrix: `inner` contiguous elements per row, `outer` rows,
// row pitch ld elements; box = box_inner x box_outer; 128-byte swizzle; OOB reads give zeros.
int make_map(CUtensorMap *map, const void *base, int dtype, int64_t inner, int64_t outer, int64_t ld,
             int box_inner, int box_outer) {
    auto fn = get_encode_fn();
    if (!fn) return set_error(SRU_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dtype == SRU_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                    const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(SRU_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return 0;
}

}  // namespace

}  // namespace srub

using namespace srub;

// Kernel choice for a problem: pair kernel or single-CTA kernel, the number of K slabs, and whether the pair kernel
// takes its tiles dynamically (option gemm_dynamic, more than one round of units).
struct GemmPlan {
    bool two_sm;
    int ksplit;        // K slabs (1: none); needs ksplit * m * n floats of workspace
    bool dynamic;      // dynamic tile order; needs sched_bytes of workspace
    int64_t units;     // work units of the persistent loop (tiles x slabs)
    int workers;       // CTAs (single-CTA kernel) or CTA pairs (pair kernel)
    size_t split_bytes, sched_bytes;
};

static int gemm_plan(int64_t m, int64_t n, int64_t k_dim, bool has_bias, GemmPlan *p) {
    int dev = 0, sms = 148;
    SRUB_CUDA_CHECK(cudaGetDevice(&dev));
    SRUB_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int64_t tiles256 = ((m + 255) / 256) * ((n + BN - 1) / BN);
    // measured: from about 32 tiles of 256 x 256 on, the pair kernel beats twice as many 128 x 256 tiles on single CTAs
    bool pair = tiles256 >= 32 && m > 160;   // a 256-row tile over at most 160 rows is mostly padding
    const int forced = option(OPT_GEMM_2SM, -1);
    if (forced >= 0) pair = forced != 0;
    const int64_t tiles = pair ? tiles256 : ((m + BM - 1) / BM) * ((n + BN - 1) / BN);
    const int nkb = (int)((k_dim + BK - 1) / BK);
    p->two_sm = pair;
    p->workers = pair ? sms / 2 : sms;
    int ksplit = has_bias ? 1 : choose_ksplit(tiles, p->workers, nkb);
    const int kbps = (nkb + ksplit - 1) / ksplit;
    ksplit = (nkb + kbps - 1) / kbps;
    p->ksplit = ksplit;
    p->units = tiles * ksplit;
    p->split_bytes = ksplit > 1 ? (size_t)ksplit * (size_t)m * (size_t)n * sizeof(float) : 0;
    const int64_t npairs = std::min<int64_t>(p->units, p->workers);
    p->dynamic = pair && option(OPT_GEMM_DYNAMIC, 0) != 0 && p->units > npairs && npairs <= kSchedMaxPairs;
    p->sched_bytes = p->dynamic ? (size_t)(1 + npairs * kSchedRing) * sizeof(unsigned long long) : 0;
    return 0;
}

static int gemm_impl(void *c, const void *a, const void *b, const float *col_bias, int64_t m, int64_t n,
                     int64_t k_dim, int64_t lda, int64_t ldb, int64_t ldc, int trans_a, int trans_b,
                     int ab_dtype, int c_dtype, int accumulate, void *workspace, size_t workspace_bytes,
                     void *stream) {
    if (m < 0 || n < 0 || k_dim < 1) return set_error(SRU_ERR_BAD_ARG, "bad gemm sizes");
    if (m == 0 || n == 0) return 0;
    if (!c || !a || !b) return set_error(SRU_ERR_BAD_ARG, "gemm pointers must not be null");
    if (ab_dtype != SRU_BF16 && ab_dtype != SRU_F16)
        return set_error(SRU_ERR_UNSUPPORTED, "gemm operands must be bf16 or fp16");
    if (c_dtype != SRU_BF16 && c_dtype != SRU_F16 && c_dtype != SRU_F32)
        return set_error(SRU_ERR_UNSUPPORTED, "gemm output must be bf16, fp16 or fp32");
    auto misaligned = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; };
    if (misaligned(a) || misaligned(b) || misaligned(c) || (col_bias && misaligned(col_bias)))
        return set_error(SRU_ERR_BAD_ARG, "gemm pointers must be 16-byte aligned");
    if (lda % 8 || ldb % 8 || ldc % 8 || n % 8)
        return set_error(SRU_ERR_BAD_ARG, "gemm leading dimensions and N must be multiples of 8 elements");
    if (m > 0x7fffffff || n > 0x7fffffff || k_dim > 0x7fffffff) return set_error(SRU_ERR_BAD_ARG, "gemm size too large");

    // the tensor-map encoder is a driver entry point: this thread needs the primary context
    if (int rc = ensure_context()) return rc;

    int dev = 0;
    SRUB_CUDA_CHECK(cudaGetDevice(&dev));
    GemmPlan plan;
    if (int prc = gemm_plan(m, n, k_dim, col_bias != nullptr, &plan)) return prc;
    const bool two_sm = plan.two_sm;
    // Both extras live in the caller's workspace ([K-slab partials][scheduler words]); what does not fit is
    // simply not used: no split, static tile order.
    const int nkb_all = (int)((k_dim + BK - 1) / BK);
    int ksplit = plan.ksplit;
    size_t ws_used = 0;
    if (ksplit > 1 && (!workspace || workspace_bytes < plan.split_bytes)) ksplit = 1;
    if (ksplit > 1) ws_used = (plan.split_bytes + 15) & ~size_t(15);
    const int kbps = (nkb_all + ksplit - 1) / ksplit;
    unsigned long long *sched = nullptr;
    if (plan.dynamic && ksplit == plan.ksplit && workspace && workspace_bytes >= ws_used + plan.sched_bytes &&
        (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0)
        sched = reinterpret_cast<unsigned long long *>(static_cast<uint8_t *>(workspace) + ws_used);

    CUtensorMap map_a, map_b;
    int rc;
    // A: K-major stored (M,K) -> inner K, box 64 x 128.  MN-major stored (K,M) -> inner M, box 64 x 64.
    if (!trans_a) rc = make_map(&map_a, a, ab_dtype, k_dim, m, lda, BK, BM);
    else rc = make_map(&map_a, a, ab_dtype, m, k_dim, lda, 64, BK);
    if (rc) return rc;
    // B: K-major stored (N,K) -> inner K, box 64 x 256 (64 x 128 per CTA of a pair).
    // MN-major stored (K,N) -> inner N, box 64 x 64.
    if (trans_b) rc = make_map(&map_b, b, ab_dtype, k_dim, n, ldb, BK, two_sm ? 128 : BN);
    else rc = make_map(&map_b, b, ab_dtype, n, k_dim, ldb, 64, BK);
    if (rc) return rc;

    GemmArgs g;
    g.c = c; g.bias = col_bias; g.M = m; g.N = n; g.K = k_dim; g.ldc = ldc;
    g.c_dtype = c_dtype; g.accumulate = accumulate ? 1 : 0;
    g.a_mn = trans_a ? 1 : 0;
    g.b_mn = trans_b ? 0 : 1;
    const uint32_t fmt = (ab_dtype == SRU_BF16) ? 1u : 0u;
    // instruction descriptor: D fp32 (bits 4-5 = 1), A/B format (bits 7-9, 10-12), operand majors
    // (bits 15, 16), N/8 (bits 17-22), M/16 (bits 24-28)
    g.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)g.a_mn << 15) | ((uint32_t)g.b_mn << 16) |
              ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    const int tile_m = two_sm ? 256 : BM;
    if (two_sm) g.idesc = (g.idesc & ~(0x1Fu << 24)) | ((uint32_t)(256 >> 4) << 24);
    g.tiles_m = (int)((m + tile_m - 1) / tile_m);
    g.tiles_n = (int)((n + BN - 1) / BN);
    g.err = device_error_flag();
    if (!g.err) return set_error(SRU_ERR_CUDA, "device error flag unavailable");
    g.ksplit = ksplit;
    g.kbps = kbps;
    const int64_t tiles_all = (int64_t)g.tiles_m * g.tiles_n;
    // Tile order: with several rounds of tiles on the persistent grid, each round sweeps one operand completely and
    // touches only a few blocks of the other; let the operand that is swept again and again be the smaller one
    // (A is M x K, B is K x N: compare M with N).  The weight gradient x^T grad_U (2048 x 6144 over 256 000) reads
    // 6 GB instead of 10 GB from HBM this way.  Option gemm_raster forces a direction.
    g.raster_m = (tiles_all > plan.workers && m < n) ? 1 : 0;
    const int raster_forced = option(OPT_GEMM_RASTER, -1);
    if (raster_forced >= 0) g.raster_m = raster_forced ? 1 : 0;
    void *final_c = c;
    const int final_dtype = c_dtype, final_acc = g.accumulate;
    if (ksplit > 1) {   // partial products go to [ksplit][M][N] fp32; splitk_reduce finishes the job
        g.c = workspace; g.ldc = n; g.c_dtype = SRU_F32; g.accumulate = 0;
    }
    const int64_t ntiles = tiles_all * ksplit;   // work units
    if (ntiles > 0x7fffffff) return set_error(SRU_ERR_BAD_ARG, "too many gemm tiles");

    static bool attr_set[64] = {false};
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        SRUB_CUDA_CHECK(cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kSmemBytes));
        SRUB_CUDA_CHECK(cudaFuncSetAttribute(gemm_tcgen05_2sm_kernel<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kSmemBytes2));
        SRUB_CUDA_CHECK(cudaFuncSetAttribute(gemm_tcgen05_2sm_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kSmemBytes2));
        SRUB_CUDA_CHECK(cudaFuncSetAttribute(gemm_tcgen05_2sm_kernel<8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kSmemBytes2));
        SRUB_CUDA_CHECK(cudaFuncSetAttribute(gemm_tcgen05_2sm_kernel<8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kSmemBytes2));
        attr_set[dev] = true;
    }
    g.sched = nullptr;
    // 16-bit output of the pair kernel leaves through tiled bulk stores where the epilogue sets the pace of a tile
    // (K <= 512).  Measured on B200, bulk stores against warp stores: 256 000 x 8192 x 120  1544 -> 1310 us,
    // 16 384 x 6144 x 512  101.9 -> 96.0, 16 384 x 4096 x 512  74.0 -> 68.7; level at K = 1024; with long reductions,
    // where four epilogue warps do both halves of a tile through one buffer and the loads keep the copy engine
    // busy, they LOSE (256 000 x 6144 x 2048  4745 -> 4973 us, 256 000 x 2048 x 6144  4413 -> 5220).
    // Option gemm_tma_store forces either way.
    CUtensorMap map_c;
    memset(&map_c, 0, sizeof(map_c));
    g.c_tma = 0;
    if (two_sm && g.c_dtype != SRU_F32 && option(OPT_GEMM_TMA_STORE, nkb_all <= 8 ? 1 : 0)) {
        rc = make_map(&map_c, g.c, g.c_dtype, n, m, g.ldc, 64, 32);
        if (rc) return rc;
        g.c_tma = 1;
    }
    g.epi_warps = (nkb_all <= 16) ? 8 : 4;      // see the epilogue of the pair kernel
    const int epi_forced = option(OPT_GEMM_EPI_WARPS, -1);
    if (epi_forced >= 0) g.epi_warps = (epi_forced == 8) ? 8 : 4;
    if (two_sm) {
        // Dynamic tile order (option gemm_dynamic) once there is more than one round of units.  It is meant for
        // products that share the GPU with another kernel (the gradient all-reduce of data-parallel training, whose
        // host side switches it on); alone on the GPU the static order is as fast or faster.  Counter and mailboxes
        // sit in the caller's workspace, so products on different streams never share them; they are refilled
        // (0xFF) on the product's stream right before its launch.
        const int64_t npairs_l = std::min<int64_t>(ntiles, plan.workers);
        if (sched) {
            g.sched = sched;
            SRUB_CUDA_CHECK(cudaMemsetAsync(g.sched, 0xFF, plan.sched_bytes, static_cast<cudaStream_t>(stream)));
        }
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3(2u * (unsigned)npairs_l, 1, 1);
        cfg.blockDim = dim3(64 + 32 * g.epi_warps, 1, 1);
        cfg.dynamicSmemBytes = kSmemBytes2;
        cfg.stream = static_cast<cudaStream_t>(stream);
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        // the accumulating 16-bit epilogue is its own instance (fp32 output accumulates in the plain chunk epilogue)
        const bool acc16 = g.accumulate && g.c_dtype != SRU_F32;
        if (g.epi_warps == 8) {
            if (acc16) SRUB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_tcgen05_2sm_kernel<8, true>, map_a, map_b, map_c, g));
            else SRUB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_tcgen05_2sm_kernel<8, false>, map_a, map_b, map_c, g));
        } else {
            if (acc16) SRUB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_tcgen05_2sm_kernel<4, true>, map_a, map_b, map_c, g));
            else SRUB_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_tcgen05_2sm_kernel<4, false>, map_a, map_b, map_c, g));
        }
    } else {
        const unsigned grid = (unsigned)std::min<int64_t>(ntiles, plan.workers);
        gemm_tcgen05_kernel<<<grid, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(map_a, map_b, g);
    }
    SRUB_CUDA_CHECK(cudaGetLastError());
    if (ksplit > 1) {
        const int64_t items = m * (n / 4);
        const unsigned blocks = (unsigned)std::min<int64_t>((items + 255) / 256, (int64_t)plan.workers * 16);
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        const float *ws = static_cast<const float *>(workspace);
        if (final_dtype == SRU_BF16)
            splitk_reduce<__nv_bfloat16><<<blocks, 256, 0, st>>>(ws, ksplit, m, n, (__nv_bfloat16 *)final_c, ldc, final_acc);
        else if (final_dtype == SRU_F16)
            splitk_reduce<__half><<<blocks, 256, 0, st>>>(ws, ksplit, m, n, (__half *)final_c, ldc, final_acc);
        else
            splitk_reduce<float><<<blocks, 256, 0, st>>>(ws, ksplit, m, n, (float *)final_c, ldc, final_acc);
        SRUB_CUDA_CHECK(cudaGetLastError());
    }
    return 0;
}

// Gate bias (2, D) -> per-column vector of U's gate-innermost layout: column (j*k + 1) gets bias[0][j], column
// (j*k + 2) gets bias[1][j], the candidate (and highway) columns get 0.
__global__ void gate_bias_columns_kernel(float *__restrict__ out, const float *__restrict__ bias, int64_t D, int k) {
    const int64_t n = D * k;
    for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < n; c += (int64_t)gridDim.x * blockDim.x) {
        const int64_t j = c / k;
        const int g = (int)(c - j * k);
        out[c] = (g == 1) ? bias[j] : (g == 2) ? bias[D + j] : 0.f;
    }
}

extern "C" int sru_b200_gate_bias_columns(float *col_bias, const float *bias, int64_t width, int k, void *stream) {
    if (!col_bias || !bias || width < 1 || (k != 3 && k != 4))
        return set_error(SRU_ERR_BAD_ARG, "gate_bias_columns: null pointer, width < 1 or k not 3 / 4");
    const int64_t n = width * k;
    const unsigned blocks = (unsigned)std::min<int64_t>((n + 255) / 256, 1024);
    gate_bias_columns_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(col_bias, bias, width, k);
    SRUB_CUDA_CHECK(cudaGetLastError());
    return 0;
}

extern "C" int sru_b200_gemm(void *c, const void *a, const void *b, const float *col_bias, int64_t m, int64_t n,
                             int64_t k_dim, int64_t lda, int64_t ldb, int64_t ldc, int trans_a, int trans_b,
                             int ab_dtype, int c_dtype, int accumulate, void *stream) {
    return gemm_impl(c, a, b, col_bias, m, n, k_dim, lda, ldb, ldc, trans_a, trans_b, ab_dtype, c_dtype, accumulate,
                     nullptr, 0, stream);
}

extern "C" size_t sru_b200_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k_dim, int has_bias) {
    if (m <= 0 || n <= 0 || k_dim <= 0) return 0;
    GemmPlan plan;
    if (gemm_plan(m, n, k_dim, has_bias != 0, &plan) != 0) return 0;
    return ((plan.split_bytes + 15) & ~size_t(15)) + plan.sched_bytes;
}

extern "C" int sru_b200_gemm_ws(void *c, const void *a, const void *b, const float *col_bias, int64_t m, int64_t n,
                                int64_t k_dim, int64_t lda, int64_t ldb, int64_t ldc, int trans_a, int trans_b,
                                int ab_dtype, int c_dtype, int accumulate, void *workspace, size_t workspace_bytes,
                                void *stream) {
    return gemm_impl(c, a, b, col_bias, m, n, k_dim, lda, ldb, ldc, trans_a, trans_b, ab_dtype, c_dtype, accumulate,
                     workspace, workspace_bytes, stream);
}
