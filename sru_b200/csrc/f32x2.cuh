// Packed float32 arithmetic (two lanes per instruction) for sm_100a.
//
// Blackwell adds add / sub / mul / fma on pairs of float32 held in a 64-bit register (PTX fma.rn.f32x2 and friends).
// The scan kernels are bound by instruction ISSUE once the SM clock drops under the power cap of a training step
// (ncu: 61 % of the issue slots busy at 1.9 GHz, i.e. about 90 % at the 1.3 GHz the step runs at), and more than half
// of their instructions are float32 arithmetic on independent columns.  Processing a thread's columns in pairs halves
// the issue slots of that arithmetic; every lane is rounded exactly like the scalar instruction.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace srub {

struct F2 {
    unsigned long long v;
};

__device__ __forceinline__ F2 f2_make(float lo, float hi) {
    F2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r.v) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ F2 f2_splat(float x) { return f2_make(x, x); }
__device__ __forceinline__ void f2_split(F2 x, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(x.v));
}
__device__ __forceinline__ F2 f2_fma(F2 a, F2 b, F2 c) {
    F2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r.v) : "l"(a.v), "l"(b.v), "l"(c.v));
    return r;
}
__device__ __forceinline__ F2 f2_mul(F2 a, F2 b) {
    F2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v));
    return r;
}
__device__ __forceinline__ F2 f2_add(F2 a, F2 b) {
    F2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v));
    return r;
}
__device__ __forceinline__ F2 f2_sub(F2 a, F2 b) {
    F2 r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v));
    return r;
}
__device__ __forceinline__ F2 f2_select(bool take_a, F2 a, F2 b) {
    F2 r;
    r.v = take_a ? a.v : b.v;
    return r;
}

}  // namespace srub
