/*
 * CPU oracle for the SRU light-recurrence scan: a plain-C restatement of the
 * reference algorithm (asappresearch/sru v2.6.0), forward and backward, uni- and
 * bidirectional, k = 3 / 4, mask_pad, mask_c, custom per-step V, tanh activation.
 *
 * THIS FILE IS TEST INFRASTRUCTURE.  It is the checker the CUDA kernels are
 * compared with, and the timed CPU baseline of the benchmark.  Nothing in the
 * shipped package calls it; the product path has no CPU fallback.
 *
 * Parity pin: the oracle is checked (tests/test_oracle.py) against golden vectors
 * produced by the reference's own Python implementation
 * (sru.ops.elementwise_recurrence_naive + autograd, and sru.SRU on CPU) and
 * against the reference's regression artifact test/regression/artifacts/2.3.5.pt,
 * re-exported by tests/golden/make_golden.py.
 *
 * Reference lines each function follows are cited in sru_oracle_body.inc.
 * Build: oracle/build.py (gcc -O2 -fno-fast-math -ffp-contract=off -fopenmp -shared -fPIC).
 */
#include <math.h>
#include <stdlib.h>

#define REAL float
#define EXPF expf
#define TANHF tanhf
#define NAME(x) x##_f32
#include "sru_oracle_body.inc"
#undef REAL
#undef EXPF
#undef TANHF
#undef NAME

#define REAL double
#define EXPF exp
#define TANHF tanh
#define NAME(x) x##_f64
#include "sru_oracle_body.inc"
#undef REAL
#undef EXPF
#undef TANHF
#undef NAME

int sru_oracle_version(void) { return 1; }
