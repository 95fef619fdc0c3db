// Argument block and launch entry points shared by the scan kernels.
#pragma once
#include "common.cuh"

namespace srub {

// One block of arguments for forward and backward; pointers not used by a pass are null.
struct ScanArgs {
    // forward outputs
    void *h;
    void *c_hist;  // forward: output (may be null); backward: input
    void *c_last;
    // backward outputs
    void *grad_u;
    void *grad_x;
    void *grad_wc;
    void *grad_bias;
    void *grad_init;
    // inputs
    const void *u;
    const void *x;
    const void *weight_c;
    const void *bias;
    const void *c_init;
    const void *mask_c;
    const uint8_t *mask_pad;
    const void *grad_h;
    const void *grad_last;
    void *workspace;
    int64_t L, B;
    int d, dirs, k;
    int activation_type, skip_type, is_custom;
    double scale_x;
    int dtype, c_dtype;
};

// Tile geometry of the pipelined kernels, chosen on the host.
struct TileCfg {
    int hw;        // hidden units per CTA tile (divides d, multiple of the copy granule)
    int br;        // batch rows per CTA tile
    int tpr;       // threads per row = hw / V
    int nht;       // hidden tiles = dirs*d / hw
    int nrt;       // row tiles = ceil(B / br)
    int nstages;   // ring depth
    int ss;        // time steps per ring stage (a multiple of 4)
    int v;         // columns per thread
    int threads;   // consumer threads (br * tpr, rounded up to a warp) + one producer warp
    size_t smem;   // dynamic shared memory bytes
};

int launch_scan_generic(const ScanArgs &a, bool backward, cudaStream_t st);

// Returns 1 if the pipelined kernels took the call, 0 if the shape is not theirs
// (caller falls back to the generic kernels), negative on error.
int launch_scan_pipelined(const ScanArgs &a, bool backward, cudaStream_t st);

// Bytes of the row-tile partials the pipelined backward writes, 0 if it would not run.
size_t pipelined_workspace_bytes(int64_t L, int64_t B, int64_t d, int dirs, int k, int dtype);

template <typename CT>
int launch_reduce_partials(const void *part, void *grad_wc, void *grad_bias, int64_t ntiles,
                           int64_t D, int write_wc, cudaStream_t st);

}  // namespace srub
