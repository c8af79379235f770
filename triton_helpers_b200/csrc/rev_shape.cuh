// Shapes, parameter pointers and the per-CTA gradient-accumulator size shared by the two
// reversible-MLP kernel families (tcgen05 and mma.sync) and their launchers.
#pragma once

#include "common.cuh"

namespace th {

constexpr int kMatFloats = 64 * 64;  // fp32 slots of one weight-gradient matrix in a CTA's private accumulator

struct RevShape {
    int half, hid;  // width of x1 / x2, hidden width of F and G (multiples of 16, <= 64)
    int blocks;
    int act;
    int has_bias;
};

struct RevParams {
    const void *w_f1, *w_f2, *w_g1, *w_g2;  // (blocks*hid, half), (blocks*half, hid), ...
    const void *b_f1, *b_f2, *b_g1, *b_g2;  // (blocks, hid), (blocks, half), ...
};

// Per-CTA accumulator layout: [block][matrix 0..3][kMatFloats] then [block][4][64] bias sums.
__host__ __device__ inline size_t rev_cta_floats(const RevShape &s) {
    return static_cast<size_t>(s.blocks) * 4 * kMatFloats + static_cast<size_t>(s.blocks) * 4 * 64;
}

// ---- tcgen05 path (reversible_mlp_tc.cu) ---------------------------------------------------------
// Each returns TH_OK when it launched, kRevTcNotApplicable when the case is outside what the
// tcgen05 kernels cover (the caller then uses the mma.sync kernels), or an error code.
constexpr int kRevTcNotApplicable = -1000;

int rev_fwd_tc(const RevShape &s, const RevParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
               int64_t rows, int dtype, cudaStream_t stream);

// Backward from the output; `workspace` (zeroed by the caller) holds one private fp32 copy of all
// weight gradients per CTA, `n_ctas` of them; writes the gradient tensors itself.
int rev_bwd_tc(const RevShape &s, const RevParams &p, const void *y, int64_t y_stride, const void *go,
               int64_t go_stride, void *gx, int64_t gx_stride, void *x_rec, int64_t xr_stride, void *const dw[4],
               float *workspace, int n_ctas, int64_t rows, int dtype, cudaStream_t stream);

}  // namespace th
