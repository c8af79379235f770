// Shapes, parameter pointers and the fp32 gradient-workspace layout shared by the two fused-MLP
// kernel families (tcgen05 and mma.sync) and their launchers.
#pragma once

#include "common.cuh"

namespace th {

struct MlpShape {
    int d_in, d_hid, d_out;
    int depth;    // activated layers: the input layer plus depth-1 hidden layers
    int ki, h, no;  // d_in, d_hid, d_out padded to multiples of 16
    int act;
    int has_bias;
};

struct MlpParams {
    const void *w_in, *w_hid, *w_out;
    const void *b_in, *b_hid, *b_out;
};

struct MlpGradWorkspace {
    float *base;  // fp32, laid out as [w_in | w_hid | w_out | b_in | b_hid | b_out], unpadded
    int w_in, w_hid, w_out, b_in, b_hid, b_out, total;
};

__host__ __device__ inline MlpGradWorkspace grad_workspace_layout(const MlpShape &s, float *base) {
    MlpGradWorkspace w{};
    w.base = base;
    int off = 0;
    w.w_in = off;
    off += s.d_hid * s.d_in;
    w.w_hid = off;
    off += (s.depth - 1) * s.d_hid * s.d_hid;
    w.w_out = off;
    off += s.d_out * s.d_hid;
    w.b_in = off;
    off += s.d_hid;
    w.b_hid = off;
    off += (s.depth - 1) * s.d_hid;
    w.b_out = off;
    off += s.d_out;
    w.total = off;
    return w;
}

// ---- tcgen05 path (fused_mlp_tc.cu) --------------------------------------------------------------
// Each returns TH_OK when it launched, kTcNotApplicable when the case is outside what the
// tcgen05 kernels cover (the caller then uses the mma.sync kernels), or an error code.
constexpr int kTcNotApplicable = -1000;

int mlp_fwd_tc(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
               int64_t rows, int dtype, cudaStream_t stream);

// Forward with the squared-error loss fused into the output epilogue: instead of (or besides, when
// `y` is given) the prediction, each output row leaves as grad = (prediction - target) * grad_scale,
// and sum (prediction - target)^2 is added to *loss_sum.  The prediction is rounded to the 16-bit
// dtype first, so the values equal those of the unfused sequence (forward, then the MSE kernel).
struct MseArgs {
    const void *target;
    long long target_stride;
    void *grad;
    long long grad_stride;
    float *loss_sum;
    float grad_scale;
};
int mlp_fwd_mse_tc(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
                   const MseArgs &mse, int64_t rows, int dtype, cudaStream_t stream);

// Accumulates the parameter gradients into `workspace` (fp32, already zeroed, laid out by
// grad_workspace_layout) and writes grad_x; the caller rounds the workspace into the gradient tensors.
int mlp_bwd_tc(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, const void *go,
               int64_t go_stride, void *gx, int64_t gx_stride, float *workspace, int64_t rows, int dtype,
               cudaStream_t stream);

}  // namespace th
