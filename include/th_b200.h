/*
 * th_b200.h - C ABI of libth_b200.so: sm_100a CUDA kernels for the three fused
 * neural-field operators of triton_helpers (multiresolution hash encoding, fully
 * fused MLP, reversible fused MLP).
 *
 * Conventions shared by every entry point
 *   - extern "C", plain pointers and sizes, no C++ or torch types.
 *   - return value: 0 = launched, < 0 = argument error (TH_ERR_*), > 0 = cudaError_t.
 *     th_last_error_string() gives a human-readable reason for the last non-zero return
 *     on the calling thread.
 *   - pointers named *_dev are device pointers owned by the caller; they must stay valid
 *     until the work queued on `stream` has finished.  Pointers named *_host are read
 *     before the call returns.
 *   - every call is asynchronous on `stream` (a cudaStream_t passed as void*), never
 *     synchronises (the two *_tc_status queries excepted), and never allocates device
 *     memory: scratch is passed in by the caller, sized by the matching *_workspace_bytes
 *     query (th_mlp_bwd_static excepted: it uses an array inside the library image, see there).
 *   - global state of the library: per-device attribute caches behind a mutex, the launch
 *     counter th_launch_count reads (atomic), one device-side status word per tensor-core
 *     kernel family, and the scratch array of th_mlp_bwd_static.  Apart from that last entry
 *     point, calls may come from several host threads and from one process per GPU.
 *   - environment switches, read once per process, for A/B runs and for testing the
 *     fall-back kernels: TH_MLP_LEGACY=1 sends the fused and the reversible MLP to their
 *     mma.sync kernels, TH_MLP_NO_TMA=1 stages weights with plain loads, TH_MLP_NO_PIPE=1
 *     disables the multi-tile tcgen05 MLP kernels, TH_MLP_NO_SLOTS=1 only the backward's
 *     shared-accumulator variant of them, TH_MLP_SLOTS=n caps the forward's row tiles in
 *     flight per CTA, TH_MLP_NO_TMEM_A=1 keeps the forward kernels' hidden activations in
 *     shared-memory operand tiles instead of tensor memory.
 *
 * dtype codes: TH_F32 = 0, TH_F16 = 1, TH_BF16 = 2.
 * activation codes: TH_ACT_NONE = 0, TH_ACT_RELU = 1, TH_ACT_SILU = 2, TH_ACT_RELU2 = 3
 *   (triton_helpers/ops.py:38-66).
 */
#ifndef TH_B200_H
#define TH_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TH_F32 0
#define TH_F16 1
#define TH_BF16 2

#define TH_ACT_NONE 0
#define TH_ACT_RELU 1
#define TH_ACT_SILU 2
#define TH_ACT_RELU2 3

#define TH_OK 0
#define TH_ERR_BAD_ARG (-1)      /* null pointer, negative size, unknown code          */
#define TH_ERR_UNSUPPORTED (-2)  /* shape / dtype combination has no kernel            */
#define TH_ERR_ALIGNMENT (-3)    /* a pointer or stride breaks a documented alignment  */
#define TH_ERR_WORKSPACE (-4)    /* scratch buffer missing or too small                */
#define TH_ERR_DEVICE (-5)       /* a kernel reported a failed internal check          */

#define TH_MAX_LEVELS 32
#define TH_MAX_DIMS 3

/* ABI version, bumped on any signature change. */
int th_version(void);

/* Text for the last non-zero return value on this host thread ("" if none). */
const char *th_last_error_string(void);

/* Kernels launched by this library in this process so far, over all entry points and threads
 * (no counterpart in triton_helpers; lets a harness state how many of its launches were these). */
long long th_launch_count(void);

/* ------------------------------------------------------------------------------------------
 * Multiresolution hash encoding
 *
 * Table layout: one (total_rows, n_feats) row-major array, level l occupying rows
 * [level_offset[l], level_offset[l] + level_rows[l]).  A level is dense when
 * (res + 1)^n_dims <= level_rows[l], hashed otherwise.  The three level arrays are what
 * triton_helpers/layers/hash_encoding/helpers.py:26-115 computes on the host.
 * ------------------------------------------------------------------------------------------ */

/*
 * Forward: replaces the Triton launch loop of HashEncoding.forward
 * (triton_helpers/layers/hash_encoding/kernel.py:575-590 -> _fwd_kernel :175-306).
 *
 *   coords_dev      (n_points, n_dims) coordinates in [0, scale], element (i, d) at
 *                   coords_dev[i * coord_stride_n + d * coord_stride_d] (strides in elements)
 *   coord_dtype     TH_F32 / TH_F16 / TH_BF16; values are promoted to float32
 *   table_dev       the concatenated table, table_dtype, rows aligned to their own size
 *   out_dev         (n_points, >= n_levels * n_feats) in table_dtype, row stride
 *                   out_stride_n elements; columns [level_begin*F, level_end*F) are written
 *   level_res_host / level_rows_host / level_offset_host   n_levels entries each
 *   primes_host     n_dims hashing primes (kernel.py:25-27)
 *   level_begin/end half-open range of levels processed by this call (the reference's
 *                   `divider` passes); 0, n_levels for everything
 */
int th_hash_fwd(const void *coords_dev, int64_t coord_stride_n, int64_t coord_stride_d, int coord_dtype,
                const void *table_dev, int table_dtype, void *out_dev, int64_t out_stride_n,
                int64_t n_points, int n_dims, int n_feats, int n_levels,
                const int32_t *level_res_host, const int64_t *level_rows_host, const int64_t *level_offset_host,
                const int64_t *primes_host, float scale, int level_begin, int level_end, void *stream);

/*
 * Backward: replaces HashEncoding.backward's launch loop
 * (triton_helpers/layers/hash_encoding/kernel.py:641-669 -> _bwd_kernel :322-440).
 * Adds weight * grad_out into grad_table_dev with warp-aggregated red.global atomics;
 * the caller zero-fills grad_table_dev first (kernel.py:636 does the same with zeros_like).
 *
 *   grad_out_dev    (n_points, >= n_levels * n_feats) in table_dtype, row stride go_stride_n
 *   grad_table_dev  same shape and dtype as the table
 */
int th_hash_bwd(const void *coords_dev, int64_t coord_stride_n, int64_t coord_stride_d, int coord_dtype,
                const void *grad_out_dev, int64_t go_stride_n, void *grad_table_dev, int table_dtype,
                int64_t n_points, int n_dims, int n_feats, int n_levels,
                const int32_t *level_res_host, const int64_t *level_rows_host, const int64_t *level_offset_host,
                const int64_t *primes_host, float scale, int level_begin, int level_end, void *stream);

/* Device-side status word of the encoding kernels: 0 = fine, 1 = a shared-memory accumulation of the
 * backward pass (compare-and-swap loop, bounded) gave up and dropped an update.  Synchronises the device.
 * No counterpart in the reference. */
int th_hash_status(void);

/*
 * Test hook for the bit-exact index check: the row index (relative to its level) and the
 * interpolation weight of every corner, computed the way the two kernels above compute them: two
 * lanes per point, each calling the kernels' own per-side index and weight functions.  Stands in for the reference's ad-hoc test kernels around
 * embedding_lookup / get_interpolation_weights
 * (tests/test_layers/test_hash_encoding.py:176-215 of the reference).
 *
 *   idx_out_dev     int64  (n_points, n_levels, 2^n_dims)
 *   weight_out_dev  float  (n_points, n_levels, 2^n_dims), may be null
 */
int th_hash_debug_indices(const void *coords_dev, int64_t coord_stride_n, int64_t coord_stride_d, int coord_dtype,
                          int64_t *idx_out_dev, float *weight_out_dev, int64_t n_points, int n_dims, int n_levels,
                          const int32_t *level_res_host, const int64_t *level_rows_host,
                          const int64_t *primes_host, float scale, void *stream);

/* ------------------------------------------------------------------------------------------
 * Fully fused MLP:  y = W_out . act(W_hid[depth-2] . ... act(W_in . x + b_in) ...) + b_out
 *
 * Weights are row-major (out, in) like nn.Linear: w_in (d_hidden, d_in), w_hid
 * ((depth-1) * d_hidden, d_hidden), w_out (d_out, d_hidden); biases b_in (d_hidden), b_hid
 * (depth-1, d_hidden), b_out (d_out), either all given or all null.  depth counts the activated
 * layers (input layer + depth-1 hidden layers), as in
 * triton_helpers/layers/fully_fused_mlp/kernel.py:534-542.  Every dimension is <= 64 and
 * d_hidden is a power of two >= 16 (kernel.py:525-531).  dtype is TH_F16 or TH_BF16 for x, all
 * parameters, outputs and gradients; accumulation is fp32 (fp16_acc is accepted and ignored).
 * x / out / grad rows are `*_stride` elements apart with unit stride inside a row.
 * ------------------------------------------------------------------------------------------ */

/* Forward: replaces the launch in _fully_fused_mlp.forward
 * (triton_helpers/layers/fully_fused_mlp/kernel.py:553-562 -> _fwd_kernel :198-261). */
int th_mlp_fwd(const void *x_dev, int64_t x_stride, const void *w_in_dev, const void *b_in_dev,
               const void *w_hid_dev, const void *b_hid_dev, const void *w_out_dev, const void *b_out_dev,
               void *out_dev, int64_t out_stride, int64_t rows, int d_in, int d_hidden, int d_out, int depth,
               int activation, int dtype, int fp16_acc, void *stream);

/* Forward with the squared-error loss fused into the output layer (no counterpart in triton_helpers;
 * the step of a training loop that follows _fully_fused_mlp.forward): grad[r, c] = (y[r, c] -
 * target[r, c]) * grad_scale in `dtype`, with y rounded to `dtype` first, and sum (y - target)^2 added
 * to *loss_sum_dev (fp32, caller-zeroed; may be null).  out_dev may be null when the prediction itself
 * is not needed.  Returns TH_ERR_UNSUPPORTED when the case is outside the tensor-core forward kernel
 * (d_in or d_out not multiples of 8, misaligned rows, float32): call th_mlp_fwd and th_mse_grad then. */
int th_mlp_fwd_mse(const void *x_dev, int64_t x_stride, const void *w_in_dev, const void *b_in_dev,
                   const void *w_hid_dev, const void *b_hid_dev, const void *w_out_dev, const void *b_out_dev,
                   void *out_dev, int64_t out_stride, const void *target_dev, int64_t target_stride, void *grad_dev,
                   int64_t grad_stride, float *loss_sum_dev, float grad_scale, int64_t rows, int d_in, int d_hidden,
                   int d_out, int depth, int activation, int dtype, void *stream);

/* Device-side status word of the tensor-core MLP kernels (th_mlp_*, th_field_*): 0 = fine, non-zero =
 * one of their bounded waits ran out (the kernel then returned early and its results are invalid).
 * Synchronises the device.  No counterpart in the reference. */
int th_mlp_tc_status(void);

/* 1 when the tensor-core MLP kernels can load their weights by TMA in this process (the driver
 * exposes cuTensorMapEncodeTiled), 0 when they stage them with plain loads.  No counterpart in the
 * reference. */
int th_mlp_tma_available(void);

/* Bytes of fp32 scratch th_mlp_bwd needs (one float per parameter); -1 for an unsupported shape. */
int64_t th_mlp_workspace_bytes(int d_in, int d_hidden, int d_out, int depth);

/* Backward: replaces the launch and the torch .sum(0) reductions of _fully_fused_mlp.backward
 * (triton_helpers/layers/fully_fused_mlp/kernel.py:599-633 -> _bwd_kernel_rfs :326-500).
 * Writes grad_x (rows, d_in) and the parameter gradients in `dtype`; any gradient pointer may be
 * null to skip it.  workspace_dev is caller-provided scratch of th_mlp_workspace_bytes() bytes;
 * the call zero-fills it, accumulates fp32 partial sums there and rounds once at the end.  When the
 * queued work has finished the workspace still holds those fp32 sums, laid out
 * [w_in | w_hid | w_out | b_in | b_hid | b_out] (each row-major, unpadded): a caller that wants the
 * gradients in fp32, or normalised before they are rounded, reads them there (th_scale_cast). */
int th_mlp_bwd(const void *x_dev, int64_t x_stride, const void *w_in_dev, const void *b_in_dev,
               const void *w_hid_dev, const void *b_hid_dev, const void *w_out_dev, const void *b_out_dev,
               const void *grad_out_dev, int64_t go_stride, void *grad_x_dev, int64_t gx_stride,
               void *grad_w_in_dev, void *grad_b_in_dev, void *grad_w_hid_dev, void *grad_b_hid_dev,
               void *grad_w_out_dev, void *grad_b_out_dev, void *workspace_dev, int64_t workspace_bytes,
               int64_t rows, int d_in, int d_hidden, int d_out, int depth, int activation, int dtype,
               int fp16_acc, void *stream);

/* Backward of the fused MLP for callers that cannot hand over scratch memory.  It has no
 * counterpart in the reference.  Arguments and results are those of th_mlp_bwd without the
 * workspace pair: the fp32 scratch is a 256 KB array that is part of the library image, so every
 * GPU that loads the library carries it until the process ends, and nothing is allocated or freed
 * by the call.  Meant for hosts where device memory cannot be requested at call time (the
 * application gave the whole device to its own pool, a latency-critical loop must avoid the
 * device-wide synchronisation an allocation implies, or a C caller has no allocator at hand).
 *   - Networks whose parameters exceed th_mlp_bwd_static_max_bytes() / 4 floats are refused with
 *     TH_ERR_WORKSPACE; use th_mlp_bwd with caller scratch for those.
 *   - The first call on a device looks up the array's device address (that device must be
 *     current); make that first call before any stream capture begins.
 *   - All calls on a device share the one array, which still holds the previous call's sums when
 *     the next begins: each call clears the part it uses on its stream before accumulating, and
 *     two calls whose GPU work overlaps (different streams or threads) race on it. */
int th_mlp_bwd_static(const void *x_dev, int64_t x_stride, const void *w_in_dev, const void *b_in_dev,
                      const void *w_hid_dev, const void *b_hid_dev, const void *w_out_dev, const void *b_out_dev,
                      const void *grad_out_dev, int64_t go_stride, void *grad_x_dev, int64_t gx_stride,
                      void *grad_w_in_dev, void *grad_b_in_dev, void *grad_w_hid_dev, void *grad_b_hid_dev,
                      void *grad_w_out_dev, void *grad_b_out_dev, int64_t rows, int d_in, int d_hidden, int d_out,
                      int depth, int activation, int dtype, int fp16_acc, void *stream);

/* Size in bytes of the built-in scratch th_mlp_bwd_static uses (262144). */
int64_t th_mlp_bwd_static_max_bytes(void);

/* ------------------------------------------------------------------------------------------
 * Reversible (additive coupling) fused MLP.  NO COUNTERPART IN THE REFERENCE: triton_helpers
 * has no reversible operator; the conventions (stacked (out, in) weights, 16-bit operands,
 * fp32 accumulation) are those of its fused MLP (fully_fused_mlp/kernel.py:503-686).
 *
 *   x = [x1 | x2] (rows, d_model), halves of width H = d_model / 2.  Block k:
 *     y1 = x1 + F_k(x2),   F_k(u) = W_f2[k] . act(W_f1[k] . u + b_f1[k]) + b_f2[k]
 *     y2 = x2 + G_k(y1),   G_k(u) = W_g2[k] . act(W_g1[k] . u + b_g1[k]) + b_g2[k]
 *   w_f1, w_g1: (blocks * d_hidden, H);  w_f2, w_g2: (blocks * H, d_hidden), row-major, 16-byte
 *   aligned; biases (blocks, d_hidden) / (blocks, H), all given or all null.  d_model is a
 *   multiple of 32 up to 128, d_hidden a multiple of 16 up to 64; dtype TH_F16 or TH_BF16.
 * ------------------------------------------------------------------------------------------ */

int th_rev_fwd(const void *x_dev, int64_t x_stride, const void *w_f1_dev, const void *w_f2_dev,
               const void *w_g1_dev, const void *w_g2_dev, const void *b_f1_dev, const void *b_f2_dev,
               const void *b_g1_dev, const void *b_g2_dev, void *out_dev, int64_t out_stride, int64_t rows,
               int d_model, int d_hidden, int blocks, int activation, int dtype, void *stream);

/* Device-side status word of the reversible tensor-core kernels (0 = fine, 1 = a bounded wait ran
 * out and results are invalid).  Synchronises the device. */
int th_rev_tc_status(void);

/* Bytes of fp32 scratch th_rev_bwd needs for `rows` rows: one private copy of all weight-gradient
 * accumulators per resident CTA (about 0.5 MB per CTA for 8 blocks of 64 x 64). */
int64_t th_rev_workspace_bytes(int64_t rows, int d_model, int d_hidden, int blocks);

/* Backward from the stack's OUTPUT y (no stored activations): reconstructs the inputs block by
 * block (x2 = y2 - G(y1), x1 = y1 - F(x2)) while forming the gradients.  Writes grad_x, the
 * eight parameter gradients (any may be null) and, when x_rec_dev is not null, the reconstructed
 * input, for checking the reconstruction error. */
int th_rev_bwd(const void *y_dev, int64_t y_stride, const void *w_f1_dev, const void *w_f2_dev,
               const void *w_g1_dev, const void *w_g2_dev, const void *b_f1_dev, const void *b_f2_dev,
               const void *b_g1_dev, const void *b_g2_dev, const void *grad_out_dev, int64_t go_stride,
               void *grad_x_dev, int64_t gx_stride, void *x_rec_dev, int64_t xr_stride, void *grad_w_f1_dev,
               void *grad_w_f2_dev, void *grad_w_g1_dev, void *grad_w_g2_dev, void *grad_b_f1_dev,
               void *grad_b_f2_dev, void *grad_b_g1_dev, void *grad_b_g2_dev, void *workspace_dev,
               int64_t workspace_bytes, int64_t rows, int d_model, int d_hidden, int blocks, int activation,
               int dtype, void *stream);

/* ------------------------------------------------------------------------------------------
 * Hash encoding and fused MLP in one kernel per direction.  NO ENTRY POINT OF THE REFERENCE
 * CORRESPONDS: triton_helpers launches the two layers separately, and only remarks that the encoding
 * "will be used with a fully fused MLP" with its L * F output columns staying on chip
 * (triton_helpers/layers/hash_encoding/kernel.py:241-243).  Semantics are those of th_hash_fwd followed
 * by th_mlp_fwd / th_mlp_fwd_mse, and of th_mlp_bwd followed by th_hash_bwd, with the MLP's input
 * width d_in = n_levels * n_feats.  Table, weights, features and gradients share one 16-bit `dtype`.
 * Covered: n_dims 2 or 3, n_feats 2 or 4, n_levels * n_feats a multiple of 16 up to 64, ReLU or no
 * activation, 16-byte aligned rows; biases in the forward only.  Anything else returns
 * TH_ERR_UNSUPPORTED and the caller runs the separate entry points.
 * ------------------------------------------------------------------------------------------ */

/* Forward.  The encoding of a 128-point tile is written straight into the first GEMM's operand tile.
 *   feats_out_dev   (n_points, n_levels * n_feats), row stride feats_stride: the encoding, written only
 *                   when not null (th_field_bwd needs it)
 *   out_dev         (n_points, d_out) prediction, may be null when a target is given
 *   target_dev      when not null: grad_dev[r, c] = (prediction - target) * grad_scale (prediction rounded
 *                   to `dtype` first) and sum (prediction - target)^2 is added to *loss_sum_dev (fp32,
 *                   caller-zeroed, may be null), as th_mlp_fwd_mse does */
int th_field_fwd(const void *coords_dev, int64_t coord_stride_n, int64_t coord_stride_d, int coord_dtype,
                 const void *table_dev, int n_dims, int n_feats, int n_levels, const int32_t *level_res_host,
                 const int64_t *level_rows_host, const int64_t *level_offset_host, const int64_t *primes_host,
                 float scale, const void *w_in_dev, const void *b_in_dev, const void *w_hid_dev,
                 const void *b_hid_dev, const void *w_out_dev, const void *b_out_dev, int d_hidden, int d_out,
                 int depth, int activation, void *feats_out_dev, int64_t feats_stride, void *out_dev,
                 int64_t out_stride, const void *target_dev, int64_t target_stride, void *grad_dev,
                 int64_t grad_stride, float *loss_sum_dev, float grad_scale, int64_t n_points, int dtype,
                 void *stream);

/* Bytes of fp32 scratch th_field_bwd needs: th_mlp_workspace_bytes of the same network. */
int64_t th_field_workspace_bytes(int n_levels, int n_feats, int d_hidden, int d_out, int depth);

/* Backward (bias-free networks).  From the encoding th_field_fwd wrote (feats_dev) and the gradient of
 * the MLP's output it recomputes the activations, forms the weight gradients (fp32 sums in
 * workspace_dev, laid out like th_mlp_bwd's: [w_in | w_hid | w_out]; the call zero-fills it first) and
 * the gradient of the encoding, which never leaves the SM: each tile's rows are scattered into
 * grad_table_dev (same shape and dtype as the table; the caller zero-fills it, as for th_hash_bwd).
 * grad_feats_dev, when not null, also receives the (n_points, n_levels * n_feats) feature gradient. */
int th_field_bwd(const void *coords_dev, int64_t coord_stride_n, int64_t coord_stride_d, int coord_dtype,
                 int n_dims, int n_feats, int n_levels, const int32_t *level_res_host,
                 const int64_t *level_rows_host, const int64_t *level_offset_host, const int64_t *primes_host,
                 float scale, const void *w_in_dev, const void *w_hid_dev, const void *w_out_dev, int d_hidden,
                 int d_out, int depth, int activation, const void *feats_dev, int64_t feats_stride,
                 const void *grad_out_dev, int64_t go_stride, void *grad_table_dev, void *grad_feats_dev,
                 int64_t gf_stride, void *workspace_dev, int64_t workspace_bytes, int64_t n_points, int dtype,
                 void *stream);

/* ------------------------------------------------------------------------------------------
 * Element-wise steps of a training step around the fused operators.  NO COUNTERPART IN THE
 * REFERENCE (triton_helpers stops at forward/backward); they keep the data-parallel
 * neural-field step on hand-written kernels from the loss to the parameter update.
 * All tensors 32-byte aligned and contiguous.
 * ------------------------------------------------------------------------------------------ */

/* grad[i] = (pred[i] - target[i]) * grad_scale in `dtype`; adds sum (pred - target)^2 to
 * *loss_sum_dev (fp32, caller-zeroed; may be null). */
int th_mse_grad(const void *pred_dev, const void *target_dev, void *grad_dev, float *loss_sum_dev,
                int64_t n_elems, float grad_scale, int dtype, void *stream);

/* One Adam step (torch.optim.Adam semantics, no weight decay, no amsgrad) on `dtype` parameters
 * with fp32 moments: g = grad * grad_scale; m, v updated; param -= lr / (1 - beta1^step) * m /
 * (sqrt(v) / sqrt(1 - beta2^step) + eps).  step counts from 1.  With zero_grad != 0 the gradient
 * buffer is cleared in the same pass (the table gradient must start at zero every step,
 * triton_helpers/layers/hash_encoding/kernel.py:636).  An element whose scaled gradient is not
 * finite keeps its parameter and moments and adds one to *skipped_dev (a device int the caller
 * zeroes and reads; may be null). */
int th_adam_step(void *param_dev, void *grad_dev, float *exp_avg_dev, float *exp_avg_sq_dev, int64_t n_elems,
                 float lr, float beta1, float beta2, float eps, int step, float grad_scale, int zero_grad,
                 int dtype, int *skipped_dev, void *stream);

/* dst[i] = src[i] * scale rounded to `dtype`: turns the fp32 sums th_mlp_bwd leaves in its workspace
 * (laid out [w_in | w_hid | w_out | b_in | b_hid | b_out]) into a normalised 16-bit gradient buffer. */
int th_scale_cast(const float *src_dev, void *dst_dev, int64_t n_elems, float scale, int dtype, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* TH_B200_H */
