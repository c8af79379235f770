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
 *     synchronises, and never allocates device memory: scratch is passed in by the
 *     caller, sized by the matching *_workspace_bytes query.
 *   - the library keeps no mutable global state besides per-device attribute caches, so
 *     it can be driven from several host threads and from one process per GPU.
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

/*
 * Test hook for the bit-exact index check: the row index (relative to its level) and the
 * interpolation weight of every corner, computed by the same device functions the two
 * kernels above use.  Stands in for the reference's ad-hoc test kernels around
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

#ifdef __cplusplus
}
#endif
#endif /* TH_B200_H */
