// Warp-level tile primitives for the small-MLP kernels: 16x8x16 tensor-core MMAs with
// fp32 accumulation, ldmatrix operand loads from padded shared-memory tiles, and the
// register shuffles that turn an accumulator tile into the next layer's A operand.
//
// Fragment conventions (lane = 4 * g + t, g in 0..7, t in 0..3), PTX mma.m16n8k16:
//   A (16 x 16, row): a0 = (row g,   k 2t..2t+1)   a1 = (row g+8, k 2t..2t+1)
//                     a2 = (row g,   k 2t+8..+9)   a3 = (row g+8, k 2t+8..+9)
//   B (16 x 8,  col): b0 = (k 2t..2t+1, n g)       b1 = (k 2t+8..+9, n g)
//   C (16 x 8):       c0,c1 = (row g, n 2t..2t+1)  c2,c3 = (row g+8, n 2t..2t+1)
// Two neighbouring C tiles (n-tiles 2j, 2j+1), rounded to 16 bits, are exactly the A
// fragment of k-tile j, so activations chain from layer to layer in registers.
#pragma once

#include "common.cuh"

namespace th {

constexpr int kMaxDim = 64;          // largest feature width of any layer
constexpr int kKTiles = kMaxDim / 16;
constexpr int kNTiles = kMaxDim / 8;
constexpr int kSmemPad = 8;          // extra 16-bit elements per row: 144-byte rows are ldmatrix conflict-free

__host__ __device__ inline int pad16(int v) { return (v + 15) & ~15; }

template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);

template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                        uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t smem_addr(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *row_ptr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr(row_ptr)));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *row_ptr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr(row_ptr)));
}

template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack_pair<__half>(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&h);
}

template <typename T>
__device__ __forceinline__ float2 unpack_pair(uint32_t v);
template <>
__device__ __forceinline__ float2 unpack_pair<__half>(uint32_t v) {
    return __half22float2(*reinterpret_cast<const __half2 *>(&v));
}
template <>
__device__ __forceinline__ float2 unpack_pair<__nv_bfloat16>(uint32_t v) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&v));
}

// Round a value to the 16-bit storage type and back (what "stored between layers" means).
template <typename T>
__device__ __forceinline__ float round_to(float v) { return to_float<T>(from_float<T>(v)); }

// ---- activations (triton_helpers/ops.py:38-66) ----------------------------------------------

__device__ __forceinline__ float sigmoidf(float z) { return 1.f / (1.f + __expf(-z)); }

__device__ __forceinline__ float activate(int act, float z) {
    switch (act) {
        case TH_ACT_RELU: return z < 0.f ? 0.f : z;
        case TH_ACT_SILU: return z * sigmoidf(z);
        case TH_ACT_RELU2: return fmaxf(z, 0.f) * z;
        default: return z;
    }
}

// d act(z) / dz * grad
__device__ __forceinline__ float activate_grad(int act, float z, float grad) {
    switch (act) {
        case TH_ACT_RELU: return z > 0.f ? grad : 0.f;
        case TH_ACT_SILU: {
            const float s = sigmoidf(z);
            return grad * s * (z * (1.f - s) + 1.f);
        }
        case TH_ACT_RELU2: return z > 0.f ? grad * (2.f * z) : 0.f;
        default: return grad;
    }
}

// ---- one dense layer on a warp's 16-row tiles ------------------------------------------------
// acc[mt][nt] += A[mt] (16 x 16*k_tiles) * W^T, W stored [n][k] row-major in shared memory with
// `stride` elements per row (zero padded to multiples of 16 in both directions).
template <typename T, int MT>
__device__ __forceinline__ void warp_gemm_nk(float (&acc)[MT][kNTiles][4], const uint32_t (&a)[MT][kKTiles][4],
                                             const T *w, int stride, int k_tiles, int n_tiles) {
    const int lane = threadIdx.x & 31;
    const int mtx = lane >> 3, r = lane & 7;
    // matrix 0/1: n-tile 2np, k halves 0/1; matrix 2/3: n-tile 2np+1
    const T *lane_ptr = w + (8 * (mtx >> 1) + r) * stride + 8 * (mtx & 1);
#pragma unroll
    for (int kt = 0; kt < kKTiles; ++kt) {
        if (kt < k_tiles) {
#pragma unroll
            for (int np = 0; np < kNTiles / 2; ++np) {
                if (2 * np < n_tiles) {
                    uint32_t b[4];
                    ldmatrix_x4(b, lane_ptr + 16 * np * stride + 16 * kt);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        mma16816<T>(acc[mt][2 * np], a[mt][kt], b[0], b[1]);
                        mma16816<T>(acc[mt][2 * np + 1], a[mt][kt], b[2], b[3]);
                    }
                }
            }
        }
    }
}

// acc[mt][nt] += A[mt] (16 x 16*k_tiles) * W, W stored [k][n] row-major (used for dgrad: the
// same [out][in] weight tile read along its other axis via ldmatrix.trans).
template <typename T, int MT>
__device__ __forceinline__ void warp_gemm_kn(float (&acc)[MT][kNTiles][4], const uint32_t (&a)[MT][kKTiles][4],
                                             const T *w, int stride, int k_tiles, int n_tiles) {
    const int lane = threadIdx.x & 31;
    const int mtx = lane >> 3, r = lane & 7;
    // matrix 0/1: k halves 0/1 of n-tile 2np; matrix 2/3: n-tile 2np+1
    const T *lane_ptr = w + (8 * (mtx & 1) + r) * stride + 8 * (mtx >> 1);
#pragma unroll
    for (int kt = 0; kt < kKTiles; ++kt) {
        if (kt < k_tiles) {
#pragma unroll
            for (int np = 0; np < kNTiles / 2; ++np) {
                if (2 * np < n_tiles) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, lane_ptr + 16 * kt * stride + 16 * np);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        mma16816<T>(acc[mt][2 * np], a[mt][kt], b[0], b[1]);
                        mma16816<T>(acc[mt][2 * np + 1], a[mt][kt], b[2], b[3]);
                    }
                }
            }
        }
    }
}

template <int MT>
__device__ __forceinline__ void fill_acc(float (&acc)[MT][kNTiles][4], const float *bias /* smem or null */) {
    const int t = threadIdx.x & 3;
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt) {
        const float b0 = bias ? bias[8 * nt + 2 * t] : 0.f;
        const float b1 = bias ? bias[8 * nt + 2 * t + 1] : 0.f;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            acc[mt][nt][0] = b0;
            acc[mt][nt][1] = b1;
            acc[mt][nt][2] = b0;
            acc[mt][nt][3] = b1;
        }
    }
}

// Accumulator tiles -> activation -> 16-bit A fragments of the next layer.
template <typename T, int MT>
__device__ __forceinline__ void acc_to_frags(uint32_t (&a)[MT][kKTiles][4], const float (&acc)[MT][kNTiles][4],
                                             int act) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int kt = 0; kt < kKTiles; ++kt) {
            a[mt][kt][0] = pack_pair<T>(activate(act, acc[mt][2 * kt][0]), activate(act, acc[mt][2 * kt][1]));
            a[mt][kt][1] = pack_pair<T>(activate(act, acc[mt][2 * kt][2]), activate(act, acc[mt][2 * kt][3]));
            a[mt][kt][2] = pack_pair<T>(activate(act, acc[mt][2 * kt + 1][0]), activate(act, acc[mt][2 * kt + 1][1]));
            a[mt][kt][3] = pack_pair<T>(activate(act, acc[mt][2 * kt + 1][2]), activate(act, acc[mt][2 * kt + 1][3]));
        }
}

// ---- global <-> fragment ---------------------------------------------------------------------
// Rows [row0, row0 + 16) x columns [0, cols) of a row-major matrix into A fragments; rows >=
// n_rows and columns >= cols read as zero.  `pairs_ok`: cols even, base and stride 4-byte aligned.
template <typename T>
__device__ __forceinline__ void load_rows_as_frags(uint32_t (&a)[kKTiles][4], const T *base, long long stride,
                                                   long long row0, long long n_rows, int cols, int k_tiles,
                                                   bool pairs_ok) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int kt = 0; kt < kKTiles; ++kt) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const long long row = row0 + g + 8 * (q & 1);
            const int col = 16 * kt + 2 * t + 8 * (q >> 1);
            uint32_t v = 0;
            if (kt < k_tiles && row < n_rows && col < cols) {
                const T *p = base + row * stride + col;
                if (pairs_ok) {
                    v = __ldcs(reinterpret_cast<const unsigned int *>(p));
                } else {
                    const unsigned short lo = *reinterpret_cast<const unsigned short *>(p);
                    const unsigned short hi = (col + 1 < cols) ? *reinterpret_cast<const unsigned short *>(p + 1) : 0;
                    v = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
                }
            }
            a[kt][q] = v;
        }
    }
}

// Accumulator tiles (fp32) -> rows of a row-major matrix, rounded to T.
template <typename T>
__device__ __forceinline__ void store_acc_rows(T *base, long long stride, long long row0, long long n_rows, int cols,
                                               int n_tiles, const float (&acc)[kNTiles][4], bool pairs_ok) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt) {
        if (nt < n_tiles) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const long long row = row0 + g + 8 * h;
                const int col = 8 * nt + 2 * t;
                if (row < n_rows && col < cols) {
                    T *p = base + row * stride + col;
                    if (pairs_ok) {
                        __stcs(reinterpret_cast<unsigned int *>(p), pack_pair<T>(acc[nt][2 * h], acc[nt][2 * h + 1]));
                    } else {
                        p[0] = from_float<T>(acc[nt][2 * h]);
                        if (col + 1 < cols) p[1] = from_float<T>(acc[nt][2 * h + 1]);
                    }
                }
            }
        }
    }
}

// A fragments <-> a padded shared-memory tile [rows][stride] (conflict-free with stride = width + 8).
__device__ __forceinline__ void frags_to_smem(void *tile, int stride, int row0, const uint32_t (&a)[kKTiles][4],
                                              int k_tiles) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    unsigned short *base = static_cast<unsigned short *>(tile);
#pragma unroll
    for (int kt = 0; kt < kKTiles; ++kt)
        if (kt < k_tiles)
#pragma unroll
            for (int q = 0; q < 4; ++q)
                *reinterpret_cast<uint32_t *>(base + (row0 + g + 8 * (q & 1)) * stride + 16 * kt + 2 * t + 8 * (q >> 1)) =
                    a[kt][q];
}

__device__ __forceinline__ void smem_to_frags(uint32_t (&a)[kKTiles][4], const void *tile, int stride, int row0,
                                              int k_tiles) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const unsigned short *base = static_cast<const unsigned short *>(tile);
#pragma unroll
    for (int kt = 0; kt < kKTiles; ++kt)
#pragma unroll
        for (int q = 0; q < 4; ++q)
            a[kt][q] = kt < k_tiles ? *reinterpret_cast<const uint32_t *>(base + (row0 + g + 8 * (q & 1)) * stride +
                                                                          16 * kt + 2 * t + 8 * (q >> 1))
                                    : 0u;
}

// Copy a row-major [rows][cols] weight matrix from global memory into a zero-padded
// shared-memory tile [rows_pad][cols_pad + kSmemPad].  All threads of the CTA take part.
template <typename T>
__device__ __forceinline__ void stage_weight(T *dst, const T *src, int rows, int cols, int rows_pad, int cols_pad) {
    const int stride = cols_pad + kSmemPad;
    for (int e = threadIdx.x; e < rows_pad * stride; e += blockDim.x) {
        const int r = e / stride, c = e - r * stride;
        dst[e] = (r < rows && c < cols) ? src[r * cols + c] : from_float<T>(0.f);
    }
}

}  // namespace th
