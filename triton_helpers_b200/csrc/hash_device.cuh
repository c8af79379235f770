// Device and host building blocks of the multiresolution hash encoding shared by the stand-alone
// kernels (hash_encoding.cu) and the kernels that fuse the encoding with the MLP (neural_field.cu):
// level parameters, coordinate loads, the per-level index / weight arithmetic, row gathers and vector
// reductions.  The arithmetic follows the CPU path of
// triton_helpers/layers/hash_encoding/kernel.py:443-479, which is the parity contract:
//   cell   = floor(x * res)                 one float32 multiply per level, no FMA contraction
//   dense  : index = sum_d corner_d * res^d
//   hashed : index = xor_d(corner_d * prime_d) mod rows
//   t      = x * res - cell ;  weight(corner) = prod_d (bit_d ? t_d : 1 - t_d), axis order 0,1,2
// Everything has internal linkage (one copy per translation unit).
#pragma once

#include "common.cuh"

#include <type_traits>

namespace th {
namespace {

constexpr int kThreads = 256;
constexpr uint32_t kAggregateMaxRes = 64;  // backward: finest grid on which warp aggregation is attempted

struct LevelParams {
    uint32_t res[TH_MAX_LEVELS];
    uint32_t rows[TH_MAX_LEVELS];
    unsigned long long offset[TH_MAX_LEVELS];  // first row of the level
    uint32_t primes[TH_MAX_DIMS];
    uint32_t hashed_mask;  // bit l: level l uses the spatial hash
    uint32_t pow2_mask;    // bit l: rows[l] is a power of two
    float scale;
};

struct CoordView {
    const void *ptr;
    long long stride_n, stride_d;  // in elements
    int dtype;
    int packed_f32;  // float32, contiguous (stride_d == 1, stride_n == D) and 16-byte aligned
};

// ---- coordinates ----------------------------------------------------------------------------

template <int D>
__device__ __forceinline__ void load_coords_strided(const CoordView &cv, long long i, float (&x)[D]) {
#pragma unroll
    for (int d = 0; d < D; ++d) {
        const long long e = i * cv.stride_n + d * cv.stride_d;
        if (cv.dtype == TH_F32) {
            x[d] = __ldcs(static_cast<const float *>(cv.ptr) + e);
        } else if (cv.dtype == TH_F16) {
            x[d] = __half2float(static_cast<const __half *>(cv.ptr)[e]);
        } else {
            x[d] = __bfloat162float(static_cast<const __nv_bfloat16 *>(cv.ptr)[e]);
        }
    }
}

// LPP lanes work on one point, so a CTA covers kThreads / LPP points.  Their D floats each are
// contiguous: fetch them as float4, then every lane picks the D values of its point.
// `tile` is the index of the CTA's point tile (blockIdx.x for one tile per CTA).  Contains a CTA barrier
// on the packed path; `stage` may be reused after the next CTA barrier.
template <int D, int LPP>
__device__ __forceinline__ bool load_coords(const CoordView &cv, long long n_points, long long tile, float (&x)[D], float *stage) {
    constexpr int kPoints = kThreads / LPP;
    const int local = threadIdx.x / LPP;
    const long long i = tile * kPoints + local;
    if (cv.packed_f32) {
        const long long first = tile * kPoints * D;  // multiple of 4
        const long long total = n_points * D;
        const float *src = static_cast<const float *>(cv.ptr);
        for (int v = threadIdx.x; v < kPoints * D / 4; v += kThreads) {
            const long long e = first + 4ll * v;
            if (e + 3 < total) {
                reinterpret_cast<float4 *>(stage)[v] = __ldcs(reinterpret_cast<const float4 *>(src + e));
            } else {
#pragma unroll
                for (int k = 0; k < 4; ++k) stage[4 * v + k] = (e + k < total) ? src[e + k] : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int d = 0; d < D; ++d) x[d] = stage[local * D + d];
    } else if (i < n_points) {
        load_coords_strided<D>(cv, i, x);
    }
    return i < n_points;
}

// ---- per-level index / weight arithmetic ----------------------------------------------------

template <int D>
__device__ __forceinline__ void locate(const float (&x)[D], uint32_t res, uint32_t (&cell)[D], float (&t)[D]) {
    const float r = static_cast<float>(res);
#pragma unroll
    for (int d = 0; d < D; ++d) {
        const float pos = __fmul_rn(x[d], r);
        const float fl = floorf(pos);
        t[d] = __fsub_rn(pos, fl);
        cell[d] = static_cast<uint32_t>(fl);  // saturating conversion: negative -> 0
    }
}

template <int D>
__device__ __forceinline__ void corner_weights(const float (&t)[D], float (&w)[1 << D]) {
    float lo[D];
#pragma unroll
    for (int d = 0; d < D; ++d) lo[d] = __fsub_rn(1.f, t[d]);
#pragma unroll
    for (int c = 0; c < (1 << D); ++c) {
        float p = (c & 1) ? t[0] : lo[0];
#pragma unroll
        for (int d = 1; d < D; ++d) p = __fmul_rn(p, ((c >> d) & 1) ? t[d] : lo[d]);
        w[c] = p;
    }
}

template <int D>
__device__ __forceinline__ void corner_indices(const uint32_t (&cell)[D], const LevelParams &P, int level,
                                               uint32_t (&idx)[1 << D]) {
    const uint32_t res = P.res[level];
    const uint32_t rows = P.rows[level];
    const bool hashed = (P.hashed_mask >> level) & 1u;
    if (!hashed) {
        // term[d][b] = (cell_d + b) * res^d
        uint32_t term[D][2];
        uint32_t stride = 1;
#pragma unroll
        for (int d = 0; d < D; ++d) {
            term[d][0] = cell[d] * stride;
            term[d][1] = term[d][0] + stride;
            stride *= res;
        }
#pragma unroll
        for (int c = 0; c < (1 << D); ++c) {
            uint32_t h = term[0][c & 1];
#pragma unroll
            for (int d = 1; d < D; ++d) h += term[d][(c >> d) & 1];
            // x == scale on every axis of a 1-D/2-D grid lands one row past the level; its weight is 0
            idx[c] = min(h, rows - 1);
        }
    } else if ((P.pow2_mask >> level) & 1u) {
        // low bits of the 64-bit products are all that survive "mod 2^k": wrap-around uint32 is exact
        uint32_t term[D][2];
#pragma unroll
        for (int d = 0; d < D; ++d) {
            term[d][0] = cell[d] * P.primes[d];
            term[d][1] = term[d][0] + P.primes[d];
        }
#pragma unroll
        for (int c = 0; c < (1 << D); ++c) {
            uint32_t h = term[0][c & 1];
#pragma unroll
            for (int d = 1; d < D; ++d) h ^= term[d][(c >> d) & 1];
            idx[c] = h & (rows - 1);
        }
    } else {
        unsigned long long term[D][2];
#pragma unroll
        for (int d = 0; d < D; ++d) {
            term[d][0] = static_cast<unsigned long long>(cell[d]) * P.primes[d];
            term[d][1] = term[d][0] + P.primes[d];
        }
#pragma unroll
        for (int c = 0; c < (1 << D); ++c) {
            unsigned long long h = term[0][c & 1];
#pragma unroll
            for (int d = 1; d < D; ++d) h ^= term[d][(c >> d) & 1];
            idx[c] = static_cast<uint32_t>(h % rows);
        }
    }
}

// The 2^(D-1) corners on one x-side of the cell (side 0: low x, side 1: high x), in the order of
// the remaining axes' bits; same arithmetic as corner_weights / corner_indices above.
template <int D>
__device__ __forceinline__ void side_weights(const float (&t)[D], int side, float (&w)[1 << (D - 1)]) {
    const float wx = side ? t[0] : __fsub_rn(1.f, t[0]);
    float lo[D];
#pragma unroll
    for (int d = 1; d < D; ++d) lo[d] = __fsub_rn(1.f, t[d]);
#pragma unroll
    for (int j = 0; j < (1 << (D - 1)); ++j) {
        float p = wx;
#pragma unroll
        for (int d = 1; d < D; ++d) p = __fmul_rn(p, ((j >> (d - 1)) & 1) ? t[d] : lo[d]);
        w[j] = p;
    }
}

template <int D>
__device__ __forceinline__ void side_indices(const uint32_t (&cell)[D], const LevelParams &P, int level, int side,
                                             uint32_t (&idx)[1 << (D - 1)]) {
    const uint32_t res = P.res[level];
    const uint32_t rows = P.rows[level];
    const bool hashed = (P.hashed_mask >> level) & 1u;
    if (!hashed) {
        uint32_t term[D][2];
        uint32_t stride = 1;
#pragma unroll
        for (int d = 0; d < D; ++d) {
            term[d][0] = cell[d] * stride;
            term[d][1] = term[d][0] + stride;
            stride *= res;
        }
#pragma unroll
        for (int j = 0; j < (1 << (D - 1)); ++j) {
            uint32_t h = side ? term[0][1] : term[0][0];
#pragma unroll
            for (int d = 1; d < D; ++d) h += term[d][(j >> (d - 1)) & 1];
            idx[j] = min(h, rows - 1);
        }
    } else if ((P.pow2_mask >> level) & 1u) {
        uint32_t term[D][2];
#pragma unroll
        for (int d = 0; d < D; ++d) {
            term[d][0] = cell[d] * P.primes[d];
            term[d][1] = term[d][0] + P.primes[d];
        }
#pragma unroll
        for (int j = 0; j < (1 << (D - 1)); ++j) {
            uint32_t h = side ? term[0][1] : term[0][0];
#pragma unroll
            for (int d = 1; d < D; ++d) h ^= term[d][(j >> (d - 1)) & 1];
            idx[j] = h & (rows - 1);
        }
    } else {
        unsigned long long term[D][2];
#pragma unroll
        for (int d = 0; d < D; ++d) {
            term[d][0] = static_cast<unsigned long long>(cell[d]) * P.primes[d];
            term[d][1] = term[d][0] + P.primes[d];
        }
#pragma unroll
        for (int j = 0; j < (1 << (D - 1)); ++j) {
            unsigned long long h = side ? term[0][1] : term[0][0];
#pragma unroll
            for (int d = 1; d < D; ++d) h ^= term[d][(j >> (d - 1)) & 1];
            idx[j] = static_cast<uint32_t>(h % rows);
        }
    }
}

// ---- row access -----------------------------------------------------------------------------

template <int BYTES>
struct Packet;
template <>
struct Packet<2> { using type = unsigned short; };
template <>
struct Packet<4> { using type = unsigned int; };
template <>
struct Packet<8> { using type = uint2; };
template <>
struct Packet<16> { using type = uint4; };

template <int BYTES>
struct PacketBytes { static constexpr int value = BYTES >= 16 ? 16 : BYTES; };

// COUNT consecutive elements of T <-> float registers, moved with the widest access that the
// element count allows (2..16 bytes).  `p` must be aligned to that width.  STREAM: 0 = read-only
// cached load, 1 = streaming (evict first).
template <typename T, int COUNT, int STREAM>
__device__ __forceinline__ void load_elems(const T *p, float (&v)[COUNT]) {
    constexpr int kBytes = COUNT * sizeof(T);
    constexpr int kPk = PacketBytes<kBytes>::value;
    using P = typename Packet<kPk>::type;
    union { P pk[kBytes / kPk]; T el[COUNT]; } u;
#pragma unroll
    for (int k = 0; k < kBytes / kPk; ++k) {
        const P *q = reinterpret_cast<const P *>(p) + k;
        if constexpr (STREAM == 1) u.pk[k] = __ldcs(q);
        else u.pk[k] = __ldg(q);
    }
#pragma unroll
    for (int k = 0; k < COUNT; ++k) v[k] = to_float<T>(u.el[k]);
}

template <typename T, int COUNT>
__device__ __forceinline__ void store_elems(T *p, const float (&v)[COUNT], bool vector_ok) {
    constexpr int kBytes = COUNT * sizeof(T);
    constexpr int kPk = PacketBytes<kBytes>::value;
    using P = typename Packet<kPk>::type;
    union { P pk[kBytes / kPk]; T el[COUNT]; } u;
#pragma unroll
    for (int k = 0; k < COUNT; ++k) u.el[k] = from_float<T>(v[k]);
    if (vector_ok) {
#pragma unroll
        for (int k = 0; k < kBytes / kPk; ++k) __stcs(reinterpret_cast<P *>(p) + k, u.pk[k]);
    } else {
#pragma unroll
        for (int k = 0; k < COUNT; ++k) p[k] = u.el[k];
    }
}

template <typename T, int COUNT>
__device__ __forceinline__ void load_elems_checked(const T *p, float (&v)[COUNT], bool vector_ok) {
    if (vector_ok) {
        load_elems<T, COUNT, 1>(p, v);
    } else {
#pragma unroll
        for (int k = 0; k < COUNT; ++k) v[k] = to_float<T>(p[k]);
    }
}

// One reduction per table row: red.global.add on F consecutive elements.
template <int F>
__device__ __forceinline__ void red_add_row(float *row, const float (&v)[F]) {
    if constexpr (F == 1) {
        asm volatile("red.global.add.f32 [%0], %1;" ::"l"(row), "f"(v[0]) : "memory");
    } else if constexpr (F == 2) {
        asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(row), "f"(v[0]), "f"(v[1]) : "memory");
    } else {
#pragma unroll
        for (int k = 0; k < F; k += 4)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(row + k), "f"(v[k]), "f"(v[k + 1]),
                         "f"(v[k + 2]), "f"(v[k + 3])
                         : "memory");
    }
}

__device__ __forceinline__ unsigned pack2(__half a, __half b) {
    return static_cast<unsigned>(__half_as_ushort(a)) | (static_cast<unsigned>(__half_as_ushort(b)) << 16);
}
__device__ __forceinline__ unsigned pack2(__nv_bfloat16 a, __nv_bfloat16 b) {
    return static_cast<unsigned>(__bfloat16_as_ushort(a)) | (static_cast<unsigned>(__bfloat16_as_ushort(b)) << 16);
}

template <int F>
__device__ __forceinline__ void red_add_row(__half *row, const float (&v)[F]) {
    if constexpr (F == 1) {
        atomicAdd(row, __float2half_rn(v[0]));
    } else if constexpr (F == 2) {
        asm volatile("red.global.add.noftz.f16x2 [%0], %1;" ::"l"(row),
                     "r"(pack2(__float2half_rn(v[0]), __float2half_rn(v[1])))
                     : "memory");
    } else {
#pragma unroll
        for (int k = 0; k < F; k += 4)
            asm volatile("red.global.add.noftz.v2.f16x2 [%0], {%1, %2};" ::"l"(row + k),
                         "r"(pack2(__float2half_rn(v[k]), __float2half_rn(v[k + 1]))),
                         "r"(pack2(__float2half_rn(v[k + 2]), __float2half_rn(v[k + 3])))
                         : "memory");
    }
}

template <int F>
__device__ __forceinline__ void red_add_row(__nv_bfloat16 *row, const float (&v)[F]) {
    if constexpr (F == 1) {
        atomicAdd(row, __float2bfloat16_rn(v[0]));
    } else if constexpr (F == 2) {
        asm volatile("red.global.add.noftz.bf16x2 [%0], %1;" ::"l"(row),
                     "r"(pack2(__float2bfloat16_rn(v[0]), __float2bfloat16_rn(v[1])))
                     : "memory");
    } else {
#pragma unroll
        for (int k = 0; k < F; k += 4)
            asm volatile("red.global.add.noftz.v2.bf16x2 [%0], {%1, %2};" ::"l"(row + k),
                         "r"(pack2(__float2bfloat16_rn(v[k]), __float2bfloat16_rn(v[k + 1]))),
                         "r"(pack2(__float2bfloat16_rn(v[k + 2]), __float2bfloat16_rn(v[k + 3])))
                         : "memory");
    }
}

// ---- accumulation in shared memory ------------------------------------------------------------
//
// Shared-memory floating-point adds are compare-and-swap loops and the unit retires about one of
// them per clock per SM, so a row is updated with as few as possible: one 16-byte or 8-byte
// compare-and-swap covers a whole row where the row has that size.

template <typename T, int N>
__device__ __forceinline__ void add_packed(const void *old_bits, const float *v, void *new_bits) {
    // old_bits/new_bits: N elements of T; v: N floats to add
    if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int k = 0; k < N; ++k) static_cast<float *>(new_bits)[k] = static_cast<const float *>(old_bits)[k] + v[k];
    } else {
        using T2 = typename std::conditional<std::is_same<T, __half>::value, __half2, __nv_bfloat162>::type;
#pragma unroll
        for (int k = 0; k < N; k += 2) {
            T2 add;
            add.x = from_float<T>(v[k]);
            add.y = from_float<T>(v[k + 1]);
            static_cast<T2 *>(new_bits)[k / 2] = __hadd2(static_cast<const T2 *>(old_bits)[k / 2], add);
        }
    }
}

__device__ __forceinline__ ulonglong2 smem_cas128(void *addr, ulonglong2 expect, ulonglong2 desired) {
    ulonglong2 old;
    const unsigned a = static_cast<unsigned>(__cvta_generic_to_shared(addr));
    asm volatile(
        "{\n\t.reg .b128 e, d, o;\n\t"
        "mov.b128 e, {%2, %3};\n\t"
        "mov.b128 d, {%4, %5};\n\t"
        "atom.relaxed.cta.shared.cas.b128 o, [%6], e, d;\n\t"
        "mov.b128 {%0, %1}, o;\n\t}"
        : "=l"(old.x), "=l"(old.y)
        : "l"(expect.x), "l"(expect.y), "l"(desired.x), "l"(desired.y), "r"(a)
        : "memory");
    return old;
}

// Set to 1 when a compare-and-swap loop below ran out of tries and dropped its update (read by
// th_hash_status).  Contention ends when the other lanes finish, so a healthy run never gets there.
__device__ int g_hash_status = 0;
constexpr int kSmemAddTries = 1 << 20;

// 16 bytes of a row: N = 16 / sizeof(T) elements
template <typename T>
__device__ __forceinline__ void smem_add16(T *p, const float *v) {
    constexpr int N = 16 / sizeof(T);
    ulonglong2 seen = *reinterpret_cast<const ulonglong2 *>(p);
    for (int tries = 0; tries < kSmemAddTries; ++tries) {
        ulonglong2 next;
        add_packed<T, N>(&seen, v, &next);
        const ulonglong2 old = smem_cas128(p, seen, next);
        if (old.x == seen.x && old.y == seen.y) return;
        seen = old;
    }
    g_hash_status = 1;
}

template <typename T>
__device__ __forceinline__ void smem_add8(T *p, const float *v) {
    constexpr int N = 8 / sizeof(T);
    unsigned long long seen = *reinterpret_cast<const unsigned long long *>(p);
    for (int tries = 0; tries < kSmemAddTries; ++tries) {
        unsigned long long next;
        add_packed<T, N>(&seen, v, &next);
        const unsigned long long old = atomicCAS(reinterpret_cast<unsigned long long *>(p), seen, next);
        if (old == seen) return;
        seen = old;
    }
    g_hash_status = 1;
}

template <typename T, int F>
__device__ __forceinline__ void smem_add_row(T *row, const float (&v)[F]) {
    constexpr int kRowBytes = F * sizeof(T);
    if constexpr (kRowBytes % 16 == 0) {
#pragma unroll
        for (int b = 0; b < kRowBytes / 16; ++b) smem_add16<T>(row + b * (16 / sizeof(T)), v + b * (16 / sizeof(T)));
    } else if constexpr (kRowBytes == 8) {
        smem_add8<T>(row, v);
    } else if constexpr (sizeof(T) == 4) {
        atomicAdd(reinterpret_cast<float *>(row), v[0]);
    } else if constexpr (F == 1) {
        atomicAdd(row, from_float<T>(v[0]));
    } else {
        using T2 = typename std::conditional<std::is_same<T, __half>::value, __half2, __nv_bfloat162>::type;
        T2 pair;
        pair.x = from_float<T>(v[0]);
        pair.y = from_float<T>(v[1]);
        atomicAdd(reinterpret_cast<T2 *>(row), pair);
    }
}

// ---- host side ------------------------------------------------------------------------------

int fill_params(LevelParams &P, int n_dims, int n_levels, const int32_t *res, const int64_t *rows,
                const int64_t *offsets, const int64_t *primes, float scale) {
    if (n_levels < 1 || n_levels > TH_MAX_LEVELS) return fail(TH_ERR_BAD_ARG, "n_levels %d outside [1, %d]", n_levels, TH_MAX_LEVELS);
    if (n_dims < 1 || n_dims > TH_MAX_DIMS) return fail(TH_ERR_UNSUPPORTED, "n_dims %d outside [1, %d]", n_dims, TH_MAX_DIMS);
    if (!res || !rows || !primes) return fail(TH_ERR_BAD_ARG, "null level array");
    if (!(scale > 0.f)) return fail(TH_ERR_BAD_ARG, "scale must be positive");
    P = LevelParams{};
    P.scale = scale;
    for (int d = 0; d < n_dims; ++d) {
        if (primes[d] < 0 || primes[d] > 0xffffffffll) return fail(TH_ERR_BAD_ARG, "prime %d does not fit 32 bits", d);
        P.primes[d] = static_cast<uint32_t>(primes[d]);
    }
    for (int l = 0; l < n_levels; ++l) {
        if (res[l] < 1 || res[l] >= (1 << 24)) return fail(TH_ERR_BAD_ARG, "level %d resolution %d outside [1, 2^24)", l, res[l]);
        if (rows[l] < 1 || rows[l] > 0xffffffffll) return fail(TH_ERR_BAD_ARG, "level %d row count out of range", l);
        P.res[l] = static_cast<uint32_t>(res[l]);
        P.rows[l] = static_cast<uint32_t>(rows[l]);
        P.offset[l] = offsets ? static_cast<unsigned long long>(offsets[l]) : 0ull;
        if (offsets && offsets[l] < 0) return fail(TH_ERR_BAD_ARG, "level %d offset is negative", l);
        // dense iff (res + 1)^D <= rows  (kernel.py:453 of the reference)
        unsigned long long dense_rows = 1;
        for (int d = 0; d < n_dims; ++d) dense_rows *= static_cast<unsigned long long>(res[l]) + 1ull;
        if (dense_rows > static_cast<unsigned long long>(rows[l])) P.hashed_mask |= 1u << l;
        if ((rows[l] & (rows[l] - 1)) == 0) P.pow2_mask |= 1u << l;
    }
    return TH_OK;
}

int make_coord_view(CoordView &cv, const void *coords, int64_t stride_n, int64_t stride_d, int dtype, int n_dims) {
    if (!coords) return fail(TH_ERR_BAD_ARG, "null coords");
    if (dtype != TH_F32 && dtype != TH_F16 && dtype != TH_BF16) return fail(TH_ERR_BAD_ARG, "unknown coord dtype %d", dtype);
    cv.ptr = coords;
    cv.stride_n = stride_n;
    cv.stride_d = stride_d;
    cv.dtype = dtype;
    cv.packed_f32 = dtype == TH_F32 && stride_d == 1 && stride_n == n_dims && aligned_to(coords, 16);
    return TH_OK;
}

}  // namespace
}  // namespace th
