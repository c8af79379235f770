// Multiresolution hash encoding for sm_100a: forward gather/interpolate and backward
// scatter-add.  Replaces the Triton kernels of
// triton_helpers/layers/hash_encoding/kernel.py:175-306 (_fwd_kernel) and :322-440 (_bwd_kernel);
// the index and weight arithmetic follows that file's CPU path (:443-479), which is the
// parity contract:
//   cell   = floor(x * res)                 one float32 multiply per level, no FMA contraction
//   dense  : index = sum_d corner_d * res^d
//   hashed : index = xor_d(corner_d * prime_d) mod rows
//   t      = x * res - cell ;  weight(corner) = prod_d (bit_d ? t_d : 1 - t_d), axis order 0,1,2
//
// Work decomposition: TWO neighbouring lanes per point, 128 points per CTA.  Lane 0 of a pair
// takes the 2^(D-1) corners on the low-x side of the cell, lane 1 those on the high-x side.
// Rows of x-neighbours are adjacent in a dense level and, because the first hashing prime is
// 1, differ only in their low bits in a hashed level, so the two addresses a lane pair
// presents in one load / reduction instruction fall into the same 32-byte sector most of the
// time (7 in 8 for 4-byte rows) and the memory system handles them as one transaction; with
// one thread per point they would be two transactions from two instructions.  The CTA stages
// its coordinates through shared memory with 128-bit coalesced loads; each lane then walks the
// levels in register groups of LG levels, so the gathers of a whole group are in flight
// together; a pair combines its two partial sums with one shuffle and each lane writes
// (forward) half of the group's slice of the [N, L*F] matrix.  Tables are read through the
// read-only path and are meant to stay L2 resident; outputs and gradients are streamed.
//
// Backward contention, coarse levels: large batches accumulate the leading dense levels per CTA in
// shared memory (hash_bwd_coarse_kernel) and flush once.  Elsewhere: lanes of a warp that work on the same cell and side are found with one
// match.any per level; their contributions are summed in registers and the first lane of
// each group issues a single vector red.global.add per corner, so a cluster of points costs
// one memory atomic per corner instead of one per point.
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
template <int D, int LPP>
__device__ __forceinline__ bool load_coords(const CoordView &cv, long long n_points, float (&x)[D], float *stage) {
    constexpr int kPoints = kThreads / LPP;
    const int local = threadIdx.x / LPP;
    const long long i = static_cast<long long>(blockIdx.x) * kPoints + local;
    if (cv.packed_f32) {
        const long long first = static_cast<long long>(blockIdx.x) * kPoints * D;  // multiple of 4
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

// ---- forward --------------------------------------------------------------------------------

template <typename T, int D, int F, int LG>
__global__ void __launch_bounds__(kThreads)
hash_fwd_kernel(const __grid_constant__ LevelParams P, const CoordView cv, const T *__restrict__ table,
                T *__restrict__ out, long long out_stride, long long n_points, int level_begin, int level_end,
                int vector_ok) {
    constexpr int kPoints = kThreads / 2;
    constexpr int kSide = 1 << (D - 1);   // corners per lane
    constexpr int kCount = LG * F;        // outputs per level group
    constexpr int kFirst = (kCount + 1) / 2;  // written by lane 0 of the pair; the rest by lane 1
    __shared__ __align__(16) float stage[kPoints * D];
    float x[D];
    const bool live = load_coords<D, 2>(cv, n_points, x, stage);
    // dead pairs of the last CTA stay in the loop: the pair shuffle below needs both lanes
    if (P.scale != 1.f) {
#pragma unroll
        for (int d = 0; d < D; ++d) x[d] = __fdiv_rn(x[d], P.scale);
    }
    if (!live) {
#pragma unroll
        for (int d = 0; d < D; ++d) x[d] = 0.f;
    }
    const int side = threadIdx.x & 1;
    const long long i = static_cast<long long>(blockIdx.x) * kPoints + (threadIdx.x >> 1);
    T *out_row = out + (live ? i : 0) * out_stride;

    // gridDim.y CTAs share a point tile and take every gridDim.y-th level group each
    for (int lg = level_begin + LG * blockIdx.y; lg < level_end; lg += LG * gridDim.y) {
        float acc[kCount];
        float e[LG][kSide][F];
        float w[LG][kSide];
        // issue every gather of the group before the first use
#pragma unroll
        for (int j = 0; j < LG; ++j) {
            const int level = lg + j;
            uint32_t cell[D], idx[kSide];
            float t[D];
            locate<D>(x, P.res[level], cell, t);
            side_weights<D>(t, side, w[j]);
            side_indices<D>(cell, P, level, side, idx);
            const T *base = table + P.offset[level] * F;
            // (loads that skip L1 allocation were tried for the hashed levels and measured slower:
            //  0.60 against 0.55 ms at 2^21 points, 3.5 against 2.2 ms with a 681 MB table)
#pragma unroll
            for (int c = 0; c < kSide; ++c) load_elems<T, F, 0>(base + static_cast<size_t>(idx[c]) * F, e[j][c]);
        }
#pragma unroll
        for (int j = 0; j < LG; ++j) {
#pragma unroll
            for (int f = 0; f < F; ++f) {
                float s = __fmul_rn(w[j][0], e[j][0][f]);
#pragma unroll
                for (int c = 1; c < kSide; ++c) s = __fadd_rn(s, __fmul_rn(w[j][c], e[j][c][f]));
                // low-x side + high-x side
                acc[j * F + f] = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, 1));
            }
        }
        if (live) {
            if (side == 0) {
                float part[kFirst];
#pragma unroll
                for (int k = 0; k < kFirst; ++k) part[k] = acc[k];
                store_elems<T, kFirst>(out_row + lg * F, part, vector_ok);
            } else if constexpr (kCount - kFirst > 0) {
                float part[kCount - kFirst];
#pragma unroll
                for (int k = 0; k < kCount - kFirst; ++k) part[k] = acc[kFirst + k];
                store_elems<T, kCount - kFirst>(out_row + lg * F + kFirst, part, vector_ok);
            }
        }
    }
}

// ---- backward -------------------------------------------------------------------------------

template <typename T, int D, int F, int LG>
__global__ void __launch_bounds__(kThreads)
hash_bwd_kernel(const __grid_constant__ LevelParams P, const CoordView cv, const T *__restrict__ grad_out,
                long long go_stride, T *__restrict__ grad_table, long long n_points, int level_begin,
                int level_end, int vector_ok, int skip_below) {
    // levels below `skip_below` were accumulated by hash_bwd_coarse_kernel and are passed over here
    constexpr int kPoints = kThreads / 2;
    constexpr int kSide = 1 << (D - 1);
    __shared__ __align__(16) float stage[kPoints * D];
    float x[D];
    const bool live = load_coords<D, 2>(cv, n_points, x, stage);
    // Dead lanes of the last CTA stay in the loop (the warp votes below need every lane)
    // with zero gradient and are never chosen to issue an atomic.
    if (P.scale != 1.f) {
#pragma unroll
        for (int d = 0; d < D; ++d) x[d] = __fdiv_rn(x[d], P.scale);
    }
    if (!live) {
#pragma unroll
        for (int d = 0; d < D; ++d) x[d] = 0.f;
    }
    const int side = threadIdx.x & 1;
    const long long i = static_cast<long long>(blockIdx.x) * kPoints + (threadIdx.x >> 1);
    const T *go_row = grad_out + (live ? i : 0) * go_stride;
    const unsigned lane = threadIdx.x & 31u;

    // gridDim.y CTAs share a point tile and take every gridDim.y-th level group each
    for (int lg = level_begin + LG * blockIdx.y; lg < level_end; lg += LG * gridDim.y) {
        float go[LG * F];
        if (live) {
            load_elems_checked<T, LG * F>(go_row + lg * F, go, vector_ok);  // both lanes of a pair: one broadcast load
        } else {
#pragma unroll
            for (int k = 0; k < LG * F; ++k) go[k] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < LG; ++j) {
            const int level = lg + j;
            if (level < skip_below) continue;
            uint32_t cell[D], idx[kSide];
            float t[D], w[kSide];
            locate<D>(x, P.res[level], cell, t);
            side_weights<D>(t, side, w);
            side_indices<D>(cell, P, level, side, idx);
            T *base = grad_table + P.offset[level] * F;

            // Lanes on the same side of the same cell share all their rows.  Looking for them costs a
            // match.any per level, which only pays on coarse grids: with res > kAggregateMaxRes even
            // tightly clustered points (sigma = 0.02) put two of a warp's 16 points in one cell less than
            // once in a hundred levels, so finer levels go straight to the atomics.  The key packs the
            // exact cell (20 bits per axis) and the side; dead lanes and cells too large to pack get a
            // key nobody else has.
            bool shared_cell = false;
            unsigned peers = 1u << lane;
            if (P.res[level] <= kAggregateMaxRes) {
                unsigned long long key = 0;
                bool packable = live;
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    packable = packable && cell[d] < (1u << 20);
                    key = (key << 20) | (cell[d] & 0xfffffu);
                }
                key = (key << 1) | static_cast<unsigned>(side);
                if (!packable) key = (1ull << 63) | lane;
                peers = __match_any_sync(0xffffffffu, key);
                shared_cell = __any_sync(0xffffffffu, (peers & (peers - 1)) != 0);
            }

            if (!shared_cell) {
                if (live) {
#pragma unroll
                    for (int c = 0; c < kSide; ++c) {
                        float v[F];
#pragma unroll
                        for (int f = 0; f < F; ++f) v[f] = __fmul_rn(w[c], go[j * F + f]);
                        red_add_row<F>(base + static_cast<size_t>(idx[c]) * F, v);
                    }
                }
            } else {
                const bool leader = (peers & ((1u << lane) - 1u)) == 0;
                // longest peer list in the warp bounds the walk below
                const int steps = __reduce_max_sync(0xffffffffu, __popc(peers));
#pragma unroll
                for (int c = 0; c < kSide; ++c) {
                    float v[F], sum[F];
#pragma unroll
                    for (int f = 0; f < F; ++f) {
                        v[f] = __fmul_rn(w[c], go[j * F + f]);
                        sum[f] = 0.f;
                    }
                    // every lane walks its own peer list and ends up with its group's total
                    unsigned rest = peers;
                    for (int s = 0; s < steps; ++s) {
                        const int src = rest ? (__ffs(rest) - 1) : static_cast<int>(lane);
#pragma unroll
                        for (int f = 0; f < F; ++f) {
                            const float pv = __shfl_sync(0xffffffffu, v[f], src);
                            if (rest) sum[f] += pv;
                        }
                        rest &= rest - 1;
                    }
                    if (live && leader) red_add_row<F>(base + static_cast<size_t>(idx[c]) * F, sum);
                }
            }
        }
    }
}

// ---- backward, coarse levels ----------------------------------------------------------------
//
// The coarsest levels have a few thousand rows that every point updates: at 2^21 points each row of
// a 16^3 grid receives thousands of reductions, and the L2 serialises reductions to one address
// (measured: the four coarsest of 16 levels cost as much as nine of the others).  For large batches
// those levels are therefore accumulated per CTA in SHARED memory - as many leading dense levels as
// fit, in the table's own dtype - by persistent CTAs that each take a contiguous slice of the
// points, and flushed once per CTA with one vector reduction per non-zero row.

constexpr int kCoarseThreads = 1024;
constexpr int kCoarseSmemBytes = 200 * 1024;

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

// 16 bytes of a row: N = 16 / sizeof(T) elements
template <typename T>
__device__ __forceinline__ void smem_add16(T *p, const float *v) {
    constexpr int N = 16 / sizeof(T);
    ulonglong2 seen = *reinterpret_cast<const ulonglong2 *>(p);
    for (int tries = 0; tries < (1 << 20); ++tries) {  // bounded: contention ends when the other lanes finish
        ulonglong2 next;
        add_packed<T, N>(&seen, v, &next);
        const ulonglong2 old = smem_cas128(p, seen, next);
        if (old.x == seen.x && old.y == seen.y) break;
        seen = old;
    }
}

template <typename T>
__device__ __forceinline__ void smem_add8(T *p, const float *v) {
    constexpr int N = 8 / sizeof(T);
    unsigned long long seen = *reinterpret_cast<const unsigned long long *>(p);
    for (int tries = 0; tries < (1 << 20); ++tries) {
        unsigned long long next;
        add_packed<T, N>(&seen, v, &next);
        const unsigned long long old = atomicCAS(reinterpret_cast<unsigned long long *>(p), seen, next);
        if (old == seen) break;
        seen = old;
    }
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

template <typename T, int D, int F>
__global__ void __launch_bounds__(kCoarseThreads, 1)
hash_bwd_coarse_kernel(const __grid_constant__ LevelParams P, const CoordView cv, const T *__restrict__ grad_out,
                       long long go_stride, T *__restrict__ grad_table, long long n_points, int level_begin,
                       int level_end, long long points_per_cta) {
    extern __shared__ __align__(16) unsigned char coarse_smem[];
    T *acc = reinterpret_cast<T *>(coarse_smem);
    const unsigned long long first_row = P.offset[level_begin];
    const unsigned long long n_rows = P.offset[level_end - 1] + P.rows[level_end - 1] - first_row;
    for (unsigned long long e = threadIdx.x; e < n_rows * F * sizeof(T) / 16; e += kCoarseThreads)
        reinterpret_cast<uint4 *>(coarse_smem)[e] = make_uint4(0, 0, 0, 0);
    for (unsigned long long e = (n_rows * F * sizeof(T) / 16) * (16 / sizeof(T)) + threadIdx.x; e < n_rows * F; e += kCoarseThreads)
        acc[e] = from_float<T>(0.f);
    __syncthreads();

    const long long begin = static_cast<long long>(blockIdx.x) * points_per_cta;
    const long long end = begin + points_per_cta < n_points ? begin + points_per_cta : n_points;
    const unsigned lane = threadIdx.x & 31u;
    // whole warps stay in the loop so that the lanes can look for peers in the same cell
    unsigned hot_levels = 0;  // warp-uniform: bit l set while level l keeps showing lanes in one cell
    int batch = 0;
    for (long long first = begin + (threadIdx.x & ~31u); first < end; first += kCoarseThreads, ++batch) {
        const long long i = first + lane;
        const bool live = i < end;
        float x[D];
#pragma unroll
        for (int d = 0; d < D; ++d) x[d] = 0.f;
        if (live) load_coords_strided<D>(cv, i, x);
        if (P.scale != 1.f) {
#pragma unroll
            for (int d = 0; d < D; ++d) x[d] = __fdiv_rn(x[d], P.scale);
        }
        for (int level = level_begin; level < level_end; ++level) {
            uint32_t cell[D], idx[1 << D];
            float t[D], w[1 << D], go[F];
            locate<D>(x, P.res[level], cell, t);
            corner_weights<D>(t, w);
            corner_indices<D>(cell, P, level, idx);
#pragma unroll
            for (int f = 0; f < F; ++f) go[f] = live ? to_float<T>(grad_out[i * go_stride + level * F + f]) : 0.f;
            T *base = acc + (P.offset[level] - first_row) * F;

            // lanes that meet in one cell (clustered inputs) are summed in registers first and one of
            // them does the shared-memory add
            // The search itself costs a match.any per level, so a warp only keeps it up on levels where
            // the last search found something, and otherwise looks again every 8th batch of points.
            unsigned peers = 1u << lane;
            bool shared_cell = false;
            if (((hot_levels >> level) & 1u) || (batch & 7) == 0) {
                unsigned long long key = 0;
#pragma unroll
                for (int d = 0; d < D; ++d) key = (key << 20) | (cell[d] & 0xfffffu);  // dense levels: res < 2^20
                if (!live) key = (1ull << 63) | lane;
                peers = __match_any_sync(0xffffffffu, key);
                shared_cell = __any_sync(0xffffffffu, (peers & (peers - 1)) != 0);
                hot_levels = shared_cell ? (hot_levels | (1u << level)) : (hot_levels & ~(1u << level));
            }
            if (!shared_cell) {
                if (live) {
#pragma unroll
                    for (int c = 0; c < (1 << D); ++c) {
                        float v[F];
#pragma unroll
                        for (int f = 0; f < F; ++f) v[f] = __fmul_rn(w[c], go[f]);
                        smem_add_row<T, F>(base + static_cast<size_t>(idx[c]) * F, v);
                    }
                }
            } else {
                const bool leader = (peers & ((1u << lane) - 1u)) == 0;
                const int steps = __reduce_max_sync(0xffffffffu, __popc(peers));
#pragma unroll
                for (int c = 0; c < (1 << D); ++c) {
                    float v[F], sum[F];
#pragma unroll
                    for (int f = 0; f < F; ++f) {
                        v[f] = __fmul_rn(w[c], go[f]);
                        sum[f] = 0.f;
                    }
                    unsigned rest = peers;
                    for (int s = 0; s < steps; ++s) {
                        const int src = rest ? (__ffs(rest) - 1) : static_cast<int>(lane);
#pragma unroll
                        for (int f = 0; f < F; ++f) {
                            const float pv = __shfl_sync(0xffffffffu, v[f], src);
                            if (rest) sum[f] += pv;
                        }
                        rest &= rest - 1;
                    }
                    if (live && leader) smem_add_row<T, F>(base + static_cast<size_t>(idx[c]) * F, sum);
                }
            }
        }
    }
    __syncthreads();
    // one reduction per row that received anything
    T *dst = grad_table + first_row * F;
    for (unsigned long long r = threadIdx.x; r < n_rows; r += kCoarseThreads) {
        float v[F];
        bool any = false;
#pragma unroll
        for (int f = 0; f < F; ++f) {
            v[f] = to_float<T>(acc[r * F + f]);
            any = any || v[f] != 0.f;
        }
        if (any) red_add_row<F>(dst + r * F, v);
    }
}

// ---- debug: indices and weights -------------------------------------------------------------

template <int D>
__global__ void __launch_bounds__(kThreads)
hash_debug_kernel(const __grid_constant__ LevelParams P, const CoordView cv, long long *__restrict__ idx_out,
                  float *__restrict__ w_out, long long n_points, int n_levels) {
    __shared__ __align__(16) float stage[kThreads * D];
    float x[D];
    if (!load_coords<D, 1>(cv, n_points, x, stage)) return;
    if (P.scale != 1.f) {
#pragma unroll
        for (int d = 0; d < D; ++d) x[d] = __fdiv_rn(x[d], P.scale);
    }
    const long long i = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
    for (int level = 0; level < n_levels; ++level) {
        uint32_t cell[D], idx[1 << D];
        float t[D], w[1 << D];
        locate<D>(x, P.res[level], cell, t);
        corner_weights<D>(t, w);
        corner_indices<D>(cell, P, level, idx);
        const long long o = (i * n_levels + level) * (1 << D);
#pragma unroll
        for (int c = 0; c < (1 << D); ++c) {
            idx_out[o + c] = idx[c];
            if (w_out) w_out[o + c] = w[c];
        }
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

// Levels per register group: as many as divide the range, capped so a group holds <= 8 features.
int pick_level_group(int level_begin, int level_end, int n_feats) {
    const int count = level_end - level_begin;
    const int cap = n_feats >= 8 ? 1 : (n_feats == 4 ? 2 : 4);
    if (cap >= 4 && count % 4 == 0 && level_begin % 4 == 0) return 4;
    if (cap >= 2 && count % 2 == 0 && level_begin % 2 == 0) return 2;
    return 1;
}

// Grid: x = point tiles (128 points each); y = how many CTAs split the level groups of a tile.
// Large batches fill the GPU with point tiles alone (y = 1: coordinates are read once per point);
// small ones (a few waves or less) would leave every thread with a serial chain of level groups and
// most of the machine idle, so their level groups are spread over y CTAs instead.
dim3 point_level_grid(int64_t n, int l0, int l1, int levels_per_group) {
    const long long tiles = (n + kThreads / 2 - 1) / (kThreads / 2);
    const int groups = (l1 - l0) / levels_per_group;
    int split = 1;
    const long long resident = static_cast<long long>(sm_count()) * 8;  // CTAs the GPU holds at once
    while (split < groups && tiles * split < 4 * resident) split *= 2;
    if (split > groups) split = groups;
    return dim3(static_cast<unsigned>(tiles), static_cast<unsigned>(split), 1);
}

// Level passes.  Rows of a level are visited at random, so a launch runs at cache speed only while
// the levels it touches stay resident in L2.  When the levels of [l0, l1) add up to more than
// kPassBytes and the batch is large, the range is cut into consecutive passes of at most kPassBytes
// each (a single level larger than that is a pass of its own).  Measured with 2^22 rows x 16 B per
// level and 2^22 points: four such levels in one launch 2.6 ms backward / 1.2 ms forward, the same
// four as one launch each 0.95 / 0.83 ms.  The reference exposes the same idea as its `divider`
// argument; here it is automatic and `level_begin/level_end` passes of the caller still work.
constexpr size_t kPassBytes = static_cast<size_t>(72) << 20;
constexpr int64_t kPassMinPoints = 1 << 16;

struct LevelPasses {
    int count = 0;
    int begin[TH_MAX_LEVELS];
    int end[TH_MAX_LEVELS];
};

LevelPasses plan_level_passes(const LevelParams &P, int64_t n, int l0, int l1, size_t row_bytes) {
    LevelPasses passes;
    size_t total = 0;
    for (int l = l0; l < l1; ++l) total += static_cast<size_t>(P.rows[l]) * row_bytes;
    if (total <= kPassBytes || n < kPassMinPoints) {
        passes.count = 1;
        passes.begin[0] = l0;
        passes.end[0] = l1;
        return passes;
    }
    int a = l0;
    while (a < l1) {
        size_t bytes = static_cast<size_t>(P.rows[a]) * row_bytes;
        int b = a + 1;
        while (b < l1 && bytes + static_cast<size_t>(P.rows[b]) * row_bytes <= kPassBytes) {
            bytes += static_cast<size_t>(P.rows[b]) * row_bytes;
            ++b;
        }
        passes.begin[passes.count] = a;
        passes.end[passes.count] = b;
        ++passes.count;
        a = b;
    }
    return passes;
}

template <typename T, int D, int F>
int launch_fwd(const LevelParams &P, const CoordView &cv, const void *table, void *out, int64_t out_stride,
               int64_t n, int l0, int l1, cudaStream_t stream) {
    const int vec = aligned_to(out, 16) && (out_stride * sizeof(T)) % 16 == 0;
    const T *tb = static_cast<const T *>(table);
    T *o = static_cast<T *>(out);
    const LevelPasses passes = plan_level_passes(P, n, l0, l1, F * sizeof(T));
    for (int p = 0; p < passes.count; ++p) {
        const int a = passes.begin[p], b = passes.end[p];
        const int lg = pick_level_group(a, b, F);
        const dim3 grid = point_level_grid(n, a, b, lg);
        switch (lg) {
            case 4: hash_fwd_kernel<T, D, F, 4><<<grid, kThreads, 0, stream>>>(P, cv, tb, o, out_stride, n, a, b, vec); break;
            case 2: hash_fwd_kernel<T, D, F, 2><<<grid, kThreads, 0, stream>>>(P, cv, tb, o, out_stride, n, a, b, vec); break;
            default: hash_fwd_kernel<T, D, F, 1><<<grid, kThreads, 0, stream>>>(P, cv, tb, o, out_stride, n, a, b, vec); break;
        }
        if (int rc = launch_status("hash_fwd_kernel launch")) return rc;
    }
    return TH_OK;
}

// How many leading levels of [l0, l1) go to the shared-memory kernel: dense levels only, as many as
// fit, and only when the batch is large enough that flushing one private copy per CTA is cheaper
// than the reductions it saves.
template <typename T, int F>
int coarse_level_end(const LevelParams &P, int64_t n, int l0, int l1) {
    if (n < (1 << 18)) return l0;
    size_t bytes = 0;
    int end = l0;
    while (end < l1 && !((P.hashed_mask >> end) & 1u)) {
        const size_t next = bytes + static_cast<size_t>(P.rows[end]) * F * sizeof(T);
        if (next > static_cast<size_t>(kCoarseSmemBytes)) break;
        bytes = next;
        ++end;
    }
    return end;
}

template <typename T, int D, int F>
int launch_bwd(const LevelParams &P, const CoordView &cv, const void *go, int64_t go_stride, void *grad_table,
               int64_t n, int l0, int l1, cudaStream_t stream) {
    const T *g = static_cast<const T *>(go);
    T *gt = static_cast<T *>(grad_table);
    // 1. coarse levels in shared memory
    const int coarse_end = coarse_level_end<T, F>(P, n, l0, l1);
    if (coarse_end > l0) {
        size_t bytes = 0;
        for (int l = l0; l < coarse_end; ++l) bytes += static_cast<size_t>(P.rows[l]) * F * sizeof(T);
        bytes = (bytes + 15) & ~static_cast<size_t>(15);
        auto kernel = hash_bwd_coarse_kernel<T, D, F>;
        if (int rc = cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)),
                                 "cudaFuncSetAttribute(hash_bwd_coarse_kernel)")) return rc;
        const int ctas = sm_count();
        const long long per_cta = (n + ctas - 1) / ctas;
        kernel<<<ctas, kCoarseThreads, bytes, stream>>>(P, cv, g, go_stride, gt, n, l0, coarse_end, per_cta);
        if (int rc = launch_status("hash_bwd_coarse_kernel launch")) return rc;
        if (coarse_end == l1) return TH_OK;
    }
    // 2. everything else with global reductions, in passes that keep the rows being updated in L2
    const int vec = aligned_to(go, 16) && (go_stride * sizeof(T)) % 16 == 0;
    const LevelPasses passes = plan_level_passes(P, n, l0, l1, F * sizeof(T));
    for (int p = 0; p < passes.count; ++p) {
        const int a = passes.begin[p], b = passes.end[p];
        if (b <= coarse_end) continue;
        const int lg = pick_level_group(a, b, F);
        const dim3 grid = point_level_grid(n, a, b, lg);
        switch (lg) {
            case 4: hash_bwd_kernel<T, D, F, 4><<<grid, kThreads, 0, stream>>>(P, cv, g, go_stride, gt, n, a, b, vec, coarse_end); break;
            case 2: hash_bwd_kernel<T, D, F, 2><<<grid, kThreads, 0, stream>>>(P, cv, g, go_stride, gt, n, a, b, vec, coarse_end); break;
            default: hash_bwd_kernel<T, D, F, 1><<<grid, kThreads, 0, stream>>>(P, cv, g, go_stride, gt, n, a, b, vec, coarse_end); break;
        }
        if (int rc = launch_status("hash_bwd_kernel launch")) return rc;
    }
    return TH_OK;
}

// Expands (dtype, D, F) into a template instantiation.
#define TH_DISPATCH_F(T, D, CALL)                                                      \
    switch (n_feats) {                                                                 \
        case 1: return CALL(T, D, 1);                                                  \
        case 2: return CALL(T, D, 2);                                                  \
        case 4: return CALL(T, D, 4);                                                  \
        case 8: return CALL(T, D, 8);                                                  \
        default: return fail(TH_ERR_UNSUPPORTED, "n_feats %d not in {1, 2, 4, 8}", n_feats); \
    }
#define TH_DISPATCH_D(T, CALL)                    \
    switch (n_dims) {                             \
        case 1: TH_DISPATCH_F(T, 1, CALL)         \
        case 2: TH_DISPATCH_F(T, 2, CALL)         \
        default: TH_DISPATCH_F(T, 3, CALL)        \
    }
#define TH_DISPATCH(CALL)                                                                  \
    switch (table_dtype) {                                                                 \
        case TH_F32: TH_DISPATCH_D(float, CALL)                                            \
        case TH_F16: TH_DISPATCH_D(__half, CALL)                                           \
        case TH_BF16: TH_DISPATCH_D(__nv_bfloat16, CALL)                                   \
        default: return fail(TH_ERR_BAD_ARG, "unknown table dtype %d", table_dtype);       \
    }

int check_range(int n_levels, int l0, int l1) {
    if (l0 < 0 || l1 > n_levels || l0 >= l1) return fail(TH_ERR_BAD_ARG, "level range [%d, %d) outside [0, %d)", l0, l1, n_levels);
    return TH_OK;
}

}  // namespace
}  // namespace th

using namespace th;

extern "C" int th_hash_fwd(const void *coords_dev, int64_t coord_stride_n, int64_t coord_stride_d, int coord_dtype,
                           const void *table_dev, int table_dtype, void *out_dev, int64_t out_stride_n,
                           int64_t n_points, int n_dims, int n_feats, int n_levels, const int32_t *level_res_host,
                           const int64_t *level_rows_host, const int64_t *level_offset_host,
                           const int64_t *primes_host, float scale, int level_begin, int level_end, void *stream) {
    if (n_points < 0) return fail(TH_ERR_BAD_ARG, "negative n_points");
    LevelParams P;
    CoordView cv;
    if (int rc = fill_params(P, n_dims, n_levels, level_res_host, level_rows_host, level_offset_host, primes_host, scale)) return rc;
    if (!level_offset_host) return fail(TH_ERR_BAD_ARG, "null level offsets");
    if (int rc = check_range(n_levels, level_begin, level_end)) return rc;
    if (n_points == 0) return TH_OK;
    if (int rc = make_coord_view(cv, coords_dev, coord_stride_n, coord_stride_d, coord_dtype, n_dims)) return rc;
    if (!table_dev || !out_dev) return fail(TH_ERR_BAD_ARG, "null table or output");
    const size_t row_bytes = n_feats * dtype_bytes(table_dtype);
    if (!aligned_to(table_dev, row_bytes < 16 ? row_bytes : 16)) return fail(TH_ERR_ALIGNMENT, "table rows must be aligned to min(row bytes, 16)");
    if (out_stride_n < static_cast<int64_t>(n_levels) * n_feats) return fail(TH_ERR_BAD_ARG, "out_stride_n smaller than n_levels * n_feats");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define TH_CALL_FWD(T, D, F) launch_fwd<T, D, F>(P, cv, table_dev, out_dev, out_stride_n, n_points, level_begin, level_end, s)
    TH_DISPATCH(TH_CALL_FWD)
#undef TH_CALL_FWD
}

extern "C" int th_hash_bwd(const void *coords_dev, int64_t coord_stride_n, int64_t coord_stride_d, int coord_dtype,
                           const void *grad_out_dev, int64_t go_stride_n, void *grad_table_dev, int table_dtype,
                           int64_t n_points, int n_dims, int n_feats, int n_levels, const int32_t *level_res_host,
                           const int64_t *level_rows_host, const int64_t *level_offset_host,
                           const int64_t *primes_host, float scale, int level_begin, int level_end, void *stream) {
    if (n_points < 0) return fail(TH_ERR_BAD_ARG, "negative n_points");
    LevelParams P;
    CoordView cv;
    if (int rc = fill_params(P, n_dims, n_levels, level_res_host, level_rows_host, level_offset_host, primes_host, scale)) return rc;
    if (!level_offset_host) return fail(TH_ERR_BAD_ARG, "null level offsets");
    if (int rc = check_range(n_levels, level_begin, level_end)) return rc;
    if (n_points == 0) return TH_OK;
    if (int rc = make_coord_view(cv, coords_dev, coord_stride_n, coord_stride_d, coord_dtype, n_dims)) return rc;
    if (!grad_out_dev || !grad_table_dev) return fail(TH_ERR_BAD_ARG, "null gradient pointer");
    const size_t row_bytes = n_feats * dtype_bytes(table_dtype);
    if (!aligned_to(grad_table_dev, row_bytes < 16 ? row_bytes : 16)) return fail(TH_ERR_ALIGNMENT, "table rows must be aligned to min(row bytes, 16)");
    if (go_stride_n < static_cast<int64_t>(n_levels) * n_feats) return fail(TH_ERR_BAD_ARG, "go_stride_n smaller than n_levels * n_feats");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define TH_CALL_BWD(T, D, F) launch_bwd<T, D, F>(P, cv, grad_out_dev, go_stride_n, grad_table_dev, n_points, level_begin, level_end, s)
    TH_DISPATCH(TH_CALL_BWD)
#undef TH_CALL_BWD
}

extern "C" int th_hash_debug_indices(const void *coords_dev, int64_t coord_stride_n, int64_t coord_stride_d,
                                     int coord_dtype, int64_t *idx_out_dev, float *weight_out_dev, int64_t n_points,
                                     int n_dims, int n_levels, const int32_t *level_res_host,
                                     const int64_t *level_rows_host, const int64_t *primes_host, float scale,
                                     void *stream) {
    if (n_points < 0) return fail(TH_ERR_BAD_ARG, "negative n_points");
    LevelParams P;
    CoordView cv;
    if (int rc = fill_params(P, n_dims, n_levels, level_res_host, level_rows_host, nullptr, primes_host, scale)) return rc;
    if (n_points == 0) return TH_OK;
    if (int rc = make_coord_view(cv, coords_dev, coord_stride_n, coord_stride_d, coord_dtype, n_dims)) return rc;
    if (!idx_out_dev) return fail(TH_ERR_BAD_ARG, "null index output");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned grid = static_cast<unsigned>((n_points + kThreads - 1) / kThreads);
    long long *io = reinterpret_cast<long long *>(idx_out_dev);
    switch (n_dims) {
        case 1: hash_debug_kernel<1><<<grid, kThreads, 0, s>>>(P, cv, io, weight_out_dev, n_points, n_levels); break;
        case 2: hash_debug_kernel<2><<<grid, kThreads, 0, s>>>(P, cv, io, weight_out_dev, n_points, n_levels); break;
        default: hash_debug_kernel<3><<<grid, kThreads, 0, s>>>(P, cv, io, weight_out_dev, n_points, n_levels); break;
    }
    return launch_status("hash_debug_kernel launch");
}
