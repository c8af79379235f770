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
#include "hash_device.cuh"

namespace th {
namespace {

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
    const bool live = load_coords<D, 2>(cv, n_points, blockIdx.x, x, stage);
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
            // (and an evict-last hint on the small dense levels changed nothing: 0.557 against 0.552 ms)
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
    const bool live = load_coords<D, 2>(cv, n_points, blockIdx.x, x, stage);
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

// Two lanes per point, exactly like the forward and backward kernels: lane `side` computes the
// corners on its x-side of the cell with side_indices / side_weights - the functions those kernels
// call - and writes them to the corner slots they stand for (corner c = side | j << 1).
template <int D>
__global__ void __launch_bounds__(kThreads)
hash_debug_kernel(const __grid_constant__ LevelParams P, const CoordView cv, long long *__restrict__ idx_out,
                  float *__restrict__ w_out, long long n_points, int n_levels) {
    constexpr int kPoints = kThreads / 2;
    constexpr int kSide = 1 << (D - 1);
    __shared__ __align__(16) float stage[kPoints * D];
    float x[D];
    if (!load_coords<D, 2>(cv, n_points, blockIdx.x, x, stage)) return;
    if (P.scale != 1.f) {
#pragma unroll
        for (int d = 0; d < D; ++d) x[d] = __fdiv_rn(x[d], P.scale);
    }
    const int side = threadIdx.x & 1;
    const long long i = static_cast<long long>(blockIdx.x) * kPoints + (threadIdx.x >> 1);
    for (int level = 0; level < n_levels; ++level) {
        uint32_t cell[D], idx[kSide];
        float t[D], w[kSide];
        locate<D>(x, P.res[level], cell, t);
        side_weights<D>(t, side, w);
        side_indices<D>(cell, P, level, side, idx);
        const long long o = (i * n_levels + level) * (1 << D);
#pragma unroll
        for (int j = 0; j < kSide; ++j) {
            const int c = side | (j << 1);
            idx_out[o + c] = idx[j];
            if (w_out) w_out[o + c] = w[j];
        }
    }
}

// ---- host side ------------------------------------------------------------------------------

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
        // the kernel addresses its shared-memory copy by (level offset - first offset): levels must follow one another
        if (end > l0 && P.offset[end] != P.offset[end - 1] + P.rows[end - 1]) break;
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

int hash_status_word() {
    int status = 0;
    if (cudaMemcpyFromSymbol(&status, g_hash_status, sizeof(int)) != cudaSuccess) return -1;
    return status;
}

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

namespace th {
int field_tc_status_word();  // neural_field.cu: bit 1 = its copy of the encoding status word
}

extern "C" int th_hash_status(void) {
    const int own = hash_status_word(), field = field_tc_status_word();
    if (own < 0 || field < 0) return -1;
    return (own | (field >> 1)) & 1;
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
    const unsigned grid = static_cast<unsigned>((n_points + kThreads / 2 - 1) / (kThreads / 2));
    long long *io = reinterpret_cast<long long *>(idx_out_dev);
    switch (n_dims) {
        case 1: hash_debug_kernel<1><<<grid, kThreads, 0, s>>>(P, cv, io, weight_out_dev, n_points, n_levels); break;
        case 2: hash_debug_kernel<2><<<grid, kThreads, 0, s>>>(P, cv, io, weight_out_dev, n_points, n_levels); break;
        default: hash_debug_kernel<3><<<grid, kThreads, 0, s>>>(P, cv, io, weight_out_dev, n_points, n_levels); break;
    }
    return launch_status("hash_debug_kernel launch");
}
