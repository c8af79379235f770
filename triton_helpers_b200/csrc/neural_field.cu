// Hash encoding and fused MLP in ONE kernel per direction (sm_100a).
//
// triton_helpers keeps the two layers apart and notes that the encoding "will be used with a fully fused
// MLP", its L * F columns small enough to stay on chip (triton_helpers/layers/hash_encoding/kernel.py:241-243).
// Here they share a kernel:
//
//   field_fwd_kernel   coordinates -> gathers / interpolation (the arithmetic of hash_fwd_kernel) -> the
//                      point tile's features land in the swizzled operand tile of the first tcgen05 GEMM
//                      -> MLP layers with accumulators in TMEM -> prediction, or (prediction - target) *
//                      scale and the squared error.  The [N, L*F] feature matrix is never read back; it is
//                      written out only when the caller wants it for the backward pass.
//   field_bwd_kernel   features + output gradient tiles -> recomputed activations, dgrad and wgrad on the
//                      tensor cores (weight gradients resident in TMEM) -> the feature gradient of the
//                      tile stays in shared memory -> scatter: weight * gradient into the table gradient
//                      with vector reductions (the arithmetic of hash_bwd_kernel), the leading dense levels
//                      accumulated per CTA in shared memory and flushed once.
//
// Why one kernel: the encoding is bound by the SM-to-L2 request path (one request per clock per SM) with the
// tensor pipe idle, the MLP by a chain of short tensor-core steps with that path idle; in one kernel the
// MLP's time can hide under the encoding's, and the feature matrix and its gradient stay on chip.  What it
// costs: the stand-alone encoding kernels need all of an SM's registers (32 warps of 64) to keep that path
// busy, and every warp given to the MLP is one they lose.
//
// Forward: one CTA per SM, three point units (gathers) and one row group (MLP) that hand tiles over through a
// ring of operand tiles; two bursts of gathers in flight per lane make up for the smaller number of warps.
// Backward: one CTA per SM made of two independent GROUPS of 512 threads that synchronise with named
// barriers; a group alternates between its MLP phase (256 of its threads) and its scatter phase (all 512),
// owns its operand tiles and 256 TMEM columns, and shares the weights and the shared-memory copy of the
// coarse levels with the other group.
//
// Every mbarrier wait is bounded; a wait that runs out raises the status word th_mlp_tc_status reads,
// the CTA stops working, keeps its barrier sequence, frees its TMEM and returns.
#include "hash_device.cuh"
#include "mlp_tc_device.cuh"

namespace th {
namespace {

constexpr int kTilePoints = kTileRows;  // 128 points = 128 MLP rows
constexpr int kChunkFeats = 8;          // features in one 16-byte chunk of a 16-bit row

// ---- forward: thread roles ---------------------------------------------------------------------------
//
// ONE CTA of 896 threads per SM:
//   3 point units of 256 threads   two lanes per point, 128 points: the encoding's gathers
//   1 row group of 128 threads     thread = tile row = TMEM lane, warp 0 issues the MMAs: the MLP
// A tile goes from a point unit to the row group through a ring of 6 operand tiles in shared memory.  The
// CTA's tiles are numbered 0, 1, 2, ...; tile q uses buffer q % 6 and is written by point unit q % 3, so a
// buffer always has the same two parties and two named barriers: FULL[r] (the unit arrives, the row group
// waits) and EMPTY[r] (the row group arrives, the unit waits, from the buffer's second use on).  Nobody else
// ever waits for anybody: while the row group walks a tile through its layers, the point units keep the
// SM-to-L2 request path busy, which is what bounds the encoding.
constexpr int kUnits = 3, kUnitThreads = 256;
constexpr int kRowGroups = 1, kRowThreads = 128;
constexpr int kRing = 6;
static_assert(kRing % kUnits == 0 && kRing % kRowGroups == 0, "a ring buffer keeps its producer and its consumer");
constexpr int kHandOver = kUnitThreads + kRowThreads;  // threads meeting at a FULL / EMPTY barrier

__device__ __forceinline__ int bar_full(int r) { return 1 + r; }
__device__ __forceinline__ int bar_empty(int r) { return 1 + kRing + r; }
__device__ __forceinline__ int bar_rows(int g) { return 1 + 2 * kRing + g; }

__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void named_barrier_arrive(int id, int threads) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// A row group waits for the MMAs committed to `mbar`: its warp 0 polls (bounded; `poller` is false when
// nothing was issued), the other three warps park at the group's barrier.  False for every thread alike
// when a wait ran out somewhere in the CTA.
__device__ __forceinline__ bool rows_wait_mma(uint32_t mbar, uint32_t &phase, volatile int *abort_flag, int barrier_id, bool poller) {
    if (poller) {
        if (!mbar_wait(mbar, phase)) {
            *abort_flag = 1;
            g_tc_status = 1;
        }
        tc_fence_after();
        tc_fence_before();
    }
    phase ^= 1;
    named_barrier(barrier_id, kRowThreads);
    tc_fence_after();
    return *abort_flag == 0;
}

// One accumulator row (out_pad a multiple of 16 columns) -> bias, activation, rounding -> 16-byte chunks handed
// to `sink(chunk index, packed values)`, 16 columns per TMEM load: half the registers of the 32-column form.
template <typename T, int ACT, bool BIAS, typename Sink>
__device__ __forceinline__ void drain_row16(uint32_t taddr, int out_pad, const float *bias, Sink sink) {
    for (int first = 0; first < out_pad; first += 16) {
        uint32_t raw[32];
        tmem_ld16(taddr + first, raw);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 2; ++u) sink(first / 8 + u, finish8<T, ACT, BIAS>(raw + 8 * u, bias + first + 8 * u));
    }
}

// Set-up shared by both kernels: barriers, TMEM allocation by warp 0, publication.
__device__ __forceinline__ uint32_t field_setup(uint32_t *tmem_holder, unsigned long long *mbars, int *abort_flag, uint32_t tmem_cols,
                                                bool weights_ok) {
    if (threadIdx.x == 0) {
        for (int g = 0; g < kRowGroups; ++g)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&mbars[g])), "r"(1u) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_holder)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (!weights_ok) {
        *abort_flag = 1;
        g_tc_status = 1;
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    return *tmem_holder;
}

__device__ __forceinline__ void field_teardown(uint32_t tmem, uint32_t tmem_cols) {
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
}

// ---- forward --------------------------------------------------------------------------------------
//
// Point units are the producers: a unit writes its tile's L * F features as 16-bit rows straight into a ring
// buffer in the operand layout of the first GEMM (and to memory when the caller wants them for the backward
// pass).  Row groups consume: the layers run in place in the ring buffer, the last epilogue writes the
// prediction or (prediction - target) * scale and sums the squared error.

constexpr int kFwdThreads = kUnits * kUnitThreads + kRowGroups * kRowThreads;

template <typename T, int D, int F, int ACT, bool BIAS>
__global__ void __launch_bounds__(kFwdThreads, 1)
field_fwd_kernel(const __grid_constant__ LevelParams P, const CoordView cv, const T *__restrict__ table, const int n_levels,
                 const MlpShape s, const MlpParams p, const __grid_constant__ WeightMaps maps, const int use_tma,
                 T *__restrict__ feats, const long long feats_stride, T *__restrict__ y, const long long y_stride,
                 const int y_vec, const MseArgs mse, const long long n_points) {
    constexpr int LG = kChunkFeats / F;      // levels per 16-byte chunk of the feature row
    constexpr int kSide = 1 << (D - 1);
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint32_t tmem_holder;
    __shared__ __align__(8) unsigned long long mbars[kRowGroups];
    __shared__ __align__(8) unsigned long long wbar;
    __shared__ int abort_flag;
    const TcPlan PL = tc_plan(s, false, kRing);  // kRing operand tiles, then weights and biases
    constexpr int bf16 = std::is_same<T, __half>::value ? 0 : 1;
    constexpr uint32_t kTmemCols = 64 * kRowGroups;  // 64 accumulator columns per row group (a power of two >= 32)
    volatile int *abort_now = &abort_flag;

    if (threadIdx.x == 0) abort_flag = 0;
    // tiles start as zeros: feature columns a narrow encoding never writes are read by the first GEMM as zeros
    for (int e = threadIdx.x; e < kRing * kTileBytes / 16; e += kFwdThreads) reinterpret_cast<uint4 *>(smem)[e] = make_uint4(0, 0, 0, 0);
    {
        float *bias = reinterpret_cast<float *>(smem + PL.bias_offset);
        for (int e = threadIdx.x; e < (s.depth + 1) * kMaxDim; e += kFwdThreads) {
            const int layer = e / kMaxDim, c = e % kMaxDim;
            float v = 0.f;
            if (BIAS) {
                if (layer == 0) {
                    if (c < s.d_hid) v = to_float<T>(static_cast<const T *>(p.b_in)[c]);
                } else if (layer < s.depth) {
                    if (c < s.d_hid) v = to_float<T>(static_cast<const T *>(p.b_hid)[(layer - 1) * s.d_hid + c]);
                } else if (c < s.d_out) {
                    v = to_float<T>(static_cast<const T *>(p.b_out)[c]);
                }
            }
            bias[e] = v;
        }
    }
    bool weights_ok = true;
    if (use_tma) {
        weights_ok = tma_stage_weights(smem, PL, s, maps, &wbar);  // contains a CTA barrier
    } else {
        if (threadIdx.x < kTcThreads) stage_all_weights<T>(smem, PL, s, p);  // its loops stride by kTcThreads
        __syncthreads();
    }
    const uint32_t tmem_base = field_setup(&tmem_holder, mbars, &abort_flag, kTmemCols, weights_ok);

    const long long n_tiles = (n_points + kTilePoints - 1) / kTilePoints;
    const long long first_tile = blockIdx.x, tile_stride = gridDim.x;
    const long long n_mine = first_tile < n_tiles ? (n_tiles - first_tile + tile_stride - 1) / tile_stride : 0;

    if (threadIdx.x < kUnits * kUnitThreads) {
        // ================= point unit: encoding of a tile into its ring buffer =================
        const int unit = threadIdx.x / kUnitThreads, v = threadIdx.x % kUnitThreads;
        const int lp = v >> 1, side = v & 1;
        const uint32_t row_off = lp * 128, swz = (lp & 7) << 4;
        for (long long q = unit; q < n_mine; q += kUnits) {
            const int r = static_cast<int>(q % kRing);
            const long long pt = (first_tile + q * tile_stride) * kTilePoints + lp;
            const bool live = pt < n_points;
            float x[D];
#pragma unroll
            for (int d = 0; d < D; ++d) x[d] = 0.f;
            if (live) load_coords_strided<D>(cv, pt, x);
            if (P.scale != 1.f) {
#pragma unroll
                for (int d = 0; d < D; ++d) x[d] = __fdiv_rn(x[d], P.scale);
            }
            if (q >= kRing) named_barrier(bar_empty(r), kHandOver);  // the row group is done with this buffer's previous tile
            if (!*abort_now) {
                const uint32_t my_row = smem_addr(smem + r * kTileBytes) + row_off;
                T *feat_row = feats && live ? feats + pt * feats_stride : nullptr;
                // Two chunks of gathers are in flight per lane: the loads of chunk c + 1 are issued before chunk c is
                // used.  A warp that waits for one burst of 16 rows at a time leaves the request path idle unless 32
                // such warps share the SM; with two bursts in flight the 24 warps of the point units keep it busy.
                // Gathered rows stay packed (F 16-bit values in F / 2 registers) until they are used, and the
                // interpolation weights are worked out when a chunk is used rather than kept across the loads.
                auto issue = [&](int lg, uint32_t(&e)[LG][kSide][F / 2]) {
#pragma unroll
                    for (int j = 0; j < LG; ++j) {
                        const int level = lg + j;
                        uint32_t cell[D], idx[kSide];
                        float t[D];
                        locate<D>(x, P.res[level], cell, t);
                        side_indices<D>(cell, P, level, side, idx);
                        const T *base = table + P.offset[level] * F;
#pragma unroll
                        for (int c = 0; c < kSide; ++c) {
                            const T *rowp = base + static_cast<size_t>(idx[c]) * F;
                            if constexpr (F == 2) {
                                e[j][c][0] = __ldg(reinterpret_cast<const unsigned int *>(rowp));
                            } else {
                                const uint2 two = __ldg(reinterpret_cast<const uint2 *>(rowp));
                                e[j][c][0] = two.x;
                                e[j][c][1] = two.y;
                            }
                        }
                    }
                };
                auto consume = [&](int lg, const uint32_t(&e)[LG][kSide][F / 2]) {
                    float acc[kChunkFeats];
#pragma unroll
                    for (int j = 0; j < LG; ++j) {
                        uint32_t cell[D];
                        float t[D], w[kSide];
                        locate<D>(x, P.res[lg + j], cell, t);
                        side_weights<D>(t, side, w);
#pragma unroll
                        for (int f2 = 0; f2 < F / 2; ++f2) {
                            float lo_sum = 0.f, hi_sum = 0.f;
#pragma unroll
                            for (int c = 0; c < kSide; ++c) {
                                const float2 pair = unpack_pair<T>(e[j][c][f2]);
                                if (c == 0) {
                                    lo_sum = __fmul_rn(w[0], pair.x);
                                    hi_sum = __fmul_rn(w[0], pair.y);
                                } else {
                                    lo_sum = __fadd_rn(lo_sum, __fmul_rn(w[c], pair.x));
                                    hi_sum = __fadd_rn(hi_sum, __fmul_rn(w[c], pair.y));
                                }
                            }
                            // low-x side + high-x side
                            acc[j * F + 2 * f2] = __fadd_rn(lo_sum, __shfl_xor_sync(0xffffffffu, lo_sum, 1));
                            acc[j * F + 2 * f2 + 1] = __fadd_rn(hi_sum, __shfl_xor_sync(0xffffffffu, hi_sum, 1));
                        }
                    }
                    // each lane of the pair keeps half of the chunk: 4 values = 8 bytes
                    const int h = side * 4;
                    const uint32_t lo = pack_pair<T>(acc[h], acc[h + 1]), hi = pack_pair<T>(acc[h + 2], acc[h + 3]);
                    const int chunk = lg / LG;
                    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(my_row + ((chunk << 4) ^ swz) + side * 8), "r"(lo), "r"(hi) : "memory");
                    if (feat_row) __stcs(reinterpret_cast<uint2 *>(feat_row + chunk * kChunkFeats + h), make_uint2(lo, hi));
                };
                uint32_t ea[LG][kSide][F / 2], eb[LG][kSide][F / 2];
                issue(0, ea);
                for (int lg = 0; lg < n_levels; lg += 2 * LG) {  // levels * features is a multiple of 16: an even number of chunks
                    issue(lg + LG, eb);
                    consume(lg, ea);
                    if (lg + 2 * LG < n_levels) issue(lg + 2 * LG, ea);
                    consume(lg + LG, eb);
                }
            }
            fence_async_smem();  // the tensor core reads the tile through the async proxy
            named_barrier_arrive(bar_full(r), kHandOver);
        }
    } else {
        // ================= row group: the MLP on a tile, in place in its ring buffer =================
        const int t = threadIdx.x - kUnits * kUnitThreads;
        const int g = t / kRowThreads, row = t % kRowThreads, warp = row >> 5;
        const bool issuer = warp == 0;
        const uint32_t acc = tmem_base + g * kAccCols;
        const uint32_t taddr = acc + (static_cast<uint32_t>(32 * warp) << 16);
        const uint32_t bar = smem_addr(&mbars[g]);
        const float *bias = reinterpret_cast<const float *>(smem + PL.bias_offset);
        uint32_t phase = 0;
        float loss = 0.f;
        for (long long q = g; q < n_mine; q += kRowGroups) {
            const int r = static_cast<int>(q % kRing);
            unsigned char *tile = smem + r * kTileBytes;
            const uint32_t tile_addr = smem_addr(tile);
            const uint32_t row_addr = tile_addr + row * 128, row_swizzle = (row & 7) << 4;
            const long long row0 = (first_tile + q * tile_stride) * kTileRows;
            named_barrier(bar_full(r), kHandOver);  // the point unit has written this tile's features
            for (int l = 0; l <= s.depth; ++l) {
                const int in_pad = l == 0 ? s.ki : s.h;
                const int out_pad = l == s.depth ? s.no : s.h;
                bool issued = false;
                if (issuer && !*abort_now) {
                    const bool leader = elect_one();
                    tc_fence_after();
                    issue_gemm(leader, acc, tile_addr, 32, smem_addr(weight_tile(smem, PL, s, l)), 32, in_pad / 16,
                               instr_desc(128, out_pad, bf16, 0, 0), false);
                    if (leader) mma_commit(bar);
                    __syncwarp();
                    issued = true;
                }
                const bool ok = rows_wait_mma(bar, phase, abort_now, bar_rows(g), issued);
                const float *layer_bias = bias + l * kMaxDim;
                if (ok && l < s.depth) {
                    drain_row16<T, ACT, BIAS>(taddr, out_pad, layer_bias, [&](int chunk, uint4 packed) {
                        st_shared_16(row_addr + ((chunk << 4) ^ row_swizzle), packed);
                    });
                    fence_async_smem();
                } else if (ok) {
                    const bool live = row0 + row < n_points;
                    const long long rr = live ? row0 + row : 0;
                    if (mse.target) {
                        // d_out is a multiple of 8 and all rows are 16-byte aligned here (checked by the launcher)
                        const T *target_row = static_cast<const T *>(mse.target) + rr * mse.target_stride;
                        T *grad_row = static_cast<T *>(mse.grad) + rr * mse.grad_stride;
                        T *out_row = y ? y + rr * y_stride : nullptr;
                        drain_row16<T, TH_ACT_NONE, BIAS>(taddr, out_pad, layer_bias, [&](int chunk, uint4 packed) {
                            if (live && 8 * chunk < s.d_out) {
                                if (out_row) __stcs(reinterpret_cast<uint4 *>(out_row + 8 * chunk), packed);
                                const uint4 tg = __ldcs(reinterpret_cast<const uint4 *>(target_row + 8 * chunk));
                                __stcs(reinterpret_cast<uint4 *>(grad_row + 8 * chunk), mse_chunk<T>(packed, tg, mse.grad_scale, loss));
                            }
                        });
                    } else {
                        T *out_row = y + rr * y_stride;
                        drain_row16<T, TH_ACT_NONE, BIAS>(taddr, out_pad, layer_bias, [&](int chunk, uint4 packed) {
                            if (live) store_chunk_to_global<T>(out_row, chunk, s.d_out, packed, y_vec);
                        });
                    }
                }
                tc_fence_before();
                named_barrier(bar_rows(g), kRowThreads);  // next layer reads what the group wrote; the accumulator is free again
            }
            if (q + kRing < n_mine) named_barrier_arrive(bar_empty(r), kHandOver);  // the buffer may take the CTA's tile q + 6
        }
        if (mse.target && mse.loss_sum) {  // one atomic per warp for the whole kernel
            for (int off = 16; off > 0; off >>= 1) loss += __shfl_xor_sync(0xffffffffu, loss, off);
            if ((threadIdx.x & 31) == 0) atomicAdd(mse.loss_sum, loss);
        }
    }
    field_teardown(tmem_base, kTmemCols);
}

// Thread groups that share an SM start in step and would stay in step - all of them scattering, then all of
// them in their MLP phase with the request path idle.  Each therefore waits a different fraction of a tile
// period once, at the start, so that their MLP phases interleave from then on.
__device__ __forceinline__ void stagger_start(long long cycles) {
    const long long t0 = clock64();
    while (clock64() - t0 < cycles) __nanosleep(200);
}

// ---- backward -------------------------------------------------------------------------------------
//
// One CTA per SM, G groups of NT threads.  Threads 0..255 of a group are its MLP threads (thread = tile
// row x column half, warp 0 issues the MMAs); all NT threads scatter.  A group's barriers: id 1 + 2g for
// all NT threads, id 2 + 2g for the 256 MLP threads.
//
// Operand tiles of a group (depth d): act[0] = features, act[l] = input of layer l (recomputed), and one
// tile for the output gradient.  Going down the layers, dz of layer l - 1 is written IN PLACE over
// act[l] once the MMAs that read act[l] have finished (dgrad and wgrad of a step are committed and
// awaited together), and the feature gradient of the tile ends up, in the operand layout, in act[1]'s
// buffer, where the scatter phase reads it: d + 2 tiles per group.

struct FieldBwdPlan {
    int group_tiles;    // operand tiles per group
    int weights;        // byte offset of the weight tiles (after all groups' tiles)
    int coarse;         // byte offset of the shared-memory copy of the coarse levels
    int coarse_bytes;
    int total;
    TcPlan w;           // weight offsets relative to `weights` come from a forward-style plan with zero tiles
};

__host__ __device__ inline FieldBwdPlan field_bwd_plan(const MlpShape &s, int groups, int coarse_bytes) {
    FieldBwdPlan f{};
    f.group_tiles = s.depth + 2;
    f.weights = groups * f.group_tiles * kTileBytes;
    f.w = tc_plan(s, false, 0);  // act_tiles = 0: offsets count from the first weight tile
    f.coarse = f.weights + ((f.w.total + 15) & ~15);
    f.coarse_bytes = (coarse_bytes + 15) & ~15;
    f.total = f.coarse + f.coarse_bytes;
    return f;
}


// The group's MLP threads wait for the MMAs committed to `mbar`: the warp that issued them polls
// (bounded; `poller` is false when nothing was issued), the others park at the MLP barrier.  False for
// every thread alike when a wait ran out somewhere in the CTA.
__device__ __forceinline__ bool group_wait_mma(uint32_t mbar, uint32_t &phase, volatile int *abort_flag, int barrier_id, bool poller) {
    if (poller) {
        if (!mbar_wait(mbar, phase)) {
            *abort_flag = 1;
            g_tc_status = 1;
        }
        tc_fence_after();
        tc_fence_before();
    }
    phase ^= 1;
    named_barrier(barrier_id, kTcThreads);
    tc_fence_after();
    return *abort_flag == 0;
}

template <typename T, int D, int F, int ACT, int G, int NT>
__global__ void __launch_bounds__(G * NT, 1)
field_bwd_kernel(const __grid_constant__ LevelParams P, const CoordView cv, const int n_levels, const int coarse_end,
                 const MlpShape s, const MlpParams p, const __grid_constant__ WeightMaps maps, const int use_tma,
                 const T *__restrict__ feats, const long long feats_stride, const T *__restrict__ go, const long long go_stride,
                 T *__restrict__ grad_table, T *__restrict__ gx, const long long gx_stride, float *__restrict__ workspace,
                 const long long n_points, const int vec_bits, const int stagger_cycles) {
    constexpr int LG = kChunkFeats / F;
    constexpr int kSide = 1 << (D - 1);
    constexpr int kHalves = NT / kTcThreads;  // how many ways a group splits a tile's chunks in the scatter phase
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint32_t tmem_holder;
    __shared__ __align__(8) unsigned long long mbars[G];
    __shared__ __align__(8) unsigned long long wbar;
    __shared__ int abort_flag;
    const int d = s.depth;
    unsigned long long coarse_rows = 0;
    if (coarse_end > 0) coarse_rows = P.offset[coarse_end - 1] + P.rows[coarse_end - 1] - P.offset[0];
    const FieldBwdPlan FP = field_bwd_plan(s, G, static_cast<int>(coarse_rows * F * sizeof(T)));
    constexpr int bf16 = std::is_same<T, __half>::value ? 0 : 1;
    const TcPlan BP = tc_plan(s, true);  // TMEM columns of a group: dgrad accumulator + one weight-gradient accumulator per layer
    const int group_cols = BP.tmem_cols;

    const int group = threadIdx.x / NT, u = threadIdx.x % NT;
    const bool mlp_thread = u < kTcThreads;
    const int bar_all = 1 + 2 * group, bar_mlp = 2 + 2 * group;
    volatile int *abort_now = &abort_flag;

    // ---- set-up ----
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int g = 0; g < G; ++g)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&mbars[g])), "r"(1u) : "memory");
    }
    // operand tiles and the coarse copy start as zeros
    for (int e = threadIdx.x; e < FP.weights / 16; e += G * NT) reinterpret_cast<uint4 *>(smem)[e] = make_uint4(0, 0, 0, 0);
    for (int e = threadIdx.x; e < FP.coarse_bytes / 16; e += G * NT) reinterpret_cast<uint4 *>(smem + FP.coarse)[e] = make_uint4(0, 0, 0, 0);
    unsigned char *wsmem = smem + FP.weights;
    bool weights_ok = true;
    if (use_tma) {
        weights_ok = tma_stage_weights(wsmem, FP.w, s, maps, &wbar);  // contains a CTA barrier
    } else {
        if (threadIdx.x < kTcThreads) stage_all_weights<T>(wsmem, FP.w, s, p);  // its loops stride by kTcThreads
        __syncthreads();
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_holder)),
                     "r"(static_cast<uint32_t>(G * group_cols))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (!weights_ok) {
        abort_flag = 1;
        g_tc_status = 1;
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_holder + group * group_cols;

    unsigned char *tiles = smem + group * FP.group_tiles * kTileBytes;
    auto act_tile = [&](int l) { return tiles + l * kTileBytes; };
    unsigned char *go_tile = tiles + (d + 1) * kTileBytes;
    auto dw_col = [&](int l) { return kAccCols + (l == 0 ? 0 : s.ki + (l - 1) * s.h); };
    auto weight_addr = [&](int l) { return smem_addr(weight_tile(wsmem, FP.w, s, l)); };
    T *coarse_acc = reinterpret_cast<T *>(smem + FP.coarse);
    const uint32_t bar = smem_addr(&mbars[group]);
    uint32_t phase = 0;
    const Seat seat_raw;  // built from threadIdx.x: valid for group-local use only through the fields below
    Seat seat = seat_raw;
    {
        const int warp = u >> 5;
        seat.row = 32 * (warp & 3) + (u & 31);
        seat.group = (warp >> 2) & 1;
        seat.lane_base = static_cast<uint32_t>(32 * (warp & 3)) << 16;
    }
    const uint32_t taddr = tmem + seat.lane_base;
    const bool issuer = u < 32;

    const long long n_tiles = (n_points + kTilePoints - 1) / kTilePoints;
    bool accumulated = false;
    // rows that can be moved as whole 16-byte chunks (checked by the launcher): bit 0 features, 1 output gradient, 2 feature gradient
    const bool x_vec = vec_bits & 1, go_vec = vec_bits & 2, gx_vec = vec_bits & 4;

    if (G > 1 && group > 0) stagger_start(static_cast<long long>(group) * stagger_cycles);

    for (long long tile = static_cast<long long>(blockIdx.x) * G + group; tile < n_tiles; tile += static_cast<long long>(gridDim.x) * G) {
        const long long row0 = tile * kTileRows;
        const bool dead = *abort_now != 0;  // keep the barrier sequence, do no work
        // ================= MLP phase (the group's first 256 threads) =================
        if (mlp_thread) {
            if (!dead) {
                if (x_vec && go_vec) {
                    // cp.async by the 256 MLP threads (tc_tiles.cuh strides by kTcThreads and uses threadIdx.x: pass u through a shifted copy)
                    const int chunks_x = s.ki / 8, chunks_g = s.no / 8;
                    for (int id = u; id < kTileRows * chunks_x; id += kTcThreads) {
                        const int r = id / chunks_x, c = id - r * chunks_x;
                        const long long row = row0 + r;
                        const bool inside = row < n_points && 8 * c < s.d_in;
                        const T *src = inside ? feats + row * feats_stride + 8 * c : feats;
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(chunk_ptr(act_tile(0), r, c))), "l"(src), "r"(inside ? 16 : 0) : "memory");
                    }
                    for (int id = u; id < kTileRows * chunks_g; id += kTcThreads) {
                        const int r = id / chunks_g, c = id - r * chunks_g;
                        const long long row = row0 + r;
                        const bool inside = row < n_points && 8 * c < s.d_out;
                        const T *src = inside ? go + row * go_stride + 8 * c : go;
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(chunk_ptr(go_tile, r, c))), "l"(src), "r"(inside ? 16 : 0) : "memory");
                    }
                    asm volatile("cp.async.commit_group;" ::: "memory");
                    async_tile_wait();
                } else {
                    const int chunks_x = s.ki / 8, chunks_g = s.no / 8;
                    for (int id = u; id < kTileRows * chunks_x; id += kTcThreads) {
                        const int r = id / chunks_x, c = id - r * chunks_x;
                        const long long row = row0 + r;
                        uint4 v = make_uint4(0, 0, 0, 0);
                        if (row < n_points && 8 * c < s.d_in) v = gather8(reinterpret_cast<const unsigned short *>(feats + row * feats_stride + 8 * c), 8 * c, s.d_in);
                        *reinterpret_cast<uint4 *>(chunk_ptr(act_tile(0), r, c)) = v;
                    }
                    for (int id = u; id < kTileRows * chunks_g; id += kTcThreads) {
                        const int r = id / chunks_g, c = id - r * chunks_g;
                        const long long row = row0 + r;
                        uint4 v = make_uint4(0, 0, 0, 0);
                        if (row < n_points && 8 * c < s.d_out) v = gather8(reinterpret_cast<const unsigned short *>(go + row * go_stride + 8 * c), 8 * c, s.d_out);
                        *reinterpret_cast<uint4 *>(chunk_ptr(go_tile, r, c)) = v;
                    }
                }
            }
            fence_async_smem();
            tc_fence_before();
            named_barrier(bar_mlp, kTcThreads);
            // ---- recompute the forward, keeping every layer's input ----
            for (int l = 0; l < d; ++l) {
                bool issued = false;
                if (issuer && !*abort_now) {
                    const bool leader = elect_one();
                    tc_fence_after();
                    issue_gemm(leader, tmem, smem_addr(act_tile(l)), 32, weight_addr(l), 32, (l == 0 ? s.ki : s.h) / 16,
                               instr_desc(128, s.h, bf16, 0, 0), false);
                    if (leader) mma_commit(bar);
                    __syncwarp();
                    issued = true;
                }
                if (group_wait_mma(bar, phase, abort_now, bar_mlp, issued))
                    hidden_epilogue<T, ACT, false>(taddr, seat, s.h, nullptr, act_tile(l + 1));
                fence_async_smem();
                tc_fence_before();
                named_barrier(bar_mlp, kTcThreads);
            }
            // ---- down the layers: dgrad + wgrad per step ----
            for (int l = d; l >= 0; --l) {
                const int in_pad = l == 0 ? s.ki : s.h;
                const int out_pad = l == d ? s.no : s.h;
                unsigned char *dz = l == d ? go_tile : act_tile(l + 1);  // dz of layer l: written over act[l + 1] one step ago
                bool issued = false;
                if (issuer && !*abort_now) {
                    const bool leader = elect_one();
                    tc_fence_after();
                    issue_gemm(leader, tmem, smem_addr(dz), 32, weight_addr(l), 2048, out_pad / 16, instr_desc(128, in_pad, bf16, 0, 1), false);
                    issue_gemm(leader, tmem + dw_col(l), smem_addr(dz), 2048, smem_addr(act_tile(l)), 2048, kTileRows / 16,
                               instr_desc(64, in_pad, bf16, 1, 1), accumulated);
                    if (leader) mma_commit(bar);
                    __syncwarp();
                    issued = true;
                }
                if (group_wait_mma(bar, phase, abort_now, bar_mlp, issued)) {
                    if (l > 0) {
                        dz_epilogue<T, ACT>(taddr, seat, in_pad, act_tile(l), act_tile(l));  // in place: mask from the parked activation
                    } else {
                        // the tile's feature gradient, rounded to T, in the operand layout in act[1]'s buffer
                        hidden_epilogue<T, TH_ACT_NONE, false>(taddr, seat, in_pad, nullptr, act_tile(1));
                        if (gx) {
                            const bool live = row0 + seat.row < n_points;
                            dx_epilogue<T>(taddr, seat, in_pad, gx + (live ? row0 + seat.row : 0) * gx_stride, s.d_in, live, gx_vec);
                        }
                    }
                }
                fence_async_smem();
                tc_fence_before();
                named_barrier(bar_mlp, kTcThreads);
            }
            accumulated = accumulated || !*abort_now;
        }
        named_barrier(bar_all, NT);  // the feature gradient is in act[1]'s buffer

        // ================= scatter phase (all NT threads of the group) =================
        if (!*abort_now) {
            const int lp = (u % kTcThreads) >> 1, side = u & 1, half = u / kTcThreads;
            const long long pt = row0 + lp;
            const bool live = pt < n_points;
            float x[D];
#pragma unroll
            for (int dd = 0; dd < D; ++dd) x[dd] = 0.f;
            if (live) load_coords_strided<D>(cv, pt, x);
            if (P.scale != 1.f) {
#pragma unroll
                for (int dd = 0; dd < D; ++dd) x[dd] = __fdiv_rn(x[dd], P.scale);
            }
            const unsigned lane = threadIdx.x & 31u;
            const uint32_t grad_row = smem_addr(act_tile(1)) + lp * 128, swz = (lp & 7) << 4;
            const int n_chunks = n_levels / LG;
            for (int chunk = half; chunk < n_chunks; chunk += kHalves) {
                float g8[kChunkFeats];
                {
                    const uint4 raw = ld_shared_16(grad_row + ((chunk << 4) ^ swz));
                    const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float2 f2 = unpack_pair<T>(wds[k]);
                        g8[2 * k] = live ? f2.x : 0.f;
                        g8[2 * k + 1] = live ? f2.y : 0.f;
                    }
                }
#pragma unroll
                for (int j = 0; j < LG; ++j) {
                    const int level = chunk * LG + j;
                    uint32_t cell[D], idx[kSide];
                    float t[D], w[kSide];
                    locate<D>(x, P.res[level], cell, t);
                    side_weights<D>(t, side, w);
                    side_indices<D>(cell, P, level, side, idx);
                    if (level < coarse_end) {
                        // leading dense levels: private copy in shared memory, flushed once at the end
                        T *base = coarse_acc + (P.offset[level] - P.offset[0]) * F;
                        if (live) {
#pragma unroll
                            for (int c = 0; c < kSide; ++c) {
                                float v[F];
#pragma unroll
                                for (int f = 0; f < F; ++f) v[f] = __fmul_rn(w[c], g8[j * F + f]);
                                smem_add_row<T, F>(base + static_cast<size_t>(idx[c]) * F, v);
                            }
                        }
                        continue;
                    }
                    T *base = grad_table + P.offset[level] * F;
                    // lanes on the same side of the same cell share all their rows: sum in registers first (coarse grids only)
                    bool shared_cell = false;
                    unsigned peers = 1u << lane;
                    if (P.res[level] <= kAggregateMaxRes) {
                        unsigned long long key = 0;
                        bool packable = live;
#pragma unroll
                        for (int dd = 0; dd < D; ++dd) {
                            packable = packable && cell[dd] < (1u << 20);
                            key = (key << 20) | (cell[dd] & 0xfffffu);
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
                                for (int f = 0; f < F; ++f) v[f] = __fmul_rn(w[c], g8[j * F + f]);
                                red_add_row<F>(base + static_cast<size_t>(idx[c]) * F, v);
                            }
                        }
                    } else {
                        const bool leader = (peers & ((1u << lane) - 1u)) == 0;
                        const int steps = __reduce_max_sync(0xffffffffu, __popc(peers));
#pragma unroll
                        for (int c = 0; c < kSide; ++c) {
                            float v[F], sum[F];
#pragma unroll
                            for (int f = 0; f < F; ++f) {
                                v[f] = __fmul_rn(w[c], g8[j * F + f]);
                                sum[f] = 0.f;
                            }
                            unsigned rest = peers;
                            for (int st = 0; st < steps; ++st) {
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
        named_barrier(bar_all, NT);  // act[1]'s buffer may be overwritten by the next tile
    }

    // ---- flush: weight gradients from TMEM, coarse levels from shared memory ----
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (!abort_flag) {
        if (mlp_thread && accumulated) {
            const MlpGradWorkspace W = grad_workspace_layout(s, workspace);
            for (int l = 0; l <= d; ++l) {
                const int in_pad = l == 0 ? s.ki : s.h;
                const int in_dim = l == 0 ? s.d_in : s.d_hid, out_dim = l == d ? s.d_out : s.d_hid;
                float *dst = W.base + (l == 0 ? W.w_in : (l == d ? W.w_out : W.w_hid + (l - 1) * s.d_hid * s.d_hid));
                // flush_dw reads threadIdx.x for lane and warp: group-local values agree with it (NT is a multiple of 128)
                flush_dw(taddr + dw_col(l), seat, in_pad, dst, out_dim, in_dim);
            }
        }
        T *dst = grad_table + P.offset[0] * F;
        for (unsigned long long r = threadIdx.x; r < coarse_rows; r += G * NT) {
            float v[F];
            bool any = false;
#pragma unroll
            for (int f = 0; f < F; ++f) {
                v[f] = to_float<T>(coarse_acc[r * F + f]);
                any = any || v[f] != 0.f;
            }
            if (any) red_add_row<F>(dst + r * F, v);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_holder), "r"(static_cast<uint32_t>(G * group_cols)) : "memory");
}

// ---- host side ------------------------------------------------------------------------------------

// Leading dense, contiguous levels whose rows fit `budget` bytes of shared memory (in the table's dtype).
// Measured at 2^21 uniform points, 16 levels x 2 float16 features: level 0 (16^3 grid, every row hit ~3 400
// times) in shared memory takes 0.22 ms off the reductions, level 1 another 0.02 ms, level 2 does not fit.
int field_coarse_end(const LevelParams &P, int n_levels, int row_bytes, int64_t n_points, int budget) {
    if (n_points < (1 << 16)) return 0;  // small batches: the flush of one private copy per CTA costs more than it saves
    size_t bytes = 0;
    int end = 0;
    while (end < n_levels && !((P.hashed_mask >> end) & 1u)) {
        if (end > 0 && P.offset[end] != P.offset[end - 1] + P.rows[end - 1]) break;
        const size_t next = bytes + static_cast<size_t>(P.rows[end]) * row_bytes;
        if (next > static_cast<size_t>(budget)) break;
        bytes = next;
        ++end;
    }
    return end;
}

struct FieldArgs {
    LevelParams P;
    CoordView cv;
    MlpShape s;
    MlpParams p;
    int n_dims, n_feats, n_levels;
};

template <typename T, int D, int F, int ACT, bool BIAS>
int launch_field_fwd(const FieldArgs &a, const void *table, void *feats, int64_t feats_stride, void *y, int64_t y_stride,
                     const MseArgs &mse, int64_t n, cudaStream_t stream) {
    const TcPlan PL = tc_plan(a.s, false, kRing);
    int need = PL.total + 1024;
    if (need + 1024 > kSmemBudget) return kTcNotApplicable;
    if (need < kSmemBudget / 2 + 1024) need = kSmemBudget / 2 + 1024;  // one CTA of 1024 threads per SM
    WeightMaps maps;
    const int use_tma = make_weight_maps(maps, a.s, a.p);
    auto kernel = field_fwd_kernel<T, D, F, ACT, BIAS>;
    if (int rc = cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, need), "cudaFuncSetAttribute(field_fwd_kernel)")) return rc;
    const long long tiles = (n + kTilePoints - 1) / kTilePoints;
    // a CTA keeps three point units and two row groups busy: give each a few tiles before spreading over more SMs
    const long long want = (tiles + kRing - 1) / kRing;
    const long long cap = sm_count();
    kernel<<<static_cast<unsigned>(want < cap ? (want < 1 ? 1 : want) : cap), kFwdThreads, need, stream>>>(
        a.P, a.cv, static_cast<const T *>(table), a.n_levels, a.s, a.p, maps, use_tma, static_cast<T *>(feats), feats_stride,
        static_cast<T *>(y), y_stride, y ? rows_vector_ok(y, y_stride, a.s.d_out) : 0, mse, n);
    return launch_status("field_fwd_kernel launch");
}

constexpr int kBwdGroupThreads = 512;
constexpr int kFieldCoarseBudget = 72 * 1024;  // shared memory the backward sets aside for leading dense levels

// A tile's reductions keep the SM's request path busy for about this many cycles: 128 points x `accesses` rows
// each at somewhat over half a request per row (two x-neighbours mostly share one).
int field_stagger_cycles(int accesses_per_point) { return 128 * accesses_per_point * 6 / 10; }

template <typename T, int D, int F, int ACT, int kBwdGroups>
int launch_field_bwd_groups(const FieldArgs &a, const void *feats, int64_t feats_stride, const void *go, int64_t go_stride, void *grad_table,
                            void *gx, int64_t gx_stride, float *workspace, int64_t n, cudaStream_t stream) {
    const TcPlan BP = tc_plan(a.s, true);
    if (BP.tmem_cols * kBwdGroups > 512) return kTcNotApplicable;
    int budget = kFieldCoarseBudget;
    int coarse_end = 0, total = 0;
    for (;;) {
        coarse_end = field_coarse_end(a.P, a.n_levels, F * sizeof(T), n, budget);
        size_t coarse_bytes = 0;
        for (int l = 0; l < coarse_end; ++l) coarse_bytes += static_cast<size_t>(a.P.rows[l]) * F * sizeof(T);
        total = field_bwd_plan(a.s, kBwdGroups, static_cast<int>(coarse_bytes)).total + 1024;
        if (total + 1024 <= kSmemBudget || coarse_end == 0) break;
        budget /= 2;  // deep networks leave less room: give up coarse levels first
    }
    if (total + 1024 > kSmemBudget) return kTcNotApplicable;
    if (total < kSmemBudget / 2 + 1024) total = kSmemBudget / 2 + 1024;  // one CTA per SM: it takes all the TMEM columns it needs at once
    WeightMaps maps;
    const int use_tma = make_weight_maps(maps, a.s, a.p);
    auto kernel = field_bwd_kernel<T, D, F, ACT, kBwdGroups, kBwdGroupThreads>;
    if (int rc = cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, total), "cudaFuncSetAttribute(field_bwd_kernel)")) return rc;
    const long long tiles = (n + kTilePoints - 1) / kTilePoints;
    const long long want = (tiles + kBwdGroups - 1) / kBwdGroups;
    const long long cap = sm_count();
    kernel<<<static_cast<unsigned>(want < cap ? want : cap), kBwdGroups * kBwdGroupThreads, total, stream>>>(
        a.P, a.cv, a.n_levels, coarse_end, a.s, a.p, maps, use_tma, static_cast<const T *>(feats), feats_stride,
        static_cast<const T *>(go), go_stride, static_cast<T *>(grad_table), static_cast<T *>(gx), gx_stride, workspace, n,
        (rows_vector_ok(feats, feats_stride, a.s.d_in) ? 1 : 0) | (rows_vector_ok(go, go_stride, a.s.d_out) ? 2 : 0) |
            (gx && rows_vector_ok(gx, gx_stride, a.s.d_in) ? 4 : 0),
        field_stagger_cycles(a.n_levels * (1 << a.n_dims)));
    return launch_status("field_bwd_kernel launch");
}

// Two groups per SM when their tensor-memory columns and operand tiles fit (networks up to two hidden
// layers of 64), one group otherwise.
template <typename T, int D, int F, int ACT>
int launch_field_bwd(const FieldArgs &a, const void *feats, int64_t feats_stride, const void *go, int64_t go_stride, void *grad_table,
                     void *gx, int64_t gx_stride, float *workspace, int64_t n, cudaStream_t stream) {
    const int rc = launch_field_bwd_groups<T, D, F, ACT, 2>(a, feats, feats_stride, go, go_stride, grad_table, gx, gx_stride, workspace, n, stream);
    if (rc != kTcNotApplicable) return rc;
    return launch_field_bwd_groups<T, D, F, ACT, 1>(a, feats, feats_stride, go, go_stride, grad_table, gx, gx_stride, workspace, n, stream);
}

int fill_field_args(FieldArgs &a, const void *coords, int64_t stride_n, int64_t stride_d, int coord_dtype, int n_dims, int n_feats,
                    int n_levels, const int32_t *res, const int64_t *rows, const int64_t *offsets, const int64_t *primes, float scale,
                    const void *w_in, const void *b_in, const void *w_hid, const void *b_hid, const void *w_out, const void *b_out,
                    int d_hidden, int d_out, int depth, int activation, int64_t n_points) {
    if (n_points < 0) return fail(TH_ERR_BAD_ARG, "negative n_points");
    if (int rc = fill_params(a.P, n_dims, n_levels, res, rows, offsets, primes, scale)) return rc;
    if (!offsets) return fail(TH_ERR_BAD_ARG, "null level offsets");
    a.n_dims = n_dims, a.n_feats = n_feats, a.n_levels = n_levels;
    const int d_in = n_levels * n_feats;
    if (d_in > kMaxDim) return fail(TH_ERR_UNSUPPORTED, "levels * features = %d exceeds %d", d_in, kMaxDim);
    if (d_hidden < 16 || d_hidden > kMaxDim || (d_hidden & (d_hidden - 1)) || d_out < 1 || d_out > kMaxDim || depth < 1)
        return fail(TH_ERR_UNSUPPORTED, "unsupported MLP shape %d -> %d x %d -> %d", d_in, depth, d_hidden, d_out);
    if (activation < TH_ACT_NONE || activation > TH_ACT_RELU2) return fail(TH_ERR_BAD_ARG, "unknown activation code %d", activation);
    const bool has_bias = b_in || b_hid || b_out;
    a.s = MlpShape{d_in, d_hidden, d_out, depth, pad16(d_in), d_hidden, pad16(d_out), activation, has_bias ? 1 : 0};
    a.p = MlpParams{w_in, w_hid, w_out, b_in, b_hid, b_out};
    if (!w_in || !w_out || (depth > 1 && !w_hid)) return fail(TH_ERR_BAD_ARG, "null weight pointer");
    if (has_bias && (!b_in || !b_out || (depth > 1 && !b_hid))) return fail(TH_ERR_BAD_ARG, "biases must be all present or all null");
    if (n_points > 0)
        if (int rc = make_coord_view(a.cv, coords, stride_n, stride_d, coord_dtype, n_dims)) return rc;
    return TH_OK;
}

// The shapes the fused kernels are built for; everything else is TH_ERR_UNSUPPORTED and the caller runs the
// separate operators.
const char *field_unsupported(const FieldArgs &a, int dtype, bool backward) {
    if (dtype != TH_F16 && dtype != TH_BF16) return "float16 or bfloat16 tables and weights only";
    if (a.n_dims != 2 && a.n_dims != 3) return "2 or 3 coordinate dimensions only";
    if (a.n_feats != 2 && a.n_feats != 4) return "2 or 4 features per level only";
    if ((a.n_levels * a.n_feats) % 16 != 0) return "levels * features must be a multiple of 16";
    if (a.s.act != TH_ACT_RELU && a.s.act != TH_ACT_NONE) return "ReLU or no activation only";
    if (backward && a.s.has_bias) return "bias-free networks only (backward)";
    if (tc_disabled()) return "tensor-core kernels disabled by TH_MLP_LEGACY";
    return nullptr;
}

}  // namespace

int field_tc_status_word() {
    int status = 0;
    if (cudaMemcpyFromSymbol(&status, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    int hash = 0;
    if (cudaMemcpyFromSymbol(&hash, g_hash_status, sizeof(int)) != cudaSuccess) return -1;
    return status | (hash << 1);
}

}  // namespace th

using namespace th;

#define TH_FIELD_DISPATCH(CALL)                                                                  \
    if (dtype == TH_F16) {                                                                       \
        if (a.n_dims == 3 && a.n_feats == 2) { CALL(__half, 3, 2) }                              \
        if (a.n_dims == 3 && a.n_feats == 4) { CALL(__half, 3, 4) }                              \
        if (a.n_dims == 2 && a.n_feats == 2) { CALL(__half, 2, 2) }                              \
        if (a.n_dims == 2 && a.n_feats == 4) { CALL(__half, 2, 4) }                              \
    } else {                                                                                     \
        if (a.n_dims == 3 && a.n_feats == 2) { CALL(__nv_bfloat16, 3, 2) }                       \
        if (a.n_dims == 3 && a.n_feats == 4) { CALL(__nv_bfloat16, 3, 4) }                       \
        if (a.n_dims == 2 && a.n_feats == 2) { CALL(__nv_bfloat16, 2, 2) }                       \
        if (a.n_dims == 2 && a.n_feats == 4) { CALL(__nv_bfloat16, 2, 4) }                       \
    }

extern "C" int th_field_fwd(const void *coords_dev, int64_t coord_stride_n, int64_t coord_stride_d, int coord_dtype,
                            const void *table_dev, int n_dims, int n_feats, int n_levels, const int32_t *level_res_host,
                            const int64_t *level_rows_host, const int64_t *level_offset_host, const int64_t *primes_host,
                            float scale, const void *w_in_dev, const void *b_in_dev, const void *w_hid_dev,
                            const void *b_hid_dev, const void *w_out_dev, const void *b_out_dev, int d_hidden, int d_out,
                            int depth, int activation, void *feats_out_dev, int64_t feats_stride, void *out_dev,
                            int64_t out_stride, const void *target_dev, int64_t target_stride, void *grad_dev,
                            int64_t grad_stride, float *loss_sum_dev, float grad_scale, int64_t n_points, int dtype,
                            void *stream) {
    FieldArgs a;
    if (int rc = fill_field_args(a, coords_dev, coord_stride_n, coord_stride_d, coord_dtype, n_dims, n_feats, n_levels, level_res_host,
                                 level_rows_host, level_offset_host, primes_host, scale, w_in_dev, b_in_dev, w_hid_dev, b_hid_dev,
                                 w_out_dev, b_out_dev, d_hidden, d_out, depth, activation, n_points)) return rc;
    if (n_points == 0) return TH_OK;
    if (!table_dev) return fail(TH_ERR_BAD_ARG, "null table");
    if (!target_dev && !out_dev) return fail(TH_ERR_BAD_ARG, "neither an output nor a target was given");
    if (target_dev && !grad_dev) return fail(TH_ERR_BAD_ARG, "a target needs a gradient output");
    if (const char *why = field_unsupported(a, dtype, false)) return fail(TH_ERR_UNSUPPORTED, "fused encoding + MLP forward: %s", why);
    const int d_in = a.s.d_in;
    if (feats_out_dev && (feats_stride < d_in || !rows_vector_ok(feats_out_dev, feats_stride, d_in)))
        return fail(TH_ERR_ALIGNMENT, "feature rows must be 16-byte aligned and at least levels * features apart");
    if (out_dev && out_stride < d_out) return fail(TH_ERR_BAD_ARG, "out_stride smaller than d_out");
    if (target_dev && (d_out % 8 != 0 || !rows_vector_ok(target_dev, target_stride, d_out) || !rows_vector_ok(grad_dev, grad_stride, d_out) ||
                       (out_dev && !rows_vector_ok(out_dev, out_stride, d_out))))
        return fail(TH_ERR_UNSUPPORTED, "fused loss needs d_out a multiple of 8 and 16-byte aligned prediction / target / gradient rows");
    if (!aligned_to(table_dev, 4)) return fail(TH_ERR_ALIGNMENT, "table rows must be aligned to their size");
    const MseArgs mse{target_dev, target_stride, grad_dev, grad_stride, loss_sum_dev, grad_scale};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = kTcNotApplicable;
#define TH_FWD_CALL(T, D, F)                                                                                                             \
    if (a.s.act == TH_ACT_RELU)                                                                                                          \
        rc = a.s.has_bias ? launch_field_fwd<T, D, F, TH_ACT_RELU, true>(a, table_dev, feats_out_dev, feats_stride, out_dev, out_stride, mse, n_points, st)   \
                          : launch_field_fwd<T, D, F, TH_ACT_RELU, false>(a, table_dev, feats_out_dev, feats_stride, out_dev, out_stride, mse, n_points, st); \
    else                                                                                                                                 \
        rc = a.s.has_bias ? launch_field_fwd<T, D, F, TH_ACT_NONE, true>(a, table_dev, feats_out_dev, feats_stride, out_dev, out_stride, mse, n_points, st)   \
                          : launch_field_fwd<T, D, F, TH_ACT_NONE, false>(a, table_dev, feats_out_dev, feats_stride, out_dev, out_stride, mse, n_points, st);
    TH_FIELD_DISPATCH(TH_FWD_CALL)
#undef TH_FWD_CALL
    if (rc == kTcNotApplicable) return fail(TH_ERR_UNSUPPORTED, "fused encoding + MLP forward: the network does not fit one CTA's shared memory");
    return rc;
}

extern "C" int64_t th_field_workspace_bytes(int n_levels, int n_feats, int d_hidden, int d_out, int depth) {
    return th_mlp_workspace_bytes(n_levels * n_feats, d_hidden, d_out, depth);
}

extern "C" int th_field_bwd(const void *coords_dev, int64_t coord_stride_n, int64_t coord_stride_d, int coord_dtype,
                            int n_dims, int n_feats, int n_levels, const int32_t *level_res_host,
                            const int64_t *level_rows_host, const int64_t *level_offset_host, const int64_t *primes_host,
                            float scale, const void *w_in_dev, const void *w_hid_dev, const void *w_out_dev, int d_hidden,
                            int d_out, int depth, int activation, const void *feats_dev, int64_t feats_stride,
                            const void *grad_out_dev, int64_t go_stride, void *grad_table_dev, void *grad_feats_dev,
                            int64_t gf_stride, void *workspace_dev, int64_t workspace_bytes, int64_t n_points, int dtype,
                            void *stream) {
    FieldArgs a;
    if (int rc = fill_field_args(a, coords_dev, coord_stride_n, coord_stride_d, coord_dtype, n_dims, n_feats, n_levels, level_res_host,
                                 level_rows_host, level_offset_host, primes_host, scale, w_in_dev, nullptr, w_hid_dev, nullptr,
                                 w_out_dev, nullptr, d_hidden, d_out, depth, activation, n_points)) return rc;
    const int64_t need = static_cast<int64_t>(sizeof(float)) * grad_workspace_layout(a.s, nullptr).total;
    if (!workspace_dev || workspace_bytes < need)
        return fail(TH_ERR_WORKSPACE, "workspace of %lld bytes needed, %lld given", (long long)need, (long long)workspace_bytes);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int rc = cuda_status(cudaMemsetAsync(workspace_dev, 0, need, st), "cudaMemsetAsync(workspace)")) return rc;
    if (n_points == 0) return TH_OK;
    if (!feats_dev || !grad_out_dev || !grad_table_dev) return fail(TH_ERR_BAD_ARG, "null features, gradient or table gradient");
    if (feats_stride < a.s.d_in || go_stride < d_out || (grad_feats_dev && gf_stride < a.s.d_in)) return fail(TH_ERR_BAD_ARG, "row stride smaller than the row");
    if (const char *why = field_unsupported(a, dtype, true)) return fail(TH_ERR_UNSUPPORTED, "fused MLP + encoding backward: %s", why);
    if (!aligned_to(grad_table_dev, 16)) return fail(TH_ERR_ALIGNMENT, "the table gradient must be 16-byte aligned");
    float *ws = static_cast<float *>(workspace_dev);
    int rc = kTcNotApplicable;
#define TH_BWD_CALL(T, D, F)                                                                                                            \
    rc = a.s.act == TH_ACT_RELU                                                                                                         \
             ? launch_field_bwd<T, D, F, TH_ACT_RELU>(a, feats_dev, feats_stride, grad_out_dev, go_stride, grad_table_dev, grad_feats_dev, gf_stride, ws, n_points, st) \
             : launch_field_bwd<T, D, F, TH_ACT_NONE>(a, feats_dev, feats_stride, grad_out_dev, go_stride, grad_table_dev, grad_feats_dev, gf_stride, ws, n_points, st);
    TH_FIELD_DISPATCH(TH_BWD_CALL)
#undef TH_BWD_CALL
    if (rc == kTcNotApplicable) return fail(TH_ERR_UNSUPPORTED, "fused MLP + encoding backward: the network does not fit one SM's shared or tensor memory");
    return rc;
}
