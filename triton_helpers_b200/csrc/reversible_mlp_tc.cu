// Reversible (additive coupling) fused MLP on the 5th-generation tensor cores.
//
// The residual stream of a 128-row tile lives in TENSOR MEMORY as fp32 for the whole stack:
// x1 in one 64-column accumulator, x2 in another.  A branch y = x + W2 . act(W1 . u) is two GEMMs,
// and the second one simply accumulates into the stream's own columns (enable-input-d), so the
// residual add costs nothing; the backward pass undoes a branch with the same GEMM and the
// A operand negated (x = y - W2 . act(W1 . u)), and the gradient stream (also fp32 in TMEM)
// receives its dgrad the same way.  Only what the tensor core must read as an operand is rounded
// to 16 bits and written to a shared-memory operand tile by the epilogue threads.
//
//   forward, per branch:   HID = U . W1^T                       U = 16-bit copy of the input stream
//                          OUT += act(HID) . W2^T               OUT = the other stream, in TMEM
//   backward, per branch:  HID = U . W1^T ,  DH = DY . W2       (one commit: recompute + dgrad)
//                          OUT += (-act(HID)) . W2^T            reconstruct the branch's input side
//                          IN_D += DZ . W1                      gradient into the input stream
//                          DW2 = DY^T . act(HID) , DW1 = DZ^T . U     (M = 64, K = the 128 rows)
//
// Weights (4 matrices per block) stream block by block through a two-stage cp.async ring in the
// operand-tile layout; the same tile is read K-major by the forward GEMMs and MN-major by dgrad.
// Weight gradients of a (tile, block, branch) leave TMEM straight into the CTA's private fp32
// accumulator in global memory (vector red.global.add, one owner per copy, L2 resident), carried
// out by four extra warps while the other eight are already in the next branch; a reduction
// kernel sums the copies.  The backward pass needs all 512 TMEM columns, so one CTA per SM; the
// forward pass needs 192 (256 allocated), two CTAs per SM.
//
// Covered here: float16 / bfloat16, 16-byte-aligned rows; backward: ReLU or no activation, no
// biases.  Everything else stays on the mma.sync kernels.
#include "rev_shape.cuh"
#include "tc_tiles.cuh"

#include <cstdlib>
#include <cstring>
#include <type_traits>

namespace th {
namespace {

constexpr int kWTileBytes = 64 * 128;            // one weight matrix as an operand tile
constexpr int kStageBytes = 4 * kWTileBytes;     // [f1 | f2 | g1 | g2]
// TMEM columns
constexpr int kS1 = 0, kS2 = 64;                 // the stream
constexpr int kFwdHid = 128;                     // forward: hidden pre-activation
constexpr int kFwdAU = 192, kFwdAH = 224;        // forward: 16-bit A operands (the branch's input, its hidden activation), 32 columns each
constexpr int kD1 = 128, kD2 = 192, kZ = 256, kDH = 320, kDW1 = 384, kDW2 = 448;  // backward

struct RevTcPlan {
    int tiles;     // operand tiles before the weight ring (2 forward, 6 backward)
    int ring;      // byte offset of the ring (2 stages)
    int bias;      // fp32 [2 stages][4][64]
    int total;
    int tmem_cols;
};

__host__ __device__ inline RevTcPlan rev_tc_plan(bool backward) {
    RevTcPlan p{};
    p.tiles = backward ? 6 : 2;
    p.ring = p.tiles * kTileBytes;
    p.bias = p.ring + 2 * kStageBytes;
    p.total = p.bias + 2 * 4 * kMaxDim * 4;
    p.tmem_cols = backward ? 512 : 256;
    return p;
}

// Queue block k's four weight matrices into ring stage `stage` (cp.async, operand-tile layout).
template <typename T>
__device__ void prefetch_weights(unsigned char *smem, const RevTcPlan &P, const RevShape &s, const RevParams &p, int k,
                                 int stage) {
    const T *src[4] = {static_cast<const T *>(p.w_f1), static_cast<const T *>(p.w_f2), static_cast<const T *>(p.w_g1),
                       static_cast<const T *>(p.w_g2)};
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const int rows = (m & 1) ? s.half : s.hid, cols = (m & 1) ? s.hid : s.half;
        unsigned char *tile = smem + P.ring + stage * kStageBytes + m * kWTileBytes;
        const T *g = src[m] + static_cast<size_t>(k) * rows * cols;
        const int chunks = cols / 8;
        for (int id = threadIdx.x; id < rows * chunks; id += kTcThreads) {
            const int r = id / chunks, c = id - r * chunks;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(chunk_ptr(tile, r, c))),
                         "l"(g + r * cols + 8 * c)
                         : "memory");
        }
    }
    if (s.has_bias) {
        float *bias = reinterpret_cast<float *>(smem + P.bias) + stage * 4 * kMaxDim;
        const T *bsrc[4] = {static_cast<const T *>(p.b_f1), static_cast<const T *>(p.b_f2), static_cast<const T *>(p.b_g1),
                            static_cast<const T *>(p.b_g2)};
        for (int e = threadIdx.x; e < 4 * kMaxDim; e += kTcThreads) {
            const int m = e / kMaxDim, c = e % kMaxDim;
            const int width = (m & 1) ? s.half : s.hid;
            bias[e] = c < width ? to_float<T>(bsrc[m][k * width + c]) : 0.f;
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// The same by TMA: one 64-column box per matrix lands in the operand-tile layout, issued by one thread
// and counted on the ring stage's mbarrier (the cp.async version above keeps every thread busy for
// ~1 800 cycles per block).  Biases, when present, still come with plain loads.
struct RevWeightMaps {
    CUtensorMap m[4];  // w_f1, w_f2, w_g1, w_g2: [blocks * rows][cols], 16-bit
};

template <typename T>
__device__ void prefetch_weights_tma(unsigned char *smem, const RevTcPlan &P, const RevShape &s, const RevParams &p,
                                     const RevWeightMaps &maps, unsigned long long *ring_bars, int k, int stage) {
    if (threadIdx.x == 64) {  // not warp 0, which is about to issue MMAs
        const uint32_t bar = smem_addr(&ring_bars[stage]);
        const uint32_t bytes = static_cast<uint32_t>(2 * (s.hid + s.half) * 128);  // four boxes of 64 columns
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int rows = (m & 1) ? s.half : s.hid;
            tma_load_2d(smem + P.ring + stage * kStageBytes + m * kWTileBytes, &maps.m[m], 0, k * rows, bar);
        }
    }
    if (s.has_bias) {
        float *bias = reinterpret_cast<float *>(smem + P.bias) + stage * 4 * kMaxDim;
        const T *bsrc[4] = {static_cast<const T *>(p.b_f1), static_cast<const T *>(p.b_f2), static_cast<const T *>(p.b_g1),
                            static_cast<const T *>(p.b_g2)};
        for (int e = threadIdx.x; e < 4 * kMaxDim; e += kTcThreads) {
            const int m = e / kMaxDim, c = e % kMaxDim;
            const int width = (m & 1) ? s.half : s.hid;
            bias[e] = c < width ? to_float<T>(bsrc[m][k * width + c]) : 0.f;
        }
    }
}

// Warp 0 waits (bounded) for the ring stage used by running step `step`; the CTA barrier that follows
// in the caller hands the result to everybody.
__device__ __forceinline__ void ring_wait(unsigned long long *ring_bars, int step, int *abort_flag) {
    if (threadIdx.x < 32 && !mbar_wait(smem_addr(&ring_bars[step & 1]), static_cast<uint32_t>((step >> 1) & 1))) *abort_flag = 1;
}

// This thread's pieces of a 16-bit operand tile row -> fp32 in TMEM (stream initialisation)
template <typename T>
__device__ __forceinline__ void tile_row_to_tmem(unsigned char *tile, const Seat &seat, int width, uint32_t taddr) {
    const int count = width / (8 * kGroups), first = seat.group * count;
#pragma unroll
    for (int u = 0; u < kMaxChunks; ++u) {
        if (u < count) {
            uint32_t wide[8];
            widen_chunk<T>(*reinterpret_cast<const uint4 *>(chunk_ptr(tile, seat.row, first + u)), wide);
            tmem_st8(taddr + 8 * (first + u), wide);
        }
    }
}

// This thread's pieces of an fp32 TMEM accumulator -> (optional bias, written back) -> rounded into an
// operand tile and / or a global row.
template <typename T, bool BIAS>
__device__ __forceinline__ void stream_epilogue(uint32_t taddr, const Seat &seat, int width, const float *bias,
                                                unsigned char *tile, T *global_row, bool live) {
    const int n = width / kGroups, first = seat.group * (n / 8);  // this thread's columns / first 8-column piece
    const uint32_t row_addr = (tile ? smem_addr(tile) : 0u) + seat.row * 128, row_swizzle = (seat.row & 7) << 4;
    for_each_piece(taddr + seat.group * n, n, [&](int u, const uint32_t(&piece)[8]) {
        uint32_t v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = piece[k];
        if constexpr (BIAS) {
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = __float_as_uint(__uint_as_float(v[k]) + bias[8 * (first + u) + k]);
            tmem_st8(taddr + 8 * (first + u), v);
        }
        const uint4 packed = finish8<T, TH_ACT_NONE, false>(v, nullptr);
        if (tile) st_shared_16(row_addr + (((first + u) << 4) ^ row_swizzle), packed);
        if (global_row && live) __stcs(reinterpret_cast<uint4 *>(global_row + 8 * (first + u)), packed);
    });
    if constexpr (BIAS) tmem_st_wait();
}

// The same with the rounded copy going to a 16-bit A operand in tensor memory (4 columns per 16-byte chunk).
template <typename T, bool BIAS>
__device__ __forceinline__ void stream_epilogue_ta(uint32_t taddr, const Seat &seat, int width, const float *bias, uint32_t a_taddr,
                                                   T *global_row, bool live) {
    const int n = width / kGroups, first = seat.group * (n / 8);
    for_each_piece(taddr + seat.group * n, n, [&](int u, const uint32_t(&piece)[8]) {
        uint32_t v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = piece[k];
        if constexpr (BIAS) {
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = __float_as_uint(__uint_as_float(v[k]) + bias[8 * (first + u) + k]);
            tmem_st8(taddr + 8 * (first + u), v);
        }
        const uint4 packed = finish8<T, TH_ACT_NONE, false>(v, nullptr);
        tmem_st4(a_taddr + 4 * (first + u), packed);
        if (global_row && live) __stcs(reinterpret_cast<uint4 *>(global_row + 8 * (first + u)), packed);
    });
    tmem_st_wait();
}

__device__ __forceinline__ bool commit_and_wait(bool leader, uint32_t bar, uint32_t &phase, int *abort_flag) {
    if (threadIdx.x < 32) {
        if (leader) mma_commit(bar);
        __syncwarp();
    }
    return cta_wait_mma(bar, phase, abort_flag);
}

__device__ __forceinline__ void publish_tiles() {
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
}

// ---- forward -----------------------------------------------------------------------------------

// TA: the two A operands of a branch (the 16-bit copy of its input stream, its hidden activation) live in tensor
// memory and never touch shared memory; the operand tiles only stage the rows as they arrive.
template <typename T, int ACT, bool BIAS, bool TA>
__global__ void __launch_bounds__(kTcThreads, 2)
rev_fwd_tc_kernel(const RevShape s, const RevParams p, const __grid_constant__ RevWeightMaps maps, const int use_tma,
                  const T *__restrict__ x, long long x_stride, T *__restrict__ y, long long y_stride, long long n_rows) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint32_t tmem_holder;
    __shared__ __align__(8) unsigned long long mbar;
    __shared__ int abort_flag;
    const RevTcPlan P = rev_tc_plan(false);
    constexpr int bf16 = std::is_same<T, __half>::value ? 0 : 1;
    unsigned char *u_tile = smem, *h_tile = smem + kTileBytes;

    __shared__ __align__(8) unsigned long long ring_bars[2];
    if (threadIdx.x == 0) {
        abort_flag = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&ring_bars[0])), "r"(1u) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&ring_bars[1])), "r"(1u) : "memory");
    }
    const long long n_tiles = (n_rows + kTileRows - 1) / kTileRows;
    if (!use_tma && static_cast<long long>(blockIdx.x) < n_tiles) prefetch_weights<T>(smem, P, s, p, 0, 0);
    const uint32_t tmem = cta_setup(&tmem_holder, &mbar, P.tmem_cols);  // publishes the barrier inits
    if (use_tma && static_cast<long long>(blockIdx.x) < n_tiles) {
        prefetch_weights_tma<T>(smem, P, s, p, maps, ring_bars, 0, 0);
        ring_wait(ring_bars, 0, &abort_flag);
    }
    const uint32_t bar = smem_addr(&mbar);
    const Seat seat;
    const uint32_t taddr = tmem + seat.lane_base;
    uint32_t phase = 0;
    int step = 0;  // running (tile, block) counter: ring stage = step & 1
    const uint32_t idesc_hid = instr_desc(128, s.hid, bf16, 0, 0), idesc_half = instr_desc(128, s.half, bf16, 0, 0);

    for (long long tile = blockIdx.x; tile < n_tiles && !abort_flag; tile += gridDim.x) {
        const long long row0 = tile * kTileRows;
        const bool live = row0 + seat.row < n_rows;
        T *y_row = y + (live ? row0 + seat.row : 0) * y_stride;
        // x1 -> scratch tile, x2 -> the first branch's operand tile; then both into the fp32 stream in TMEM
        async_tile_load<T>(h_tile, x, x_stride, row0, n_rows, s.half, s.half);
        async_tile_load<T>(u_tile, x + s.half, x_stride, row0, n_rows, s.half, s.half);
        async_tile_wait();  // also the weights queued for this step
        __syncthreads();
        tile_row_to_tmem<T>(h_tile, seat, s.half, taddr + kS1);
        tile_row_to_tmem<T>(u_tile, seat, s.half, taddr + kS2);
        if constexpr (TA) {  // x2 as the first branch's A operand
            const int count = s.half / (8 * kGroups), first = seat.group * count;
            for (int u = 0; u < count; ++u)
                tmem_st4(taddr + kFwdAU + 4 * (first + u), *reinterpret_cast<const uint4 *>(chunk_ptr(u_tile, seat.row, first + u)));
        }
        tmem_st_wait();
        publish_tiles();

        for (int k = 0; k < s.blocks && !abort_flag; ++k, ++step) {
            const int stage = step & 1;
            // the other stage was last read by the previous block, whose GEMMs have all completed
            const bool more = k + 1 < s.blocks || tile + gridDim.x < n_tiles;
            if (more) {
                if (use_tma) prefetch_weights_tma<T>(smem, P, s, p, maps, ring_bars, (k + 1) % s.blocks, stage ^ 1);
                else prefetch_weights<T>(smem, P, s, p, (k + 1) % s.blocks, stage ^ 1);
            }
            const unsigned char *w = smem + P.ring + stage * kStageBytes;
            const float *bias = reinterpret_cast<const float *>(smem + P.bias) + stage * 4 * kMaxDim;
#pragma unroll 1
            for (int branch = 0; branch < 2; ++branch) {
                // branch 0: x1 += F(x2) (U holds x2), branch 1: x2 += G(x1) (U holds x1)
                const uint32_t w1 = smem_addr(w + (2 * branch) * kWTileBytes), w2 = smem_addr(w + (2 * branch + 1) * kWTileBytes);
                const uint32_t out_col = branch == 0 ? kS1 : kS2;
                bool leader = false;
                if (threadIdx.x < 32) {
                    leader = elect_one();
                    tc_fence_after();
                    if constexpr (TA) issue_gemm_ta(leader, tmem + kFwdHid, tmem + kFwdAU, w1, 32, s.half / 16, idesc_hid, false);
                    else issue_gemm(leader, tmem + kFwdHid, smem_addr(u_tile), 32, w1, 32, s.half / 16, idesc_hid, false);
                }
                commit_and_wait(leader, bar, phase, &abort_flag);
                {
                    const int n = s.hid / kGroups, first = seat.group * (n / 8);
                    const uint32_t row_addr = smem_addr(h_tile) + seat.row * 128, row_swizzle = (seat.row & 7) << 4;
                    const float *layer_bias = bias + (2 * branch) * kMaxDim;
                    for_each_piece(taddr + kFwdHid + seat.group * n, n, [&](int u, const uint32_t(&piece)[8]) {
                        const uint4 packed = finish8<T, ACT, BIAS>(piece, layer_bias + 8 * (first + u));
                        if constexpr (TA) tmem_st4(taddr + kFwdAH + 4 * (first + u), packed);
                        else st_shared_16(row_addr + (((first + u) << 4) ^ row_swizzle), packed);
                    });
                    if constexpr (TA) tmem_st_wait();
                }
                publish_tiles();
                if (threadIdx.x < 32) {
                    leader = elect_one();
                    tc_fence_after();
                    if constexpr (TA) issue_gemm_ta(leader, tmem + out_col, tmem + kFwdAH, w2, 32, s.hid / 16, idesc_half, true);
                    else issue_gemm(leader, tmem + out_col, smem_addr(h_tile), 32, w2, 32, s.hid / 16, idesc_half, true);
                }
                commit_and_wait(leader, bar, phase, &abort_flag);
                // the updated stream: rounded copy for the next branch, and the output after the last block
                const bool last = k == s.blocks - 1;
                if constexpr (TA)
                    stream_epilogue_ta<T, BIAS>(taddr + out_col, seat, s.half, bias + (2 * branch + 1) * kMaxDim, taddr + kFwdAU,
                                                last ? y_row + branch * s.half : nullptr, live);
                else
                    stream_epilogue<T, BIAS>(taddr + out_col, seat, s.half, bias + (2 * branch + 1) * kMaxDim, u_tile,
                                             last ? y_row + branch * s.half : nullptr, live);
                if (branch == 1) {  // next block's weights have landed
                    if (!use_tma) async_tile_wait();
                    else if (more) ring_wait(ring_bars, step + 1, &abort_flag);
                }
                publish_tiles();
            }
        }
    }
    if (abort_flag) g_tc_status = 1;
    cta_teardown(tmem, P.tmem_cols);
}

// ---- backward ----------------------------------------------------------------------------------

// One weight-gradient accumulator (M = 64 layout) out of TMEM, added into this CTA's private copy.
// The copy of a matrix is stored [column / 4][row][column % 4]: the 16 lanes of a warp that hold rows
// m .. m + 15 of one column quad then add to 256 contiguous bytes (8 full sectors per instruction
// instead of 16 half-used ones), which is what the L2's reduction rate is counted in.
__host__ __device__ inline int dw_private_index(int row, int col) { return ((col >> 2) * 64 + row) * 4 + (col & 3); }

// The backward kernel runs 256 "main" threads (the chain: issue, wait, epilogue) and 128 "flush" threads
// that carry the weight gradients of a pass out of TMEM while the main threads are already in the next pass.
constexpr int kRevFlushThreads = 128;

// CTA barrier of the main threads only
__device__ __forceinline__ void main_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__device__ __forceinline__ void main_publish() {
    fence_async_smem();
    tc_fence_before();
    main_sync();
}

// Bounded wait that also gives up when somebody else has: false = do not go on.
__device__ __forceinline__ bool rev_wait(uint32_t bar, uint32_t parity, int *abort_flag) {
    for (int poll = 0; poll < kWaitPolls; ++poll) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
        if ((poll & 63) == 63 && *reinterpret_cast<volatile int *>(abort_flag)) return false;
    }
    *reinterpret_cast<volatile int *>(abort_flag) = 1;
    return false;
}

// cta_wait_mma for the main threads: warp 0 polls, the others park at the main barrier
__device__ __forceinline__ bool main_wait_mma(uint32_t mbar, uint32_t &phase, int *abort_flag) {
    if (threadIdx.x < 32) {
        rev_wait(mbar, phase, abort_flag);
        tc_fence_after();
        tc_fence_before();
    }
    phase ^= 1;
    main_sync();
    tc_fence_after();
    return *reinterpret_cast<volatile int *>(abort_flag) == 0;
}

// One flush warp's share (TMEM lanes 32 q .. 32 q + 15 = gradient rows 16 q .. 16 q + 15) of one accumulator
__device__ __forceinline__ void flush_dw_quadrant(uint32_t tmem, int q, uint32_t col, int out_dim, int in_dim, float *dst) {
    const int lane = threadIdx.x & 31;
    const int m = 16 * q + lane;
    const bool owner = lane < 16 && m < out_dim;
    const uint32_t taddr = tmem + (static_cast<uint32_t>(32 * q) << 16) + col;
    // The private copies (0.5 MB per CTA) are revisited once per row tile while a gigabyte of rows streams through
    // L2: ask the L2 to keep their lines (evict-last), or most of the reductions end up in DRAM.
    unsigned long long keep;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(keep));
    for (int first = 0; first < in_dim; first += 16) {
        uint32_t raw[32];
        tmem_ld16(taddr + first, raw);
        tmem_ld_wait();
        if (owner) {
#pragma unroll
            for (int h = 0; h < 4; ++h)
                asm volatile("red.global.add.L2::cache_hint.v4.f32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(dst + dw_private_index(m, first + 4 * h)),
                             "f"(__uint_as_float(raw[4 * h])), "f"(__uint_as_float(raw[4 * h + 1])),
                             "f"(__uint_as_float(raw[4 * h + 2])), "f"(__uint_as_float(raw[4 * h + 3])), "l"(keep)
                             : "memory");
        }
    }
}

template <typename T, int ACT>
__global__ void __launch_bounds__(kTcThreads + kRevFlushThreads, 1)
rev_bwd_tc_kernel(const RevShape s, const RevParams p, const __grid_constant__ RevWeightMaps maps, const int use_tma,
                  const T *__restrict__ y, long long y_stride,
                  const T *__restrict__ go, long long go_stride, T *__restrict__ gx, long long gx_stride,
                  T *__restrict__ x_rec, long long xr_stride, float *__restrict__ workspace, long long n_rows) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint32_t tmem_holder;
    __shared__ __align__(8) unsigned long long mbar;
    __shared__ int abort_flag;
    const RevTcPlan P = rev_tc_plan(true);
    constexpr int bf16 = std::is_same<T, __half>::value ? 0 : 1;
    // U (the branch's input, 16-bit) and DY (the gradient of its output) alternate between two tiles each: the
    // epilogue of a pass writes the next pass's copies while this pass's weight-gradient MMAs still read theirs
    unsigned char *u_tiles = smem, *h_tile = smem + 2 * kTileBytes, *dy_tiles = smem + 3 * kTileBytes, *dz_tile = smem + 5 * kTileBytes;
    const bool is_flush = threadIdx.x >= kTcThreads;

    __shared__ __align__(8) unsigned long long ring_bars[2];
    // wgrad_bar: the weight-gradient MMAs of a pass are done (one commit per pass); flushed_bar: the flush warps
    // have read them out (one arrival per flush warp), so the next pass may overwrite the accumulators
    __shared__ __align__(8) unsigned long long wgrad_bar, flushed_bar;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&ring_bars[0])), "r"(1u) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&ring_bars[1])), "r"(1u) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&wgrad_bar)), "r"(1u) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&flushed_bar)), "r"(static_cast<uint32_t>(kRevFlushThreads / 32)) : "memory");
    }
    for (int e = threadIdx.x; e < P.tiles * kTileBytes / 16; e += blockDim.x) reinterpret_cast<uint4 *>(smem)[e] = make_uint4(0, 0, 0, 0);
    const long long n_tiles = (n_rows + kTileRows - 1) / kTileRows;
    if (!is_flush && !use_tma && static_cast<long long>(blockIdx.x) < n_tiles) prefetch_weights<T>(smem, P, s, p, s.blocks - 1, 0);
    const uint32_t tmem = cta_setup(&tmem_holder, &mbar, P.tmem_cols);  // publishes the barrier inits
    float *cta_acc = workspace + static_cast<size_t>(blockIdx.x) * rev_cta_floats(s);
    const uint32_t wgrad_addr = smem_addr(&wgrad_bar), flushed_addr = smem_addr(&flushed_bar);

    if (is_flush) {
        // ================= weight gradients out of TMEM, one pass behind the main threads =================
        const int q = (threadIdx.x >> 5) & 3;
        uint32_t n = 0;  // passes flushed so far
        bool alive = true;
        for (long long tile = blockIdx.x; alive && tile < n_tiles; tile += gridDim.x) {
            for (int k = s.blocks - 1; alive && k >= 0; --k) {
                float *block_acc = cta_acc + static_cast<size_t>(k) * 4 * kMatFloats;
                for (int pass = 0; pass < 2; ++pass, ++n) {
                    alive = __all_sync(0xffffffffu, rev_wait(wgrad_addr, n & 1u, &abort_flag));
                    if (!alive) break;
                    tc_fence_after();
                    const int m1 = pass == 0 ? 2 : 0;
                    flush_dw_quadrant(tmem, q, kDW1, s.hid, s.half, block_acc + m1 * kMatFloats);
                    flush_dw_quadrant(tmem, q, kDW2, s.half, s.hid, block_acc + (m1 + 1) * kMatFloats);
                    tc_fence_before();
                    __syncwarp();
                    if ((threadIdx.x & 31) == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(flushed_addr) : "memory");
                }
            }
        }
    } else {
        // ================= the chain =================
        if (use_tma && static_cast<long long>(blockIdx.x) < n_tiles) {
            prefetch_weights_tma<T>(smem, P, s, p, maps, ring_bars, s.blocks - 1, 0);
            ring_wait(ring_bars, 0, &abort_flag);
        }
        const uint32_t bar = smem_addr(&mbar);
        const Seat seat;
        const uint32_t taddr = tmem + seat.lane_base;
        uint32_t phase = 0;
        int step = 0;
        uint32_t n = 0;  // passes started so far; pass n reads U / DY copy n & 1 and writes copy (n + 1) & 1
        // instruction descriptors: forward-type, dgrad (B MN-major), reconstruction (A negated), wgrad (both MN-major, M = 64)
        const uint32_t id_z = instr_desc(128, s.hid, bf16, 0, 0);
        const uint32_t id_dh = instr_desc(128, s.hid, bf16, 0, 1);
        const uint32_t id_undo = instr_desc(128, s.half, bf16, 0, 0) | (1u << 13);
        const uint32_t id_din = instr_desc(128, s.half, bf16, 0, 1);
        const uint32_t id_dw2 = instr_desc(64, s.hid, bf16, 1, 1), id_dw1 = instr_desc(64, s.half, bf16, 1, 1);
        volatile int *abort_now = &abort_flag;

        for (long long tile = blockIdx.x; tile < n_tiles && !*abort_now; tile += gridDim.x) {
            const long long row0 = tile * kTileRows;
            const bool live = row0 + seat.row < n_rows;
            unsigned char *u_in = u_tiles + (n & 1u) * kTileBytes, *dy_in = dy_tiles + (n & 1u) * kTileBytes;
            // the scratch tiles below were operands of the previous tile's last weight-gradient MMAs
            if (n > 0) {
                if (threadIdx.x < 32) rev_wait(wgrad_addr, (n - 1) & 1u, &abort_flag);
                main_sync();
            }
            // y1 -> U (input of the last G), y2 -> scratch, go1 -> scratch, go2 -> DY (gradient of G's output)
            async_tile_load<T>(u_in, y, y_stride, row0, n_rows, s.half, s.half);
            async_tile_load<T>(h_tile, y + s.half, y_stride, row0, n_rows, s.half, s.half);
            async_tile_load<T>(dz_tile, go, go_stride, row0, n_rows, s.half, s.half);
            async_tile_load<T>(dy_in, go + s.half, go_stride, row0, n_rows, s.half, s.half);
            async_tile_wait();
            main_sync();
            tile_row_to_tmem<T>(u_in, seat, s.half, taddr + kS1);
            tile_row_to_tmem<T>(h_tile, seat, s.half, taddr + kS2);
            tile_row_to_tmem<T>(dz_tile, seat, s.half, taddr + kD1);
            tile_row_to_tmem<T>(dy_in, seat, s.half, taddr + kD2);
            tmem_st_wait();
            main_publish();

            for (int k = s.blocks - 1; k >= 0 && !*abort_now; --k, ++step) {
                const int stage = step & 1;
                const bool more = k > 0 || tile + gridDim.x < n_tiles;
                if (more) {
                    if (use_tma) prefetch_weights_tma<T>(smem, P, s, p, maps, ring_bars, k > 0 ? k - 1 : s.blocks - 1, stage ^ 1);
                    else prefetch_weights<T>(smem, P, s, p, k > 0 ? k - 1 : s.blocks - 1, stage ^ 1);
                }
                const unsigned char *w = smem + P.ring + stage * kStageBytes;
#pragma unroll 1
                for (int pass = 0; pass < 2; ++pass, ++n) {
                    // pass 0 undoes y2 = x2 + G(y1): input stream S1, output stream S2, gradient flows D2 -> D1
                    // pass 1 undoes y1 = x1 + F(x2): input stream S2, output stream S1, gradient flows D1 -> D2
                    const int m1 = pass == 0 ? 2 : 0, m2 = m1 + 1;
                    const uint32_t w1 = smem_addr(w + m1 * kWTileBytes), w2 = smem_addr(w + m2 * kWTileBytes);
                    const uint32_t out_col = pass == 0 ? kS2 : kS1, in_d_col = pass == 0 ? kD1 : kD2;
                    const uint32_t u_cur = smem_addr(u_tiles + (n & 1u) * kTileBytes), dy_cur = smem_addr(dy_tiles + (n & 1u) * kTileBytes);
                    unsigned char *u_next = u_tiles + ((n + 1) & 1u) * kTileBytes, *dy_next = dy_tiles + ((n + 1) & 1u) * kTileBytes;
                    // step A: z = U . W1^T and dh = DY . W2 together.  This commit also covers the previous pass's
                    // weight-gradient MMAs (a commit tracks everything its thread issued before), which read the
                    // h and dz tiles the epilogue below overwrites.
                    if (threadIdx.x < 32) {
                        const bool leader = elect_one();
                        tc_fence_after();
                        issue_gemm(leader, tmem + kZ, u_cur, 32, w1, 32, s.half / 16, id_z, false);
                        issue_gemm(leader, tmem + kDH, dy_cur, 32, w2, 2048, s.half / 16, id_dh, false);
                        if (leader) mma_commit(bar);
                        __syncwarp();
                    }
                    main_wait_mma(bar, phase, &abort_flag);
                    {
                        // h = act(z) first (also the ReLU mask), then dz = dh where h > 0
                        const int nn = s.hid / kGroups, first = seat.group * (nn / 8);
                        const uint32_t row_off = seat.row * 128, row_swizzle = (seat.row & 7) << 4;
                        const uint32_t h_row = smem_addr(h_tile) + row_off, dz_row = smem_addr(dz_tile) + row_off;
                        for_each_piece(taddr + kZ + seat.group * nn, nn, [&](int u, const uint32_t(&piece)[8]) {
                            st_shared_16(h_row + (((first + u) << 4) ^ row_swizzle), finish8<T, ACT, false>(piece, nullptr));
                        });
                        for_each_piece(taddr + kDH + seat.group * nn, nn, [&](int u, const uint32_t(&piece)[8]) {
                            const uint32_t off = ((first + u) << 4) ^ row_swizzle;
                            uint4 g = finish8<T, TH_ACT_NONE, false>(piece, nullptr);
                            if constexpr (ACT == TH_ACT_RELU) {
                                const uint4 h = ld_shared_16(h_row + off);  // this thread's own store above
                                g.x = keep_where_positive<T>(g.x, h.x);
                                g.y = keep_where_positive<T>(g.y, h.y);
                                g.z = keep_where_positive<T>(g.z, h.z);
                                g.w = keep_where_positive<T>(g.w, h.w);
                            }
                            st_shared_16(dz_row + off, g);
                        });
                    }
                    main_publish();
                    // step B: undo the branch and push the gradient through (waited for below); then both weight
                    // gradients, committed on their own for the flush warps
                    if (threadIdx.x < 32) {
                        const bool leader = elect_one();
                        tc_fence_after();
                        issue_gemm(leader, tmem + out_col, smem_addr(h_tile), 32, w2, 32, s.hid / 16, id_undo, true);
                        issue_gemm(leader, tmem + in_d_col, smem_addr(dz_tile), 32, w1, 2048, s.hid / 16, id_din, true);
                        if (leader) mma_commit(bar);
                        // the accumulators still hold the previous pass's sums until the flush warps have read them
                        const bool free_dw = n == 0 || __all_sync(0xffffffffu, rev_wait(flushed_addr, (n - 1) & 1u, &abort_flag));
                        if (free_dw) {
                            tc_fence_after();
                            issue_gemm(leader, tmem + kDW2, dy_cur, 2048, smem_addr(h_tile), 2048, kTileRows / 16, id_dw2, false);
                            issue_gemm(leader, tmem + kDW1, smem_addr(dz_tile), 2048, u_cur, 2048, kTileRows / 16, id_dw1, false);
                            if (leader) mma_commit(wgrad_addr);
                        }
                        __syncwarp();
                    }
                    main_wait_mma(bar, phase, &abort_flag);
                    // next pass: its input is the stream just reconstructed, its output gradient the one just updated
                    stream_epilogue<T, false>(taddr + out_col, seat, s.half, nullptr, u_next, nullptr, false);
                    stream_epilogue<T, false>(taddr + in_d_col, seat, s.half, nullptr, dy_next, nullptr, false);
                    if (pass == 1) {  // next block's weights have landed
                        if (!use_tma) async_tile_wait();
                        else if (more) ring_wait(ring_bars, step + 1, &abort_flag);
                    }
                    main_publish();
                }
            }
            // the stream is now the reconstructed input, the gradient stream the input gradient
            if (!*abort_now) {
#pragma unroll 1
                for (int q = 0; q < 4; ++q) {
                    // q: 0 = dx1 (D1), 1 = dx2 (D2), 2 = x1 (S1), 3 = x2 (S2)
                    T *base = q < 2 ? gx : x_rec;
                    const long long stride = q < 2 ? gx_stride : xr_stride;
                    const uint32_t col = q == 0 ? kD1 : (q == 1 ? kD2 : (q == 2 ? kS1 : kS2));
                    if (base != nullptr)
                        stream_epilogue<T, false>(taddr + col, seat, s.half, nullptr, nullptr,
                                                  base + (live ? row0 + seat.row : 0) * stride + (q & 1) * s.half, live);
                }
                tc_fence_before();
                main_sync();
            }
        }
    }
    if (abort_flag) g_tc_status = 1;
    cta_teardown(tmem, P.tmem_cols);
}

// Sum the per-CTA accumulators ([cta][block][matrix][64][64]) into the gradient tensors.
template <typename T>
__global__ void rev_grad_reduce_tc_kernel(const RevShape s, const float *__restrict__ workspace, int n_ctas, T *dw_f1,
                                          T *dw_f2, T *dw_g1, T *dw_g2) {
    const size_t per_cta = rev_cta_floats(s);
    const size_t mat_total = static_cast<size_t>(s.blocks) * 4 * kMatFloats;
    T *dw[4] = {dw_f1, dw_f2, dw_g1, dw_g2};
    for (size_t e = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < mat_total;
         e += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int k = static_cast<int>(e / (4 * kMatFloats));
        const int m = static_cast<int>((e / kMatFloats) % 4);
        const int row = static_cast<int>((e % kMatFloats) / 64), col = static_cast<int>(e % 64);
        const int out_dim = (m & 1) ? s.half : s.hid, in_dim = (m & 1) ? s.hid : s.half;
        if (row >= out_dim || col >= in_dim || !dw[m]) continue;
        const size_t at = (e / kMatFloats) * kMatFloats + dw_private_index(row, col);
        float sum = 0.f;
        for (int c = 0; c < n_ctas; ++c) sum += workspace[c * per_cta + at];
        dw[m][(static_cast<size_t>(k) * out_dim + row) * in_dim + col] = from_float<T>(sum);
    }
}

// ---- host side ---------------------------------------------------------------------------------

bool rev_tc_disabled() {
    static const bool off = [] {
        const char *v = getenv("TH_MLP_LEGACY");
        return v && v[0] == '1';
    }();
    return off;
}

bool rows16_ok(const void *p, int64_t stride) { return p && stride % 8 == 0 && aligned_to(p, 16); }

// Dynamic shared memory to request so that no more than `ctas` CTAs share an SM.
int smem_request(const RevTcPlan &P, int ctas) {
    const int need = P.total + 1024;
    const int floor_bytes = kSmemBudget / (ctas + 1) + 1;
    return need > floor_bytes ? need : floor_bytes;
}

// Tensor maps of the four stacked weight arrays (box = 64 columns x one block's rows); 0 when one of
// them cannot be described (then the kernels stage the weights with cp.async) or TH_MLP_NO_TMA=1.
int make_rev_maps(RevWeightMaps &maps, const RevShape &s, const RevParams &p) {
    memset(&maps, 0, sizeof(maps));
    static const bool off = [] {
        const char *v = getenv("TH_MLP_NO_TMA");
        return v && v[0] == '1';
    }();
    if (off) return 0;
    const void *w[4] = {p.w_f1, p.w_f2, p.w_g1, p.w_g2};
    for (int m = 0; m < 4; ++m) {
        const int rows = (m & 1) ? s.half : s.hid, cols = (m & 1) ? s.hid : s.half;
        if (!make_map(&maps.m[m], w[m], static_cast<long long>(s.blocks) * rows, cols, rows)) return 0;
    }
    return 1;
}

// TH_MLP_NO_TMEM_A=1 keeps the A operands of the forward GEMMs in shared memory (for A/B runs).
bool rev_tmem_a_enabled() {
    static const bool on = [] {
        const char *v = getenv("TH_MLP_NO_TMEM_A");
        return !(v && v[0] == '1');
    }();
    return on;
}

template <typename T, int ACT, bool BIAS, bool TA>
int launch_rev_fwd_ta(const RevShape &s, const RevParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
                      int64_t rows, cudaStream_t stream) {
    const RevTcPlan P = rev_tc_plan(false);
    const int ctas = 2;  // 256 of the 512 TMEM columns each
    const int smem = smem_request(P, ctas);
    auto kernel = rev_fwd_tc_kernel<T, ACT, BIAS, TA>;
    if (int rc = cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                             "cudaFuncSetAttribute(rev_fwd_tc_kernel)")) return rc;
    const long long tiles = (rows + kTileRows - 1) / kTileRows;
    const long long cap = static_cast<long long>(sm_count()) * ctas;
    RevWeightMaps maps;
    const int use_tma = make_rev_maps(maps, s, p);
    kernel<<<static_cast<unsigned>(tiles < cap ? tiles : cap), kTcThreads, smem, stream>>>(
        s, p, maps, use_tma, static_cast<const T *>(x), x_stride, static_cast<T *>(y), y_stride, rows);
    return launch_status("rev_fwd_tc_kernel launch");
}

template <typename T, int ACT, bool BIAS>
int launch_rev_fwd_t(const RevShape &s, const RevParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
                     int64_t rows, cudaStream_t stream) {
    return rev_tmem_a_enabled() ? launch_rev_fwd_ta<T, ACT, BIAS, true>(s, p, x, x_stride, y, y_stride, rows, stream)
                                : launch_rev_fwd_ta<T, ACT, BIAS, false>(s, p, x, x_stride, y, y_stride, rows, stream);
}

template <typename T, bool BIAS>
int launch_rev_fwd_act(const RevShape &s, const RevParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
                       int64_t rows, cudaStream_t stream) {
    switch (s.act) {
        case TH_ACT_RELU: return launch_rev_fwd_t<T, TH_ACT_RELU, BIAS>(s, p, x, x_stride, y, y_stride, rows, stream);
        case TH_ACT_SILU: return launch_rev_fwd_t<T, TH_ACT_SILU, BIAS>(s, p, x, x_stride, y, y_stride, rows, stream);
        case TH_ACT_RELU2: return launch_rev_fwd_t<T, TH_ACT_RELU2, BIAS>(s, p, x, x_stride, y, y_stride, rows, stream);
        default: return launch_rev_fwd_t<T, TH_ACT_NONE, BIAS>(s, p, x, x_stride, y, y_stride, rows, stream);
    }
}

template <typename T>
int launch_rev_fwd(const RevShape &s, const RevParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
                   int64_t rows, cudaStream_t stream) {
    return s.has_bias ? launch_rev_fwd_act<T, true>(s, p, x, x_stride, y, y_stride, rows, stream)
                      : launch_rev_fwd_act<T, false>(s, p, x, x_stride, y, y_stride, rows, stream);
}

template <typename T, int ACT>
int launch_rev_bwd_t(const RevShape &s, const RevParams &p, const void *y, int64_t y_stride, const void *go,
                     int64_t go_stride, void *gx, int64_t gx_stride, void *x_rec, int64_t xr_stride, void *const dw[4],
                     float *workspace, int n_ctas, int64_t rows, cudaStream_t stream) {
    const RevTcPlan P = rev_tc_plan(true);
    const int smem = smem_request(P, 1);  // all 512 TMEM columns: one CTA per SM
    auto kernel = rev_bwd_tc_kernel<T, ACT>;
    if (int rc = cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                             "cudaFuncSetAttribute(rev_bwd_tc_kernel)")) return rc;
    RevWeightMaps maps;
    const int use_tma = make_rev_maps(maps, s, p);
    kernel<<<n_ctas, kTcThreads + kRevFlushThreads, smem, stream>>>(s, p, maps, use_tma, static_cast<const T *>(y), y_stride,
                                                static_cast<const T *>(go), go_stride, static_cast<T *>(gx), gx_stride,
                                                static_cast<T *>(x_rec), xr_stride, workspace, rows);
    if (int rc = launch_status("rev_bwd_tc_kernel launch")) return rc;
    const size_t mat_total = static_cast<size_t>(s.blocks) * 4 * kMatFloats;
    rev_grad_reduce_tc_kernel<T><<<static_cast<unsigned>((mat_total + 255) / 256), 256, 0, stream>>>(
        s, workspace, n_ctas, static_cast<T *>(dw[0]), static_cast<T *>(dw[1]), static_cast<T *>(dw[2]),
        static_cast<T *>(dw[3]));
    return launch_status("rev_grad_reduce_tc_kernel launch");
}

}  // namespace

int rev_fwd_tc(const RevShape &s, const RevParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
               int64_t rows, int dtype, cudaStream_t stream) {
    if (rev_tc_disabled() || rows <= 0) return kRevTcNotApplicable;
    if (!rows16_ok(x, x_stride) || !rows16_ok(y, y_stride)) return kRevTcNotApplicable;
    switch (dtype) {
        case TH_F16: return launch_rev_fwd<__half>(s, p, x, x_stride, y, y_stride, rows, stream);
        case TH_BF16: return launch_rev_fwd<__nv_bfloat16>(s, p, x, x_stride, y, y_stride, rows, stream);
        default: return kRevTcNotApplicable;
    }
}

int rev_bwd_tc(const RevShape &s, const RevParams &p, const void *y, int64_t y_stride, const void *go, int64_t go_stride,
               void *gx, int64_t gx_stride, void *x_rec, int64_t xr_stride, void *const dw[4], float *workspace,
               int n_ctas, int64_t rows, int dtype, cudaStream_t stream) {
    if (rev_tc_disabled() || rows <= 0) return kRevTcNotApplicable;
    if (s.has_bias || (s.act != TH_ACT_RELU && s.act != TH_ACT_NONE)) return kRevTcNotApplicable;
    if (!rows16_ok(y, y_stride) || !rows16_ok(go, go_stride) || (gx && !rows16_ok(gx, gx_stride)) ||
        (x_rec && !rows16_ok(x_rec, xr_stride)))
        return kRevTcNotApplicable;
#define TH_REV_BWD(T)                                                                                                        \
    (s.act == TH_ACT_RELU ? launch_rev_bwd_t<T, TH_ACT_RELU>(s, p, y, y_stride, go, go_stride, gx, gx_stride, x_rec,         \
                                                            xr_stride, dw, workspace, n_ctas, rows, stream)                 \
                          : launch_rev_bwd_t<T, TH_ACT_NONE>(s, p, y, y_stride, go, go_stride, gx, gx_stride, x_rec,         \
                                                            xr_stride, dw, workspace, n_ctas, rows, stream))
    switch (dtype) {
        case TH_F16: return TH_REV_BWD(__half);
        case TH_BF16: return TH_REV_BWD(__nv_bfloat16);
        default: return kRevTcNotApplicable;
    }
#undef TH_REV_BWD
}

}  // namespace th

// Device-side status of the reversible tensor-core kernels: 0 = fine, 1 = a bounded wait ran out.
extern "C" int th_rev_tc_status(void) {
    int status = 0;
    if (cudaMemcpyFromSymbol(&status, th::g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    return status;
}

