// Fully fused MLP on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM).
//
// A 128-row tile of the batch is the unit of work (M = 128 = the TMEM lanes; a thread that reads an
// accumulator reads the TMEM lanes of its warp quarter, thread = lane = tile row).  Every operand
// tile lives in shared memory in ONE layout: rows 128 bytes apart (64 16-bit features), 16-byte
// chunk c of row r stored at chunk position c ^ (r & 7), tile base 1024-byte aligned.  That is the
// canonical 128-byte-swizzle layout of the tensor core, and the same bytes can be described to it
// two ways:
//   K-major  (the row index is M or N, features are K)  - forward GEMMs, the A side of dgrad;
//   MN-major (the row index is K, features are M or N)  - wgrad (K = the tile's 128 rows) and
//            the weight side of dgrad (K = a layer's outputs, N = its inputs),
// so neither activations nor weights are ever transposed or stored twice.
//
//   forward : ACC[128 x out] = ACT_l[128 x in] . W_l^T        A K-major, B K-major
//   dgrad   : ACC[128 x in]  = DZ_l[128 x out] . W_l          A K-major, B MN-major
//   wgrad   : DW_l[out x in] += DZ_l^T[out x 128] . ACT_l     A, B MN-major, M = 64
//
// An elected lane issues the MMAs and commits them to an mbarrier; the epilogue threads read their
// part of the accumulator row with tcgen05.ld, apply bias / activation / ReLU mask on packed 16-bit
// pairs and write the next operand tile straight back to shared memory (fence.proxy.async before
// the tensor core reads it).  Weight gradients stay in TMEM columns for the whole life of the CTA
// (wgrad MMAs accumulate tile after tile) and leave once, at the end, as red.global.add.f32.
//
// Four kernels, in the order of the file:
//   mlp_fwd_tc_kernel   one tile per CTA of 256 threads, several CTAs per SM; the forward for rows
//                       TMA cannot describe
//   mlp_fwd_pipe_kernel one CTA per SM, up to four independent 128-thread slots with a tile each in
//                       flight, sharing the weights; input tiles by TMA - the usual forward
//   mlp_bwd_tc_kernel   one tile per CTA of 256 threads; the backward when only one CTA fits an SM
//   mlp_bwd_pipe_kernel 256 epilogue threads + an issuer warp, dgrad and wgrad committed separately,
//                       the next tile's inputs prefetched by TMA - the usual backward
//
// Weights reach shared memory by TMA (cp.async.bulk.tensor.2d, one box per layer, 128-byte swizzle:
// the box lands directly in the operand-tile layout, zero filled where a layer is narrower than its
// padded tile); arrays TMA cannot describe (inner dimension not a multiple of 8 elements) are staged
// with plain loads instead.  No multicast: every CTA loads its own copy.
//
// Every wait is bounded: a stuck mbarrier sets a device-side status word and the CTA frees its
// TMEM and returns.  tcgen05.alloc cannot block for good because the launcher sizes shared
// memory so that the CTAs resident on one SM never ask for more than its 512 TMEM columns.
#include "mlp_tc_device.cuh"

namespace th {
namespace {

// ---- forward -----------------------------------------------------------------------------------
template <typename T, int ACT, bool BIAS>
__global__ void __launch_bounds__(kTcThreads, 3)
mlp_fwd_tc_kernel(const MlpShape s, const MlpParams p, const __grid_constant__ WeightMaps maps, const int use_tma,
                  const T *__restrict__ x, long long x_stride, T *__restrict__ y, long long y_stride, long long n_rows,
                  int x_vec, int y_vec) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint32_t tmem_holder;
    __shared__ __align__(8) unsigned long long mbar;
    __shared__ int abort_flag;
    const TcPlan P = tc_plan(s, false);
    constexpr int bf16 = std::is_same<T, __half>::value ? 0 : 1;

    __shared__ __align__(8) unsigned long long wbar;
    if (threadIdx.x == 0) abort_flag = 0;
    stage_biases<T>(smem, P, s, p);
    bool weights_ok = true;
    if (use_tma) weights_ok = tma_stage_weights(smem, P, s, maps, &wbar);
    else stage_all_weights<T>(smem, P, s, p);
    const uint32_t tmem = cta_setup(&tmem_holder, &mbar, P.tmem_cols);
    if (!weights_ok) {  // the bytes never arrived: report and leave (after the barrier inside cta_setup)
        abort_flag = 1;
        g_tc_status = 1;
    }
    __syncthreads();
    const uint32_t bar = smem_addr(&mbar);
    const float *bias = reinterpret_cast<const float *>(smem + P.bias_offset);
    const Seat seat;
    const uint32_t taddr = tmem + seat.lane_base;
    uint32_t phase = 0;
    const long long n_tiles = (n_rows + kTileRows - 1) / kTileRows;

    // Input tiles alternate between two buffers: while tile t runs through its layers in place in
    // buffer t & 1, tile t + 1 streams into the other one.
    auto start_input = [&](long long t, int b) {
        unsigned char *dst = smem + b * kTileBytes;
        if (x_vec) {
            async_tile_load<T>(dst, x, x_stride, t * kTileRows, n_rows, s.d_in, s.ki);
        } else {
            TileRegs regs;
            fetch_tile<T>(regs, x, x_stride, t * kTileRows, n_rows, s.d_in, s.ki, false);
            commit_tile(dst, regs, s.ki);
        }
    };
    int cur = 0;
    if (static_cast<long long>(blockIdx.x) < n_tiles) start_input(blockIdx.x, 0);
    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, cur ^= 1) {
        const long long row0 = tile * kTileRows;
        unsigned char *act_tile = smem + cur * kTileBytes;
        const uint32_t act_addr = smem_addr(act_tile);
        async_tile_wait();
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (abort_flag) break;
        // the other buffer is free (its tile finished before the barrier above): start the next input
        if (tile + gridDim.x < n_tiles) start_input(tile + gridDim.x, cur ^ 1);
        for (int l = 0; l <= s.depth; ++l) {
            const int in_pad = l == 0 ? s.ki : s.h;
            const int out_pad = l == s.depth ? s.no : s.h;
            if (threadIdx.x < 32) {
                const bool leader = elect_one();
                tc_fence_after();
                issue_gemm(leader, tmem, act_addr, 32, smem_addr(weight_tile(smem, P, s, l)), 32, in_pad / 16,
                           instr_desc(128, out_pad, bf16, 0, 0), false);
                if (leader) mma_commit(bar);
                __syncwarp();
            }
            const bool ok = cta_wait_mma(bar, phase, &abort_flag);
            if (!ok) {
                g_tc_status = 1;
            } else if (l < s.depth) {
                hidden_epilogue<T, ACT, BIAS>(taddr, seat, out_pad, bias + l * kMaxDim, act_tile);
            } else {
                const bool live = row0 + seat.row < n_rows;
                output_epilogue<T, BIAS>(taddr, seat, out_pad, bias + l * kMaxDim, y + (live ? row0 + seat.row : 0) * y_stride,
                                         s.d_out, live, y_vec);
            }
            if (l < s.depth) {
                fence_async_smem();
                tc_fence_before();
                __syncthreads();
                if (abort_flag) break;
            }
        }
        tc_fence_before();
        if (abort_flag) break;
    }
    cta_teardown(tmem, P.tmem_cols);
}

// ---- forward, several row tiles per CTA ------------------------------------------------------------
//
// The kernel above keeps one row tile per CTA in flight and every thread walks the same chain
// (issue, wait, epilogue, barrier); only co-resident CTAs overlap, and each of them needs its own
// copy of the weights.  Here one CTA per SM runs S independent "slots" of 128 threads (4 warps).
// A slot is what a CTA is above - it owns 64 TMEM columns, two operand tiles and two mbarriers, and
// walks its row tiles layer by layer - but the slots share the weights, and they never meet at a
// CTA-wide barrier after set-up, so one slot's MMAs run under the other slots' epilogues:
//
//   warp 0 of the slot  : fetches the slot's next input tile by TMA (a box of 64 columns x 128 rows
//                         lands in the operand-tile layout; rows past the end and columns past
//                         d_in arrive as zeros), waits for the current one, issues each layer's
//                         GEMM, commits it to `acc_full` and polls that barrier;
//   all 4 warps         : meet at the slot's named barrier (the three other warps park there while
//                         the MMAs run), turn their accumulator rows (thread = tile row =
//                         TMEM lane) into the next layer's operand rows in place, or into output
//                         rows in global memory, and meet at the slot's named barrier.
//
// Tile k of a slot computes in buffer k & 1 while the prefetch of tile k + 1 lands in the other.
// Every mbarrier wait is bounded and watches a shared abort flag; after an abort a slot keeps the
// SAME sequence of named barriers (doing no work) so nobody is left waiting at one.

constexpr int kMaxSlots = 5;

struct SlotBarriers {
    unsigned long long in_full[kMaxSlots][2];
    unsigned long long acc_full[kMaxSlots];
};

// Bounded by wall-clock time (the nanosecond global timer, looked at every 64 polls): two seconds are
// orders of magnitude above any wait of a healthy run, also under a profiler's replay.
constexpr unsigned long long kPipeWaitNs = 2000000000ull;

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ bool pipe_wait(uint32_t bar, uint32_t parity, int *abort_flag) {
    if (*reinterpret_cast<volatile int *>(abort_flag)) return false;
    unsigned long long deadline = 0;
    for (unsigned poll = 0;; ++poll) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
        if ((poll & 63u) == 63u) {
            if (*reinterpret_cast<volatile int *>(abort_flag)) return false;
            const unsigned long long now = global_ns();
            if (deadline == 0) deadline = now + kPipeWaitNs;
            else if (now > deadline) break;
        }
    }
    *reinterpret_cast<volatile int *>(abort_flag) = 1;
    g_tc_status = 1;
    return false;
}

__device__ __forceinline__ void slot_barrier(int slot) {
    asm volatile("bar.sync %0, 128;" ::"r"(slot + 1) : "memory");
}

// One accumulator row (out_pad = 16, 32 or 64 columns) -> bias, activation, rounding -> 16-byte
// chunks, each handed to `sink(chunk index, packed values)`; 32 columns per TMEM load.
// TA: hidden activations go back to the tensor core through tensor memory (32 more columns per slot) instead of
// the operand tile in shared memory; the first layer still reads the TMA-fetched input tile.
template <typename T, int ACT, bool BIAS, int S, bool MSE, bool TA>
__global__ void __launch_bounds__(128 * S, 1)
mlp_fwd_pipe_kernel(const MlpShape s, const MlpParams p, const __grid_constant__ WeightMaps maps,
                    const __grid_constant__ CUtensorMap x_map, T *__restrict__ y, long long y_stride, long long n_rows,
                    int y_vec, const MseArgs mse) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint32_t tmem_holder;
    __shared__ int abort_flag;
    __shared__ __align__(8) unsigned long long wbar;
    __shared__ __align__(8) SlotBarriers bars;
    const TcPlan P = tc_plan(s, false, 2 * S);
    constexpr int bf16 = std::is_same<T, __half>::value ? 0 : 1;
    constexpr uint32_t kTmemCols = S * (kAccCols + (TA ? 32 : 0)) <= 256 ? 256 : 512;
    const int warp = threadIdx.x >> 5;

    // ---- set-up: barriers, biases, weights, TMEM ----
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < S; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars.in_full[i][0])), "r"(1u) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars.in_full[i][1])), "r"(1u) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars.acc_full[i])), "r"(1u) : "memory");
        }
    }
    {
        float *bias = reinterpret_cast<float *>(smem + P.bias_offset);
        for (int e = threadIdx.x; e < (s.depth + 1) * kMaxDim; e += blockDim.x) {
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
    const bool weights_ok = tma_stage_weights(smem, P, s, maps, &wbar);  // contains the barrier that publishes the inits
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_holder)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (!weights_ok) {
        abort_flag = 1;
        g_tc_status = 1;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_holder;
    const float *bias = reinterpret_cast<const float *>(smem + P.bias_offset);

    const long long n_tiles = (n_rows + kTileRows - 1) / kTileRows;
    const long long first_tile = blockIdx.x;
    const long long n_mine = first_tile < n_tiles ? (n_tiles - first_tile + gridDim.x - 1) / gridDim.x : 0;

    // ---- the slot's life; nothing below depends on other slots ----
    const int slot = warp >> 2;
    const bool issuer = (warp & 3) == 0;
    const int row = 32 * (warp & 3) + (threadIdx.x & 31);
    const uint32_t acc = tmem + slot * kAccCols;
    const uint32_t taddr = acc + (static_cast<uint32_t>(32 * (warp & 3)) << 16);
    const uint32_t act_tmem = tmem + S * kAccCols + slot * 32;  // TA: the slot's hidden activations, 16-bit pairs
    const uint32_t act_taddr = act_tmem + (static_cast<uint32_t>(32 * (warp & 3)) << 16);
    const uint32_t acc_bar = smem_addr(&bars.acc_full[slot]);
    unsigned char *buffers = smem + 2 * slot * kTileBytes;
    uint32_t acc_phase = 0;  // tracked by the issuer warp
    float loss = 0.f;        // MSE: this thread's share of sum (prediction - target)^2

    auto fetch_input = [&](int b, long long k) {  // by the issuer warp
        if (elect_one()) {
            const uint32_t bar = smem_addr(&bars.in_full[slot][b]);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(static_cast<uint32_t>(kTileBytes))
                         : "memory");
            tma_load_2d(buffers + b * kTileBytes, &x_map, 0, static_cast<int>((first_tile + k * gridDim.x) * kTileRows), bar);
        }
        __syncwarp();
    };
    if (issuer && slot < n_mine && !abort_flag) fetch_input(0, slot);

    for (long long k = slot, q = 0; k < n_mine; k += S, ++q) {
        const int b = static_cast<int>(q & 1);
        const long long row0 = (first_tile + k * gridDim.x) * kTileRows;
        unsigned char *tile = buffers + b * kTileBytes;
        const uint32_t tile_addr = smem_addr(tile);
        const uint32_t row_addr = tile_addr + row * 128, row_swizzle = (row & 7) << 4;  // chunk c of the row: row_addr + ((c << 4) ^ row_swizzle)
        if (issuer) {
            // the other buffer's last reader was the previous tile of this slot: finished
            if (k + S < n_mine && !*reinterpret_cast<volatile int *>(&abort_flag)) fetch_input(b ^ 1, k + S);
            pipe_wait(smem_addr(&bars.in_full[slot][b]), static_cast<uint32_t>((q >> 1) & 1), &abort_flag);
        }
        for (int l = 0; l <= s.depth; ++l) {
            const int in_pad = l == 0 ? s.ki : s.h;
            const int out_pad = l == s.depth ? s.no : s.h;
            // Only the issuer warp polls the mbarrier; the slot's other warps park at the named barrier,
            // which costs no issue slots.  A wait that gives up raises the abort flag, and everybody
            // reads it after the barrier: work stops, the barrier sequence goes on.
            if (issuer) {
                if (__all_sync(0xffffffffu, !*reinterpret_cast<volatile int *>(&abort_flag))) {
                    const bool leader = elect_one();
                    tc_fence_after();
                    if (TA && l > 0)
                        issue_gemm_ta(leader, acc, act_tmem, smem_addr(weight_tile(smem, P, s, l)), 32, in_pad / 16,
                                      instr_desc(128, out_pad, bf16, 0, 0), false);
                    else
                        issue_gemm(leader, acc, tile_addr, 32, smem_addr(weight_tile(smem, P, s, l)), 32, in_pad / 16,
                                   instr_desc(128, out_pad, bf16, 0, 0), false);
                    if (leader) mma_commit(acc_bar);
                    __syncwarp();
                    pipe_wait(acc_bar, acc_phase, &abort_flag);
                    acc_phase ^= 1u;
                }
            }
            slot_barrier(slot);
            if (!*reinterpret_cast<volatile int *>(&abort_flag)) {
                tc_fence_after();
                const float *layer_bias = bias + l * kMaxDim;
                if (l < s.depth) {
                    if constexpr (TA) {
                        drain_row<T, ACT, BIAS>(taddr, out_pad, layer_bias, [&](int chunk, uint4 packed) { tmem_st4(act_taddr + 4 * chunk, packed); });
                        tmem_st_wait();
                    } else {
                        drain_row<T, ACT, BIAS>(taddr, out_pad, layer_bias, [&](int chunk, uint4 packed) {
                            st_shared_16(row_addr + ((chunk << 4) ^ row_swizzle), packed);
                        });
                        fence_async_smem();
                    }
                } else {
                    const bool live = row0 + row < n_rows;
                    if constexpr (MSE) {
                        // d_out is a multiple of 8 and all rows are 16-byte aligned here (checked by the launcher)
                        const long long r = live ? row0 + row : 0;
                        const T *target_row = static_cast<const T *>(mse.target) + r * mse.target_stride;
                        T *grad_row = static_cast<T *>(mse.grad) + r * mse.grad_stride;
                        T *out_row = y ? y + r * y_stride : nullptr;
                        drain_row<T, TH_ACT_NONE, BIAS>(taddr, out_pad, layer_bias, [&](int chunk, uint4 packed) {
                            if (live && 8 * chunk < s.d_out) {
                                if (out_row) __stcs(reinterpret_cast<uint4 *>(out_row + 8 * chunk), packed);
                                const uint4 t = __ldcs(reinterpret_cast<const uint4 *>(target_row + 8 * chunk));
                                __stcs(reinterpret_cast<uint4 *>(grad_row + 8 * chunk), mse_chunk<T>(packed, t, mse.grad_scale, loss));
                            }
                        });
                    } else {
                        T *out_row = y + (live ? row0 + row : 0) * y_stride;
                        drain_row<T, TH_ACT_NONE, BIAS>(taddr, out_pad, layer_bias, [&](int chunk, uint4 packed) {
                            if (live) store_chunk_to_global<T>(out_row, chunk, s.d_out, packed, y_vec);
                        });
                    }
                }
                tc_fence_before();
            }
            slot_barrier(slot);
        }
    }

    if constexpr (MSE) {
        // one atomic per warp for the whole kernel
        for (int off = 16; off > 0; off >>= 1) loss += __shfl_xor_sync(0xffffffffu, loss, off);
        if ((threadIdx.x & 31) == 0 && mse.loss_sum) atomicAdd(mse.loss_sum, loss);
    }

    // ---- teardown ----
    tc_fence_before();
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
}

// ---- backward ----------------------------------------------------------------------------------
//
// Biases and activations that need the pre-activation (SiLU, ReLU^2) stay on the tensor cores:
//   * bias gradient of layer l = column sums of dz_l over the tile's rows = dz_l^T . ONES, one more small
//     MMA per step (A = the dz tile MN-major as for wgrad, B = a tile of ones, N = 16) into 16 TMEM columns
//     per layer that live as long as the weight-gradient accumulators and are flushed with them;
//   * SiLU' and ReLU^2' want z_{l-1}, which nobody kept: the step that needs it issues the layer's forward
//     GEMM again (act[l-1] . W_{l-1}^T, four MMAs) into a second accumulator, and the epilogue reads dy and
//     z side by side, rounds z to the storage dtype as the forward pass did (reference: activation
//     derivatives are taken at the dtype-rounded pre-activation, fully_fused_mlp/kernel.py:278-281) and
//     applies the derivative.  The tensor pipe has the room; shared memory does not.

// dz of the layer below from dy (accumulator) and the recomputed pre-activation (second accumulator)
template <typename T, int ACT, bool BIAS>
__device__ __forceinline__ void dz_epilogue_preact(uint32_t taddr_dy, uint32_t taddr_z, const Seat &seat, int pad, const float *bias,
                                                   unsigned char *dz_tile) {
    const int n = pad / kGroups, first = seat.group * (n / 8);
    const uint32_t dz_row = smem_addr(dz_tile) + seat.row * 128, row_swizzle = (seat.row & 7) << 4;
    for (int u = 0; u < n / 8; ++u) {
        uint32_t dy[8], zz[8];
        tmem_ld8(taddr_dy + seat.group * n + 8 * u, dy);
        tmem_ld8(taddr_z + seat.group * n + 8 * u, zz);
        tmem_ld_wait();
        float g[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            float z = __uint_as_float(zz[k]);
            if constexpr (BIAS) z += bias[8 * (first + u) + k];
            z = to_float<T>(from_float<T>(z));  // the forward pass stored z rounded
            g[k] = activate_grad(ACT, z, __uint_as_float(dy[k]));
        }
        st_shared_16(dz_row + (((first + u) << 4) ^ row_swizzle),
                     make_uint4(pack_pair<T>(g[0], g[1]), pack_pair<T>(g[2], g[3]), pack_pair<T>(g[4], g[5]), pack_pair<T>(g[6], g[7])));
    }
}

// Column 0 of a bias-gradient accumulator (M = 64 layout, see flush_dw) -> float32 sums
__device__ __forceinline__ void flush_db(uint32_t taddr, float *dst, int out_dim) {
    uint32_t raw[8];
    tmem_ld8(taddr, raw);
    tmem_ld_wait();
    const int lane = threadIdx.x & 31;
    const int m = 16 * ((threadIdx.x >> 5) & 3) + lane;
    if (threadIdx.x < 128 && lane < 16 && m < out_dim) atomicAdd(dst + m, __uint_as_float(raw[0]));
}

template <typename T, int ACT, int MINB, bool BIAS>
__global__ void __launch_bounds__(kTcThreads, MINB)
mlp_bwd_tc_kernel(const MlpShape s, const MlpParams p, const __grid_constant__ WeightMaps maps, const int use_tma,
                  const T *__restrict__ x, long long x_stride,
                  const T *__restrict__ go, long long go_stride, T *__restrict__ gx, long long gx_stride,
                  float *__restrict__ workspace, long long n_rows, int x_vec, int go_vec, int gx_vec) {
    constexpr bool kPreact = ACT == TH_ACT_SILU || ACT == TH_ACT_RELU2;
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint32_t tmem_holder;
    __shared__ __align__(8) unsigned long long mbar;
    __shared__ int abort_flag;
    __shared__ __align__(8) unsigned long long wbar;
    const TcPlan P = tc_plan(s, true);
    constexpr int bf16 = std::is_same<T, __half>::value ? 0 : 1;

    if (threadIdx.x == 0) abort_flag = 0;
    // operand tiles start out as zeros: columns a layer does not use are still read as MMA rows
    for (int e = threadIdx.x; e < (P.act_tiles + P.dz_tiles) * kTileBytes / 16; e += kTcThreads)
        reinterpret_cast<uint4 *>(smem)[e] = make_uint4(0, 0, 0, 0);
    unsigned char *ones_tile = smem + (P.act_tiles + P.dz_tiles) * kTileBytes;
    if constexpr (BIAS) {
        // 128 rows x 16 columns of ones (logical chunks 0 and 1 of every row), zeros elsewhere
        const uint32_t one2 = pack_pair<T>(1.f, 1.f);
        for (int e = threadIdx.x; e < kTileBytes / 16; e += kTcThreads) {
            const int r = e >> 3, c = (e & 7) ^ (r & 7);  // physical chunk e & 7 of row r holds logical chunk c
            reinterpret_cast<uint4 *>(ones_tile)[e] = c < 2 ? make_uint4(one2, one2, one2, one2) : make_uint4(0, 0, 0, 0);
        }
    }
    stage_biases<T>(smem, P, s, p);
    bool weights_ok = true;
    if (use_tma) weights_ok = tma_stage_weights(smem, P, s, maps, &wbar);
    else stage_all_weights<T>(smem, P, s, p);
    const uint32_t tmem = cta_setup(&tmem_holder, &mbar, P.tmem_cols);
    if (!weights_ok) {
        abort_flag = 1;
        g_tc_status = 1;
    }
    __syncthreads();
    const uint32_t bar = smem_addr(&mbar);
    const float *bias = reinterpret_cast<const float *>(smem + P.bias_offset);
    unsigned char *dz_tiles = smem + P.act_tiles * kTileBytes;
    const Seat seat;
    const uint32_t taddr = tmem + seat.lane_base;
    uint32_t phase = 0;
    bool first_tile = true;
    const long long n_tiles = (n_rows + kTileRows - 1) / kTileRows;
    auto act_tile = [&](int l) { return smem + l * kTileBytes; };
    auto dw_col = [&](int l) { return kAccCols + (l == 0 ? 0 : s.ki + (l - 1) * s.h); };
    auto db_col = [&](int l) { return P.db_col + 16 * l; };

    // With one CTA per SM (MINB == 1: shared memory bound, registers to spare) the next tile's inputs
    // are fetched into registers while the current tile computes; with two CTAs per SM the other
    // CTA covers the latency and the registers are needed elsewhere.
    constexpr bool kPrefetch = MINB == 1;
    TileRegs x_next, go_next;
    if (kPrefetch && static_cast<long long>(blockIdx.x) < n_tiles) {
        fetch_tile<T>(x_next, x, x_stride, static_cast<long long>(blockIdx.x) * kTileRows, n_rows, s.d_in, s.ki, x_vec);
        fetch_tile<T>(go_next, go, go_stride, static_cast<long long>(blockIdx.x) * kTileRows, n_rows, s.d_out, s.no, go_vec);
    }
    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const long long row0 = tile * kTileRows;
        // ---- phase 1: recompute the forward, parking every layer input ----
        if (kPrefetch) {
            commit_tile(act_tile(0), x_next, s.ki);
            commit_tile(dz_tiles, go_next, s.no);  // dz of the output layer = grad_out
        } else {
            fetch_tile<T>(x_next, x, x_stride, row0, n_rows, s.d_in, s.ki, x_vec);
            commit_tile(act_tile(0), x_next, s.ki);
            fetch_tile<T>(x_next, go, go_stride, row0, n_rows, s.d_out, s.no, go_vec);
            commit_tile(dz_tiles, x_next, s.no);
        }
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (abort_flag) break;
        if (kPrefetch && tile + gridDim.x < n_tiles) {
            fetch_tile<T>(x_next, x, x_stride, (tile + gridDim.x) * kTileRows, n_rows, s.d_in, s.ki, x_vec);
            fetch_tile<T>(go_next, go, go_stride, (tile + gridDim.x) * kTileRows, n_rows, s.d_out, s.no, go_vec);
        }
        for (int l = 0; l < s.depth; ++l) {
            const int in_pad = l == 0 ? s.ki : s.h;
            if (threadIdx.x < 32) {
                const bool leader = elect_one();
                tc_fence_after();
                issue_gemm(leader, tmem, smem_addr(act_tile(l)), 32, smem_addr(weight_tile(smem, P, s, l)), 32, in_pad / 16,
                           instr_desc(128, s.h, bf16, 0, 0), false);
                if (leader) mma_commit(bar);
                __syncwarp();
            }
            const bool ok = cta_wait_mma(bar, phase, &abort_flag);
            if (!ok) {
                g_tc_status = 1;
            } else {
                hidden_epilogue<T, ACT, BIAS>(taddr, seat, s.h, bias + l * kMaxDim, act_tile(l + 1));
            }
            fence_async_smem();
            tc_fence_before();
            __syncthreads();
            if (abort_flag) break;
        }
        if (abort_flag) break;

        // ---- phase 2: walk the layers backwards ----
        int buf = 0;
        for (int l = s.depth; l >= 0; --l) {
            const int in_pad = l == 0 ? s.ki : s.h;
            const int out_pad = l == s.depth ? s.no : s.h;
            unsigned char *dz = dz_tiles + buf * kTileBytes;
            const bool need_dgrad = l > 0 || gx != nullptr;
            if (threadIdx.x < 32) {
                const bool leader = elect_one();
                tc_fence_after();
                // dgrad first (the epilogue waits for it): ACC[128 x in] = DZ . W_l (A K-major over the
                // layer's outputs, W_l tile MN-major)
                if (need_dgrad)
                    issue_gemm(leader, tmem, smem_addr(dz), 32, smem_addr(weight_tile(smem, P, s, l)), 2048, out_pad / 16,
                               instr_desc(128, in_pad, bf16, 0, 1), false);
                // the pre-activation of the layer below, for its activation's derivative
                if (kPreact && l > 0)
                    issue_gemm(leader, tmem + P.z_col, smem_addr(act_tile(l - 1)), 32, smem_addr(weight_tile(smem, P, s, l - 1)), 32,
                               (l == 1 ? s.ki : s.h) / 16, instr_desc(128, s.h, bf16, 0, 0), false);
                // wgrad: DW_l[out x in] += DZ^T . ACT_l over the tile's 128 rows (both operands MN-major)
                issue_gemm(leader, tmem + dw_col(l), smem_addr(dz), 2048, smem_addr(act_tile(l)), 2048, kTileRows / 16,
                           instr_desc(64, in_pad, bf16, 1, 1), !first_tile);
                // bias gradient: DB_l[out x 16] += DZ^T . ONES (every column holds the column sums of dz)
                if (BIAS)
                    issue_gemm(leader, tmem + db_col(l), smem_addr(dz), 2048, smem_addr(ones_tile), 2048, kTileRows / 16,
                               instr_desc(64, 16, bf16, 1, 1), !first_tile);
                if (leader) mma_commit(bar);
                __syncwarp();
            }
            const bool ok = cta_wait_mma(bar, phase, &abort_flag);
            if (!ok) {
                g_tc_status = 1;
            } else if (l > 0) {
                // in_pad == s.h here: the layer below produced ACT_l
                if constexpr (kPreact)
                    dz_epilogue_preact<T, ACT, BIAS>(taddr, taddr + P.z_col, seat, in_pad, bias + (l - 1) * kMaxDim, dz_tiles + (buf ^ 1) * kTileBytes);
                else
                    dz_epilogue<T, ACT>(taddr, seat, in_pad, act_tile(l), dz_tiles + (buf ^ 1) * kTileBytes);
            } else if (gx != nullptr) {
                const bool live = row0 + seat.row < n_rows;
                dx_epilogue<T>(taddr, seat, in_pad, gx + (live ? row0 + seat.row : 0) * gx_stride, s.d_in, live, gx_vec);
            }
            fence_async_smem();
            tc_fence_before();
            __syncthreads();
            if (abort_flag) break;
            buf ^= 1;
        }
        if (abort_flag) break;
        first_tile = false;
    }

    // ---- flush the weight (and bias) gradients this CTA accumulated in TMEM ----
    if (!abort_flag && !first_tile) {
        tc_fence_after();
        const MlpGradWorkspace W = grad_workspace_layout(s, workspace);
        for (int l = 0; l <= s.depth; ++l) {
            const int in_pad = l == 0 ? s.ki : s.h;
            const int in_dim = l == 0 ? s.d_in : s.d_hid, out_dim = l == s.depth ? s.d_out : s.d_hid;
            float *dst = W.base + (l == 0 ? W.w_in : (l == s.depth ? W.w_out : W.w_hid + (l - 1) * s.d_hid * s.d_hid));
            flush_dw(taddr + dw_col(l), seat, in_pad, dst, out_dim, in_dim);
            if constexpr (BIAS) {
                float *bdst = W.base + (l == 0 ? W.b_in : (l == s.depth ? W.b_out : W.b_hid + (l - 1) * s.d_hid));
                flush_db(taddr + db_col(l), bdst, out_dim);
            }
        }
    }
    cta_teardown(tmem, P.tmem_cols);
}

// ---- backward, issuer warp + prefetched inputs ----------------------------------------------------
//
// Same dataflow as mlp_bwd_tc_kernel above (recompute and park, then dgrad + wgrad per layer with the
// weight gradients resident in TMEM), reorganised so that less of it sits on the serial chain:
//
//   * warp 8 is the ISSUER.  It waits for an operand (mbarrier `ready`, 256 arrivals of the epilogue
//     threads, or a TMA barrier), issues the layer's MMAs and commits: dgrad to `acc_full`, which the
//     epilogue waits for, and wgrad after it to `wgrad_done`, which only the issuer itself waits for,
//     one step later, before it reuses a buffer.  The 256 epilogue threads never issue or wait on wgrad.
//   * the next row tile's x and grad_out tiles are fetched by TMA while the current tile is still in
//     its last steps, into operand tiles the current tile has finished with: x into the buffer that
//     held the input of the output layer (free once that layer's wgrad is done), grad_out into the dz
//     buffer that held dz of layer 1 (free during the last step).  The activation buffers therefore
//     rotate from tile to tile: layer l's input lives in buffer (base + l) mod (depth + 1).
//   * epilogues read up to 32 accumulator columns per tcgen05.ld, convert with the ReLU fused into
//     the rounding, and address shared memory with 32-bit shared addresses.
//
// Waiting for `acc_full`: warp 0 polls, the other seven epilogue warps park at named barrier 1 (256
// threads).  All mbarrier waits are bounded and watch the abort flag; after an abort everybody keeps
// the same barrier sequence without doing work.

struct BwdBarriers {
    // wgrad_done alternates between two barriers from step to step: the issuer waits for a step's
    // wgrad one step late, after committing the next one, and a single barrier could then complete
    // two phases between two looks at it, which a parity wait cannot tell from none.
    unsigned long long in_x, in_go, acc_full, wgrad_done[2], ready;
};

template <typename T, int ACT>
__global__ void __launch_bounds__(kTcThreads + 32, 2)
mlp_bwd_pipe_kernel(const MlpShape s, const MlpParams p, const __grid_constant__ WeightMaps maps,
                    const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap go_map,
                    T *__restrict__ gx, long long gx_stride, float *__restrict__ workspace, long long n_rows, int gx_vec) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint32_t tmem_holder;
    __shared__ int abort_flag;
    __shared__ __align__(8) unsigned long long wbar;
    __shared__ __align__(8) BwdBarriers bars;
    const TcPlan P = tc_plan(s, true);
    constexpr int bf16 = std::is_same<T, __half>::value ? 0 : 1;
    const int warp = threadIdx.x >> 5;
    const int d = s.depth;  // layers 0 .. d; layer d is the output layer
    const int n_act = d + 1;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars.in_x)), "r"(1u) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars.in_go)), "r"(1u) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars.acc_full)), "r"(1u) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars.wgrad_done[0])), "r"(1u) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars.wgrad_done[1])), "r"(1u) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars.ready)), "r"(static_cast<uint32_t>(kTcThreads / 32)) : "memory");
    }
    // operand tiles start out as zeros: columns a layer does not use are still read as MMA rows
    for (int e = threadIdx.x; e < (P.act_tiles + P.dz_tiles) * kTileBytes / 16; e += blockDim.x)
        reinterpret_cast<uint4 *>(smem)[e] = make_uint4(0, 0, 0, 0);
    fence_async_smem();
    const bool weights_ok = tma_stage_weights(smem, P, s, maps, &wbar);  // contains the barrier that publishes the inits
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_holder)),
                     "r"(static_cast<uint32_t>(P.tmem_cols))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (!weights_ok) {
        abort_flag = 1;
        g_tc_status = 1;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_holder;

    const long long n_tiles = (n_rows + kTileRows - 1) / kTileRows;
    const long long first_tile = blockIdx.x;
    const long long n_mine = first_tile < n_tiles ? (n_tiles - first_tile + gridDim.x - 1) / gridDim.x : 0;
    const uint32_t smem_base = smem_addr(smem);
    const uint32_t dz_base = smem_base + P.act_tiles * kTileBytes;
    auto dw_col = [&](int l) { return kAccCols + (l == 0 ? 0 : s.ki + (l - 1) * s.h); };
    auto weight_addr = [&](int l) { return smem_addr(weight_tile(smem, P, s, l)); };
    const uint32_t acc_bar = smem_addr(&bars.acc_full), ready_bar = smem_addr(&bars.ready);
    volatile int *abort_now = &abort_flag;

    if (warp == 8) {
        // ================= issuer =================
        const uint32_t x_bar = smem_addr(&bars.in_x), go_bar = smem_addr(&bars.in_go);
        const uint32_t wg_bar[2] = {smem_addr(&bars.wgrad_done[0]), smem_addr(&bars.wgrad_done[1])};
        uint32_t wg_phases = 0;  // bit b: parity of the next phase of wgrad_done[b] to wait for
        unsigned step = 0;       // counts backward steps over all tiles; step j commits to wgrad_done[j & 1]
        auto wait_wgrad = [&](unsigned j) {  // wgrad of step j has finished
            const unsigned b = j & 1u;
            const bool ok = __all_sync(0xffffffffu, pipe_wait(wg_bar[b], (wg_phases >> b) & 1u, &abort_flag));
            wg_phases ^= 1u << b;
            return ok;
        };
        auto fetch = [&](const CUtensorMap *map, uint32_t dst, uint32_t bar, long long k) {
            if (elect_one()) {
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(static_cast<uint32_t>(kTileBytes)) : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                    "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(static_cast<int>((first_tile + k * gridDim.x) * kTileRows)), "r"(bar)
                    : "memory");
            }
            __syncwarp();
        };
        int base = 0, zs = 0;
        uint32_t ready_phase = 0, in_phase = 0;
        bool alive = !*abort_now;
        if (alive && n_mine > 0) {
            fetch(&x_map, smem_base, x_bar, 0);
            fetch(&go_map, dz_base, go_bar, 0);
        }
        for (long long k = 0; alive && k < n_mine; ++k) {
            auto act_addr = [&](int l) { return smem_base + static_cast<uint32_t>((base + l) % n_act) * kTileBytes; };
            // ---- phase 1: recompute ----
            for (int l = 0; alive && l < d; ++l) {
                if (l > 0 || k > 0) {
                    alive = pipe_wait(ready_bar, ready_phase, &abort_flag);
                    ready_phase ^= 1u;
                }
                if (alive && l == 0) alive = pipe_wait(x_bar, in_phase, &abort_flag);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) break;
                const bool leader = elect_one();
                tc_fence_after();
                issue_gemm(leader, tmem, act_addr(l), 32, weight_addr(l), 32, (l == 0 ? s.ki : s.h) / 16,
                           instr_desc(128, s.h, bf16, 0, 0), false);
                if (leader) mma_commit(acc_bar);
                __syncwarp();
            }
            // ---- phase 2: layers backwards ----
            for (int l = d; alive && l >= 0; --l) {
                const int in_pad = l == 0 ? s.ki : s.h;
                const int out_pad = l == d ? s.no : s.h;
                const uint32_t dz = dz_base + static_cast<uint32_t>(zs ^ ((d - l) & 1)) * kTileBytes;
                if (d > 0 || k > 0) {
                    alive = pipe_wait(ready_bar, ready_phase, &abort_flag);
                    ready_phase ^= 1u;
                }
                if (alive && d == 0) alive = pipe_wait(x_bar, in_phase, &abort_flag);  // no recompute phase: x is first used here
                if (alive && l == d) alive = pipe_wait(go_bar, in_phase, &abort_flag);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) break;
                const bool leader = elect_one();
                tc_fence_after();
                if (l > 0 || gx != nullptr)
                    issue_gemm(leader, tmem, dz, 32, weight_addr(l), 2048, out_pad / 16, instr_desc(128, in_pad, bf16, 0, 1), false);
                if (leader) mma_commit(acc_bar);
                issue_gemm(leader, tmem + dw_col(l), dz, 2048, act_addr(l), 2048, kTileRows / 16, instr_desc(64, in_pad, bf16, 1, 1),
                           k > 0);
                if (leader) mma_commit(wg_bar[step & 1u]);
                __syncwarp();
                ++step;
                // Buffers of step l + 1 are free once its wgrad is done (committed one step ago).
                if (l < d) {
                    alive = wait_wgrad(step - 2);
                    if (!alive) break;
                    if (k + 1 < n_mine) {
                        if (l == d - 1) fetch(&x_map, act_addr(d), x_bar, k + 1);  // becomes the next tile's buffer 0
                        if (l == 0) fetch(&go_map, dz_base + static_cast<uint32_t>(zs ^ ((d - 1) & 1)) * kTileBytes, go_bar, k + 1);
                    }
                }
            }
            if (!alive) break;
            if (d == 0) {
                // a single layer: nothing above freed its buffers early; wait for this tile's wgrad, then fetch
                alive = wait_wgrad(step - 1);
                if (alive && k + 1 < n_mine) {
                    fetch(&x_map, smem_base, x_bar, k + 1);
                    fetch(&go_map, dz_base + static_cast<uint32_t>(zs) * kTileBytes, go_bar, k + 1);
                }
            } else {
                // the last step's wgrad: every commit is waited for exactly once, in order
                alive = wait_wgrad(step - 1);
                base = (base + d) % n_act;
                zs ^= (d - 1) & 1;
            }
            in_phase ^= 1u;
        }
    } else {
        // ================= epilogue threads =================
        const Seat seat;
        const uint32_t taddr = tmem + seat.lane_base;
        const uint32_t row_off = seat.row * 128, row_swizzle = (seat.row & 7) << 4;
        uint32_t acc_phase = 0;
        int base = 0, zs = 0;
        // wait for the accumulator: warp 0 polls, everybody meets at named barrier 1
        auto wait_acc = [&]() {
            if (warp == 0) {
                pipe_wait(acc_bar, acc_phase, &abort_flag);
                tc_fence_after();
                tc_fence_before();
            }
            acc_phase ^= 1u;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            tc_fence_after();
            return !*abort_now;
        };
        auto publish = [&]() {
            fence_async_smem();
            tc_fence_before();
            __syncwarp();  // one arrival per warp: arrivals on one mbarrier are serialised, a hundred of them cost a microsecond
            if ((threadIdx.x & 31) == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ready_bar) : "memory");
        };
        for (long long k = 0; k < n_mine; ++k) {
            const long long row0 = (first_tile + k * gridDim.x) * kTileRows;
            auto act_addr = [&](int l) { return smem_base + static_cast<uint32_t>((base + l) % n_act) * kTileBytes; };
            // ---- phase 1 ----
            for (int l = 0; l < d; ++l) {
                const bool ok1 = wait_acc();
                if (ok1) {
                    const int n = s.h / kGroups;  // this thread's columns
                    const uint32_t dst = act_addr(l + 1) + row_off;
                    const int first = seat.group * (n / 8);
                    for_each_piece(taddr + seat.group * n, n, [&](int u, const uint32_t(&piece)[8]) {
                        st_shared_16(dst + (((first + u) << 4) ^ row_swizzle), finish8<T, ACT, false>(piece, nullptr));
                    });
                }
                publish();
            }
            // ---- phase 2 ----
            for (int l = d; l >= 0; --l) {
                const int in_pad = l == 0 ? s.ki : s.h;
                const bool ok = wait_acc();
                const int n = in_pad / kGroups;
                const int first = seat.group * (n / 8);
                if (ok && l > 0) {
                    const uint32_t parked = act_addr(l) + row_off;
                    const uint32_t dst = dz_base + static_cast<uint32_t>(zs ^ ((d - l) & 1) ^ 1) * kTileBytes + row_off;
                    for_each_piece(taddr + seat.group * n, n, [&](int u, const uint32_t(&piece)[8]) {
                        const uint32_t off = ((first + u) << 4) ^ row_swizzle;
                        uint4 g = finish8<T, TH_ACT_NONE, false>(piece, nullptr);
                        if constexpr (ACT == TH_ACT_RELU) {
                            const uint4 a = ld_shared_16(parked + off);
                            g.x = keep_where_positive<T>(g.x, a.x);
                            g.y = keep_where_positive<T>(g.y, a.y);
                            g.z = keep_where_positive<T>(g.z, a.z);
                            g.w = keep_where_positive<T>(g.w, a.w);
                        }
                        st_shared_16(dst + off, g);
                    });
                } else if (ok && gx != nullptr) {
                    const bool live = row0 + seat.row < n_rows;
                    T *row_ptr = gx + (live ? row0 + seat.row : 0) * gx_stride;
                    for_each_piece(taddr + seat.group * n, n, [&](int u, const uint32_t(&piece)[8]) {
                        if (live) store_chunk_to_global<T>(row_ptr, first + u, s.d_in, finish8<T, TH_ACT_NONE, false>(piece, nullptr), gx_vec);
                    });
                }
                publish();
            }
            if (d > 0) {
                base = (base + d) % n_act;
                zs ^= (d - 1) & 1;
            }
        }
    }

    // ---- flush the weight gradients this CTA accumulated in TMEM ----
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (!abort_flag && n_mine > 0 && warp < 8) {
        const Seat seat;
        const MlpGradWorkspace W = grad_workspace_layout(s, workspace);
        for (int l = 0; l <= d; ++l) {
            const int in_pad = l == 0 ? s.ki : s.h;
            const int in_dim = l == 0 ? s.d_in : s.d_hid, out_dim = l == d ? s.d_out : s.d_hid;
            float *dst = W.base + (l == 0 ? W.w_in : (l == d ? W.w_out : W.w_hid + (l - 1) * s.d_hid * s.d_hid));
            flush_dw(tmem + seat.lane_base + dw_col(l), seat, in_pad, dst, out_dim, in_dim);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(static_cast<uint32_t>(P.tmem_cols)) : "memory");
}

// ---- backward, several row tiles per CTA -------------------------------------------------------------
//
// The two kernels above keep at most two row tiles per SM in flight (one per CTA), because every CTA holds
// its own weight-gradient accumulators (ki + depth x 64 TMEM columns) and depth + 3 operand tiles, and each
// tile is a chain of 2 depth + 1 short steps that are mostly latency.  Here ONE CTA per SM runs S independent
// SLOTS of 128 threads (thread = tile row = TMEM lane) plus one WGRAD warp:
//   * a slot's warp 0 issues the slot's recompute and dgrad MMAs into the slot's own 64 accumulator columns
//     (as in the forward kernel), so that chain never leaves the slot;
//   * the wgrad warp issues the weight-gradient MMAs of every slot.  MMAs of one thread execute in order, so
//     all slots accumulate into ONE shared set of TMEM columns instead of one set per tile in flight;
//   * dz of layer l - 1 is written in place over the parked input of layer l once both MMAs that read it have
//     finished, so a slot needs depth + 2 operand tiles;
//   * when features and output gradient are at most 32 wide, the output-gradient tile of a slot lives in
//     the logical chunks 4..7 of its feature tile (which uses chunks 0..3): depth + 1 tiles per slot.  The
//     output layer's wgrad then reads the whole feature tile as its A operand, and the real gradient rows
//     sit at rows 32.. of that layer's accumulator (rows 0..31 are products nobody reads).
// Per slot three mbarriers: `ready` (one arrival: the operands of the slot's next backward step are in place),
// `acc` (the slot's own MMAs of the step are done) and `wdone` (the step's wgrad is done).  The wgrad warp
// polls all `ready` barriers at once, one lane per slot, without blocking; a slot's warp 0 polls `acc` and
// `wdone`, its other warps park at the slot's named barrier.  Every wait is bounded by the global timer and
// watches the CTA's abort flag; after an abort everybody keeps the same barrier sequence without doing work.

struct BwdSlotPlan {
    int packed;          // the output gradient shares the feature tile
    int tiles_per_slot;
    int slots;
    int weights;         // byte offset of the weight tiles
    int total;           // dynamic shared memory without the alignment slack
    int tmem_cols;
    TcPlan w;            // weight offsets relative to `weights`
};

inline BwdSlotPlan bwd_slot_plan(const MlpShape &s, int slots) {
    BwdSlotPlan b{};
    b.packed = (s.ki <= 32 && s.no <= 32) ? 1 : 0;
    b.tiles_per_slot = s.depth + 1 + (b.packed ? 0 : 1);
    b.slots = slots;
    b.weights = slots * b.tiles_per_slot * kTileBytes;
    b.w = tc_plan(s, false, 0);
    b.total = b.weights + b.w.total;
    const int cols = slots * kAccCols + s.ki + s.depth * s.h;
    int alloc = 32;
    while (alloc < cols) alloc <<= 1;
    b.tmem_cols = alloc;
    return b;
}

struct BwdSlotBarriers {
    unsigned long long ready[kMaxSlots];
    unsigned long long acc[kMaxSlots];
    unsigned long long wdone[kMaxSlots];
};

// What the issuing warps need for one step of a tile, worked out once per CTA: both issue paths are on the
// critical chain of every tile, and each address or descriptor computed there is paid 2 depth + 1 times per tile.
struct __align__(16) SlotStep {
    uint32_t a_off;    // the slot's own GEMM: A operand, relative to the slot's first tile
    uint32_t b_addr;   //   B operand (a weight tile)
    uint32_t idesc;    //   instruction descriptor; 0 = the step has no GEMM of its own
    uint32_t k_steps;  //   bits 0..7: K steps of 16; bit 8: B is read MN-major
    uint32_t wa_off;   // weight gradient: A operand (dz, MN-major), relative to the slot's first tile
    uint32_t wb_off;   //   B operand (the layer's input, MN-major)
    uint32_t widesc;   //   instruction descriptor
    uint32_t dw_col;   //   accumulator column
};
constexpr int kMaxSlotSteps = 16;  // 2 depth + 1 steps; deeper networks do not fit two slots anyway

__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                 : "=r"(done)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return done != 0;
}

template <typename T, int ACT, int S>
__global__ void __launch_bounds__(128 * S + 32, 1)
mlp_bwd_slots_kernel(const MlpShape s, const MlpParams p, const __grid_constant__ WeightMaps maps, const int packed,
                     const T *__restrict__ x, long long x_stride, const T *__restrict__ go, long long go_stride,
                     T *__restrict__ gx, long long gx_stride, float *__restrict__ workspace, long long n_rows, int gx_vec) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint32_t tmem_holder;
    __shared__ int abort_flag;
    __shared__ __align__(8) unsigned long long wbar;
    __shared__ __align__(8) BwdSlotBarriers bars;
    __shared__ SlotStep steps[kMaxSlotSteps];
    constexpr int bf16 = std::is_same<T, __half>::value ? 0 : 1;
    const int d = s.depth;
    const int tiles_per_slot = d + 1 + (packed ? 0 : 1);
    const int weights_off = S * tiles_per_slot * kTileBytes;
    const TcPlan WP = tc_plan(s, false, 0);
    unsigned char *wsmem = smem + weights_off;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool is_wgrad_warp = warp == 4 * S;
    int dw_cols = S * kAccCols + s.ki + d * s.h, tmem_cols = 32;
    while (tmem_cols < dw_cols) tmem_cols <<= 1;
    volatile int *abort_now = &abort_flag;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < S; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars.ready[i])), "r"(1u) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars.acc[i])), "r"(1u) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&bars.wdone[i])), "r"(1u) : "memory");
        }
    }
    // operand tiles start out as zeros: columns a layer does not use are still read as MMA rows
    for (int e = threadIdx.x; e < weights_off / 16; e += blockDim.x) reinterpret_cast<uint4 *>(smem)[e] = make_uint4(0, 0, 0, 0);
    fence_async_smem();
    const bool weights_ok = tma_stage_weights(wsmem, WP, s, maps, &wbar);  // contains the barrier that publishes the inits
    if (is_wgrad_warp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_holder)),
                     "r"(static_cast<uint32_t>(tmem_cols))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (!weights_ok) {
        abort_flag = 1;
        g_tc_status = 1;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_holder;

    const long long n_tiles = (n_rows + kTileRows - 1) / kTileRows;
    const long long first_tile = blockIdx.x, tile_stride = gridDim.x;
    const long long n_mine = first_tile < n_tiles ? (n_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
    const uint32_t smem_base = smem_addr(smem);
    const uint32_t slot_bytes = static_cast<uint32_t>(tiles_per_slot) * kTileBytes;
    // the output gradient of a slot: its own tile, or logical chunks 4.. of the slot's feature tile
    const uint32_t go_off = packed ? 64u : static_cast<uint32_t>(d + 1) * kTileBytes;
    const int go_chunk0 = packed ? 4 : 0;
    const int n_steps = 2 * d + 1;  // steps 0 .. d - 1 recompute layers 0 .. d - 1, step j >= d is the backward step of layer 2 d - j
    auto dw_col = [&](int l) { return S * kAccCols + (l == 0 ? 0 : s.ki + (l - 1) * s.h); };
    if (static_cast<int>(threadIdx.x) < n_steps) {
        const int j = threadIdx.x;
        SlotStep st{};
        if (j < d) {
            st.a_off = static_cast<uint32_t>(j) * kTileBytes;
            st.b_addr = smem_addr(weight_tile(wsmem, WP, s, j));
            st.idesc = instr_desc(128, s.h, bf16, 0, 0);
            st.k_steps = static_cast<uint32_t>((j == 0 ? s.ki : s.h) / 16);
        } else {
            const int l = 2 * d - j;
            const int in_pad = l == 0 ? s.ki : s.h, out_pad = l == d ? s.no : s.h;
            const uint32_t dz_off = l == d ? go_off : static_cast<uint32_t>(l + 1) * kTileBytes;
            if (l > 0 || gx != nullptr) {
                st.a_off = dz_off;
                st.b_addr = smem_addr(weight_tile(wsmem, WP, s, l));
                st.idesc = instr_desc(128, in_pad, bf16, 0, 1);
                st.k_steps = static_cast<uint32_t>(out_pad / 16) | 256u;
            }
            st.wa_off = (l == d && packed) ? 0u : dz_off;  // packed output gradient: the whole feature tile is the A operand
            st.wb_off = static_cast<uint32_t>(l) * kTileBytes;
            st.widesc = instr_desc(64, in_pad, bf16, 1, 1);
            st.dw_col = static_cast<uint32_t>(dw_col(l));
        }
        steps[j] = st;
    }
    __syncthreads();

    if (is_wgrad_warp) {
        // ================= weight gradients of every slot =================
        // lane i < S keeps slot i's state: its next backward step, the tiles it still has, the parity to wait for
        int my_step = d;
        long long my_tiles = lane < S && lane < n_mine ? (n_mine - lane + S - 1) / S : 0;
        uint32_t my_parity = 0, dw_started = 0;
        const uint32_t my_bar = smem_addr(&bars.ready[lane < S ? lane : 0]);
        unsigned long long deadline = 0;
        unsigned idle = 0;
        const bool leader = elect_one();  // the same lane every time: MMAs of one thread execute in order
        while (__any_sync(0xffffffffu, my_tiles > 0)) {
            uint32_t mask = __ballot_sync(0xffffffffu, my_tiles > 0 && mbar_test(my_bar, my_parity));
            if (mask == 0) {
                if ((++idle & 63u) == 0) {
                    if (*abort_now) break;
                    const unsigned long long now = global_ns();
                    if (deadline == 0) deadline = now + kPipeWaitNs;
                    else if (now > deadline) {
                        *abort_now = 1;
                        g_tc_status = 1;
                        break;
                    }
                }
                continue;
            }
            idle = 0;
            deadline = 0;
            const bool mine = (mask >> lane) & 1u;
            tc_fence_after();
            while (mask) {
                const int i = __ffs(mask) - 1;
                mask &= mask - 1;
                const int j = __shfl_sync(0xffffffffu, my_step, i);
                const uint4 w = *reinterpret_cast<const uint4 *>(&steps[j].wa_off);
                const uint32_t tile0 = smem_base + static_cast<uint32_t>(i) * slot_bytes;
                issue_gemm(leader, tmem + w.w, tile0 + w.x, 2048, tile0 + w.y, 2048, kTileRows / 16, w.z, (dw_started >> (j - d)) & 1u);
                dw_started |= 1u << (j - d);
                if (leader) mma_commit(smem_addr(&bars.wdone[i]));
            }
            __syncwarp();
            if (mine) {
                my_parity ^= 1u;
                if (++my_step == n_steps) {
                    my_step = d;
                    --my_tiles;
                }
            }
        }
    } else {
        // ================= slots: loads, own MMAs, epilogues =================
        const int slot = warp >> 2, wq = warp & 3;
        const int row = threadIdx.x - slot * 128;
        const uint32_t acc = tmem + slot * kAccCols;
        const uint32_t taddr = acc + (static_cast<uint32_t>(32 * wq) << 16);
        const uint32_t acc_bar = smem_addr(&bars.acc[slot]), ready_bar = smem_addr(&bars.ready[slot]), wdone_bar = smem_addr(&bars.wdone[slot]);
        const uint32_t tile0 = smem_base + static_cast<uint32_t>(slot) * slot_bytes;
        auto act_addr = [&](int l) { return tile0 + static_cast<uint32_t>(l) * kTileBytes; };
        const uint32_t row_off = row * 128, row_swizzle = (row & 7) << 4;
        const int chunks_x = s.ki / 8, chunks_g = s.no / 8;
        uint32_t acc_phase = 0, wdone_phase = 0;
        const bool leader = wq == 0 && elect_one();
        // operands written -> the slot's warp 0 issues the step's own MMAs (and hands the wgrad to the wgrad warp)
        auto start_step = [&](int j) {
            fence_async_smem();
            tc_fence_before();
            slot_barrier(slot);
            if (wq == 0 && !*abort_now) {
                tc_fence_after();
                if (j >= d && leader) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ready_bar) : "memory");
                const uint4 own = *reinterpret_cast<const uint4 *>(&steps[j].a_off);
                if (own.z != 0) {
                    issue_gemm(leader, acc, tile0 + own.x, 32, own.y, (own.w & 256u) ? 2048 : 32, static_cast<int>(own.w & 255u), own.z, false);
                    if (leader) mma_commit(acc_bar);
                }
                __syncwarp();
            }
        };
        auto finish_step = [&](bool own, bool wgrad) {
            if (wq == 0) {
                if (own) pipe_wait(acc_bar, acc_phase, &abort_flag);
                if (wgrad) pipe_wait(wdone_bar, wdone_phase, &abort_flag);
                tc_fence_after();
                tc_fence_before();
            }
            if (own) acc_phase ^= 1u;
            if (wgrad) wdone_phase ^= 1u;
            slot_barrier(slot);
            tc_fence_after();
            return !*abort_now;
        };
        for (long long k = slot; k < n_mine; k += S) {
            const long long row0 = (first_tile + k * tile_stride) * kTileRows;
            if (!*abort_now) {
                for (int id = row; id < kTileRows * chunks_x; id += 128) {
                    const int r = id / chunks_x, c = id - r * chunks_x;
                    const long long grow = row0 + r;
                    const bool inside = grow < n_rows && 8 * c < s.d_in;
                    const T *src = inside ? x + grow * x_stride + 8 * c : x;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(tile0 + r * 128 + ((c ^ (r & 7)) << 4)), "l"(src), "r"(inside ? 16 : 0) : "memory");
                }
                const uint32_t go_tile = packed ? tile0 : act_addr(d + 1);
                for (int id = row; id < kTileRows * chunks_g; id += 128) {
                    const int r = id / chunks_g, c = id - r * chunks_g;
                    const long long grow = row0 + r;
                    const bool inside = grow < n_rows && 8 * c < s.d_out;
                    const T *src = inside ? go + grow * go_stride + 8 * c : go;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(go_tile + r * 128 + (((go_chunk0 + c) ^ (r & 7)) << 4)), "l"(src), "r"(inside ? 16 : 0) : "memory");
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
                async_tile_wait();
            }
            for (int l = 0; l < d; ++l) {  // recomputed activation of layer l -> input tile of layer l + 1
                start_step(l);
                if (finish_step(true, false)) {
                    const uint32_t dst = act_addr(l + 1) + row_off;
                    drain_row<T, ACT, false>(taddr, s.h, nullptr, [&](int chunk, uint4 packed_v) { st_shared_16(dst + ((chunk << 4) ^ row_swizzle), packed_v); });
                }
            }
            for (int l = d; l >= 0; --l) {
                const int in_pad = l == 0 ? s.ki : s.h;
                const bool own = l > 0 || gx != nullptr;
                start_step(2 * d - l);
                const bool ok = finish_step(own, true);
                if (l > 0) {
                    if (ok) {  // dz of the layer below = dy * act'(its parked output), in place over that output
                        const uint32_t parked = act_addr(l) + row_off;
                        drain_row<T, TH_ACT_NONE, false>(taddr, in_pad, nullptr, [&](int chunk, uint4 gq) {
                            const uint32_t off = (chunk << 4) ^ row_swizzle;
                            if constexpr (ACT == TH_ACT_RELU) {
                                const uint4 a = ld_shared_16(parked + off);
                                gq.x = keep_where_positive<T>(gq.x, a.x);
                                gq.y = keep_where_positive<T>(gq.y, a.y);
                                gq.z = keep_where_positive<T>(gq.z, a.z);
                                gq.w = keep_where_positive<T>(gq.w, a.w);
                            }
                            st_shared_16(parked + off, gq);
                        });
                    }
                } else if (ok && gx != nullptr) {
                    const bool live = row0 + row < n_rows;
                    T *row_ptr = gx + (live ? row0 + row : 0) * gx_stride;
                    drain_row<T, TH_ACT_NONE, false>(taddr, in_pad, nullptr, [&](int chunk, uint4 packed_v) {
                        if (live && 8 * chunk < in_pad) store_chunk_to_global<T>(row_ptr, chunk, s.d_in, packed_v, gx_vec);
                    });
                    tc_fence_before();
                }
            }
        }
    }

    // ---- flush the weight gradients (slot 0's threads; M = 64 layout: lanes 0..15 of warp w hold rows 16 w ..) ----
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (!abort_flag && n_mine > 0 && threadIdx.x < 128) {
        const MlpGradWorkspace W = grad_workspace_layout(s, workspace);
        const int wq = warp & 3;
        const uint32_t lane_base = static_cast<uint32_t>(32 * wq) << 16;
        for (int l = 0; l <= d; ++l) {
            const int in_pad = l == 0 ? s.ki : s.h;
            const int in_dim = l == 0 ? s.d_in : s.d_hid, out_dim = l == d ? s.d_out : s.d_hid;
            float *dst = W.base + (l == 0 ? W.w_in : (l == d ? W.w_out : W.w_hid + (l - 1) * s.d_hid * s.d_hid));
            const int o = 16 * wq + lane - ((l == d && packed) ? 32 : 0);  // output row this lane holds
            for (int first = 0; first < in_pad; first += 16) {
                uint32_t raw[32];
                tmem_ld16(tmem + lane_base + dw_col(l) + first, raw);
                tmem_ld_wait();
                if (lane < 16 && o >= 0 && o < out_dim) {
#pragma unroll
                    for (int c = 0; c < 16; ++c)
                        if (first + c < in_dim) atomicAdd(dst + o * in_dim + first + c, __uint_as_float(raw[c]));
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (is_wgrad_warp)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(static_cast<uint32_t>(tmem_cols)) : "memory");
}

bool pipe_disabled() {
    static const bool off = [] {
        const char *v = getenv("TH_MLP_NO_PIPE");
        return v && v[0] == '1';
    }();
    return off;
}

bool tmem_a_enabled() {
    static const bool on = [] {
        const char *v = getenv("TH_MLP_NO_TMEM_A");
        return !(v && v[0] == '1');
    }();
    return on;
}

template <typename T, int ACT, bool BIAS, int S, bool MSE, bool TA>
int launch_fwd_pipe(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
                    int64_t rows, cudaStream_t stream, const MseArgs &mse = MseArgs{}) {
    const TcPlan P = tc_plan(s, false, 2 * S);
    const int smem = P.total + 1024;
    if (smem > kSmemBudget || pipe_disabled()) return kTcNotApplicable;
    if (rows >= (1ll << 31) - kTileRows) return kTcNotApplicable;  // TMA coordinates are 32-bit
    WeightMaps maps;
    CUtensorMap x_map;
    if (!make_weight_maps(maps, s, p)) return kTcNotApplicable;
    if (!make_map(&x_map, x, rows, s.d_in, kTileRows, x_stride)) return kTcNotApplicable;
    if (S * (kAccCols + (TA ? 32 : 0)) > 512) return kTcNotApplicable;
    auto kernel = mlp_fwd_pipe_kernel<T, ACT, BIAS, S, MSE, TA>;
    if (int rc = cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                             "cudaFuncSetAttribute(mlp_fwd_pipe_kernel)")) return rc;
    const long long tiles = (rows + kTileRows - 1) / kTileRows;
    const long long cap = sm_count();
    kernel<<<static_cast<unsigned>(tiles < cap ? tiles : cap), 128 * S, smem, stream>>>(
        s, p, maps, x_map, static_cast<T *>(y), y_stride, rows, y ? rows_vector_ok(y, y_stride, s.d_out) : 0, mse);
    return launch_status("mlp_fwd_pipe_kernel launch");
}

// Slots per CTA, measured (2^21 rows, 32-64-64-16, with the loss; 2^20 rows, 32-4x64-16):
//   activations through shared memory: 3 slots 0.136 ms, 4: 0.122 / 0.083, 5: 0.127 / 0.098, 6: 0.153 - MMA operand reads and
//     epilogue stores share the SM's shared-memory bandwidth, and beyond four tiles in flight they only queue up;
//   activations through tensor memory: 3 slots 0.128 / 0.088, 4: 0.104 / 0.069, 5: 0.092 / 0.064 - five slots x 96 columns are
//     what tensor memory holds.
// TH_MLP_SLOTS=n lowers the cap (0 = never), TH_MLP_NO_TMEM_A=1 keeps the activations in shared memory.
template <typename T, int ACT, bool BIAS, bool MSE>
int launch_fwd_slots(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
                     int64_t rows, cudaStream_t stream, const MseArgs &mse) {
    static const int cap = [] {
        const char *v = getenv("TH_MLP_SLOTS");
        return v ? atoi(v) : 5;
    }();
    int rc = kTcNotApplicable;
    if (tmem_a_enabled()) {
        if (cap >= 5) rc = launch_fwd_pipe<T, ACT, BIAS, 5, MSE, true>(s, p, x, x_stride, y, y_stride, rows, stream, mse);
        if (rc == kTcNotApplicable && cap >= 4) rc = launch_fwd_pipe<T, ACT, BIAS, 4, MSE, true>(s, p, x, x_stride, y, y_stride, rows, stream, mse);
        if (rc == kTcNotApplicable && cap >= 3) rc = launch_fwd_pipe<T, ACT, BIAS, 3, MSE, true>(s, p, x, x_stride, y, y_stride, rows, stream, mse);
        return rc;
    }
    if (cap >= 4) rc = launch_fwd_pipe<T, ACT, BIAS, 4, MSE, false>(s, p, x, x_stride, y, y_stride, rows, stream, mse);
    if (rc == kTcNotApplicable && cap >= 3) rc = launch_fwd_pipe<T, ACT, BIAS, 3, MSE, false>(s, p, x, x_stride, y, y_stride, rows, stream, mse);
    return rc;
}

template <typename T, int ACT, bool BIAS>
int launch_fwd_t(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
                 int64_t rows, cudaStream_t stream) {
    {
        const int rc = launch_fwd_slots<T, ACT, BIAS, false>(s, p, x, x_stride, y, y_stride, rows, stream, MseArgs{});
        if (rc != kTcNotApplicable) return rc;
    }
    const TcPlan P = tc_plan(s, false);
    int ctas = 0;
    const int smem = occupancy_plan(P, &ctas);
    if (ctas < 1) return kTcNotApplicable;
    auto kernel = mlp_fwd_tc_kernel<T, ACT, BIAS>;
    if (int rc = cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                             "cudaFuncSetAttribute(mlp_fwd_tc_kernel)")) return rc;
    const long long tiles = (rows + kTileRows - 1) / kTileRows;
    const long long cap = static_cast<long long>(sm_count()) * ctas;
    WeightMaps maps;
    const int use_tma = make_weight_maps(maps, s, p);
    kernel<<<static_cast<unsigned>(tiles < cap ? tiles : cap), kTcThreads, smem, stream>>>(
        s, p, maps, use_tma, static_cast<const T *>(x), x_stride, static_cast<T *>(y), y_stride, rows,
        rows_vector_ok(x, x_stride, s.d_in), rows_vector_ok(y, y_stride, s.d_out));
    return launch_status("mlp_fwd_tc_kernel launch");
}

template <typename T, bool BIAS>
int launch_fwd_act(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
                   int64_t rows, cudaStream_t stream) {
    switch (s.act) {
        case TH_ACT_RELU: return launch_fwd_t<T, TH_ACT_RELU, BIAS>(s, p, x, x_stride, y, y_stride, rows, stream);
        case TH_ACT_SILU: return launch_fwd_t<T, TH_ACT_SILU, BIAS>(s, p, x, x_stride, y, y_stride, rows, stream);
        case TH_ACT_RELU2: return launch_fwd_t<T, TH_ACT_RELU2, BIAS>(s, p, x, x_stride, y, y_stride, rows, stream);
        default: return launch_fwd_t<T, TH_ACT_NONE, BIAS>(s, p, x, x_stride, y, y_stride, rows, stream);
    }
}

template <typename T>
int launch_fwd(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
               int64_t rows, cudaStream_t stream) {
    return s.has_bias ? launch_fwd_act<T, true>(s, p, x, x_stride, y, y_stride, rows, stream)
                      : launch_fwd_act<T, false>(s, p, x, x_stride, y, y_stride, rows, stream);
}

template <typename T, int ACT>
int launch_bwd_pipe(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, const void *go, int64_t go_stride,
                    void *gx, int64_t gx_stride, float *workspace, int64_t rows, cudaStream_t stream) {
    if (pipe_disabled() || rows >= (1ll << 31) - kTileRows) return kTcNotApplicable;
    const TcPlan P = tc_plan(s, true);
    if (P.tmem_cols > 512) return kTcNotApplicable;
    int ctas = 0;
    const int smem = occupancy_plan(P, &ctas);
    // With a single CTA per SM (deep networks: depth + 3 operand tiles) one row tile is in flight and the
    // extra barrier round trips between issuer and epilogue cost more than the overlap gains (2^20 rows,
    // 32-64x4-16: 0.534 ms against 0.494 ms for the kernel above); with two CTAs it is 0.378 against 0.470
    // (2^21 rows, 32-64-64-16).
    if (ctas < 2) return kTcNotApplicable;
    if (ctas > 2) ctas = 2;  // the kernel is compiled for two CTAs of 288 threads per SM
    WeightMaps maps;
    CUtensorMap x_map, go_map;
    if (!make_weight_maps(maps, s, p)) return kTcNotApplicable;
    if (!make_map(&x_map, x, rows, s.d_in, kTileRows, x_stride)) return kTcNotApplicable;
    if (!make_map(&go_map, go, rows, s.d_out, kTileRows, go_stride)) return kTcNotApplicable;
    auto kernel = mlp_bwd_pipe_kernel<T, ACT>;
    if (int rc = cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                             "cudaFuncSetAttribute(mlp_bwd_pipe_kernel)")) return rc;
    const long long tiles = (rows + kTileRows - 1) / kTileRows;
    const long long cap = static_cast<long long>(sm_count()) * ctas;
    kernel<<<static_cast<unsigned>(tiles < cap ? tiles : cap), kTcThreads + 32, smem, stream>>>(
        s, p, maps, x_map, go_map, static_cast<T *>(gx), gx_stride, workspace, rows, gx ? rows_vector_ok(gx, gx_stride, s.d_in) : 0);
    return launch_status("mlp_bwd_pipe_kernel launch");
}

bool slots_disabled() {
    static const bool off = [] {
        const char *v = getenv("TH_MLP_NO_SLOTS");
        return v && v[0] == '1';
    }();
    return off;
}

// Slots that fit one SM: shared memory for their tiles next to the weights, tensor memory for their
// accumulators next to the shared weight-gradient columns.
template <typename T, int ACT, int S>
int launch_bwd_slots_n(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, const void *go, int64_t go_stride,
                       void *gx, int64_t gx_stride, float *workspace, int64_t rows, cudaStream_t stream) {
    const BwdSlotPlan B = bwd_slot_plan(s, S);
    int smem = B.total + 1024;
    if (smem + 1024 > kSmemBudget || B.tmem_cols > 512 || 2 * s.depth + 1 > kMaxSlotSteps) return kTcNotApplicable;
    if (smem < kSmemBudget / 2 + 1024) smem = kSmemBudget / 2 + 1024;  // one CTA per SM
    WeightMaps maps;
    if (!make_weight_maps(maps, s, p)) return kTcNotApplicable;
    auto kernel = mlp_bwd_slots_kernel<T, ACT, S>;
    if (int rc = cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                             "cudaFuncSetAttribute(mlp_bwd_slots_kernel)")) return rc;
    const long long tiles = (rows + kTileRows - 1) / kTileRows;
    const long long want = (tiles + S - 1) / S;
    const long long cap = sm_count();
    kernel<<<static_cast<unsigned>(want < cap ? want : cap), 128 * S + 32, smem, stream>>>(
        s, p, maps, B.packed, static_cast<const T *>(x), x_stride, static_cast<const T *>(go), go_stride, static_cast<T *>(gx), gx_stride,
        workspace, rows, gx ? rows_vector_ok(gx, gx_stride, s.d_in) : 0);
    return launch_status("mlp_bwd_slots_kernel launch");
}

template <typename T, int ACT>
int launch_bwd_slots(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, const void *go, int64_t go_stride,
                     void *gx, int64_t gx_stride, float *workspace, int64_t rows, cudaStream_t stream) {
    if (pipe_disabled() || slots_disabled()) return kTcNotApplicable;
    // rows must move as whole 16-byte chunks (cp.async)
    if (!rows_vector_ok(x, x_stride, s.d_in) || !rows_vector_ok(go, go_stride, s.d_out)) return kTcNotApplicable;
    int rc = launch_bwd_slots_n<T, ACT, 4>(s, p, x, x_stride, go, go_stride, gx, gx_stride, workspace, rows, stream);
    if (rc == kTcNotApplicable) rc = launch_bwd_slots_n<T, ACT, 3>(s, p, x, x_stride, go, go_stride, gx, gx_stride, workspace, rows, stream);
    if (rc == kTcNotApplicable) rc = launch_bwd_slots_n<T, ACT, 2>(s, p, x, x_stride, go, go_stride, gx, gx_stride, workspace, rows, stream);
    return rc;
}

template <typename T, int ACT, bool BIAS>
int launch_bwd_t(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, const void *go, int64_t go_stride,
                 void *gx, int64_t gx_stride, float *workspace, int64_t rows, cudaStream_t stream) {
    // the issuer-warp kernel is built for bias-free networks whose activation derivative needs no pre-activation
    if constexpr (!BIAS && (ACT == TH_ACT_RELU || ACT == TH_ACT_NONE)) {
        int rc = launch_bwd_slots<T, ACT>(s, p, x, x_stride, go, go_stride, gx, gx_stride, workspace, rows, stream);
        if (rc != kTcNotApplicable) return rc;
        rc = launch_bwd_pipe<T, ACT>(s, p, x, x_stride, go, go_stride, gx, gx_stride, workspace, rows, stream);
        if (rc != kTcNotApplicable) return rc;
    }
    const TcPlan P = tc_plan(s, true);
    if (P.tmem_cols > 512) return kTcNotApplicable;
    int ctas = 0;
    const int smem = occupancy_plan(P, &ctas);
    if (ctas < 1) return kTcNotApplicable;
    // one CTA per SM (shared memory bound): let it keep its prefetched tiles in registers
    auto kernel = ctas >= 2 ? mlp_bwd_tc_kernel<T, ACT, 2, BIAS> : mlp_bwd_tc_kernel<T, ACT, 1, BIAS>;
    if (int rc = cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                             "cudaFuncSetAttribute(mlp_bwd_tc_kernel)")) return rc;
    const long long tiles = (rows + kTileRows - 1) / kTileRows;
    const long long cap = static_cast<long long>(sm_count()) * ctas;
    WeightMaps maps;
    const int use_tma = make_weight_maps(maps, s, p);
    kernel<<<static_cast<unsigned>(tiles < cap ? tiles : cap), kTcThreads, smem, stream>>>(
        s, p, maps, use_tma, static_cast<const T *>(x), x_stride, static_cast<const T *>(go), go_stride, static_cast<T *>(gx), gx_stride,
        workspace, rows, rows_vector_ok(x, x_stride, s.d_in), rows_vector_ok(go, go_stride, s.d_out),
        gx ? rows_vector_ok(gx, gx_stride, s.d_in) : 0);
    return launch_status("mlp_bwd_tc_kernel launch");
}

template <typename T>
int launch_bwd(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, const void *go, int64_t go_stride,
               void *gx, int64_t gx_stride, float *workspace, int64_t rows, cudaStream_t stream) {
#define TH_BWD_ACT(A)                                                                                                   \
    (s.has_bias ? launch_bwd_t<T, A, true>(s, p, x, x_stride, go, go_stride, gx, gx_stride, workspace, rows, stream)    \
                : launch_bwd_t<T, A, false>(s, p, x, x_stride, go, go_stride, gx, gx_stride, workspace, rows, stream))
    switch (s.act) {
        case TH_ACT_RELU: return TH_BWD_ACT(TH_ACT_RELU);
        case TH_ACT_SILU: return TH_BWD_ACT(TH_ACT_SILU);
        case TH_ACT_RELU2: return TH_BWD_ACT(TH_ACT_RELU2);
        default: return TH_BWD_ACT(TH_ACT_NONE);
    }
#undef TH_BWD_ACT
}

// ---- forward with the fused MSE epilogue: only the multi-slot kernel has it ----

template <typename T, bool BIAS>
int launch_fwd_mse_act(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
                       const MseArgs &mse, int64_t rows, cudaStream_t stream) {
    switch (s.act) {
        case TH_ACT_RELU: return launch_fwd_slots<T, TH_ACT_RELU, BIAS, true>(s, p, x, x_stride, y, y_stride, rows, stream, mse);
        case TH_ACT_SILU: return launch_fwd_slots<T, TH_ACT_SILU, BIAS, true>(s, p, x, x_stride, y, y_stride, rows, stream, mse);
        case TH_ACT_RELU2: return launch_fwd_slots<T, TH_ACT_RELU2, BIAS, true>(s, p, x, x_stride, y, y_stride, rows, stream, mse);
        default: return launch_fwd_slots<T, TH_ACT_NONE, BIAS, true>(s, p, x, x_stride, y, y_stride, rows, stream, mse);
    }
}

template <typename T>
int launch_fwd_mse(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
                   const MseArgs &mse, int64_t rows, cudaStream_t stream) {
    return s.has_bias ? launch_fwd_mse_act<T, true>(s, p, x, x_stride, y, y_stride, mse, rows, stream)
                      : launch_fwd_mse_act<T, false>(s, p, x, x_stride, y, y_stride, mse, rows, stream);
}

}  // namespace

int mlp_fwd_mse_tc(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
                   const MseArgs &mse, int64_t rows, int dtype, cudaStream_t stream) {
    if (tc_disabled() || rows <= 0) return kTcNotApplicable;
    if (s.h != 16 && s.h != 32 && s.h != 64) return kTcNotApplicable;
    // whole 16-byte chunks of every row: prediction (if kept), target and gradient
    if (s.d_out % 8 != 0 || !rows_vector_ok(mse.target, mse.target_stride, s.d_out) ||
        !rows_vector_ok(mse.grad, mse.grad_stride, s.d_out) || (y && !rows_vector_ok(y, y_stride, s.d_out)))
        return kTcNotApplicable;
    switch (dtype) {
        case TH_F16: return launch_fwd_mse<__half>(s, p, x, x_stride, y, y_stride, mse, rows, stream);
        case TH_BF16: return launch_fwd_mse<__nv_bfloat16>(s, p, x, x_stride, y, y_stride, mse, rows, stream);
        default: return kTcNotApplicable;
    }
}

int mlp_fwd_tc(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
               int64_t rows, int dtype, cudaStream_t stream) {
    if (tc_disabled() || rows <= 0) return kTcNotApplicable;
    if (s.h != 16 && s.h != 32 && s.h != 64) return kTcNotApplicable;
    switch (dtype) {
        case TH_F16: return launch_fwd<__half>(s, p, x, x_stride, y, y_stride, rows, stream);
        case TH_BF16: return launch_fwd<__nv_bfloat16>(s, p, x, x_stride, y, y_stride, rows, stream);
        default: return kTcNotApplicable;
    }
}

int mlp_bwd_tc(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, const void *go, int64_t go_stride,
               void *gx, int64_t gx_stride, float *workspace, int64_t rows, int dtype, cudaStream_t stream) {
    if (tc_disabled() || rows <= 0) return kTcNotApplicable;
    if (s.h != 16 && s.h != 32 && s.h != 64) return kTcNotApplicable;
    switch (dtype) {
        case TH_F16: return launch_bwd<__half>(s, p, x, x_stride, go, go_stride, gx, gx_stride, workspace, rows, stream);
        case TH_BF16: return launch_bwd<__nv_bfloat16>(s, p, x, x_stride, go, go_stride, gx, gx_stride, workspace, rows, stream);
        default: return kTcNotApplicable;
    }
}

}  // namespace th


// 1 when tensor maps can be built in this process (the driver exposes cuTensorMapEncodeTiled), i.e.
// when the tensor-core MLP kernels load their weights by TMA; 0 when they fall back to plain loads.
extern "C" int th_mlp_tma_available(void) { return th::encode_tiled_fn() != nullptr ? 1 : 0; }

namespace th {
int field_tc_status_word();  // neural_field.cu: the fused encoding + MLP kernels' copy of the status word
}

// Device-side status of the tcgen05 kernels: 0 = fine, non-zero = a bounded wait ran out.  Synchronises.
extern "C" int th_mlp_tc_status(void) {
    int status = 0;
    if (cudaMemcpyFromSymbol(&status, th::g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    const int field = th::field_tc_status_word();
    if (field < 0) return -1;
    return status | ((field & 1) << 1);
}
