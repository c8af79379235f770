// Pieces of the tcgen05 fused-MLP kernels shared by fused_mlp_tc.cu and the kernels that fuse the MLP
// with the hash encoding (neural_field.cu): the shared-memory plan of a CTA (operand tiles, weight tiles,
// biases), weight staging by TMA or plain loads, the per-layer epilogues between accumulator and operand
// tile, the weight-gradient flush, and the host-side helpers around tensor maps and occupancy.
// Internal linkage throughout (one copy per translation unit, including the status word of tc_tiles.cuh).
#pragma once

#include "mlp_shape.cuh"
#include "tc_tiles.cuh"

#include <cstdlib>
#include <cstring>
#include <type_traits>

namespace th {
namespace {

constexpr int kAccCols = 64;  // TMEM columns of the forward / dgrad accumulator

// ---- shared-memory plan ------------------------------------------------------------------------

struct TcPlan {
    int act_tiles;      // operand tiles for activations (2 forward, depth + 1 backward)
    int dz_tiles;       // 0 forward, 2 backward
    int ones_tile;      // backward with biases: one tile of ones, the B operand that turns dz into its column sums
    int db_col;         // backward with biases: first TMEM column of the bias-gradient accumulators (16 per layer)
    int z_col;          // backward with SiLU / ReLU^2: TMEM column of the recomputed pre-activation (64 columns)
    int w_offset[3];    // byte offsets of W_in, W_hid[0], W_out tiles (after the activation / dz tiles)
    int w_hid_each;
    int bias_offset;    // fp32 [(depth + 1)][64]
    int total;          // bytes, excluding the 1 KB alignment slack
    int tmem_cols;      // power of two >= 32
};

__host__ __device__ inline TcPlan tc_plan(const MlpShape &s, bool backward, int forward_tiles = 2) {
    TcPlan p{};
    p.act_tiles = backward ? s.depth + 1 : forward_tiles;  // forward: two tiles per row tile in flight, alternating, so the next input can stream in
    p.dz_tiles = backward ? 2 : 0;
    p.ones_tile = backward && s.has_bias ? 1 : 0;
    int off = (p.act_tiles + p.dz_tiles + p.ones_tile) * kTileBytes;
    p.w_offset[0] = off;
    off += s.h * 128;
    p.w_offset[1] = off;
    p.w_hid_each = s.h * 128;
    off += (s.depth - 1) * p.w_hid_each;
    p.w_offset[2] = off;
    off += s.no * 128;
    p.bias_offset = off;
    off += (s.depth + 1) * kMaxDim * 4;
    p.total = off;
    int cols = kAccCols;
    if (backward) cols += s.ki + s.depth * s.h;  // one accumulator of in_pad columns per layer
    p.db_col = cols;
    if (backward && s.has_bias) cols += 16 * (s.depth + 1);
    p.z_col = cols;
    if (backward && (s.act == TH_ACT_SILU || s.act == TH_ACT_RELU2)) cols += kAccCols;
    int alloc = 32;
    while (alloc < cols) alloc <<= 1;
    p.tmem_cols = alloc;
    return p;
}

__device__ __forceinline__ unsigned char *weight_tile(unsigned char *smem, const TcPlan &P, const MlpShape &s, int l) {
    if (l == 0) return smem + P.w_offset[0];
    if (l == s.depth) return smem + P.w_offset[2];
    return smem + P.w_offset[1] + (l - 1) * P.w_hid_each;
}

// Tensor maps of the three weight arrays (see make_weight_maps): 2-D, 16-bit elements, box = 64
// columns x one layer's rows, 128-byte swizzle, zero fill outside the array.  A TMA box lands in
// shared memory exactly in the operand-tile layout (row pitch 128 B, chunk ^ (row & 7)).
struct WeightMaps {
    CUtensorMap w_in, w_hid, w_out;
};

// All weight tiles of the network by TMA: thread 0 arms the barrier with the byte count and issues
// one box per layer; everybody waits (bounded) for the bytes to land.  Returns false on a timeout.
__device__ bool tma_stage_weights(unsigned char *smem, const TcPlan &P, const MlpShape &s, const WeightMaps &maps,
                                  unsigned long long *wbar) {
    const uint32_t bar = smem_addr(wbar);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(1u) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t bytes = static_cast<uint32_t>((s.h + (s.depth - 1) * s.h + s.no) * 128);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
        tma_load_2d(smem + P.w_offset[0], &maps.w_in, 0, 0, bar);
        for (int i = 0; i < s.depth - 1; ++i) tma_load_2d(smem + P.w_offset[1] + i * P.w_hid_each, &maps.w_hid, 0, i * s.d_hid, bar);
        tma_load_2d(smem + P.w_offset[2], &maps.w_out, 0, 0, bar);
    }
    return mbar_wait(bar, 0);
}

template <typename T>
__device__ void stage_biases(unsigned char *smem, const TcPlan &P, const MlpShape &s, const MlpParams &p) {
    float *bias = reinterpret_cast<float *>(smem + P.bias_offset);
    for (int e = threadIdx.x; e < (s.depth + 1) * kMaxDim; e += kTcThreads) {
        const int layer = e / kMaxDim, c = e % kMaxDim;
        float v = 0.f;
        if (s.has_bias) {
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

// Weights without TMA (inner dimension not a multiple of 8 elements, or a misaligned pointer): plain
// loads and swizzled stores by all threads.
template <typename T>
__device__ void stage_all_weights(unsigned char *smem, const TcPlan &P, const MlpShape &s, const MlpParams &p) {
    stage_weight_tile<T>(smem + P.w_offset[0], static_cast<const T *>(p.w_in), s.d_hid, s.d_in, s.h, s.ki);
    for (int i = 0; i < s.depth - 1; ++i)
        stage_weight_tile<T>(smem + P.w_offset[1] + i * P.w_hid_each,
                             static_cast<const T *>(p.w_hid) + static_cast<size_t>(i) * s.d_hid * s.d_hid, s.d_hid,
                             s.d_hid, s.h, s.h);
    stage_weight_tile<T>(smem + P.w_offset[2], static_cast<const T *>(p.w_out), s.d_out, s.d_hid, s.no, s.h);
}

// ---- epilogues: forward ------------------------------------------------------------------------

// A hidden layer's accumulator -> bias, activation, rounding -> this thread's chunks of the next operand tile
template <typename T, int ACT, bool BIAS>
__device__ __forceinline__ void hidden_epilogue(uint32_t taddr, const Seat &seat, int pad, const float *bias,
                                                unsigned char *next_tile) {
    const int n = pad / kGroups, first = seat.group * (n / 8);  // this thread's columns / first 8-column piece
    const uint32_t row_addr = smem_addr(next_tile) + seat.row * 128, row_swizzle = (seat.row & 7) << 4;
    for_each_piece(taddr + seat.group * n, n, [&](int u, const uint32_t(&piece)[8]) {
        st_shared_16(row_addr + (((first + u) << 4) ^ row_swizzle), finish8<T, ACT, BIAS>(piece, bias + 8 * (first + u)));
    });
}

template <typename T, bool BIAS>
__device__ __forceinline__ void output_epilogue(uint32_t taddr, const Seat &seat, int pad, const float *bias, T *row_ptr,
                                                int cols, bool live, bool vector_ok) {
    const int n = pad / kGroups, first = seat.group * (n / 8);
    for_each_piece(taddr + seat.group * n, n, [&](int u, const uint32_t(&piece)[8]) {
        if (live)
            store_chunk_to_global<T>(row_ptr, first + u, cols, finish8<T, TH_ACT_NONE, BIAS>(piece, bias + 8 * (first + u)), vector_ok);
    });
}

template <typename T, int ACT, bool BIAS, typename Sink>
__device__ __forceinline__ void drain_row(uint32_t taddr, int out_pad, const float *bias, Sink sink) {
    uint32_t raw[32];
    if (out_pad == 16) {
        tmem_ld16(taddr, raw);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 2; ++u) sink(u, finish8<T, ACT, BIAS>(raw + 8 * u, bias + 8 * u));
        return;
    }
    for (int first = 0; first < out_pad; first += 32) {
        tmem_ld32(taddr + first, raw);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 4; ++u) sink(first / 8 + u, finish8<T, ACT, BIAS>(raw + 8 * u, bias + first + 8 * u));
    }
}

// One 16-byte chunk of a prediction row against the same chunk of the target row: the scaled difference
// (rounded to T) and the sum of the eight squared differences.
template <typename T>
__device__ __forceinline__ uint4 mse_chunk(uint4 pred, uint4 target, float grad_scale, float &loss) {
    const uint32_t pw[4] = {pred.x, pred.y, pred.z, pred.w}, tw[4] = {target.x, target.y, target.z, target.w};
    uint32_t gw[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 a = unpack_pair<T>(pw[k]), b = unpack_pair<T>(tw[k]);
        const float d0 = a.x - b.x, d1 = a.y - b.y;
        loss += d0 * d0 + d1 * d1;
        gw[k] = pack_pair<T>(d0 * grad_scale, d1 * grad_scale);
    }
    return make_uint4(gw[0], gw[1], gw[2], gw[3]);
}

// ---- epilogues: backward -----------------------------------------------------------------------

// Epilogue of a dgrad: dz of the layer below = dy * act'(that layer's parked output), rounded.
template <typename T, int ACT>
__device__ __forceinline__ void dz_epilogue(uint32_t taddr, const Seat &seat, int pad, unsigned char *parked,
                                            unsigned char *dz_tile) {
    const int n = pad / kGroups, first = seat.group * (n / 8);
    const uint32_t row_off = seat.row * 128, row_swizzle = (seat.row & 7) << 4;
    const uint32_t parked_row = smem_addr(parked) + row_off, dz_row = smem_addr(dz_tile) + row_off;
    for_each_piece(taddr + seat.group * n, n, [&](int u, const uint32_t(&piece)[8]) {
        const uint32_t off = ((first + u) << 4) ^ row_swizzle;
        uint4 g = finish8<T, TH_ACT_NONE, false>(piece, nullptr);
        if constexpr (ACT == TH_ACT_RELU) {
            const uint4 a = ld_shared_16(parked_row + off);
            g.x = keep_where_positive<T>(g.x, a.x);
            g.y = keep_where_positive<T>(g.y, a.y);
            g.z = keep_where_positive<T>(g.z, a.z);
            g.w = keep_where_positive<T>(g.w, a.w);
        }
        st_shared_16(dz_row + off, g);
    });
}

template <typename T>
__device__ __forceinline__ void dx_epilogue(uint32_t taddr, const Seat &seat, int pad, T *row_ptr, int cols, bool live,
                                            bool vector_ok) {
    const int n = pad / kGroups, first = seat.group * (n / 8);
    for_each_piece(taddr + seat.group * n, n, [&](int u, const uint32_t(&piece)[8]) {
        if (live) store_chunk_to_global<T>(row_ptr, first + u, cols, finish8<T, TH_ACT_NONE, false>(piece, nullptr), vector_ok);
    });
}

// Flush one layer's weight-gradient accumulator (M = 64 layout: gradient row m sits in TMEM lane
// 32 * (m / 16) + m % 16, so lanes 0..15 of a warp's 32 carry rows 16 * (warp % 4) .. + 15).
__device__ __forceinline__ void flush_dw(uint32_t taddr, const Seat &seat, int pad, float *dst, int out_dim, int in_dim) {
    const int count = pad / (8 * kGroups), first = seat.group * count;
    uint32_t raw[kMaxChunks][8];
    load_pieces(taddr, first, count, raw);
    const int lane = threadIdx.x & 31;
    const int m = 16 * ((threadIdx.x >> 5) & 3) + lane;
    if (lane < 16 && m < out_dim) {
#pragma unroll
        for (int u = 0; u < kMaxChunks; ++u)
            if (u < count)
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int c = 8 * (first + u) + k;
                    if (c < in_dim) atomicAdd(dst + m * in_dim + c, __uint_as_float(raw[u][k]));
                }
    }
}

// ---- host side ---------------------------------------------------------------------------------

bool rows_vector_ok(const void *p, int64_t stride, int cols) {
    return cols % 8 == 0 && stride % 8 == 0 && aligned_to(p, 16);
}

// CTAs per SM so that (a) shared memory fits and (b) the CTAs on one SM never need more than 512
// TMEM columns; returns the dynamic shared-memory size to request (padded to enforce (b)).
int occupancy_plan(const TcPlan &P, int *ctas_per_sm) {
    const int need = P.total + 1024;  // alignment slack
    int by_smem = kSmemBudget / need;
    const int by_tmem = 512 / P.tmem_cols;
    int ctas = by_smem < by_tmem ? by_smem : by_tmem;
    if (ctas > 8) ctas = 8;
    *ctas_per_sm = ctas;
    if (ctas < 1) return need;
    // the smallest request for which ctas + 1 CTAs no longer fit
    const int floor_bytes = kSmemBudget / (ctas + 1) + 1;
    return need > floor_bytes ? need : floor_bytes;
}

// ---- tensor maps for the weights ---------------------------------------------------------------

// Returns 1 when all three maps could be built (then the kernels load the weights by TMA), else 0.
int make_weight_maps(WeightMaps &maps, const MlpShape &s, const MlpParams &p) {
    memset(&maps, 0, sizeof(maps));
    static const bool off = [] {
        const char *v = getenv("TH_MLP_NO_TMA");
        return v && v[0] == '1';
    }();
    if (off) return 0;
    if (!make_map(&maps.w_in, p.w_in, s.d_hid, s.d_in, s.h)) return 0;
    if (s.depth > 1) {
        if (!make_map(&maps.w_hid, p.w_hid, (s.depth - 1) * s.d_hid, s.d_hid, s.h)) return 0;
    } else {
        maps.w_hid = maps.w_in;  // never used
    }
    if (!make_map(&maps.w_out, p.w_out, s.d_out, s.d_hid, s.no)) return 0;
    return 1;
}

bool tc_disabled() {
    static const bool off = [] {
        const char *v = getenv("TH_MLP_LEGACY");
        return v && v[0] == '1';
    }();
    return off;
}

// The pipelined kernel needs TMA for the weights and for the input rows, and enough shared memory
// for two operand tiles per slot; anything else goes to the one-tile-per-CTA kernel below.

}  // namespace
}  // namespace th
