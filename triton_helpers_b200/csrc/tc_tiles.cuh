// Building blocks shared by the tcgen05 kernels (fused MLP, reversible MLP): PTX wrappers for
// tcgen05 / TMEM / mbarrier, the one shared-memory operand-tile layout, packed 16-bit epilogue
// arithmetic, and the CTA set-up / tear-down around a TMEM allocation.
//
// Operand-tile layout: 128 rows x 128 bytes (64 16-bit features), 16-byte chunk c of row r at chunk
// position c ^ (r & 7), tile base 1024-byte aligned: the tensor core's canonical 128-byte-swizzle
// layout.  The same bytes serve as a K-major operand (row = M or N index, features = K: descriptor
// start address advances 32 B per 16-deep K step) and as an MN-major operand (row = K index,
// features = M or N: start address advances 2048 B per K step).
//
// Thread organisation: 256 threads; warp w owns TMEM lanes 32 * (w % 4) .. + 31 (thread = lane =
// tile row) and the column half w / 4; accumulators are read in 8-column pieces, one piece = one
// 16-byte chunk of an operand tile.
//
// Everything here has internal linkage: each translation unit gets its own copy, including its own
// device-side status word.
#pragma once

#include "mma_tiles.cuh"

#include <cuda.h>  // CUtensorMap and its enums only; the driver entry point is looked up at run time

#include <mutex>

namespace th {
namespace {

constexpr int kGroups = 2;                    // column halves of a row, one per warpgroup
constexpr int kTcThreads = 128 * kGroups;
constexpr int kMaxChunks = 8 / kGroups;       // 16-byte chunks (8 columns) per thread at the widest layer
constexpr int kTileRows = 128;
constexpr int kTileBytes = kTileRows * 128;  // one operand tile: 128 rows x 128 B
constexpr int kSmemBudget = 227 * 1024;
constexpr int kWaitPolls = 1 << 20;

__device__ int g_tc_status = 0;  // 0 = fine, 1 = an mbarrier wait ran out

// ---- PTX wrappers ------------------------------------------------------------------------------

// Shared-memory matrix descriptor = {low word, high word}.  High word (constant for every tile here):
// SBO 1024 B (8 rows of 128 B), descriptor version 1, layout type 2 = 128-byte swizzle.  Low word:
// start address >> 4 in bits 0..13, LBO 0 (one 128-byte atom along the contiguous dimension).
constexpr uint32_t kDescHigh = (1024u >> 4) | (1u << 14) | (2u << 29);

__device__ __forceinline__ uint32_t desc_low(uint32_t addr) { return (addr >> 4) & 0x3fffu; }

__device__ __forceinline__ uint64_t smem_desc(uint32_t low) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(low), "r"(kDescHigh));
    return d;
}

// kind::f16 instruction descriptor: fp32 accumulate, A/B format 0 = f16 / 1 = bf16
__host__ __device__ constexpr uint32_t instr_desc(int m, int n, int bf16, int a_mn_major, int b_mn_major) {
    return (1u << 4) | (static_cast<uint32_t>(bf16) << 7) | (static_cast<uint32_t>(bf16) << 10) |
           (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// One lane of a converged warp.  MMAs are issued from warp-uniform code (all of warp 0 computes the
// descriptors, one elected lane executes the instruction) so the descriptors live in uniform
// registers, which is where tcgen05.mma takes them from.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}\n" : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ void mma_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar) : "memory");
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Waits for the given phase of the barrier; gives up after kWaitPolls polls.
__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity) {
    uint32_t done = 0;
    for (int poll = 0; poll < kWaitPolls && !done; ++poll) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(done)
            : "r"(mbar), "r"(parity)
            : "memory");
    }
    return done != 0;
}

// CTA-wide wait for the MMAs committed to `mbar`: only warp 0 polls the mbarrier (bounded); the other
// warps park at the CTA barrier, which costs no issue slots while they wait.  Returns false (for
// every thread alike) when the wait ran out; `abort_flag` lives in shared memory.
__device__ __forceinline__ bool cta_wait_mma(uint32_t mbar, uint32_t &phase, int *abort_flag) {
    if (threadIdx.x < 32) {
        if (!mbar_wait(mbar, phase)) *abort_flag = 1;
        tc_fence_after();
        tc_fence_before();
    }
    phase ^= 1;
    __syncthreads();
    tc_fence_after();
    return *abort_flag == 0;
}

// 8 consecutive accumulator columns of this thread's lane
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 8 consecutive columns of this thread's lane, register -> TMEM (complete after tmem_st_wait)
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(v[0]), "r"(v[1]),
                 "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// A 16-byte chunk of 16-bit values -> 8 fp32 bit patterns
template <typename T>
__device__ __forceinline__ void widen_chunk(uint4 packed, uint32_t (&out)[8]) {
    const uint32_t w[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 f = unpack_pair<T>(w[k]);
        out[2 * k] = __float_as_uint(f.x);
        out[2 * k + 1] = __float_as_uint(f.y);
    }
}

// This thread's `count` (<= kMaxChunks) 8-column pieces starting at piece `first`, all in flight together.
__device__ __forceinline__ void load_pieces(uint32_t taddr, int first, int count, uint32_t (&raw)[kMaxChunks][8]) {
#pragma unroll
    for (int u = 0; u < kMaxChunks; ++u)
        if (u < count) tmem_ld8(taddr + 8 * (first + u), raw[u]);
    tmem_ld_wait();
}

// ---- packed 16-bit arithmetic --------------------------------------------------------------------

template <typename T>
__device__ __forceinline__ uint32_t relu_pair(uint32_t v);
template <>
__device__ __forceinline__ uint32_t relu_pair<__half>(uint32_t v) {
    const __half2 r = __hmax2(*reinterpret_cast<const __half2 *>(&v), __float2half2_rn(0.f));
    return *reinterpret_cast<const uint32_t *>(&r);
}
template <>
__device__ __forceinline__ uint32_t relu_pair<__nv_bfloat16>(uint32_t v) {
    const __nv_bfloat162 r = __hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&v), __float2bfloat162_rn(0.f));
    return *reinterpret_cast<const uint32_t *>(&r);
}

// keep each 16-bit half of `grad` where the matching half of `post` is > 0
template <typename T>
__device__ __forceinline__ uint32_t keep_where_positive(uint32_t grad, uint32_t post);
template <>
__device__ __forceinline__ uint32_t keep_where_positive<__half>(uint32_t grad, uint32_t post) {
    return grad & __hgt2_mask(*reinterpret_cast<const __half2 *>(&post), __float2half2_rn(0.f));
}
template <>
__device__ __forceinline__ uint32_t keep_where_positive<__nv_bfloat16>(uint32_t grad, uint32_t post) {
    return grad & __hgt2_mask(*reinterpret_cast<const __nv_bfloat162 *>(&post), __float2bfloat162_rn(0.f));
}

// 8 fp32 accumulator columns (+ bias) -> activation -> one 16-byte chunk of 16-bit values
template <typename T, int ACT, bool BIAS>
__device__ __forceinline__ uint4 finish_piece(const uint32_t (&raw)[8], const float *bias8) {
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = __uint_as_float(raw[k]);
    if constexpr (BIAS) {
        const float4 b0 = *reinterpret_cast<const float4 *>(bias8), b1 = *reinterpret_cast<const float4 *>(bias8 + 4);
        v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
        v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
    }
    if constexpr (ACT == TH_ACT_SILU || ACT == TH_ACT_RELU2) {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = activate(ACT, v[k]);
    }
    uint32_t w[4] = {pack_pair<T>(v[0], v[1]), pack_pair<T>(v[2], v[3]), pack_pair<T>(v[4], v[5]), pack_pair<T>(v[6], v[7])};
    if constexpr (ACT == TH_ACT_RELU) {
        // round, then clamp: the same value as clamp, then round
#pragma unroll
        for (int k = 0; k < 4; ++k) w[k] = relu_pair<T>(w[k]);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---- lean epilogue pieces: 32 columns per TMEM load, fused convert + ReLU, 32-bit shared addresses ----

// 32 consecutive accumulator columns of this thread's lane in one instruction
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

// two fp32 -> one packed 16-bit pair (lo in the low half), rounding to nearest even, with ReLU fused
// into the conversion (negative results become +0; the same values as round-then-clamp)
template <typename T>
__device__ __forceinline__ uint32_t pack_pair_relu(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack_pair_relu<__half>(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.relu.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
template <>
__device__ __forceinline__ uint32_t pack_pair_relu<__nv_bfloat16>(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.relu.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

__device__ __forceinline__ void st_shared_16(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ uint4 ld_shared_16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

// N (8, 16, 24 or 32) consecutive accumulator columns of this thread's lane, then `fn(u, eight values)`
// for each 8-column piece u; everything is sized at compile time so the values stay in registers.
__device__ __forceinline__ void tmem_ld8_at(uint32_t taddr, uint32_t *r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

template <int N, typename Fn>
__device__ __forceinline__ void for_each_piece_n(uint32_t taddr, Fn fn) {
    uint32_t raw[32];
    if constexpr (N == 32) {
        tmem_ld32(taddr, raw);
    } else if constexpr (N == 24) {
        tmem_ld16(taddr, raw);
        tmem_ld8_at(taddr + 16, raw + 16);
    } else if constexpr (N == 16) {
        tmem_ld16(taddr, raw);
    } else {
        tmem_ld8_at(taddr, raw);
    }
    tmem_ld_wait();
#pragma unroll
    for (int u = 0; u < N / 8; ++u) {
        const uint32_t piece[8] = {raw[8 * u], raw[8 * u + 1], raw[8 * u + 2], raw[8 * u + 3],
                                   raw[8 * u + 4], raw[8 * u + 5], raw[8 * u + 6], raw[8 * u + 7]};
        fn(u, piece);
    }
}
// the same for a run-time n in {8, 16, 24, 32} (warp uniform; padded widths are multiples of 16 and
// two threads share a row)
template <typename Fn>
__device__ __forceinline__ void for_each_piece(uint32_t taddr, int n, Fn fn) {
    if (n == 32) for_each_piece_n<32>(taddr, fn);
    else if (n == 24) for_each_piece_n<24>(taddr, fn);
    else if (n == 16) for_each_piece_n<16>(taddr, fn);
    else for_each_piece_n<8>(taddr, fn);
}

// 8 fp32 accumulator columns (+ bias) -> activation -> one 16-byte chunk; the ReLU-without-bias case
// is four instructions
template <typename T, int ACT, bool BIAS>
__device__ __forceinline__ uint4 finish8(const uint32_t *raw, const float *bias8) {
    if constexpr (ACT == TH_ACT_RELU) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = __uint_as_float(raw[k]);
        if constexpr (BIAS) {
            const float4 b0 = *reinterpret_cast<const float4 *>(bias8), b1 = *reinterpret_cast<const float4 *>(bias8 + 4);
            v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
            v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
        }
        return make_uint4(pack_pair_relu<T>(v[0], v[1]), pack_pair_relu<T>(v[2], v[3]), pack_pair_relu<T>(v[4], v[5]),
                          pack_pair_relu<T>(v[6], v[7]));
    } else {
        uint32_t r8[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) r8[k] = raw[k];
        return finish_piece<T, ACT, BIAS>(r8, bias8);
    }
}

// ---- operand tiles -----------------------------------------------------------------------------

__device__ __forceinline__ unsigned char *chunk_ptr(unsigned char *tile, int row, int chunk) {
    return tile + row * 128 + ((chunk ^ (row & 7)) << 4);
}

__device__ __forceinline__ uint4 gather8(const unsigned short *p, int first_col, int cols) {
    unsigned short e[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) e[k] = (first_col + k < cols) ? p[k] : static_cast<unsigned short>(0);
    return make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
}

// Rows [row0, row0 + 128) x cols [0, cols) of a row-major global matrix -> operand tile, zero padded
// to `pad_cols`, in two steps so the global loads of the NEXT tile can be in flight while the
// current one is computed: fetch_tile pulls this thread's 16-byte chunks into registers (coalesced:
// consecutive threads fetch consecutive chunks), commit_tile writes them to their swizzled places.
constexpr int kFetchIters = kTileRows * 8 / kTcThreads;
struct TileRegs {
    uint4 v[kFetchIters];
};

template <typename T>
__device__ __forceinline__ void fetch_tile(TileRegs &t, const T *src, long long stride, long long row0, long long n_rows,
                                           int cols, int pad_cols, bool vector_ok) {
    const int chunks = pad_cols / 8;
    const int total = kTileRows * chunks;
#pragma unroll
    for (int it = 0; it < kFetchIters; ++it) {
        const int id = it * kTcThreads + threadIdx.x;
        t.v[it] = make_uint4(0, 0, 0, 0);
        if (id < total) {
            const int r = id / chunks, c = id - r * chunks;
            const long long row = row0 + r;
            if (row < n_rows && 8 * c < cols) {
                const T *p = src + row * stride + 8 * c;
                t.v[it] = vector_ok ? __ldcs(reinterpret_cast<const uint4 *>(p))
                                    : gather8(reinterpret_cast<const unsigned short *>(p), 8 * c, cols);
            }
        }
    }
}

// The same copy with cp.async: global -> swizzled shared memory without passing through registers
// (rows past the end and padding columns are zero-filled by a zero source size).  Needs the
// 16-byte-aligned layout (`vector_ok`); completion is awaited with async_tile_wait().
template <typename T>
__device__ __forceinline__ void async_tile_load(unsigned char *tile, const T *src, long long stride, long long row0,
                                                long long n_rows, int cols, int pad_cols) {
    const int chunks = pad_cols / 8;
    const int total = kTileRows * chunks;
#pragma unroll
    for (int it = 0; it < kFetchIters; ++it) {
        const int id = it * kTcThreads + threadIdx.x;
        if (id < total) {
            const int r = id / chunks, c = id - r * chunks;
            const long long row = row0 + r;
            const bool inside = row < n_rows && 8 * c < cols;
            const T *p = inside ? src + row * stride + 8 * c : src;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(chunk_ptr(tile, r, c))), "l"(p),
                         "r"(inside ? 16 : 0)
                         : "memory");
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void async_tile_wait() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void commit_tile(unsigned char *tile, const TileRegs &t, int pad_cols) {
    const int chunks = pad_cols / 8;
    const int total = kTileRows * chunks;
#pragma unroll
    for (int it = 0; it < kFetchIters; ++it) {
        const int id = it * kTcThreads + threadIdx.x;
        if (id < total) {
            const int r = id / chunks, c = id - r * chunks;
            *reinterpret_cast<uint4 *>(chunk_ptr(tile, r, c)) = t.v[it];
        }
    }
}

// A weight matrix [rows][cols] (row-major, contiguous) -> operand tile [rows_pad][cols_pad], zero padded.
template <typename T>
__device__ __forceinline__ void stage_weight_tile(unsigned char *tile, const T *w, int rows, int cols, int rows_pad,
                                                  int cols_pad) {
    const int chunks = cols_pad / 8;
    const bool vector_ok = (cols % 8 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    for (int id = threadIdx.x; id < rows_pad * chunks; id += kTcThreads) {
        const int r = id / chunks, c = id - r * chunks;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows && 8 * c < cols) {
            const T *p = w + r * cols + 8 * c;
            v = vector_ok ? *reinterpret_cast<const uint4 *>(p) : gather8(reinterpret_cast<const unsigned short *>(p), 8 * c, cols);
        }
        *reinterpret_cast<uint4 *>(chunk_ptr(tile, r, c)) = v;
    }
}

// One 16-byte chunk (8 values) of this thread's row -> row-major global matrix
template <typename T>
__device__ __forceinline__ void store_chunk_to_global(T *row_ptr, int chunk, int cols, uint4 packed, bool vector_ok) {
    if (8 * chunk >= cols) return;
    if (vector_ok) {
        __stcs(reinterpret_cast<uint4 *>(row_ptr + 8 * chunk), packed);
    } else {
        const uint32_t w[4] = {packed.x, packed.y, packed.z, packed.w};
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (8 * chunk + k < cols)
                reinterpret_cast<unsigned short *>(row_ptr)[8 * chunk + k] = static_cast<unsigned short>(w[k >> 1] >> (16 * (k & 1)));
    }
}

// TMEM allocation by warp 0, mbarrier init by thread 0, then a CTA-wide hand-over.
__device__ __forceinline__ uint32_t cta_setup(uint32_t *tmem_holder, unsigned long long *mbar, uint32_t cols) {
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_holder)),
                     "r"(cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(mbar)), "r"(1u) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    return *tmem_holder;
}

__device__ __forceinline__ void cta_teardown(uint32_t tmem, uint32_t cols) {
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(cols) : "memory");
}

// Issue the K-loop of one GEMM; called by all of warp 0, `leader` marks the elected lane.
// a_step / b_step: bytes the operand's start address advances per 16-deep K step (32 for a K-major
// operand, 2048 for an MN-major one).
__device__ __forceinline__ void issue_gemm(bool leader, uint32_t tmem_d, uint32_t a_addr, uint32_t a_step, uint32_t b_addr,
                                           uint32_t b_step, int k_steps, uint32_t idesc, bool accumulate) {
    uint32_t a_low = desc_low(a_addr), b_low = desc_low(b_addr);
    uint32_t acc = accumulate ? 1u : 0u;
    for (int k = 0; k < k_steps; ++k) {
        if (leader) mma_f16(tmem_d, smem_desc(a_low), smem_desc(b_low), idesc, acc);
        a_low += a_step >> 4;
        b_low += b_step >> 4;
        acc = 1u;
    }
}

// A-operand in tensor memory: [d] += [a_tmem] * b(smem).  Row i of A sits in lane i, two consecutive K elements per
// 32-bit column, so a 16-deep K step is 8 columns.
__device__ __forceinline__ void mma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void issue_gemm_ta(bool leader, uint32_t tmem_d, uint32_t tmem_a, uint32_t b_addr, uint32_t b_step, int k_steps,
                                              uint32_t idesc, bool accumulate) {
    uint32_t b_low = desc_low(b_addr);
    for (int k = 0; k < k_steps; ++k) {
        if (leader) mma_f16_ta(tmem_d, tmem_a + 8 * k, smem_desc(b_low), idesc, (accumulate || k > 0) ? 1u : 0u);
        b_low += b_step >> 4;
    }
}

__device__ __forceinline__ void tmem_st4(uint32_t taddr, uint4 v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Which rows / columns a thread looks after: TMEM lanes 32 * (warp % 4) .. + 31, column half warp / 4.
struct Seat {
    int row;            // tile row = TMEM lane
    int group;          // column half
    uint32_t lane_base; // lane field of the TMEM address
    __device__ Seat() {
        const int warp = threadIdx.x >> 5;
        row = 32 * (warp & 3) + (threadIdx.x & 31);
        group = warp >> 2;
        lane_base = static_cast<uint32_t>(32 * (warp & 3)) << 16;
    }
};

// ---- TMA: tensor maps (host) and the 2-D tile load (device) -------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver-entry-point lookup (no link against libcuda).
EncodeTiledFn encode_tiled_fn() {
    static std::mutex guard;
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    std::lock_guard<std::mutex> lock(guard);
    if (!tried) {
        tried = true;
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) == cudaSuccess &&
            status == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// One map per weight array: [rows][cols] 16-bit row-major, box = 64 columns x box_rows rows.
bool make_map(CUtensorMap *map, const void *base, long long rows, int cols, int box_rows, long long row_stride = 0) {
    EncodeTiledFn encode = encode_tiled_fn();
    if (row_stride == 0) row_stride = cols;
    if (!encode || !base || cols % 8 != 0 || row_stride % 8 != 0 || !aligned_to(base, 16)) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_stride) * 2};
    const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void *>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// One box of `map` at element coordinates (x, y) into shared memory, completion counted on `mbar`.
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int x, int y, uint32_t mbar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_addr(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(mbar)
        : "memory");
}

}  // namespace
}  // namespace th
