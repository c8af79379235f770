// Fully fused MLP on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM).
//
// One CTA of 128 threads owns a 128-row tile at a time (M = 128 = the TMEM lanes); several CTAs
// share an SM, so one CTA's epilogue overlaps another's MMAs.  Every operand tile lives in
// shared memory in ONE layout: rows 128 bytes apart (64 16-bit features), 16-byte chunk c of
// row r stored at chunk position c ^ (r & 7), tile base 1024-byte aligned.  That is the
// canonical 128-byte-swizzle layout of the tensor core, and the same bytes can be described
// to it two ways:
//   K-major  (the row index is M or N, features are K)  - forward GEMMs, the A side of dgrad;
//   MN-major (the row index is K, features are M or N)  - wgrad (K = the tile's 128 rows) and
//            the weight side of dgrad (K = a layer's outputs, N = its inputs),
// so neither activations nor weights are ever transposed or stored twice.
//
//   forward : ACC[128 x out] = ACT_l[128 x in] . W_l^T        A K-major, B K-major
//   dgrad   : ACC[128 x in]  = DZ_l[128 x out] . W_l          A K-major, B MN-major
//   wgrad   : DW_l[out x in] += DZ_l^T[out x 128] . ACT_l     A, B MN-major, M = 64
//
// Thread 0 issues the MMAs and commits them to an mbarrier; all 128 threads wait on it,
// read their row of the accumulator with tcgen05.ld (thread = TMEM lane = tile row), apply
// bias / activation / ReLU mask in registers and write the next operand tile straight back
// to shared memory (fence.proxy.async before the tensor core reads it).  Weight gradients
// stay in TMEM columns for the whole life of the CTA (wgrad MMAs accumulate tile after tile
// and are never waited on individually) and leave once, at the end, as red.global.add.f32.
//
// Every wait is bounded: a stuck mbarrier sets a device-side status word and the CTA frees its
// TMEM and returns.  tcgen05.alloc cannot block for good because the launcher sizes shared
// memory so that the CTAs resident on one SM never ask for more than its 512 TMEM columns.
#include "mlp_shape.cuh"
#include "mma_tiles.cuh"

#include <cstdlib>
#include <type_traits>

namespace th {
namespace {

constexpr int kTcThreads = 128;
constexpr int kTileRows = 128;
constexpr int kTileBytes = kTileRows * 128;  // one operand tile: 128 rows x 128 B
constexpr int kAccCols = 64;                 // TMEM columns of the forward / dgrad accumulator
constexpr int kSmemBudget = 227 * 1024;
constexpr int kWaitPolls = 1 << 22;

__device__ int g_tc_status = 0;  // 0 = fine, 1 = an mbarrier wait ran out

// ---- PTX wrappers ------------------------------------------------------------------------------

__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    // start address, LBO 0 (one 128-byte atom along the contiguous dimension), SBO 1024 B (8 rows),
    // descriptor version 1, layout type 2 = 128-byte swizzle
    return static_cast<uint64_t>((addr >> 4) & 0x3fff) | (static_cast<uint64_t>(1024 >> 4) << 32) |
           (static_cast<uint64_t>(1) << 46) | (static_cast<uint64_t>(2) << 61);
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

// 16 consecutive accumulator columns of this thread's lane
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// COLS (16, 32, 48 or 64) accumulator columns of this thread's row, as floats
template <int COLS>
__device__ __forceinline__ void load_acc_row(uint32_t taddr, float (&v)[COLS]) {
    uint32_t raw[COLS / 16][16];
#pragma unroll
    for (int c = 0; c < COLS / 16; ++c) tmem_ld16(taddr + 16 * c, raw[c]);
    tmem_ld_wait();
#pragma unroll
    for (int c = 0; c < COLS; ++c) v[c] = __uint_as_float(raw[c / 16][c % 16]);
}

// ---- operand tiles -----------------------------------------------------------------------------

__device__ __forceinline__ unsigned char *chunk_ptr(unsigned char *tile, int row, int chunk) {
    return tile + row * 128 + ((chunk ^ (row & 7)) << 4);
}

// Rows [row0, row0 + 128) x cols [0, cols) of a row-major global matrix -> operand tile, zero padded
// to `pad_cols`.  Coalesced: consecutive threads fetch consecutive 16-byte chunks.
template <typename T>
__device__ __forceinline__ void load_tile(unsigned char *tile, const T *src, long long stride, long long row0,
                                          long long n_rows, int cols, int pad_cols, bool vector_ok) {
    const int chunks = pad_cols / 8;
    for (int id = threadIdx.x; id < kTileRows * chunks; id += kTcThreads) {
        const int r = id / chunks, c = id - r * chunks;
        const long long row = row0 + r;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < n_rows) {
            const T *p = src + row * stride + 8 * c;
            if (vector_ok) {
                if (8 * c < cols) v = __ldcs(reinterpret_cast<const uint4 *>(p));
            } else {
                unsigned short e[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) e[k] = (8 * c + k < cols) ? reinterpret_cast<const unsigned short *>(p)[k] : 0;
                v = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
            }
        }
        *reinterpret_cast<uint4 *>(chunk_ptr(tile, r, c)) = v;
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
        if (r < rows) {
            const T *p = w + r * cols + 8 * c;
            if (vector_ok) {
                if (8 * c < cols) v = *reinterpret_cast<const uint4 *>(p);
            } else {
                unsigned short e[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) e[k] = (8 * c + k < cols) ? reinterpret_cast<const unsigned short *>(p)[k] : 0;
                v = make_uint4(e[0] | (e[1] << 16), e[2] | (e[3] << 16), e[4] | (e[5] << 16), e[6] | (e[7] << 16));
            }
        }
        *reinterpret_cast<uint4 *>(chunk_ptr(tile, r, c)) = v;
    }
}

// This thread's row (COLS floats) -> 16-bit, into its row of an operand tile
template <typename T, int COLS>
__device__ __forceinline__ void store_row_to_tile(unsigned char *tile, int row, const float (&v)[COLS]) {
#pragma unroll
    for (int c = 0; c < COLS / 8; ++c) {
        const uint4 packed = make_uint4(pack_pair<T>(v[8 * c], v[8 * c + 1]), pack_pair<T>(v[8 * c + 2], v[8 * c + 3]),
                                        pack_pair<T>(v[8 * c + 4], v[8 * c + 5]), pack_pair<T>(v[8 * c + 6], v[8 * c + 7]));
        *reinterpret_cast<uint4 *>(chunk_ptr(tile, row, c)) = packed;
    }
}

// This thread's row (COLS floats) -> 16-bit, to a row-major global matrix
template <typename T, int COLS>
__device__ __forceinline__ void store_row_to_global(T *dst, int cols, const float (&v)[COLS], bool vector_ok) {
    if (vector_ok) {
#pragma unroll
        for (int c = 0; c < COLS / 8; ++c) {
            if (8 * c < cols) {
                const uint4 packed = make_uint4(pack_pair<T>(v[8 * c], v[8 * c + 1]), pack_pair<T>(v[8 * c + 2], v[8 * c + 3]),
                                                pack_pair<T>(v[8 * c + 4], v[8 * c + 5]), pack_pair<T>(v[8 * c + 6], v[8 * c + 7]));
                __stcs(reinterpret_cast<uint4 *>(dst + 8 * c), packed);
            }
        }
    } else {
#pragma unroll
        for (int c = 0; c < COLS; ++c)
            if (c < cols) dst[c] = from_float<T>(v[c]);
    }
}

// ---- shared-memory plan ------------------------------------------------------------------------

struct TcPlan {
    int act_tiles;      // operand tiles for activations (1 forward, depth + 1 backward)
    int dz_tiles;       // 0 forward, 2 backward
    int w_offset[3];    // byte offsets of W_in, W_hid[0], W_out tiles (after the activation / dz tiles)
    int w_hid_each;
    int bias_offset;    // fp32 [(depth + 1)][64]
    int total;          // bytes, excluding the 1 KB alignment slack
    int tmem_cols;      // power of two >= 32
};

__host__ __device__ inline TcPlan tc_plan(const MlpShape &s, bool backward) {
    TcPlan p{};
    p.act_tiles = backward ? s.depth + 1 : 1;
    p.dz_tiles = backward ? 2 : 0;
    int off = (p.act_tiles + p.dz_tiles) * kTileBytes;
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

template <typename T>
__device__ void stage_all_weights(unsigned char *smem, const TcPlan &P, const MlpShape &s, const MlpParams &p) {
    stage_weight_tile<T>(smem + P.w_offset[0], static_cast<const T *>(p.w_in), s.d_hid, s.d_in, s.h, s.ki);
    for (int i = 0; i < s.depth - 1; ++i)
        stage_weight_tile<T>(smem + P.w_offset[1] + i * P.w_hid_each,
                             static_cast<const T *>(p.w_hid) + static_cast<size_t>(i) * s.d_hid * s.d_hid, s.d_hid,
                             s.d_hid, s.h, s.h);
    stage_weight_tile<T>(smem + P.w_offset[2], static_cast<const T *>(p.w_out), s.d_out, s.d_hid, s.no, s.h);
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

// Issue (thread 0 only) the K-loop of one GEMM.  a_step / b_step: bytes the operand's start address
// advances per 16-deep K step (32 for a K-major operand, 2048 for an MN-major one).
__device__ __forceinline__ void issue_gemm(uint32_t tmem_d, uint32_t a_addr, uint32_t a_step, uint32_t b_addr,
                                           uint32_t b_step, int k_steps, uint32_t idesc, bool accumulate) {
    for (int k = 0; k < k_steps; ++k)
        mma_f16(tmem_d, smem_desc(a_addr + k * a_step), smem_desc(b_addr + k * b_step), idesc, (accumulate || k > 0) ? 1u : 0u);
}

// bias + activation on this thread's accumulator row
template <int COLS>
__device__ __forceinline__ void bias_act(float (&v)[COLS], const float *bias, int act) {
#pragma unroll
    for (int c = 0; c < COLS; ++c) v[c] = activate(act, v[c] + bias[c]);
}

// ---- forward -----------------------------------------------------------------------------------

template <typename T, int COLS>
__device__ __forceinline__ void fwd_epilogue(uint32_t taddr, const float *bias, int act, unsigned char *next_tile,
                                             int row) {
    float v[COLS];
    load_acc_row<COLS>(taddr, v);
    bias_act<COLS>(v, bias, act);
    store_row_to_tile<T, COLS>(next_tile, row, v);
}

template <typename T, int COLS>
__device__ __forceinline__ void fwd_output(uint32_t taddr, const float *bias, T *dst, int cols, bool live, bool vector_ok) {
    float v[COLS];
    load_acc_row<COLS>(taddr, v);
    bias_act<COLS>(v, bias, TH_ACT_NONE);
    if (live) store_row_to_global<T, COLS>(dst, cols, v, vector_ok);
}

template <typename T>
__global__ void __launch_bounds__(kTcThreads)
mlp_fwd_tc_kernel(const MlpShape s, const MlpParams p, const T *__restrict__ x, long long x_stride, T *__restrict__ y,
                  long long y_stride, long long n_rows, int x_vec, int y_vec) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint32_t tmem_holder;
    __shared__ __align__(8) unsigned long long mbar;
    __shared__ int abort_flag;
    const TcPlan P = tc_plan(s, false);
    constexpr int bf16 = sizeof(T) == 2 && !std::is_same<T, __half>::value;

    if (threadIdx.x == 0) abort_flag = 0;
    stage_all_weights<T>(smem, P, s, p);
    const uint32_t tmem = cta_setup(&tmem_holder, &mbar, P.tmem_cols);
    const uint32_t bar = smem_addr(&mbar);
    const float *bias = reinterpret_cast<const float *>(smem + P.bias_offset);
    unsigned char *act_tile = smem;
    const uint32_t act_addr = smem_addr(act_tile);
    const int row = threadIdx.x;
    const uint32_t taddr = tmem + (static_cast<uint32_t>(row & ~31) << 16);  // this warp's 32 lanes
    uint32_t phase = 0;
    const long long n_tiles = (n_rows + kTileRows - 1) / kTileRows;

    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const long long row0 = tile * kTileRows;
        load_tile<T>(act_tile, x, x_stride, row0, n_rows, s.d_in, s.ki, x_vec);
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (abort_flag) break;
        for (int l = 0; l <= s.depth; ++l) {
            const int in_pad = l == 0 ? s.ki : s.h;
            const int out_pad = l == s.depth ? s.no : s.h;
            if (threadIdx.x == 0) {
                tc_fence_after();
                issue_gemm(tmem, act_addr, 32, smem_addr(weight_tile(smem, P, s, l)), 32, in_pad / 16,
                           instr_desc(128, out_pad, bf16, 0, 0), false);
                mma_commit(bar);
            }
            const bool ok = mbar_wait(bar, phase);
            phase ^= 1;
            tc_fence_after();
            if (!ok) {
                abort_flag = 1;
                g_tc_status = 1;
            } else if (l < s.depth) {
                const float *b = bias + l * kMaxDim;
                switch (out_pad) {
                    case 16: fwd_epilogue<T, 16>(taddr, b, s.act, act_tile, row); break;
                    case 32: fwd_epilogue<T, 32>(taddr, b, s.act, act_tile, row); break;
                    default: fwd_epilogue<T, 64>(taddr, b, s.act, act_tile, row); break;
                }
            } else {
                const float *b = bias + l * kMaxDim;
                const bool live = row0 + row < n_rows;
                T *dst = y + (live ? row0 + row : 0) * y_stride;
                switch (out_pad) {
                    case 16: fwd_output<T, 16>(taddr, b, dst, s.d_out, live, y_vec); break;
                    case 32: fwd_output<T, 32>(taddr, b, dst, s.d_out, live, y_vec); break;
                    case 48: fwd_output<T, 48>(taddr, b, dst, s.d_out, live, y_vec); break;
                    default: fwd_output<T, 64>(taddr, b, dst, s.d_out, live, y_vec); break;
                }
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

// ---- backward ----------------------------------------------------------------------------------

// Epilogue of a recomputed forward layer: park the layer output in its own tile.
// Epilogue of a dgrad: dz of the layer below = dy * act'(parked output of that layer).
template <typename T, int COLS>
__device__ __forceinline__ void bwd_dz_epilogue(uint32_t taddr, int act, const unsigned char *parked, unsigned char *dz_tile,
                                                int row) {
    float v[COLS];
    load_acc_row<COLS>(taddr, v);
    if (act == TH_ACT_RELU) {
#pragma unroll
        for (int c = 0; c < COLS / 8; ++c) {
            const uint4 a = *reinterpret_cast<const uint4 *>(chunk_ptr(const_cast<unsigned char *>(parked), row, c));
            const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 post = unpack_pair<T>(w[k]);
                if (!(post.x > 0.f)) v[8 * c + 2 * k] = 0.f;
                if (!(post.y > 0.f)) v[8 * c + 2 * k + 1] = 0.f;
            }
        }
    }
    store_row_to_tile<T, COLS>(dz_tile, row, v);
}

template <typename T, int COLS>
__device__ __forceinline__ void bwd_dx_epilogue(uint32_t taddr, T *dst, int cols, bool live, bool vector_ok) {
    float v[COLS];
    load_acc_row<COLS>(taddr, v);
    if (live) store_row_to_global<T, COLS>(dst, cols, v, vector_ok);
}

// Flush one layer's weight-gradient accumulator (M = 64 layout: gradient row m sits in TMEM lane
// 32 * (m / 16) + m % 16, so lanes 0..15 of each warp carry rows 16 * warp .. 16 * warp + 15).
template <int COLS>
__device__ __forceinline__ void flush_dw(uint32_t taddr, float *dst, int out_dim, int in_dim) {
    float v[COLS];
    load_acc_row<COLS>(taddr, v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int m = 16 * warp + lane;
    if (lane < 16 && m < out_dim) {
#pragma unroll
        for (int c = 0; c < COLS; ++c)
            if (c < in_dim) atomicAdd(dst + m * in_dim + c, v[c]);
    }
}

template <typename T>
__global__ void __launch_bounds__(kTcThreads)
mlp_bwd_tc_kernel(const MlpShape s, const MlpParams p, const T *__restrict__ x, long long x_stride,
                  const T *__restrict__ go, long long go_stride, T *__restrict__ gx, long long gx_stride,
                  float *__restrict__ workspace, long long n_rows, int x_vec, int go_vec, int gx_vec) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint32_t tmem_holder;
    __shared__ __align__(8) unsigned long long mbar;
    __shared__ int abort_flag;
    const TcPlan P = tc_plan(s, true);
    constexpr int bf16 = sizeof(T) == 2 && !std::is_same<T, __half>::value;

    if (threadIdx.x == 0) abort_flag = 0;
    // operand tiles start out as zeros: columns a layer does not use are still read as MMA rows
    for (int e = threadIdx.x; e < (P.act_tiles + P.dz_tiles) * kTileBytes / 16; e += kTcThreads)
        reinterpret_cast<uint4 *>(smem)[e] = make_uint4(0, 0, 0, 0);
    stage_all_weights<T>(smem, P, s, p);
    const uint32_t tmem = cta_setup(&tmem_holder, &mbar, P.tmem_cols);
    const uint32_t bar = smem_addr(&mbar);
    unsigned char *dz_tiles = smem + P.act_tiles * kTileBytes;
    const int row = threadIdx.x;
    const uint32_t lane_base = static_cast<uint32_t>(row & ~31) << 16;
    const uint32_t taddr = tmem + lane_base;
    uint32_t phase = 0;
    bool first_tile = true;
    const long long n_tiles = (n_rows + kTileRows - 1) / kTileRows;
    auto act_tile = [&](int l) { return smem + l * kTileBytes; };
    auto dw_col = [&](int l) { return kAccCols + (l == 0 ? 0 : s.ki + (l - 1) * s.h); };

    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const long long row0 = tile * kTileRows;
        // ---- phase 1: recompute the forward, parking every layer input ----
        load_tile<T>(act_tile(0), x, x_stride, row0, n_rows, s.d_in, s.ki, x_vec);
        load_tile<T>(dz_tiles, go, go_stride, row0, n_rows, s.d_out, s.no, go_vec);  // dz of the output layer = grad_out
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        if (abort_flag) break;
        for (int l = 0; l < s.depth; ++l) {
            const int in_pad = l == 0 ? s.ki : s.h;
            if (threadIdx.x == 0) {
                tc_fence_after();
                issue_gemm(tmem, smem_addr(act_tile(l)), 32, smem_addr(weight_tile(smem, P, s, l)), 32, in_pad / 16,
                           instr_desc(128, s.h, bf16, 0, 0), false);
                mma_commit(bar);
            }
            const bool ok = mbar_wait(bar, phase);
            phase ^= 1;
            tc_fence_after();
            if (!ok) {
                abort_flag = 1;
                g_tc_status = 1;
            } else {
                const float *b = reinterpret_cast<const float *>(smem + P.bias_offset) + l * kMaxDim;
                switch (s.h) {
                    case 16: fwd_epilogue<T, 16>(taddr, b, s.act, act_tile(l + 1), row); break;
                    case 32: fwd_epilogue<T, 32>(taddr, b, s.act, act_tile(l + 1), row); break;
                    default: fwd_epilogue<T, 64>(taddr, b, s.act, act_tile(l + 1), row); break;
                }
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
            if (threadIdx.x == 0) {
                tc_fence_after();
                // wgrad: DW_l[out x in] += DZ^T . ACT_l over the tile's 128 rows (both operands MN-major)
                issue_gemm(tmem + dw_col(l), smem_addr(dz), 2048, smem_addr(act_tile(l)), 2048, kTileRows / 16,
                           instr_desc(64, in_pad, bf16, 1, 1), !first_tile);
                // dgrad: ACC[128 x in] = DZ . W_l (A K-major over the layer's outputs, W_l tile MN-major)
                if (need_dgrad)
                    issue_gemm(tmem, smem_addr(dz), 32, smem_addr(weight_tile(smem, P, s, l)), 2048, out_pad / 16,
                               instr_desc(128, in_pad, bf16, 0, 1), false);
                mma_commit(bar);
            }
            const bool ok = mbar_wait(bar, phase);
            phase ^= 1;
            tc_fence_after();
            if (!ok) {
                abort_flag = 1;
                g_tc_status = 1;
            } else if (l > 0) {
                // in_pad == s.h here: the layer below produced ACT_l
                unsigned char *next = dz_tiles + (buf ^ 1) * kTileBytes;
                switch (s.h) {
                    case 16: bwd_dz_epilogue<T, 16>(taddr, s.act, act_tile(l), next, row); break;
                    case 32: bwd_dz_epilogue<T, 32>(taddr, s.act, act_tile(l), next, row); break;
                    default: bwd_dz_epilogue<T, 64>(taddr, s.act, act_tile(l), next, row); break;
                }
            } else if (gx != nullptr) {
                const bool live = row0 + row < n_rows;
                T *dst = gx + (live ? row0 + row : 0) * gx_stride;
                switch (in_pad) {
                    case 16: bwd_dx_epilogue<T, 16>(taddr, dst, s.d_in, live, gx_vec); break;
                    case 32: bwd_dx_epilogue<T, 32>(taddr, dst, s.d_in, live, gx_vec); break;
                    case 48: bwd_dx_epilogue<T, 48>(taddr, dst, s.d_in, live, gx_vec); break;
                    default: bwd_dx_epilogue<T, 64>(taddr, dst, s.d_in, live, gx_vec); break;
                }
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

    // ---- flush the weight gradients this CTA accumulated in TMEM ----
    if (!abort_flag && !first_tile) {
        tc_fence_after();
        const MlpGradWorkspace W = grad_workspace_layout(s, workspace);
        for (int l = 0; l <= s.depth; ++l) {
            const int in_pad = l == 0 ? s.ki : s.h;
            const int in_dim = l == 0 ? s.d_in : s.d_hid, out_dim = l == s.depth ? s.d_out : s.d_hid;
            float *dst = W.base + (l == 0 ? W.w_in : (l == s.depth ? W.w_out : W.w_hid + (l - 1) * s.d_hid * s.d_hid));
            const uint32_t t = taddr + dw_col(l);
            switch (in_pad) {
                case 16: flush_dw<16>(t, dst, out_dim, in_dim); break;
                case 32: flush_dw<32>(t, dst, out_dim, in_dim); break;
                case 48: flush_dw<48>(t, dst, out_dim, in_dim); break;
                default: flush_dw<64>(t, dst, out_dim, in_dim); break;
            }
        }
    }
    cta_teardown(tmem, P.tmem_cols);
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

bool tc_disabled() {
    static const bool off = [] {
        const char *v = getenv("TH_MLP_LEGACY");
        return v && v[0] == '1';
    }();
    return off;
}

template <typename T>
int launch_fwd(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
               int64_t rows, cudaStream_t stream) {
    const TcPlan P = tc_plan(s, false);
    int ctas = 0;
    const int smem = occupancy_plan(P, &ctas);
    if (ctas < 1) return kTcNotApplicable;
    if (int rc = cuda_status(cudaFuncSetAttribute(mlp_fwd_tc_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                             "cudaFuncSetAttribute(mlp_fwd_tc_kernel)")) return rc;
    const long long tiles = (rows + kTileRows - 1) / kTileRows;
    const long long cap = static_cast<long long>(sm_count()) * ctas;
    mlp_fwd_tc_kernel<T><<<static_cast<unsigned>(tiles < cap ? tiles : cap), kTcThreads, smem, stream>>>(
        s, p, static_cast<const T *>(x), x_stride, static_cast<T *>(y), y_stride, rows, rows_vector_ok(x, x_stride, s.d_in),
        rows_vector_ok(y, y_stride, s.d_out));
    return cuda_status(cudaGetLastError(), "mlp_fwd_tc_kernel launch");
}

template <typename T>
int launch_bwd(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, const void *go, int64_t go_stride,
               void *gx, int64_t gx_stride, float *workspace, int64_t rows, cudaStream_t stream) {
    const TcPlan P = tc_plan(s, true);
    if (P.tmem_cols > 512) return kTcNotApplicable;
    int ctas = 0;
    const int smem = occupancy_plan(P, &ctas);
    if (ctas < 1) return kTcNotApplicable;
    if (int rc = cuda_status(cudaFuncSetAttribute(mlp_bwd_tc_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem),
                             "cudaFuncSetAttribute(mlp_bwd_tc_kernel)")) return rc;
    const long long tiles = (rows + kTileRows - 1) / kTileRows;
    const long long cap = static_cast<long long>(sm_count()) * ctas;
    mlp_bwd_tc_kernel<T><<<static_cast<unsigned>(tiles < cap ? tiles : cap), kTcThreads, smem, stream>>>(
        s, p, static_cast<const T *>(x), x_stride, static_cast<const T *>(go), go_stride, static_cast<T *>(gx), gx_stride,
        workspace, rows, rows_vector_ok(x, x_stride, s.d_in), rows_vector_ok(go, go_stride, s.d_out),
        gx ? rows_vector_ok(gx, gx_stride, s.d_in) : 0);
    return cuda_status(cudaGetLastError(), "mlp_bwd_tc_kernel launch");
}

}  // namespace

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
    // bias gradients and activations that need the pre-activation stay on the mma.sync kernels
    if (s.has_bias || (s.act != TH_ACT_RELU && s.act != TH_ACT_NONE)) return kTcNotApplicable;
    switch (dtype) {
        case TH_F16: return launch_bwd<__half>(s, p, x, x_stride, go, go_stride, gx, gx_stride, workspace, rows, stream);
        case TH_BF16: return launch_bwd<__nv_bfloat16>(s, p, x, x_stride, go, go_stride, gx, gx_stride, workspace, rows, stream);
        default: return kTcNotApplicable;
    }
}

}  // namespace th

// Device-side status of the tcgen05 kernels: 0 = fine, 1 = a bounded wait ran out.  Synchronises.
extern "C" int th_mlp_tc_status(void) {
    int status = 0;
    if (cudaMemcpyFromSymbol(&status, th::g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    return status;
}
