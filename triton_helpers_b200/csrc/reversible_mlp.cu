// Reversible (additive coupling) fused MLP for sm_100a.  No counterpart exists in
// triton_helpers; the calling conventions follow its fused MLP
// (triton_helpers/layers/fully_fused_mlp/kernel.py:503-686): stacked (out, in) weights,
// 16-bit operands, fp32 accumulation, activations rounded to the storage dtype between layers.
//
//   block k:   y1 = x1 + F_k(x2)      F_k(u) = W_f2[k] . act(W_f1[k] . u + b_f1[k]) + b_f2[k]
//              y2 = x2 + G_k(y1)      G_k(u) = W_g2[k] . act(W_g1[k] . u + b_g1[k]) + b_g2[k]
//
// The residual stream (x1, x2) of a row lives in fp32 registers of the warp that owns the row
// for the whole stack; only branch inputs and hidden activations are rounded to 16 bits for
// the tensor cores.  Weights do not fit in shared memory for the full stack (8 blocks x 4 x
// 64 x 64 x 2 B = 256 KB), so each CTA streams them block by block through a two-stage
// cp.async ring while the previous block computes.
//
// Backward stores no activations: starting from the stack's OUTPUT it undoes one block at a
// time, x2 = y2 - G(y1), x1 = y1 - F(x2), recomputing the branch it needs for the gradients
// on the way.  Per block and 128-row tile the four weight gradients are formed cooperatively
// (K = 128 rows) and added into CTA-private fp32 accumulators that live in global memory and
// stay L2 resident (no atomics: one CTA owns one copy); a reduction kernel sums the copies.
#include "rev_shape.cuh"
#include "mma_tiles.cuh"

#include <type_traits>

namespace th {
namespace {

constexpr int kRevWarps = 8;
constexpr int kRevThreads = kRevWarps * 32;
constexpr int kRevRows = kRevWarps * 16;  // rows per CTA tile

struct RevSmem {
    int w_stage;       // bytes of one ring stage: [w_f1 | w_f2 | w_g1 | w_g2]
    int w1_bytes, w2_bytes;
    int ring;          // offset of stage 0; stage 1 follows
    int bias;          // fp32 [2 stages][4][64]
    int tile_in, tile_h, tile_dz, tile_dy, tile_bytes;  // backward: 16-bit [128][64 + 8] operand tiles
    int total;
};

__host__ __device__ inline RevSmem rev_smem_layout(const RevShape &s, bool backward) {
    RevSmem m{};
    m.w1_bytes = s.hid * (s.half + kSmemPad) * 2;   // [hid][half + pad]
    m.w2_bytes = s.half * (s.hid + kSmemPad) * 2;   // [half][hid + pad]
    m.w_stage = 2 * (m.w1_bytes + m.w2_bytes);
    int off = 0;
    m.ring = off;
    off += 2 * m.w_stage;
    m.bias = off;
    off += 2 * 4 * kMaxDim * 4;
    if (backward) {
        m.tile_bytes = kRevRows * (kMaxDim + kSmemPad) * 2;
        m.tile_in = off;
        m.tile_h = off + m.tile_bytes;
        m.tile_dz = off + 2 * m.tile_bytes;
        m.tile_dy = off + 3 * m.tile_bytes;
        off += 4 * m.tile_bytes;
    }
    m.total = off;
    return m;
}

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Queue the copy of block k's four weight matrices (and biases) into ring stage `stage`.
template <typename T>
__device__ void prefetch_block(unsigned char *smem, const RevSmem &L, const RevShape &s, const RevParams &p, int k,
                               int stage) {
    unsigned char *dst = smem + L.ring + stage * L.w_stage;
    const T *src[4] = {static_cast<const T *>(p.w_f1), static_cast<const T *>(p.w_f2),
                       static_cast<const T *>(p.w_g1), static_cast<const T *>(p.w_g2)};
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const bool first = (m & 1) == 0;  // (hid x half) matrices first in each branch
        const int rows = first ? s.hid : s.half, cols = first ? s.half : s.hid;
        const int stride = cols + kSmemPad;
        T *tile = reinterpret_cast<T *>(dst + (m >> 1) * (L.w1_bytes + L.w2_bytes) + (first ? 0 : L.w1_bytes));
        const T *g = src[m] + static_cast<size_t>(k) * rows * cols;
        const int chunks = cols / 8;  // 16-byte pieces per row
        for (int e = threadIdx.x; e < rows * chunks; e += blockDim.x) {
            const int r = e / chunks, c = e - r * chunks;
            cp_async16(tile + r * stride + 8 * c, g + r * cols + 8 * c);
        }
    }
    if (s.has_bias) {
        float *bias = reinterpret_cast<float *>(smem + L.bias) + stage * 4 * kMaxDim;
        const T *bsrc[4] = {static_cast<const T *>(p.b_f1), static_cast<const T *>(p.b_f2),
                            static_cast<const T *>(p.b_g1), static_cast<const T *>(p.b_g2)};
        for (int e = threadIdx.x; e < 4 * kMaxDim; e += blockDim.x) {
            const int m = e / kMaxDim, c = e % kMaxDim;
            const int width = (m & 1) == 0 ? s.hid : s.half;
            bias[e] = c < width ? to_float<T>(bsrc[m][k * width + c]) : 0.f;
        }
    }
    cp_async_commit();
}

struct StageView {
    const unsigned char *w;
    const float *bias;  // null when the stack has no biases
    int w1_bytes, w2_bytes;
    template <typename T>
    __device__ const T *mat(int m) const {  // 0: f1, 1: f2, 2: g1, 3: g2
        return reinterpret_cast<const T *>(w + (m >> 1) * (w1_bytes + w2_bytes) + ((m & 1) ? w1_bytes : 0));
    }
    __device__ const float *b(int m) const { return bias ? bias + m * kMaxDim : nullptr; }
};

// fp32 stream registers (C layout) <-> 16-bit A fragments / global rows
template <typename T>
__device__ __forceinline__ void stream_to_frags(uint32_t (&a)[1][kKTiles][4], const float (&v)[1][kNTiles][4]) {
    acc_to_frags<T, 1>(a, v, TH_ACT_NONE);
}

template <typename T>
__device__ __forceinline__ void frags_to_stream(float (&v)[1][kNTiles][4], const uint32_t (&a)[kKTiles][4]) {
#pragma unroll
    for (int kt = 0; kt < kKTiles; ++kt)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 f = unpack_pair<T>(a[kt][q]);
            v[0][2 * kt + (q >> 1)][2 * (q & 1)] = f.x;
            v[0][2 * kt + (q >> 1)][2 * (q & 1) + 1] = f.y;
        }
}

// ---- forward --------------------------------------------------------------------------------

template <typename T>
__global__ void __launch_bounds__(kRevThreads)
rev_fwd_kernel(const RevShape s, const RevParams p, const T *__restrict__ x, long long x_stride, T *__restrict__ y,
               long long y_stride, long long n_rows) {
    extern __shared__ __align__(16) unsigned char smem[];
    const RevSmem L = rev_smem_layout(s, false);
    const int warp = threadIdx.x >> 5;
    const long long n_tiles = (n_rows + kRevRows - 1) / kRevRows;
    const int k_half = s.half / 16, k_hid = s.hid / 16;

    int step = 0;  // running (tile, block) counter: ring stage = step & 1
    if (static_cast<long long>(blockIdx.x) < n_tiles) prefetch_block<T>(smem, L, s, p, 0, 0);
    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const long long row0 = tile * kRevRows + warp * 16;
        float x1[1][kNTiles][4], x2[1][kNTiles][4], acc[1][kNTiles][4];
        uint32_t a[1][kKTiles][4];
        load_rows_as_frags<T>(a[0], x, x_stride, row0, n_rows, s.half, k_half, true);
        frags_to_stream<T>(x1, a[0]);
        load_rows_as_frags<T>(a[0], x + s.half, x_stride, row0, n_rows, s.half, k_half, true);
        frags_to_stream<T>(x2, a[0]);

        for (int k = 0; k < s.blocks; ++k, ++step) {
            cp_async_wait_all();
            __syncthreads();  // stage (step & 1) is filled; everyone is done with the other stage
            const bool more = k + 1 < s.blocks || tile + gridDim.x < n_tiles;
            if (more) prefetch_block<T>(smem, L, s, p, (k + 1) % s.blocks, (step + 1) & 1);
            const StageView W{smem + L.ring + (step & 1) * L.w_stage,
                              s.has_bias ? reinterpret_cast<const float *>(smem + L.bias) + (step & 1) * 4 * kMaxDim : nullptr,
                              L.w1_bytes, L.w2_bytes};
#pragma unroll
            for (int branch = 0; branch < 2; ++branch) {
                // branch 0: x1 += F(x2); branch 1: x2 += G(x1)
                stream_to_frags<T>(a, branch == 0 ? x2 : x1);
                fill_acc<1>(acc, W.b(2 * branch));
                warp_gemm_nk<T, 1>(acc, a, W.mat<T>(2 * branch), s.half + kSmemPad, k_half, s.hid / 8);
                acc_to_frags<T, 1>(a, acc, s.act);
                fill_acc<1>(acc, W.b(2 * branch + 1));
                warp_gemm_nk<T, 1>(acc, a, W.mat<T>(2 * branch + 1), s.hid + kSmemPad, k_hid, s.half / 8);
#pragma unroll
                for (int nt = 0; nt < kNTiles; ++nt)
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        if (branch == 0) x1[0][nt][q] += acc[0][nt][q];
                        else x2[0][nt][q] += acc[0][nt][q];
                    }
            }
        }
        store_acc_rows<T>(y, y_stride, row0, n_rows, s.half, s.half / 8, x1[0], true);
        store_acc_rows<T>(y + s.half, y_stride, row0, n_rows, s.half, s.half / 8, x2[0], true);
    }
}

// ---- backward -------------------------------------------------------------------------------

// dW[out][in] += A^T . B over the tile's 128 rows; A tile = [128][out], B tile = [128][in] (16-bit,
// stride kMaxDim + kSmemPad).  Warp `unit` owns a 16 x 32 patch; the patch is added into its
// fragment-native slot of the CTA-private accumulator.
template <typename T>
__device__ __forceinline__ void tile_wgrad(const T *a_tile, const T *b_tile, int out_pad, int in_pad, float *slots) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mtx = lane >> 3, r8 = lane & 7;
    constexpr int stride = kMaxDim + kSmemPad;
    const int halves = (in_pad + 31) / 32;
    if (warp >= (out_pad / 16) * halves) return;
    const int mt = warp / halves, nh = warp % halves;
    float c[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) c[i][j] = 0.f;
    const T *a_lane = a_tile + (8 * (mtx >> 1) + r8) * stride + 16 * mt + 8 * (mtx & 1);
    const T *b_lane = b_tile + (8 * (mtx & 1) + r8) * stride + 32 * nh + 8 * (mtx >> 1);
#pragma unroll
    for (int kt = 0; kt < kRevRows / 16; ++kt) {
        uint32_t af[4];
        ldmatrix_x4_trans(af, a_lane + 16 * kt * stride);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
            if (32 * nh + 16 * np < in_pad) {
                uint32_t bf[4];
                ldmatrix_x4_trans(bf, b_lane + 16 * kt * stride + 16 * np);
                mma16816<T>(c[2 * np], af, bf[0], bf[1]);
                mma16816<T>(c[2 * np + 1], af, bf[2], bf[3]);
            }
        }
    }
    float *mine = slots + warp * 512 + lane;
#pragma unroll
    for (int i = 0; i < 16; ++i) mine[32 * i] += c[i >> 2][i & 3];
}

template <typename T>
__device__ __forceinline__ void tile_bias_grad(const T *tile, int width, float *dst) {
    constexpr int stride = kMaxDim + kSmemPad;
    const int col = threadIdx.x & 63, part = threadIdx.x >> 6;
    if (col >= width) return;
    float sum = 0.f;
    for (int r = 0; r < kRevRows / 4; ++r) sum += to_float<T>(tile[(part * (kRevRows / 4) + r) * stride + col]);
    atomicAdd(dst + col, sum);
}

template <typename T>
__global__ void __launch_bounds__(kRevThreads, 1)
rev_bwd_kernel(const RevShape s, const RevParams p, const T *__restrict__ y, long long y_stride,
               const T *__restrict__ go, long long go_stride, T *__restrict__ gx, long long gx_stride,
               T *__restrict__ x_rec, long long xr_stride, float *__restrict__ workspace, long long n_rows) {
    extern __shared__ __align__(16) unsigned char smem[];
    const RevSmem L = rev_smem_layout(s, true);
    const int warp = threadIdx.x >> 5;
    const int wrow = warp * 16;
    const long long n_tiles = (n_rows + kRevRows - 1) / kRevRows;
    const int k_half = s.half / 16, k_hid = s.hid / 16;
    constexpr int tstride = kMaxDim + kSmemPad;
    T *t_in = reinterpret_cast<T *>(smem + L.tile_in);
    T *t_h = reinterpret_cast<T *>(smem + L.tile_h);
    T *t_dz = reinterpret_cast<T *>(smem + L.tile_dz);
    T *t_dy = reinterpret_cast<T *>(smem + L.tile_dy);
    float *cta_acc = workspace + static_cast<size_t>(blockIdx.x) * rev_cta_floats(s);
    float *cta_bias = cta_acc + static_cast<size_t>(s.blocks) * 4 * kMatFloats;

    int step = 0;
    if (static_cast<long long>(blockIdx.x) < n_tiles) prefetch_block<T>(smem, L, s, p, s.blocks - 1, 0);
    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const long long row0 = tile * kRevRows + wrow;
        float s1[1][kNTiles][4], s2[1][kNTiles][4];  // stream: y1, y2 turning into x1, x2
        float d1[1][kNTiles][4], d2[1][kNTiles][4];  // gradients with respect to the stream
        uint32_t a[1][kKTiles][4], zf[1][kKTiles][4];
        float acc[1][kNTiles][4];
        load_rows_as_frags<T>(a[0], y, y_stride, row0, n_rows, s.half, k_half, true);
        frags_to_stream<T>(s1, a[0]);
        load_rows_as_frags<T>(a[0], y + s.half, y_stride, row0, n_rows, s.half, k_half, true);
        frags_to_stream<T>(s2, a[0]);
        load_rows_as_frags<T>(a[0], go, go_stride, row0, n_rows, s.half, k_half, true);
        frags_to_stream<T>(d1, a[0]);
        load_rows_as_frags<T>(a[0], go + s.half, go_stride, row0, n_rows, s.half, k_half, true);
        frags_to_stream<T>(d2, a[0]);

        for (int k = s.blocks - 1; k >= 0; --k, ++step) {
            cp_async_wait_all();
            __syncthreads();
            const bool more = k > 0 || tile + gridDim.x < n_tiles;
            if (more) prefetch_block<T>(smem, L, s, p, k > 0 ? k - 1 : s.blocks - 1, (step + 1) & 1);
            const StageView W{smem + L.ring + (step & 1) * L.w_stage,
                              s.has_bias ? reinterpret_cast<const float *>(smem + L.bias) + (step & 1) * 4 * kMaxDim : nullptr,
                              L.w1_bytes, L.w2_bytes};
#pragma unroll
            for (int pass = 0; pass < 2; ++pass) {
                // pass 0 undoes y2 = x2 + G(y1): input s1, output side (s2, d2), gradient flows into d1
                // pass 1 undoes y1 = x1 + F(x2): input s2, output side (s1, d1), gradient flows into d2
                const int m1 = pass == 0 ? 2 : 0, m2 = m1 + 1;
                float(&in_s)[1][kNTiles][4] = pass == 0 ? s1 : s2;
                float(&out_s)[1][kNTiles][4] = pass == 0 ? s2 : s1;
                float(&in_d)[1][kNTiles][4] = pass == 0 ? d1 : d2;
                float(&out_d)[1][kNTiles][4] = pass == 0 ? d2 : d1;

                // recompute the branch: z = W1 . in + b1, h = act(z), out -= W2 . h + b2
                stream_to_frags<T>(a, in_s);
                frags_to_smem(t_in, tstride, wrow, a[0], k_half);
                fill_acc<1>(acc, W.b(m1));
                warp_gemm_nk<T, 1>(acc, a, W.mat<T>(m1), s.half + kSmemPad, k_half, s.hid / 8);
                acc_to_frags<T, 1>(zf, acc, TH_ACT_NONE);  // pre-activation, rounded
                acc_to_frags<T, 1>(a, acc, s.act);         // hidden activation, rounded
                frags_to_smem(t_h, tstride, wrow, a[0], k_hid);
                fill_acc<1>(acc, W.b(m2));
                warp_gemm_nk<T, 1>(acc, a, W.mat<T>(m2), s.hid + kSmemPad, k_hid, s.half / 8);
#pragma unroll
                for (int nt = 0; nt < kNTiles; ++nt)
#pragma unroll
                    for (int q = 0; q < 4; ++q) out_s[0][nt][q] -= acc[0][nt][q];

                // gradient of the branch output is the stream gradient on the output side
                stream_to_frags<T>(a, out_d);
                frags_to_smem(t_dy, tstride, wrow, a[0], k_half);
                fill_acc<1>(acc, nullptr);
                warp_gemm_kn<T, 1>(acc, a, W.mat<T>(m2), s.hid + kSmemPad, k_half, s.hid / 8);  // dh = dy . W2
#pragma unroll
                for (int kt = 0; kt < kKTiles; ++kt)
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int nt = 2 * kt + (q >> 1), c = 2 * (q & 1);
                        const float2 z = unpack_pair<T>(zf[0][kt][q]);
                        a[0][kt][q] = pack_pair<T>(activate_grad(s.act, z.x, acc[0][nt][c]),
                                                   activate_grad(s.act, z.y, acc[0][nt][c + 1]));
                    }
                frags_to_smem(t_dz, tstride, wrow, a[0], k_hid);
                warp_gemm_kn<T, 1>(in_d, a, W.mat<T>(m1), s.half + kSmemPad, k_hid, s.half / 8);  // d_in += dz . W1
                __syncthreads();  // the four operand tiles hold all 128 rows

                float *slots = cta_acc + (static_cast<size_t>(k) * 4) * kMatFloats;
                tile_wgrad<T>(t_dz, t_in, s.hid, s.half, slots + m1 * kMatFloats);
                tile_wgrad<T>(t_dy, t_h, s.half, s.hid, slots + m2 * kMatFloats);
                if (s.has_bias) {
                    tile_bias_grad<T>(t_dz, s.hid, cta_bias + (k * 4 + m1) * kMaxDim);
                    tile_bias_grad<T>(t_dy, s.half, cta_bias + (k * 4 + m2) * kMaxDim);
                }
                __syncthreads();  // tiles may be overwritten
            }
        }
        if (gx) {
            store_acc_rows<T>(gx, gx_stride, row0, n_rows, s.half, s.half / 8, d1[0], true);
            store_acc_rows<T>(gx + s.half, gx_stride, row0, n_rows, s.half, s.half / 8, d2[0], true);
        }
        if (x_rec) {
            store_acc_rows<T>(x_rec, xr_stride, row0, n_rows, s.half, s.half / 8, s1[0], true);
            store_acc_rows<T>(x_rec + s.half, xr_stride, row0, n_rows, s.half, s.half / 8, s2[0], true);
        }
    }
}

// Sum the per-CTA accumulators and write the gradients in the parameter dtype.
template <typename T>
__global__ void rev_grad_reduce_kernel(const RevShape s, const float *__restrict__ workspace, int n_ctas, T *dw_f1,
                                       T *dw_f2, T *dw_g1, T *dw_g2, T *db_f1, T *db_f2, T *db_g1, T *db_g2) {
    const size_t per_cta = rev_cta_floats(s);
    const size_t mat_total = static_cast<size_t>(s.blocks) * 4 * kMatFloats;
    T *dw[4] = {dw_f1, dw_f2, dw_g1, dw_g2};
    T *db[4] = {db_f1, db_f2, db_g1, db_g2};
    for (size_t e = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; e < per_cta;
         e += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float sum = 0.f;
        for (int c = 0; c < n_ctas; ++c) sum += workspace[c * per_cta + e];
        if (e < mat_total) {
            const int k = static_cast<int>(e / (4 * kMatFloats));
            const int m = static_cast<int>((e / kMatFloats) % 4);
            const int f = static_cast<int>(e % kMatFloats);
            const int u = f / 512, i = (f % 512) / 32, ln = f % 32;
            const int out_dim = (m & 1) == 0 ? s.hid : s.half, in_dim = (m & 1) == 0 ? s.half : s.hid;
            const int halves = (in_dim + 31) / 32;
            const int mt = u / halves, nh = u % halves;
            const int row = 16 * mt + (ln >> 2) + 8 * ((i >> 1) & 1);
            const int col = 32 * nh + 8 * (i >> 2) + 2 * (ln & 3) + (i & 1);
            if (u < (out_dim / 16) * halves && row < out_dim && col < in_dim && dw[m])
                dw[m][(static_cast<size_t>(k) * out_dim + row) * in_dim + col] = from_float<T>(sum);
        } else {
            const size_t b = e - mat_total;
            const int k = static_cast<int>(b / (4 * kMaxDim)), m = static_cast<int>((b / kMaxDim) % 4);
            const int c = static_cast<int>(b % kMaxDim);
            const int width = (m & 1) == 0 ? s.hid : s.half;
            if (c < width && db[m]) db[m][k * width + c] = from_float<T>(sum);
        }
    }
}

// ---- host side ------------------------------------------------------------------------------

int make_rev_shape(RevShape &s, int d_model, int d_hidden, int blocks, int act, bool has_bias) {
    if (d_model < 32 || d_model > 2 * kMaxDim || d_model % 32)
        return fail(TH_ERR_UNSUPPORTED, "d_model %d must be a multiple of 32 in [32, %d]", d_model, 2 * kMaxDim);
    if (d_hidden < 16 || d_hidden > kMaxDim || d_hidden % 16)
        return fail(TH_ERR_UNSUPPORTED, "hidden width %d must be a multiple of 16 in [16, %d]", d_hidden, kMaxDim);
    if (blocks < 1 || blocks > 1024) return fail(TH_ERR_BAD_ARG, "block count %d outside [1, 1024]", blocks);
    if (act < TH_ACT_NONE || act > TH_ACT_RELU2) return fail(TH_ERR_BAD_ARG, "unknown activation code %d", act);
    s = RevShape{d_model / 2, d_hidden, blocks, act, has_bias ? 1 : 0};
    return TH_OK;
}

int check_rev_params(const RevParams &p, bool has_bias) {
    if (!p.w_f1 || !p.w_f2 || !p.w_g1 || !p.w_g2) return fail(TH_ERR_BAD_ARG, "null weight pointer");
    if (!aligned_to(p.w_f1, 16) || !aligned_to(p.w_f2, 16) || !aligned_to(p.w_g1, 16) || !aligned_to(p.w_g2, 16))
        return fail(TH_ERR_ALIGNMENT, "weight pointers must be 16-byte aligned");
    if (has_bias && (!p.b_f1 || !p.b_f2 || !p.b_g1 || !p.b_g2))
        return fail(TH_ERR_BAD_ARG, "biases must be all present or all null");
    return TH_OK;
}

int check_rows(const void *ptr, int64_t stride, int d_model, const char *what) {
    if (!ptr) return fail(TH_ERR_BAD_ARG, "null %s", what);
    if (stride < d_model) return fail(TH_ERR_BAD_ARG, "%s row stride smaller than the row", what);
    if (stride % 2 || !aligned_to(ptr, 4)) return fail(TH_ERR_ALIGNMENT, "%s rows must be 4-byte aligned", what);
    return TH_OK;
}

int rev_grid(int64_t rows) {
    const long long tiles = (rows + kRevRows - 1) / kRevRows;
    return static_cast<int>(tiles < sm_count() ? (tiles > 0 ? tiles : 1) : sm_count());
}

template <typename T>
int launch_rev_fwd(const RevShape &s, const RevParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
                   int64_t rows, cudaStream_t stream) {
    const RevSmem L = rev_smem_layout(s, false);
    if (int rc = cuda_status(cudaFuncSetAttribute(rev_fwd_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total),
                             "cudaFuncSetAttribute(rev_fwd_kernel)")) return rc;
    const long long tiles = (rows + kRevRows - 1) / kRevRows;
    const long long cap = static_cast<long long>(sm_count()) * 2;
    rev_fwd_kernel<T><<<static_cast<unsigned>(tiles < cap ? tiles : cap), kRevThreads, L.total, stream>>>(
        s, p, static_cast<const T *>(x), x_stride, static_cast<T *>(y), y_stride, rows);
    return launch_status("rev_fwd_kernel launch");
}

template <typename T>
int launch_rev_bwd(const RevShape &s, const RevParams &p, const void *y, int64_t y_stride, const void *go,
                   int64_t go_stride, void *gx, int64_t gx_stride, void *x_rec, int64_t xr_stride, void *const dw[4],
                   void *const db[4], float *workspace, int64_t rows, cudaStream_t stream) {
    const RevSmem L = rev_smem_layout(s, true);
    if (int rc = cuda_status(cudaFuncSetAttribute(rev_bwd_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total),
                             "cudaFuncSetAttribute(rev_bwd_kernel)")) return rc;
    const int grid = rev_grid(rows);
    const size_t bytes = sizeof(float) * rev_cta_floats(s) * grid;
    if (int rc = cuda_status(cudaMemsetAsync(workspace, 0, bytes, stream), "cudaMemsetAsync(workspace)")) return rc;
    // tensor-core kernels first (they also reduce and write the gradients); mma.sync kernels otherwise
    const int tc = rows > 0 ? rev_bwd_tc(s, p, y, y_stride, go, go_stride, gx, gx_stride, x_rec, xr_stride, dw, workspace, grid,
                                         rows, std::is_same<T, __half>::value ? TH_F16 : TH_BF16, stream)
                            : kRevTcNotApplicable;
    if (tc != kRevTcNotApplicable) return tc;
    if (rows > 0) {
        rev_bwd_kernel<T><<<grid, kRevThreads, L.total, stream>>>(
            s, p, static_cast<const T *>(y), y_stride, static_cast<const T *>(go), go_stride, static_cast<T *>(gx),
            gx_stride, static_cast<T *>(x_rec), xr_stride, workspace, rows);
        if (int rc = launch_status("rev_bwd_kernel launch")) return rc;
    }
    const unsigned rgrid = static_cast<unsigned>((rev_cta_floats(s) + 255) / 256);
    rev_grad_reduce_kernel<T><<<rgrid, 256, 0, stream>>>(
        s, workspace, grid, static_cast<T *>(dw[0]), static_cast<T *>(dw[1]), static_cast<T *>(dw[2]),
        static_cast<T *>(dw[3]), static_cast<T *>(db[0]), static_cast<T *>(db[1]), static_cast<T *>(db[2]),
        static_cast<T *>(db[3]));
    return launch_status("rev_grad_reduce_kernel launch");
}

}  // namespace
}  // namespace th

using namespace th;

extern "C" int64_t th_rev_workspace_bytes(int64_t rows, int d_model, int d_hidden, int blocks) {
    RevShape s;
    if (rows < 0 || make_rev_shape(s, d_model, d_hidden, blocks, TH_ACT_RELU, true)) return -1;
    return static_cast<int64_t>(sizeof(float) * rev_cta_floats(s)) * rev_grid(rows);
}

extern "C" int th_rev_fwd(const void *x_dev, int64_t x_stride, const void *w_f1_dev, const void *w_f2_dev,
                          const void *w_g1_dev, const void *w_g2_dev, const void *b_f1_dev, const void *b_f2_dev,
                          const void *b_g1_dev, const void *b_g2_dev, void *out_dev, int64_t out_stride, int64_t rows,
                          int d_model, int d_hidden, int blocks, int activation, int dtype, void *stream) {
    if (rows < 0) return fail(TH_ERR_BAD_ARG, "negative row count");
    const bool has_bias = b_f1_dev || b_f2_dev || b_g1_dev || b_g2_dev;
    RevShape s;
    if (int rc = make_rev_shape(s, d_model, d_hidden, blocks, activation, has_bias)) return rc;
    RevParams p{w_f1_dev, w_f2_dev, w_g1_dev, w_g2_dev, b_f1_dev, b_f2_dev, b_g1_dev, b_g2_dev};
    if (int rc = check_rev_params(p, has_bias)) return rc;
    if (rows == 0) return TH_OK;
    if (int rc = check_rows(x_dev, x_stride, d_model, "input")) return rc;
    if (int rc = check_rows(out_dev, out_stride, d_model, "output")) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (const int tc = rev_fwd_tc(s, p, x_dev, x_stride, out_dev, out_stride, rows, dtype, st); tc != kRevTcNotApplicable) return tc;
    switch (dtype) {
        case TH_F16: return launch_rev_fwd<__half>(s, p, x_dev, x_stride, out_dev, out_stride, rows, st);
        case TH_BF16: return launch_rev_fwd<__nv_bfloat16>(s, p, x_dev, x_stride, out_dev, out_stride, rows, st);
        default: return fail(TH_ERR_UNSUPPORTED, "reversible MLP kernels take float16 or bfloat16 (dtype code %d)", dtype);
    }
}

extern "C" int th_rev_bwd(const void *y_dev, int64_t y_stride, const void *w_f1_dev, const void *w_f2_dev,
                          const void *w_g1_dev, const void *w_g2_dev, const void *b_f1_dev, const void *b_f2_dev,
                          const void *b_g1_dev, const void *b_g2_dev, const void *grad_out_dev, int64_t go_stride,
                          void *grad_x_dev, int64_t gx_stride, void *x_rec_dev, int64_t xr_stride, void *grad_w_f1_dev,
                          void *grad_w_f2_dev, void *grad_w_g1_dev, void *grad_w_g2_dev, void *grad_b_f1_dev,
                          void *grad_b_f2_dev, void *grad_b_g1_dev, void *grad_b_g2_dev, void *workspace_dev,
                          int64_t workspace_bytes, int64_t rows, int d_model, int d_hidden, int blocks, int activation,
                          int dtype, void *stream) {
    if (rows < 0) return fail(TH_ERR_BAD_ARG, "negative row count");
    const bool has_bias = b_f1_dev || b_f2_dev || b_g1_dev || b_g2_dev;
    RevShape s;
    if (int rc = make_rev_shape(s, d_model, d_hidden, blocks, activation, has_bias)) return rc;
    RevParams p{w_f1_dev, w_f2_dev, w_g1_dev, w_g2_dev, b_f1_dev, b_f2_dev, b_g1_dev, b_g2_dev};
    if (int rc = check_rev_params(p, has_bias)) return rc;
    const int64_t need = th_rev_workspace_bytes(rows, d_model, d_hidden, blocks);
    if (!workspace_dev || workspace_bytes < need)
        return fail(TH_ERR_WORKSPACE, "workspace of %lld bytes needed, %lld given", (long long)need, (long long)workspace_bytes);
    if (rows > 0) {
        if (int rc = check_rows(y_dev, y_stride, d_model, "output")) return rc;
        if (int rc = check_rows(grad_out_dev, go_stride, d_model, "output gradient")) return rc;
        if (grad_x_dev) if (int rc = check_rows(grad_x_dev, gx_stride, d_model, "input gradient")) return rc;
        if (x_rec_dev) if (int rc = check_rows(x_rec_dev, xr_stride, d_model, "reconstructed input")) return rc;
    }
    void *const dw[4] = {grad_w_f1_dev, grad_w_f2_dev, grad_w_g1_dev, grad_w_g2_dev};
    void *const db[4] = {grad_b_f1_dev, grad_b_f2_dev, grad_b_g1_dev, grad_b_g2_dev};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float *ws = static_cast<float *>(workspace_dev);
    switch (dtype) {
        case TH_F16:
            return launch_rev_bwd<__half>(s, p, y_dev, y_stride, grad_out_dev, go_stride, grad_x_dev, gx_stride,
                                          x_rec_dev, xr_stride, dw, db, ws, rows, st);
        case TH_BF16:
            return launch_rev_bwd<__nv_bfloat16>(s, p, y_dev, y_stride, grad_out_dev, go_stride, grad_x_dev, gx_stride,
                                                 x_rec_dev, xr_stride, dw, db, ws, rows, st);
        default: return fail(TH_ERR_UNSUPPORTED, "reversible MLP kernels take float16 or bfloat16 (dtype code %d)", dtype);
    }
}
