// Fully fused small MLP for sm_100a, forward and backward, 16-bit operands with fp32
// accumulation.  Replaces the Triton kernels of
// triton_helpers/layers/fully_fused_mlp/kernel.py:198-261 (_fwd_kernel) and :326-500
// (_bwd_kernel_rfs).
//
//   y = W_out . act( W_hid[d-2] . ... act( W_in . x + b_in ) ... ) + b_out
//
// Semantics kept from the reference: activations are rounded to the input dtype after every
// layer (kernel.py:47); the output layer is never activated (:250); in the backward pass dz
// and dx are rounded to the gradient dtype between layers (:64,:74) and act' is evaluated
// on the dtype-rounded pre-activation (:278-281).
//
// Forward: persistent CTAs of 8 warps; all weights are staged once per CTA into padded
// shared-memory tiles; each warp owns 32 rows and keeps the activations of those rows in
// registers from the first layer to the last (accumulator tiles are converted in place into
// the next layer's A fragments), so a row costs one read of x and one write of y.
//
// Backward: one pass per 128-row tile instead of the reference's depth-many forward re-runs
// (kernel.py:345) and per-program dW copies (:599-633).  Phase 1 recomputes the forward and
// parks every layer input in shared memory; phase 2 walks the layers backwards: dz from the
// parked activations, dgrad warp-locally in registers, wgrad cooperatively over the tile's
// 128 rows, accumulated in fp32 shared-memory slots that live for the whole kernel and are
// flushed once per CTA with red.global.add into an fp32 workspace.  A small second kernel
// rounds the workspace into the gradient tensors.
#include "mlp_shape.cuh"
#include "mma_tiles.cuh"

#include <mutex>
#include <type_traits>

namespace th {
namespace {

constexpr int kWarps = 8;
constexpr int kThreadsMlp = kWarps * 32;
constexpr int kFwdMT = 2;                       // 16-row tiles per warp in the forward kernel
constexpr int kFwdRows = kWarps * 16 * kFwdMT;  // rows per CTA iteration (forward)
constexpr int kBwdRows = kWarps * 16;           // rows per CTA iteration (backward)
constexpr int kSmemLimit = 227 * 1024;

// Shared-memory layout, computed identically on host and device.
struct MlpSmem {
    int w_in, w_hid, w_hid_each, w_out;  // byte offsets of the 16-bit weight tiles
    int bias;                            // fp32 [depth + 1][64]
    int stash0, stash, stash_each;       // backward only: layer inputs, 16-bit [128][width + 8]
    int dz;                              // backward only: 16-bit [128][max(h, no) + 8]
    int acc, acc_total;                  // backward only: fp32 wgrad slots
    int dbias;                           // backward only: fp32 [depth + 1][64]
    int total;
};

__host__ __device__ inline int wgrad_units(int out_pad, int in_pad) { return (out_pad / 16) * ((in_pad + 31) / 32); }

__host__ __device__ inline MlpSmem mlp_smem_layout(const MlpShape &s, bool backward) {
    MlpSmem m{};
    int off = 0;
    m.w_in = off;
    off += s.h * (s.ki + kSmemPad) * 2;
    m.w_hid = off;
    m.w_hid_each = s.h * (s.h + kSmemPad) * 2;
    off += (s.depth - 1) * m.w_hid_each;
    m.w_out = off;
    off += s.no * (s.h + kSmemPad) * 2;
    m.bias = off;
    off += (s.depth + 1) * kMaxDim * 4;
    if (backward) {
        m.stash0 = off;
        off += kBwdRows * (s.ki + kSmemPad) * 2;
        m.stash = off;
        m.stash_each = kBwdRows * (s.h + kSmemPad) * 2;
        off += s.depth * m.stash_each;
        m.dz = off;
        off += kBwdRows * ((s.h > s.no ? s.h : s.no) + kSmemPad) * 2;
        m.acc = off;
        m.acc_total = wgrad_units(s.h, s.ki) + (s.depth - 1) * wgrad_units(s.h, s.h) + wgrad_units(s.no, s.h);
        off += m.acc_total * 512 * 4;
        m.dbias = off;
        off += (s.depth + 1) * kMaxDim * 4;
    }
    m.total = off;
    return m;
}

template <typename T>
__device__ void stage_parameters(unsigned char *smem, const MlpSmem &L, const MlpShape &s, const MlpParams &p) {
    stage_weight<T>(reinterpret_cast<T *>(smem + L.w_in), static_cast<const T *>(p.w_in), s.d_hid, s.d_in, s.h, s.ki);
    for (int i = 0; i < s.depth - 1; ++i)
        stage_weight<T>(reinterpret_cast<T *>(smem + L.w_hid + i * L.w_hid_each),
                        static_cast<const T *>(p.w_hid) + static_cast<size_t>(i) * s.d_hid * s.d_hid, s.d_hid, s.d_hid,
                        s.h, s.h);
    stage_weight<T>(reinterpret_cast<T *>(smem + L.w_out), static_cast<const T *>(p.w_out), s.d_out, s.d_hid, s.no,
                    s.h);
    float *bias = reinterpret_cast<float *>(smem + L.bias);
    for (int e = threadIdx.x; e < (s.depth + 1) * kMaxDim; e += blockDim.x) {
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

// ---- forward --------------------------------------------------------------------------------

template <typename T>
__global__ void __launch_bounds__(kThreadsMlp)
mlp_fwd_kernel(const MlpShape s, const MlpParams p, const T *__restrict__ x, long long x_stride, T *__restrict__ y,
               long long y_stride, long long n_rows, int x_pairs_ok, int y_pairs_ok) {
    extern __shared__ __align__(16) unsigned char smem[];
    const MlpSmem L = mlp_smem_layout(s, false);
    stage_parameters<T>(smem, L, s, p);
    __syncthreads();

    const int warp = threadIdx.x >> 5;
    const T *w_in = reinterpret_cast<const T *>(smem + L.w_in);
    const T *w_out = reinterpret_cast<const T *>(smem + L.w_out);
    const float *bias = reinterpret_cast<const float *>(smem + L.bias);
    const long long n_tiles = (n_rows + kFwdRows - 1) / kFwdRows;

    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const long long row0 = tile * kFwdRows + warp * 16 * kFwdMT;
        if (row0 >= n_rows) continue;
        uint32_t a[kFwdMT][kKTiles][4];
        float acc[kFwdMT][kNTiles][4];
#pragma unroll
        for (int mt = 0; mt < kFwdMT; ++mt)
            load_rows_as_frags<T>(a[mt], x, x_stride, row0 + 16 * mt, n_rows, s.d_in, s.ki / 16, x_pairs_ok);

        fill_acc<kFwdMT>(acc, s.has_bias ? bias : nullptr);
        warp_gemm_nk<T, kFwdMT>(acc, a, w_in, s.ki + kSmemPad, s.ki / 16, s.h / 8);
        acc_to_frags<T, kFwdMT>(a, acc, s.act);
        for (int i = 0; i < s.depth - 1; ++i) {
            fill_acc<kFwdMT>(acc, s.has_bias ? bias + (i + 1) * kMaxDim : nullptr);
            warp_gemm_nk<T, kFwdMT>(acc, a, reinterpret_cast<const T *>(smem + L.w_hid + i * L.w_hid_each),
                                    s.h + kSmemPad, s.h / 16, s.h / 8);
            acc_to_frags<T, kFwdMT>(a, acc, s.act);
        }
        fill_acc<kFwdMT>(acc, s.has_bias ? bias + s.depth * kMaxDim : nullptr);
        warp_gemm_nk<T, kFwdMT>(acc, a, w_out, s.h + kSmemPad, s.h / 16, s.no / 8);
#pragma unroll
        for (int mt = 0; mt < kFwdMT; ++mt)
            store_acc_rows<T>(y, y_stride, row0 + 16 * mt, n_rows, s.d_out, s.no / 8, acc[mt], y_pairs_ok);
    }
}

// ---- backward -------------------------------------------------------------------------------

template <typename T>
__global__ void __launch_bounds__(kThreadsMlp, 1)
mlp_bwd_kernel(const MlpShape s, const MlpParams p, const T *__restrict__ x, long long x_stride,
               const T *__restrict__ go, long long go_stride, T *__restrict__ gx, long long gx_stride,
               float *__restrict__ workspace, long long n_rows, int x_pairs_ok, int go_pairs_ok, int gx_pairs_ok) {
    extern __shared__ __align__(16) unsigned char smem[];
    const MlpSmem L = mlp_smem_layout(s, true);
    stage_parameters<T>(smem, L, s, p);
    float *acc_slots = reinterpret_cast<float *>(smem + L.acc);
    float *dbias = reinterpret_cast<float *>(smem + L.dbias);
    for (int e = threadIdx.x; e < L.acc_total * 512; e += blockDim.x) acc_slots[e] = 0.f;
    for (int e = threadIdx.x; e < (s.depth + 1) * kMaxDim; e += blockDim.x) dbias[e] = 0.f;
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mtx = lane >> 3, r8 = lane & 7;
    const int wrow = warp * 16;
    const float *bias = reinterpret_cast<const float *>(smem + L.bias);
    T *dz_tile = reinterpret_cast<T *>(smem + L.dz);
    const int dz_stride = (s.h > s.no ? s.h : s.no) + kSmemPad;
    const long long n_tiles = (n_rows + kBwdRows - 1) / kBwdRows;

    for (long long tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const long long row0 = tile * kBwdRows + wrow;
        uint32_t a[1][kKTiles][4];
        float acc[1][kNTiles][4];

        // ---- phase 1: forward, parking every layer input ----
        load_rows_as_frags<T>(a[0], x, x_stride, row0, n_rows, s.d_in, s.ki / 16, x_pairs_ok);
        frags_to_smem(smem + L.stash0, s.ki + kSmemPad, wrow, a[0], s.ki / 16);
        for (int l = 0; l < s.depth; ++l) {
            const T *w = reinterpret_cast<const T *>(l == 0 ? smem + L.w_in : smem + L.w_hid + (l - 1) * L.w_hid_each);
            const int in_pad = l == 0 ? s.ki : s.h;
            fill_acc<1>(acc, s.has_bias ? bias + l * kMaxDim : nullptr);
            warp_gemm_nk<T, 1>(acc, a, w, in_pad + kSmemPad, in_pad / 16, s.h / 8);
            acc_to_frags<T, 1>(a, acc, s.act);
            frags_to_smem(smem + L.stash + l * L.stash_each, s.h + kSmemPad, wrow, a[0], s.h / 16);
        }

        // ---- phase 2: backward ----
        uint32_t dy[1][kKTiles][4];
        load_rows_as_frags<T>(dy[0], go, go_stride, row0, n_rows, s.d_out, s.no / 16, go_pairs_ok);
        int slot = L.acc_total;  // slots are laid out in layer order; walk them backwards
        for (int l = s.depth; l >= 0; --l) {
            const int in_pad = l == 0 ? s.ki : s.h;
            const int out_pad = l == s.depth ? s.no : s.h;
            const unsigned char *w_bytes =
                l == 0 ? smem + L.w_in : (l == s.depth ? smem + L.w_out : smem + L.w_hid + (l - 1) * L.w_hid_each);
            const T *w = reinterpret_cast<const T *>(w_bytes);
            const unsigned char *in_stash = l == 0 ? smem + L.stash0 : smem + L.stash + (l - 1) * L.stash_each;
            const int in_stride = in_pad + kSmemPad;

            // dz = dy * act'(z)
            if (l < s.depth && s.act != TH_ACT_NONE) {
                if (s.act == TH_ACT_RELU) {
                    // relu(z) > 0 exactly when the rounded z > 0: the parked output is the mask
                    uint32_t post[kKTiles][4];
                    smem_to_frags(post, smem + L.stash + l * L.stash_each, s.h + kSmemPad, wrow, s.h / 16);
#pragma unroll
                    for (int kt = 0; kt < kKTiles; ++kt)
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float2 av = unpack_pair<T>(post[kt][q]);
                            const float2 gv = unpack_pair<T>(dy[0][kt][q]);
                            dy[0][kt][q] = pack_pair<T>(av.x > 0.f ? gv.x : 0.f, av.y > 0.f ? gv.y : 0.f);
                        }
                } else {
                    // recompute the pre-activation from the parked layer input
                    smem_to_frags(a[0], in_stash, in_stride, wrow, in_pad / 16);
                    fill_acc<1>(acc, s.has_bias ? bias + l * kMaxDim : nullptr);
                    warp_gemm_nk<T, 1>(acc, a, w, in_stride, in_pad / 16, s.h / 8);
#pragma unroll
                    for (int kt = 0; kt < kKTiles; ++kt)
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int nt = 2 * kt + (q >> 1), c = 2 * (q & 1);
                            const float2 gv = unpack_pair<T>(dy[0][kt][q]);
                            dy[0][kt][q] = pack_pair<T>(activate_grad(s.act, round_to<T>(acc[0][nt][c]), gv.x),
                                                        activate_grad(s.act, round_to<T>(acc[0][nt][c + 1]), gv.y));
                        }
                }
            }
            frags_to_smem(dz_tile, dz_stride, wrow, dy[0], out_pad / 16);

            // dgrad, warp-local: dy_prev = dz . W   (K = out, N = in)
            fill_acc<1>(acc, nullptr);
            warp_gemm_kn<T, 1>(acc, dy, w, in_stride, out_pad / 16, in_pad / 8);
            __syncthreads();  // dz tile and this layer's parked input are complete for all 128 rows

            // wgrad, cooperative: dW[out][in] += dz^T . a   (K = the tile's 128 rows)
            const int halves = (in_pad + 31) / 32;
            const int units = (out_pad / 16) * halves;
            slot -= units;
            if (warp < units) {
                const int mt = warp / halves, nh = warp % halves;
                float c[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) c[i][j] = 0.f;
                const T *dz_lane = dz_tile + (8 * (mtx >> 1) + r8) * dz_stride + 16 * mt + 8 * (mtx & 1);
                const T *in_lane = reinterpret_cast<const T *>(in_stash) + (8 * (mtx & 1) + r8) * in_stride + 32 * nh +
                                   8 * (mtx >> 1);
#pragma unroll
                for (int kt = 0; kt < kBwdRows / 16; ++kt) {
                    uint32_t af[4];
                    ldmatrix_x4_trans(af, dz_lane + 16 * kt * dz_stride);
#pragma unroll
                    for (int np = 0; np < 2; ++np) {
                        if (32 * nh + 16 * np < in_pad) {
                            uint32_t bf[4];
                            ldmatrix_x4_trans(bf, in_lane + 16 * kt * in_stride + 16 * np);
                            mma16816<T>(c[2 * np], af, bf[0], bf[1]);
                            mma16816<T>(c[2 * np + 1], af, bf[2], bf[3]);
                        }
                    }
                }
                float *mine = acc_slots + (slot + warp) * 512 + lane;
#pragma unroll
                for (int i = 0; i < 16; ++i) mine[32 * i] += c[i >> 2][i & 3];
            }
            if (s.has_bias) {
                const int col = threadIdx.x & 63, part = threadIdx.x >> 6;
                if (col < out_pad) {
                    float sum = 0.f;
                    for (int rr = 0; rr < kBwdRows / 4; ++rr)
                        sum += to_float<T>(dz_tile[(part * (kBwdRows / 4) + rr) * dz_stride + col]);
                    atomicAdd(dbias + l * kMaxDim + col, sum);
                }
            }
            // next layer's dy: rounded to the gradient dtype, no activation
            acc_to_frags<T, 1>(dy, acc, TH_ACT_NONE);
            __syncthreads();  // dz tile may be overwritten
        }
        if (gx) {
            float dxacc[kNTiles][4];
#pragma unroll
            for (int kt = 0; kt < kKTiles; ++kt)
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 v = unpack_pair<T>(dy[0][kt][q]);
                    dxacc[2 * kt + (q >> 1)][2 * (q & 1)] = v.x;
                    dxacc[2 * kt + (q >> 1)][2 * (q & 1) + 1] = v.y;
                }
            store_acc_rows<T>(gx, gx_stride, row0, n_rows, s.d_in, s.ki / 8, dxacc, gx_pairs_ok);
        }
    }

    // ---- flush this CTA's partial sums ----
    __syncthreads();
    const MlpGradWorkspace W = grad_workspace_layout(s, workspace);
    int slot = 0;
    for (int l = 0; l <= s.depth; ++l) {
        const int in_pad = l == 0 ? s.ki : s.h, out_pad = l == s.depth ? s.no : s.h;
        const int in_dim = l == 0 ? s.d_in : s.d_hid, out_dim = l == s.depth ? s.d_out : s.d_hid;
        const int halves = (in_pad + 31) / 32;
        const int units = (out_pad / 16) * halves;
        float *dst = W.base + (l == 0 ? W.w_in : (l == s.depth ? W.w_out : W.w_hid + (l - 1) * s.d_hid * s.d_hid));
        for (int e = threadIdx.x; e < units * 512; e += blockDim.x) {
            const int u = e / 512, i = (e % 512) / 32, ln = e % 32;
            const int mt = u / halves, nh = u % halves;
            const int m = 16 * mt + (ln >> 2) + 8 * ((i >> 1) & 1);
            const int n = 32 * nh + 8 * (i >> 2) + 2 * (ln & 3) + (i & 1);
            const float v = acc_slots[(slot + u) * 512 + i * 32 + ln];
            if (m < out_dim && n < in_dim && v != 0.f) atomicAdd(dst + m * in_dim + n, v);
        }
        slot += units;
        if (s.has_bias) {
            float *bdst = W.base + (l == 0 ? W.b_in : (l == s.depth ? W.b_out : W.b_hid + (l - 1) * s.d_hid));
            for (int c = threadIdx.x; c < out_dim; c += blockDim.x) atomicAdd(bdst + c, dbias[l * kMaxDim + c]);
        }
    }
}

// fp32 workspace -> gradient tensors in the parameter dtype (any destination may be null).
template <typename T>
__global__ void mlp_grad_convert_kernel(const MlpShape s, const float *__restrict__ ws, T *dw_in, T *dw_hid, T *dw_out,
                                        T *db_in, T *db_hid, T *db_out) {
    const MlpGradWorkspace W = grad_workspace_layout(s, const_cast<float *>(ws));
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < W.total; e += gridDim.x * blockDim.x) {
        T *dst;
        int off;
        if (e < W.w_hid) { dst = dw_in; off = e - W.w_in; }
        else if (e < W.w_out) { dst = dw_hid; off = e - W.w_hid; }
        else if (e < W.b_in) { dst = dw_out; off = e - W.w_out; }
        else if (e < W.b_hid) { dst = db_in; off = e - W.b_in; }
        else if (e < W.b_out) { dst = db_hid; off = e - W.b_hid; }
        else { dst = db_out; off = e - W.b_out; }
        if (dst) dst[off] = from_float<T>(ws[e]);
    }
}

// ---- host side ------------------------------------------------------------------------------

int make_shape(MlpShape &s, int d_in, int d_hid, int d_out, int depth, int act, bool has_bias) {
    if (d_in < 1 || d_in > kMaxDim) return fail(TH_ERR_UNSUPPORTED, "input dimension %d outside [1, %d]", d_in, kMaxDim);
    if (d_out < 1 || d_out > kMaxDim) return fail(TH_ERR_UNSUPPORTED, "output dimension %d outside [1, %d]", d_out, kMaxDim);
    if (d_hid < 16 || d_hid > kMaxDim || (d_hid & (d_hid - 1)))
        return fail(TH_ERR_UNSUPPORTED, "hidden dimension %d must be a power of two in [16, %d]", d_hid, kMaxDim);
    if (depth < 1) return fail(TH_ERR_BAD_ARG, "depth %d < 1", depth);
    if (act < TH_ACT_NONE || act > TH_ACT_RELU2) return fail(TH_ERR_BAD_ARG, "unknown activation code %d", act);
    s = MlpShape{d_in, d_hid, d_out, depth, pad16(d_in), d_hid, pad16(d_out), act, has_bias ? 1 : 0};
    return TH_OK;
}

int check_params(const MlpShape &s, const MlpParams &p, bool has_bias) {
    if (!p.w_in || !p.w_out || (s.depth > 1 && !p.w_hid)) return fail(TH_ERR_BAD_ARG, "null weight pointer");
    if (has_bias && (!p.b_in || !p.b_out || (s.depth > 1 && !p.b_hid)))
        return fail(TH_ERR_BAD_ARG, "biases must be all present or all null");
    return TH_OK;
}

bool pairs_ok(const void *p, int64_t stride, int cols) {
    return cols % 2 == 0 && stride % 2 == 0 && aligned_to(p, 4);
}

template <typename T>
int set_smem_limit(const void *kernel, int bytes) {
    if (bytes > kSmemLimit) return fail(TH_ERR_UNSUPPORTED, "layer stack needs %d bytes of shared memory, limit %d", bytes, kSmemLimit);
    return cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes),
                       "cudaFuncSetAttribute(max dynamic shared memory)");
}

template <typename T>
int launch_mlp_fwd(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, void *y, int64_t y_stride,
                   int64_t rows, cudaStream_t stream) {
    const MlpSmem L = mlp_smem_layout(s, false);
    if (int rc = set_smem_limit<T>(reinterpret_cast<const void *>(mlp_fwd_kernel<T>), L.total)) return rc;
    const long long tiles = (rows + kFwdRows - 1) / kFwdRows;
    const int per_sm = L.total <= 100 * 1024 ? 2 : 1;
    const unsigned grid = static_cast<unsigned>(tiles < static_cast<long long>(sm_count()) * per_sm ? tiles : sm_count() * per_sm);
    mlp_fwd_kernel<T><<<grid, kThreadsMlp, L.total, stream>>>(s, p, static_cast<const T *>(x), x_stride,
                                                             static_cast<T *>(y), y_stride, rows,
                                                             pairs_ok(x, x_stride, s.d_in), pairs_ok(y, y_stride, s.d_out));
    return launch_status("mlp_fwd_kernel launch");
}

template <typename T>
int launch_mlp_bwd(const MlpShape &s, const MlpParams &p, const void *x, int64_t x_stride, const void *go,
                   int64_t go_stride, void *gx, int64_t gx_stride, void *dw_in, void *db_in, void *dw_hid, void *db_hid,
                   void *dw_out, void *db_out, float *workspace, int64_t rows, cudaStream_t stream) {
    const MlpSmem L = mlp_smem_layout(s, true);
    const MlpGradWorkspace W = grad_workspace_layout(s, workspace);
    if (int rc = cuda_status(cudaMemsetAsync(workspace, 0, sizeof(float) * W.total, stream), "cudaMemsetAsync(workspace)")) return rc;
    const int tc = rows > 0 ? mlp_bwd_tc(s, p, x, x_stride, go, go_stride, gx, gx_stride, workspace, rows,
                                         std::is_same<T, __half>::value ? TH_F16 : TH_BF16, stream)
                            : kTcNotApplicable;
    if (tc != kTcNotApplicable && tc != TH_OK) return tc;
    if (rows > 0 && tc == kTcNotApplicable) {
        if (int rc = set_smem_limit<T>(reinterpret_cast<const void *>(mlp_bwd_kernel<T>), L.total)) return rc;
        const long long tiles = (rows + kBwdRows - 1) / kBwdRows;
        const unsigned grid = static_cast<unsigned>(tiles < sm_count() ? tiles : sm_count());
        mlp_bwd_kernel<T><<<grid, kThreadsMlp, L.total, stream>>>(
            s, p, static_cast<const T *>(x), x_stride, static_cast<const T *>(go), go_stride, static_cast<T *>(gx),
            gx_stride, workspace, rows, pairs_ok(x, x_stride, s.d_in), pairs_ok(go, go_stride, s.d_out),
            gx ? pairs_ok(gx, gx_stride, s.d_in) : 0);
        if (int rc = launch_status("mlp_bwd_kernel launch")) return rc;
    }
    mlp_grad_convert_kernel<T><<<(W.total + 255) / 256, 256, 0, stream>>>(
        s, workspace, static_cast<T *>(dw_in), static_cast<T *>(dw_hid), static_cast<T *>(dw_out),
        static_cast<T *>(db_in), static_cast<T *>(db_hid), static_cast<T *>(db_out));
    return launch_status("mlp_grad_convert_kernel launch");
}

}  // namespace
}  // namespace th

using namespace th;

extern "C" int64_t th_mlp_workspace_bytes(int d_in, int d_hidden, int d_out, int depth) {
    MlpShape s;
    if (make_shape(s, d_in, d_hidden, d_out, depth, TH_ACT_RELU, true)) return -1;
    return static_cast<int64_t>(sizeof(float)) * grad_workspace_layout(s, nullptr).total;
}

extern "C" int th_mlp_fwd(const void *x_dev, int64_t x_stride, const void *w_in_dev, const void *b_in_dev,
                          const void *w_hid_dev, const void *b_hid_dev, const void *w_out_dev, const void *b_out_dev,
                          void *out_dev, int64_t out_stride, int64_t rows, int d_in, int d_hidden, int d_out, int depth,
                          int activation, int dtype, int fp16_acc, void *stream) {
    (void)fp16_acc;  // accepted for signature parity; accumulation is always fp32
    if (rows < 0) return fail(TH_ERR_BAD_ARG, "negative row count");
    const bool has_bias = b_in_dev || b_hid_dev || b_out_dev;
    MlpShape s;
    if (int rc = make_shape(s, d_in, d_hidden, d_out, depth, activation, has_bias)) return rc;
    MlpParams p{w_in_dev, w_hid_dev, w_out_dev, b_in_dev, b_hid_dev, b_out_dev};
    if (int rc = check_params(s, p, has_bias)) return rc;
    if (rows == 0) return TH_OK;
    if (!x_dev || !out_dev) return fail(TH_ERR_BAD_ARG, "null input or output");
    if (x_stride < d_in || out_stride < d_out) return fail(TH_ERR_BAD_ARG, "row stride smaller than the row");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // tcgen05 kernels first; the mma.sync kernels take what they do not cover
    if (const int tc = mlp_fwd_tc(s, p, x_dev, x_stride, out_dev, out_stride, rows, dtype, st); tc != kTcNotApplicable) return tc;
    switch (dtype) {
        case TH_F16: return launch_mlp_fwd<__half>(s, p, x_dev, x_stride, out_dev, out_stride, rows, st);
        case TH_BF16: return launch_mlp_fwd<__nv_bfloat16>(s, p, x_dev, x_stride, out_dev, out_stride, rows, st);
        default: return fail(TH_ERR_UNSUPPORTED, "fused MLP kernels take float16 or bfloat16 (dtype code %d)", dtype);
    }
}

extern "C" int th_mlp_fwd_mse(const void *x_dev, int64_t x_stride, const void *w_in_dev, const void *b_in_dev,
                              const void *w_hid_dev, const void *b_hid_dev, const void *w_out_dev, const void *b_out_dev,
                              void *out_dev, int64_t out_stride, const void *target_dev, int64_t target_stride,
                              void *grad_dev, int64_t grad_stride, float *loss_sum_dev, float grad_scale, int64_t rows,
                              int d_in, int d_hidden, int d_out, int depth, int activation, int dtype, void *stream) {
    if (rows < 0) return fail(TH_ERR_BAD_ARG, "negative row count");
    const bool has_bias = b_in_dev || b_hid_dev || b_out_dev;
    MlpShape s;
    if (int rc = make_shape(s, d_in, d_hidden, d_out, depth, activation, has_bias)) return rc;
    MlpParams p{w_in_dev, w_hid_dev, w_out_dev, b_in_dev, b_hid_dev, b_out_dev};
    if (int rc = check_params(s, p, has_bias)) return rc;
    if (rows == 0) return TH_OK;
    if (!x_dev || !target_dev || !grad_dev) return fail(TH_ERR_BAD_ARG, "null input, target or gradient");
    if (x_stride < d_in || target_stride < d_out || grad_stride < d_out || (out_dev && out_stride < d_out))
        return fail(TH_ERR_BAD_ARG, "row stride smaller than the row");
    const MseArgs mse{target_dev, target_stride, grad_dev, grad_stride, loss_sum_dev, grad_scale};
    const int rc = mlp_fwd_mse_tc(s, p, x_dev, x_stride, out_dev, out_stride, mse, rows, dtype, static_cast<cudaStream_t>(stream));
    if (rc == kTcNotApplicable)
        return fail(TH_ERR_UNSUPPORTED, "fused forward + MSE needs float16 / bfloat16 rows of whole 16-byte chunks "
                                        "(d_in, d_out multiples of 8, aligned) and a network the multi-slot kernel holds");
    return rc;
}

extern "C" int th_mlp_bwd(const void *x_dev, int64_t x_stride, const void *w_in_dev, const void *b_in_dev,
                          const void *w_hid_dev, const void *b_hid_dev, const void *w_out_dev, const void *b_out_dev,
                          const void *grad_out_dev, int64_t go_stride, void *grad_x_dev, int64_t gx_stride,
                          void *grad_w_in_dev, void *grad_b_in_dev, void *grad_w_hid_dev, void *grad_b_hid_dev,
                          void *grad_w_out_dev, void *grad_b_out_dev, void *workspace_dev, int64_t workspace_bytes,
                          int64_t rows, int d_in, int d_hidden, int d_out, int depth, int activation, int dtype,
                          int fp16_acc, void *stream) {
    (void)fp16_acc;
    if (rows < 0) return fail(TH_ERR_BAD_ARG, "negative row count");
    const bool has_bias = b_in_dev || b_hid_dev || b_out_dev;
    MlpShape s;
    if (int rc = make_shape(s, d_in, d_hidden, d_out, depth, activation, has_bias)) return rc;
    MlpParams p{w_in_dev, w_hid_dev, w_out_dev, b_in_dev, b_hid_dev, b_out_dev};
    if (int rc = check_params(s, p, has_bias)) return rc;
    const int64_t need = static_cast<int64_t>(sizeof(float)) * grad_workspace_layout(s, nullptr).total;
    if (!workspace_dev || workspace_bytes < need)
        return fail(TH_ERR_WORKSPACE, "workspace of %lld bytes needed, %lld given", (long long)need, (long long)workspace_bytes);
    if (rows > 0) {
        if (!x_dev || !grad_out_dev) return fail(TH_ERR_BAD_ARG, "null input or gradient");
        if (x_stride < d_in || go_stride < d_out || (grad_x_dev && gx_stride < d_in))
            return fail(TH_ERR_BAD_ARG, "row stride smaller than the row");
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float *ws = static_cast<float *>(workspace_dev);
    switch (dtype) {
        case TH_F16:
            return launch_mlp_bwd<__half>(s, p, x_dev, x_stride, grad_out_dev, go_stride, grad_x_dev, gx_stride,
                                          grad_w_in_dev, grad_b_in_dev, grad_w_hid_dev, grad_b_hid_dev, grad_w_out_dev,
                                          grad_b_out_dev, ws, rows, st);
        case TH_BF16:
            return launch_mlp_bwd<__nv_bfloat16>(s, p, x_dev, x_stride, grad_out_dev, go_stride, grad_x_dev, gx_stride,
                                                 grad_w_in_dev, grad_b_in_dev, grad_w_hid_dev, grad_b_hid_dev,
                                                 grad_w_out_dev, grad_b_out_dev, ws, rows, st);
        default: return fail(TH_ERR_UNSUPPORTED, "fused MLP kernels take float16 or bfloat16 (dtype code %d)", dtype);
    }
}

// ---- backward without caller-provided scratch ------------------------------------------------
//
// th_mlp_bwd needs one fp32 per parameter of scratch and asks the caller for it.  Some callers
// have no way to get device memory at call time: a plug-in inside a host application that
// handed the whole device to its own memory pool, a latency-critical loop that must not run
// into the device-wide synchronisation cudaMalloc implies, or a plain C caller with no
// allocator at hand.  For them the scratch below is part of the library image: every GPU
// that loads the library holds these 256 KB until the process exits.

namespace {

constexpr int kStaticScratchFloats = 64 * 1024;  // 256 KB: e.g. fourteen 64 x 64 layers

static __device__ __align__(256) float g_mlp_bwd_scratch[kStaticScratchFloats];

// In host code `g_mlp_bwd_scratch` is only a handle for the runtime, not a device address, so the
// address the kernels get is looked up once per device (with that device current) and cached.
int static_scratch_address(float **out) {
    static std::mutex guard;
    static float *cache[64] = {nullptr};
    int dev = -1;
    if (int rc = th::cuda_status(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    if (dev < 0 || dev >= 64) return th::fail(TH_ERR_UNSUPPORTED, "device ordinal %d outside [0, 64)", dev);
    std::lock_guard<std::mutex> lock(guard);
    if (!cache[dev]) {
        void *address = nullptr;
        if (int rc = th::cuda_status(cudaGetSymbolAddress(&address, g_mlp_bwd_scratch), "cudaGetSymbolAddress(scratch)"))
            return rc;
        cache[dev] = static_cast<float *>(address);
    }
    *out = cache[dev];
    return TH_OK;
}

}  // namespace

extern "C" int64_t th_mlp_bwd_static_max_bytes(void) { return static_cast<int64_t>(sizeof(float)) * kStaticScratchFloats; }

extern "C" int th_mlp_bwd_static(const void *x_dev, int64_t x_stride, const void *w_in_dev, const void *b_in_dev,
                                 const void *w_hid_dev, const void *b_hid_dev, const void *w_out_dev,
                                 const void *b_out_dev, const void *grad_out_dev, int64_t go_stride, void *grad_x_dev,
                                 int64_t gx_stride, void *grad_w_in_dev, void *grad_b_in_dev, void *grad_w_hid_dev,
                                 void *grad_b_hid_dev, void *grad_w_out_dev, void *grad_b_out_dev, int64_t rows,
                                 int d_in, int d_hidden, int d_out, int depth, int activation, int dtype, int fp16_acc,
                                 void *stream) {
    const int64_t need = th_mlp_workspace_bytes(d_in, d_hidden, d_out, depth);
    if (need < 0) return fail(TH_ERR_UNSUPPORTED, "unsupported layer shape %d -> %d x %d -> %d", d_in, depth, d_hidden, d_out);
    if (need > th_mlp_bwd_static_max_bytes())
        return fail(TH_ERR_WORKSPACE,
                    "this network needs %lld bytes of scratch, the built-in buffer holds %lld: use th_mlp_bwd with caller scratch",
                    (long long)need, (long long)th_mlp_bwd_static_max_bytes());
    float *scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    // same launch sequence as th_mlp_bwd; it zero-fills the part of the scratch it uses first
    return th_mlp_bwd(x_dev, x_stride, w_in_dev, b_in_dev, w_hid_dev, b_hid_dev, w_out_dev, b_out_dev, grad_out_dev,
                      go_stride, grad_x_dev, gx_stride, grad_w_in_dev, grad_b_in_dev, grad_w_hid_dev, grad_b_hid_dev,
                      grad_w_out_dev, grad_b_out_dev, scratch, need, rows, d_in, d_hidden, d_out, depth, activation,
                      dtype, fp16_acc, stream);
}
