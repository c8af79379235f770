// The two element-wise steps either side of the fused operators in a neural-field training
// step: the scaled MSE gradient that feeds the MLP backward, and an Adam update for 16-bit
// parameters with fp32 moments.  triton_helpers has no counterpart (its benchmarks stop at
// forward/backward, triton_helpers/benchmark.py:175-187); these exist so the data-parallel
// training step never leaves hand-written kernels between the forward and the next step.
//
// Both are pure streaming kernels: 128-bit loads and stores, grid-stride over 8-element packets.
#include "common.cuh"

namespace th {
namespace {

constexpr int kOptThreads = 256;

template <typename T>
struct Vec8 {
    T v[8];
};
template <>
struct __align__(16) Vec8<__half> {
    __half v[8];
};
template <>
struct __align__(16) Vec8<__nv_bfloat16> {
    __nv_bfloat16 v[8];
};
template <>
struct __align__(32) Vec8<float> {
    float v[8];
};

// grad = (pred - target) * grad_scale ;  *loss_sum += sum (pred - target)^2
template <typename T>
__global__ void __launch_bounds__(kOptThreads)
mse_grad_kernel(const T *__restrict__ pred, const T *__restrict__ target, T *__restrict__ grad,
                float *__restrict__ loss_sum, long long n, float grad_scale) {
    float local = 0.f;
    const long long packets = n / 8;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < packets;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const Vec8<T> p = reinterpret_cast<const Vec8<T> *>(pred)[i];
        const Vec8<T> t = reinterpret_cast<const Vec8<T> *>(target)[i];
        Vec8<T> g;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float d = to_float<T>(p.v[k]) - to_float<T>(t.v[k]);
            local += d * d;
            g.v[k] = from_float<T>(d * grad_scale);
        }
        reinterpret_cast<Vec8<T> *>(grad)[i] = g;
    }
    // ragged tail
    for (long long i = packets * 8 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const float d = to_float<T>(pred[i]) - to_float<T>(target[i]);
        local += d * d;
        grad[i] = from_float<T>(d * grad_scale);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) local += __shfl_xor_sync(0xffffffffu, local, off);
    __shared__ float warp_sum[kOptThreads / 32];
    if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < kOptThreads / 32; ++w) total += warp_sum[w];
        if (loss_sum) atomicAdd(loss_sum, total);
    }
}

struct AdamScalars {
    float lr, beta1, beta2, eps;
    float bias1, bias2_sqrt;  // 1 - beta1^t, sqrt(1 - beta2^t)
    float grad_scale;         // multiplies the stored gradient (1 / loss scale / world size)
    int zero_grad;            // write zeros back into the gradient buffer
};

// One element.  A gradient that is not finite (a 16-bit sum that overflowed, a NaN from upstream)
// leaves the parameter and both moments as they were and is counted in `skipped`: one bad element
// must not turn into inf / inf = NaN in the parameter and poison every later step.
template <typename T>
__device__ __forceinline__ T adam_one(T p, T g_in, float &m, float &v, const AdamScalars &a, int &skipped) {
    const float g = to_float<T>(g_in) * a.grad_scale;
    if (!isfinite(g)) {
        ++skipped;
        return p;
    }
    m = a.beta1 * m + (1.f - a.beta1) * g;
    v = a.beta2 * v + (1.f - a.beta2) * g * g;
    const float denom = sqrtf(v) / a.bias2_sqrt + a.eps;
    return from_float<T>(to_float<T>(p) - (a.lr / a.bias1) * (m / denom));
}

template <typename T>
__global__ void __launch_bounds__(kOptThreads)
adam_kernel(T *__restrict__ param, T *__restrict__ grad, float *__restrict__ exp_avg, float *__restrict__ exp_avg_sq,
            long long n, const AdamScalars a, int *__restrict__ skipped_total) {
    int skipped = 0;
    const long long packets = n / 8;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < packets;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        Vec8<T> p = reinterpret_cast<Vec8<T> *>(param)[i];
        const Vec8<T> g = reinterpret_cast<const Vec8<T> *>(grad)[i];
        Vec8<float> m = reinterpret_cast<Vec8<float> *>(exp_avg)[i];
        Vec8<float> v = reinterpret_cast<Vec8<float> *>(exp_avg_sq)[i];
#pragma unroll
        for (int k = 0; k < 8; ++k) p.v[k] = adam_one<T>(p.v[k], g.v[k], m.v[k], v.v[k], a, skipped);
        reinterpret_cast<Vec8<T> *>(param)[i] = p;
        reinterpret_cast<Vec8<float> *>(exp_avg)[i] = m;
        reinterpret_cast<Vec8<float> *>(exp_avg_sq)[i] = v;
        if (a.zero_grad) {
            Vec8<T> z;
#pragma unroll
            for (int k = 0; k < 8; ++k) z.v[k] = from_float<T>(0.f);
            reinterpret_cast<Vec8<T> *>(grad)[i] = z;
        }
    }
    for (long long i = packets * 8 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        param[i] = adam_one<T>(param[i], grad[i], exp_avg[i], exp_avg_sq[i], a, skipped);
        if (a.zero_grad) grad[i] = from_float<T>(0.f);
    }
    if (skipped_total && skipped) atomicAdd(skipped_total, skipped);
}

// dst[i] = round(src[i] * scale): the float32 sums a backward pass left in its workspace, normalised
// and rounded into a 16-bit (or float32) gradient buffer.
template <typename T>
__global__ void __launch_bounds__(kOptThreads)
scale_cast_kernel(const float *__restrict__ src, T *__restrict__ dst, long long n, float scale) {
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        dst[i] = from_float<T>(src[i] * scale);
}

unsigned stream_grid(long long n) {
    const long long blocks = (n / 8 + kOptThreads - 1) / kOptThreads + 1;
    const long long cap = static_cast<long long>(sm_count()) * 8;
    return static_cast<unsigned>(blocks < cap ? blocks : cap);
}

}  // namespace
}  // namespace th

using namespace th;

extern "C" int th_mse_grad(const void *pred_dev, const void *target_dev, void *grad_dev, float *loss_sum_dev,
                           int64_t n_elems, float grad_scale, int dtype, void *stream) {
    if (n_elems < 0) return fail(TH_ERR_BAD_ARG, "negative element count");
    if (n_elems == 0) return TH_OK;
    if (!pred_dev || !target_dev || !grad_dev) return fail(TH_ERR_BAD_ARG, "null tensor pointer");
    if (!aligned_to(pred_dev, 32) || !aligned_to(target_dev, 32) || !aligned_to(grad_dev, 32))
        return fail(TH_ERR_ALIGNMENT, "tensors must be 32-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = stream_grid(n_elems);
    switch (dtype) {
        case TH_F32:
            mse_grad_kernel<float><<<grid, kOptThreads, 0, st>>>(static_cast<const float *>(pred_dev), static_cast<const float *>(target_dev),
                                                                  static_cast<float *>(grad_dev), loss_sum_dev, n_elems, grad_scale);
            break;
        case TH_F16:
            mse_grad_kernel<__half><<<grid, kOptThreads, 0, st>>>(static_cast<const __half *>(pred_dev), static_cast<const __half *>(target_dev),
                                                                   static_cast<__half *>(grad_dev), loss_sum_dev, n_elems, grad_scale);
            break;
        case TH_BF16:
            mse_grad_kernel<__nv_bfloat16><<<grid, kOptThreads, 0, st>>>(static_cast<const __nv_bfloat16 *>(pred_dev), static_cast<const __nv_bfloat16 *>(target_dev),
                                                                          static_cast<__nv_bfloat16 *>(grad_dev), loss_sum_dev, n_elems, grad_scale);
            break;
        default: return fail(TH_ERR_BAD_ARG, "unknown dtype %d", dtype);
    }
    return launch_status("mse_grad_kernel launch");
}

extern "C" int th_adam_step(void *param_dev, void *grad_dev, float *exp_avg_dev, float *exp_avg_sq_dev, int64_t n_elems,
                            float lr, float beta1, float beta2, float eps, int step, float grad_scale, int zero_grad,
                            int dtype, int *skipped_dev, void *stream) {
    if (n_elems < 0) return fail(TH_ERR_BAD_ARG, "negative element count");
    if (step < 1) return fail(TH_ERR_BAD_ARG, "step counts from 1");
    if (n_elems == 0) return TH_OK;
    if (!param_dev || !grad_dev || !exp_avg_dev || !exp_avg_sq_dev) return fail(TH_ERR_BAD_ARG, "null tensor pointer");
    if (!aligned_to(param_dev, 32) || !aligned_to(grad_dev, 32) || !aligned_to(exp_avg_dev, 32) || !aligned_to(exp_avg_sq_dev, 32))
        return fail(TH_ERR_ALIGNMENT, "tensors must be 32-byte aligned");
    AdamScalars a{lr, beta1, beta2, eps, 0.f, 0.f, grad_scale, zero_grad};
    a.bias1 = static_cast<float>(1.0 - pow(static_cast<double>(beta1), step));
    a.bias2_sqrt = static_cast<float>(sqrt(1.0 - pow(static_cast<double>(beta2), step)));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = stream_grid(n_elems);
    switch (dtype) {
        case TH_F32:
            adam_kernel<float><<<grid, kOptThreads, 0, st>>>(static_cast<float *>(param_dev), static_cast<float *>(grad_dev), exp_avg_dev, exp_avg_sq_dev, n_elems, a, skipped_dev);
            break;
        case TH_F16:
            adam_kernel<__half><<<grid, kOptThreads, 0, st>>>(static_cast<__half *>(param_dev), static_cast<__half *>(grad_dev), exp_avg_dev, exp_avg_sq_dev, n_elems, a, skipped_dev);
            break;
        case TH_BF16:
            adam_kernel<__nv_bfloat16><<<grid, kOptThreads, 0, st>>>(static_cast<__nv_bfloat16 *>(param_dev), static_cast<__nv_bfloat16 *>(grad_dev), exp_avg_dev, exp_avg_sq_dev, n_elems, a, skipped_dev);
            break;
        default: return fail(TH_ERR_BAD_ARG, "unknown dtype %d", dtype);
    }
    return launch_status("adam_kernel launch");
}

extern "C" int th_scale_cast(const float *src_dev, void *dst_dev, int64_t n_elems, float scale, int dtype, void *stream) {
    if (n_elems < 0) return fail(TH_ERR_BAD_ARG, "negative element count");
    if (n_elems == 0) return TH_OK;
    if (!src_dev || !dst_dev) return fail(TH_ERR_BAD_ARG, "null tensor pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long blocks = (n_elems + kOptThreads - 1) / kOptThreads;
    const long long cap = static_cast<long long>(sm_count()) * 8;
    const unsigned grid = static_cast<unsigned>(blocks < cap ? blocks : cap);
    switch (dtype) {
        case TH_F32: scale_cast_kernel<float><<<grid, kOptThreads, 0, st>>>(src_dev, static_cast<float *>(dst_dev), n_elems, scale); break;
        case TH_F16: scale_cast_kernel<__half><<<grid, kOptThreads, 0, st>>>(src_dev, static_cast<__half *>(dst_dev), n_elems, scale); break;
        case TH_BF16: scale_cast_kernel<__nv_bfloat16><<<grid, kOptThreads, 0, st>>>(src_dev, static_cast<__nv_bfloat16 *>(dst_dev), n_elems, scale); break;
        default: return fail(TH_ERR_BAD_ARG, "unknown dtype %d", dtype);
    }
    return launch_status("scale_cast_kernel launch");
}
