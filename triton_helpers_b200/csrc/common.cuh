// Shared host/device helpers for libth_b200.so.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/th_b200.h"

namespace th {

// ---- error reporting -----------------------------------------------------------------------
// One message per host thread; set on every non-zero return of an entry point.
char *last_error_buffer();
constexpr int kErrorBufferBytes = 512;

inline int fail(int code, const char *fmt, ...) {
    va_list args;
    va_start(args, fmt);
    vsnprintf(last_error_buffer(), kErrorBufferBytes, fmt, args);
    va_end(args);
    return code;
}

inline int cuda_status(cudaError_t err, const char *what) {
    if (err == cudaSuccess) return TH_OK;
    return fail(static_cast<int>(err), "%s: %s", what, cudaGetErrorString(err));
}

// After every kernel launch: counts it (th_launch_count) and reports a launch error, if any.
void note_launch();
inline int launch_status(const char *what) {
    note_launch();
    return cuda_status(cudaGetLastError(), what);
}

// Number of SMs of the current device (cached per device).
int sm_count();

inline bool aligned_to(const void *p, size_t bytes) { return (reinterpret_cast<uintptr_t>(p) % bytes) == 0; }

// ---- dtype helpers -------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

inline size_t dtype_bytes(int code) { return code == TH_F32 ? 4 : 2; }

}  // namespace th
