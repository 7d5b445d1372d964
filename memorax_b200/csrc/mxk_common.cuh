// Shared host/device helpers for the mxk kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "mxk.h"

namespace mxk {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized against this

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? MXK_OK : static_cast<int>(e);
}

// 16-byte streaming accesses: data that is touched once should not displace
// reusable lines (the carried state, chunk tiles) from L1/L2.
__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ float2 ld_stream(const float2* p) { return __ldcs(p); }
__device__ __forceinline__ float ld_stream(const float* p) { return __ldcs(p); }
__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4* p, float4 v) { __stcs(p, v); }
__device__ __forceinline__ void st_stream(float2* p, float2 v) { __stcs(p, v); }
__device__ __forceinline__ void st_stream(float* p, float v) { __stcs(p, v); }

}  // namespace mxk
