// Shared helpers for the kmb200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <math.h>

#include "../../include/kmb200.h"

namespace kmb {

void set_error(const char* fmt, ...);

#define KMB_CHECK_CUDA(expr)                                                             \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess) {                                                             \
      kmb::set_error("%s failed at %s:%d: %s", #expr, __FILE__, __LINE__,               \
                     cudaGetErrorString(_e));                                            \
      return KMB_ERR_CUDA;                                                               \
    }                                                                                    \
  } while (0)

#define KMB_REQUIRE(cond, ...)                                                           \
  do {                                                                                   \
    if (!(cond)) {                                                                       \
      kmb::set_error(__VA_ARGS__);                                                       \
      return KMB_ERR_INVALID;                                                            \
    }                                                                                    \
  } while (0)

#define KMB_CHECK_LAUNCH() KMB_CHECK_CUDA(cudaGetLastError())

// Runs `body` with T bound to float or double.
#define KMB_DISPATCH_DTYPE(dtype, ...)                                                   \
  do {                                                                                   \
    if ((dtype) == KMB_F32) {                                                            \
      using T = float;                                                                   \
      __VA_ARGS__                                                                        \
    } else if ((dtype) == KMB_F64) {                                                     \
      using T = double;                                                                  \
      __VA_ARGS__                                                                        \
    } else {                                                                             \
      kmb::set_error("dtype must be KMB_F32 or KMB_F64, got %d", (int)(dtype));          \
      return KMB_ERR_INVALID;                                                            \
    }                                                                                    \
  } while (0)

inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
      v = 148;
    cached[dev] = v;
  }
  return cached[dev];
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Lanes that cooperate on one sample row in the row-scan kernels: the smallest power of
// two >= d, capped at 32.
inline int lanes_per_row(int d) {
  int g = 1;
  while (g < d && g < 32) g <<= 1;
  return g;
}

template <typename T>
__device__ __forceinline__ T inf_value();
template <>
__device__ __forceinline__ float inf_value<float>() { return __int_as_float(0x7f800000); }
template <>
__device__ __forceinline__ double inf_value<double>() {
  return __longlong_as_double(0x7ff0000000000000LL);
}

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum of `v` over the block, valid in thread 0. `red` holds >= 32 doubles of shared memory.
__device__ __forceinline__ double block_sum(double v, double* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  v = (threadIdx.x < nw) ? red[threadIdx.x] : 0.0;
  if (wid == 0) v = warp_sum(v);
  return v;
}

}  // namespace kmb
