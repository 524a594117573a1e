// Shared helpers for the kmb200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_pipeline.h>
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

// Control block shared by the fused step and the finalize kernel.  It opens the Lloyd
// workspace and is cleared by kmb_lloyd_workspace_init, never by a step.
struct LloydControl {
  int wait_error;        // raised by a bounded wait of the tensor-core kernel that ran out; sticky
  unsigned int ticket;   // CTAs of the finalize kernel that have finished; reset by the last one
};

// Layout of the Lloyd workspace: [control block, 256 B | C_hi | C_lo | padded half norms], the
// two matrices (k_pad x d_pad, fp32, rounded to tf32) being the B operands of the tensor-core
// step.  k_pad = k rounded up to 128, d_pad = d rounded up to 32.
struct LloydWorkspace {
  LloydControl* ctl;
  float* chi;
  float* clo;
  float* h_pad;
  int k_pad, d_pad;
  size_t bytes;          // from the caller's pointer to the end of the last array
};

// The tensor-core step can fold the half norms into the contraction when the padded feature
// count leaves two spare features: the sample operand carries 1.0 in features d and d + 1, the
// centroid operands carry -h split over the same two features, and the accumulator comes out
// as x.c - h directly (one argmax, no half-norm loads, no subtraction per element).
// Index of the first of the two fold features, or -1 when the step does not fold.  `pad` trailing
// features of the rows are zero padding of the caller (0..3): two or more of them take the fold
// features; otherwise they follow the data, which needs spare room in the last 32-feature chunk.
__host__ __device__ inline int lloyd_tc_fold_at(int d, int pad) {
  if (d % 4 != 0) return -1;
  if (pad >= 2 && pad <= 3 && d >= 4) return d - pad;
  return ((d % 32) != 0 && (d % 32) <= 28) ? d : -1;
}

// Round-to-nearest (ties away) to the 10-bit mantissa of tf32.
__device__ __forceinline__ float tf32_rna(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// Values of the two fold features of a centroid with half norm h: (hi, lo) pairs, each a tf32
// number, whose sum is -h to beyond fp32 precision.
__device__ __forceinline__ void lloyd_tc_fold_values(float h, float (&hi)[2], float (&lo)[2]) {
  const float nh = -h;
  hi[0] = tf32_rna(nh);
  const float r0 = nh - hi[0];
  lo[0] = tf32_rna(r0);
  const float r1 = r0 - lo[0];
  hi[1] = tf32_rna(r1);
  lo[1] = tf32_rna(r1 - hi[1]);
}

inline LloydWorkspace lloyd_carve(void* workspace, int d, int k) {
  LloydWorkspace w;
  w.d_pad = (d + 31) / 32 * 32;
  w.k_pad = (k + 127) / 128 * 128;
  unsigned char* p = (unsigned char*)(((uintptr_t)workspace + 255) & ~(uintptr_t)255);
  const size_t mat = ((size_t)w.k_pad * w.d_pad * sizeof(float) + 255) / 256 * 256;
  const size_t hb = ((size_t)w.k_pad * sizeof(float) + 255) / 256 * 256;
  w.ctl = (LloydControl*)p;
  w.chi = (float*)(p + 256);
  w.clo = (float*)(p + 256 + mat);
  w.h_pad = (float*)(p + 256 + 2 * mat);
  w.bytes = (size_t)(p - (unsigned char*)workspace) + 256 + 2 * mat + hb;
  return w;
}

// 16-byte vectors of consecutive features: 4 floats or 2 doubles per lane.
template <typename T>
struct RowVec;
template <>
struct RowVec<float> {
  static constexpr int VEC = 4;
};
template <>
struct RowVec<double> {
  static constexpr int VEC = 2;
};

// v[j] = p[f0 + j] for f0 + j < d, else 0.  `aligned` = the row pitch and the base pointer
// allow one 16-byte load (d a multiple of VEC, base 16-byte aligned).
template <typename T>
__device__ __forceinline__ void load_row_vec(const T* __restrict__ p, int f0, int d, bool aligned,
                                             T (&v)[RowVec<T>::VEC]) {
  constexpr int VEC = RowVec<T>::VEC;
  if (aligned && f0 + VEC <= d) {
    if constexpr (sizeof(T) == 4) {
      const float4 q = *reinterpret_cast<const float4*>(p + f0);
      v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    } else {
      const double2 q = *reinterpret_cast<const double2*>(p + f0);
      v[0] = q.x; v[1] = q.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < VEC; ++j) v[j] = (f0 + j < d) ? p[f0 + j] : T(0);
  }
}

// Row pitch (in elements) of a staged tile: the row length rounded up so that the pitch is an
// odd number of 16-byte chunks (or of words when rows cannot be copied in 16-byte chunks), which
// makes "every thread reads chunk q of its own row" free of bank conflicts while all threads
// walk the features in the same ascending order.
template <typename T>
__host__ __device__ inline int tile_row_pitch(int d, bool vec) {
  constexpr int VEC = RowVec<T>::VEC;
  if (vec) return (((d + VEC - 1) / VEC) | 1) * VEC;
  return d | 1;
}

// Copies rows [r0, r0 + rows) of X (rows x d, contiguous in global memory) to a shared-memory
// tile with row pitch `ld`.  With `vec` (d a multiple of VEC and X 16-byte aligned) the copy is
// made of 16-byte asynchronous copies; otherwise of plain loads.  Every thread commits exactly
// one group per call (possibly empty).
template <typename T, int THREADS>
__device__ __forceinline__ void issue_row_tile(T* __restrict__ dst, const T* __restrict__ X,
                                               int64_t r0, int rows, int d, int ld, bool vec) {
  constexpr int VEC = RowVec<T>::VEC;
  if (rows > 0) {
    const T* src = X + r0 * (int64_t)d;
    if (vec) {
      const int nq = d / VEC;
      const int total = rows * nq;
      for (int ch = threadIdx.x; ch < total; ch += THREADS) {
        const int row = ch / nq, q = ch - row * nq;
        __pipeline_memcpy_async(dst + (size_t)row * ld + q * VEC, src + (size_t)ch * VEC, 16);
      }
    } else {
      const int total = rows * d;
      for (int e = threadIdx.x; e < total; e += THREADS) {
        const int row = e / d, f = e - row * d;
        dst[(size_t)row * ld + f] = src[e];
      }
    }
  }
  __pipeline_commit();
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
