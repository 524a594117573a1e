// Test hook for the distance contraction alone: out = X * Y^T.
// Stands for make_matmul_2d_kernel of sklearn_numba_dpex/common/matmul.py:13-489, which the
// KMeans path itself never calls.  The CUDA-core variant below is a plain shared-memory
// tiled product; the tensor-core variant reuses the 3xTF32 pipeline of the fused step.
#include "kmb_common.cuh"

namespace kmb {

int lloyd_tc_matmul(const float* X, const float* Y, float* out, int64_t m, int n, int kdim,
                    void* workspace, size_t workspace_bytes, cudaStream_t stream);
bool lloyd_tc_supported(int dtype, int64_t n, int d, int k);

constexpr int MM_TILE = 32;

template <typename T>
__global__ void __launch_bounds__(MM_TILE * MM_TILE / 4)
matmul_nt_kernel(const T* __restrict__ X, const T* __restrict__ Y, T* __restrict__ out, int64_t m,
                 int n, int kdim) {
  // 32x32 output tile, 256 threads, 4 outputs (one column, 4 rows) per thread.
  __shared__ T Xs[MM_TILE][MM_TILE + 1];
  __shared__ T Ys[MM_TILE][MM_TILE + 1];
  const int tx = threadIdx.x % MM_TILE, ty = threadIdx.x / MM_TILE;  // ty in [0, 8)
  const int64_t i0 = (int64_t)blockIdx.y * MM_TILE;
  const int j0 = blockIdx.x * MM_TILE;
  T acc[4] = {T(0), T(0), T(0), T(0)};
  for (int k0 = 0; k0 < kdim; k0 += MM_TILE) {
    for (int r = ty; r < MM_TILE; r += 8) {
      Xs[r][tx] = (i0 + r < m && k0 + tx < kdim) ? X[(i0 + r) * (int64_t)kdim + k0 + tx] : T(0);
      Ys[r][tx] = (j0 + r < n && k0 + tx < kdim) ? Y[(int64_t)(j0 + r) * kdim + k0 + tx] : T(0);
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < MM_TILE; ++kk) {
      const T b = Ys[tx][kk];
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[q] = fma(Xs[ty + 8 * q][kk], b, acc[q]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int64_t i = i0 + ty + 8 * q;
    if (i < m && j0 + tx < n) out[i * (int64_t)n + j0 + tx] = acc[q];
  }
}

}  // namespace kmb

using namespace kmb;

extern "C" int kmb_matmul_nt(int dtype, int algo, const void* X, const void* Y, void* out,
                             int64_t m, int n, int kdim, void* workspace, size_t workspace_bytes,
                             void* stream) {
  KMB_REQUIRE(X && Y && out, "kmb_matmul_nt: NULL argument");
  KMB_REQUIRE(m >= 0 && n > 0 && kdim > 0, "kmb_matmul_nt: bad sizes");
  if (m == 0) return KMB_OK;
  if (algo == KMB_ALGO_TF32X3) {
    if (!lloyd_tc_supported(dtype, m, kdim, n)) {
      set_error("kmb_matmul_nt: KMB_ALGO_TF32X3 does not support dtype=%d m=%lld n=%d k=%d", dtype,
                (long long)m, n, kdim);
      return KMB_ERR_UNSUPPORTED;
    }
    return lloyd_tc_matmul((const float*)X, (const float*)Y, (float*)out, m, n, kdim, workspace,
                           workspace_bytes, (cudaStream_t)stream);
  }
  KMB_REQUIRE(ceil_div(m, MM_TILE) <= 65535, "kmb_matmul_nt: m too large for the test hook");
  KMB_DISPATCH_DTYPE(dtype, {
    dim3 grid((unsigned)ceil_div(n, MM_TILE), (unsigned)ceil_div(m, MM_TILE));
    matmul_nt_kernel<T><<<grid, MM_TILE * MM_TILE / 4, 0, (cudaStream_t)stream>>>(
        (const T*)X, (const T*)Y, (T*)out, m, n, kdim);
    KMB_CHECK_LAUNCH();
  });
  return KMB_OK;
}

// ---- measurement hook: FMA issue rate of the CUDA cores ------------------------------------
// Every thread runs 16 independent register-resident FMA chains; nothing touches memory until
// the final store, so the figure is the pipe's own ceiling for the CUDA-core step.
namespace kmb {
template <typename T>
__global__ void __launch_bounds__(256) fma_peak_kernel(T* out, int iters, T a, T b) {
  T acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = (T)(threadIdx.x + i);
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = fma(acc[i], a, b);
  }
  T s = T(0);
#pragma unroll
  for (int i = 0; i < 16; ++i) s += acc[i];
  if (s == (T)-1.2345) out[blockIdx.x * blockDim.x + threadIdx.x] = s;   // keeps the chains alive
}
}  // namespace kmb

extern "C" int kmb_measure_fma_peak(int dtype, int repeats, double* tflops, void* scratch,
                                    void* stream) {
  KMB_REQUIRE(tflops && scratch && repeats >= 1, "kmb_measure_fma_peak: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  const int blocks = sm_count() * 8, threads = 256;
  const int iters = dtype == KMB_F32 ? 16384 : 2048;
  cudaEvent_t e0, e1;
  KMB_CHECK_CUDA(cudaEventCreate(&e0));
  KMB_CHECK_CUDA(cudaEventCreate(&e1));
  double best = 0.0;
  int rc = KMB_OK;
  for (int r = 0; r < repeats + 2 && rc == KMB_OK; ++r) {
    cudaEventRecord(e0, s);
    if (dtype == KMB_F32)
      fma_peak_kernel<float><<<blocks, threads, 0, s>>>((float*)scratch, iters, 0.999f, 0.001f);
    else if (dtype == KMB_F64)
      fma_peak_kernel<double><<<blocks, threads, 0, s>>>((double*)scratch, iters, 0.999, 0.001);
    else {
      set_error("dtype must be KMB_F32 or KMB_F64, got %d", dtype);
      rc = KMB_ERR_INVALID;
      break;
    }
    cudaEventRecord(e1, s);
    if (cudaEventSynchronize(e1) != cudaSuccess || cudaGetLastError() != cudaSuccess) {
      set_error("kmb_measure_fma_peak: kernel failed");
      rc = KMB_ERR_CUDA;
      break;
    }
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    const double tf = 2.0 * 16.0 * iters * (double)blocks * threads / (ms * 1e-3) / 1e12;
    if (r >= 2 && tf > best) best = tf;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  *tflops = best;
  return rc;
}
