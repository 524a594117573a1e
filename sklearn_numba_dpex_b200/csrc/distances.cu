// Euclidean distances between every sample and every centroid (the transform back end).
//
// out_t[j * ldo + i] = sqrt(sum_f (Y[j, f] - X[i, f])^2): the (k, n) array whose transpose the
// reference returns.  The squared differences are accumulated directly, feature by feature,
// as the reference does (no |x|^2 + |y|^2 - 2 x.y expansion, which cancels badly for nearby
// points), so the kernel is bound by the FMA pipe: 2 instructions per (sample, centroid,
// feature).  It is tiled like the fused step: a CTA owns 128 samples x BN centroids, a thread a
// 4 x TN register tile; 16-feature (fp64: 8) chunks of both operands are fetched with vector loads
// one chunk ahead and staged feature-major in shared memory.  The finished tile is transposed
// through shared memory so that every output row (one centroid, 128 consecutive samples) is
// written as whole 128-byte lines.
//
// Replaces make_compute_euclidean_distances_fixed_window_kernel,
// sklearn_numba_dpex/kmeans/kernels/compute_euclidean_distances.py:16-161.
#include "cc_tile.cuh"

namespace kmb {

template <typename T>
__global__ void __launch_bounds__(CC_THREADS, 2)
distances_tile_kernel(const T* __restrict__ X, const T* __restrict__ Y, T* __restrict__ out_t,
                      int64_t n, int d, int k, int64_t ldo, int xvec, int yvec) {
  using Cfg = CcTile<T>;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, TM = Cfg::TM, TN = Cfg::TN;
  constexpr int V = Cfg::V, PAD = Cfg::PAD;
  constexpr int NTX = BN / TN, NTY = BM / TM;
  constexpr int LDX = BM + PAD, LDC = BN + PAD, LDO = BM + 1;
  constexpr int KK_UNROLL = sizeof(T) == 8 ? 1 : 2;

  __shared__ __align__(16) T Xs[BK * LDX];
  __shared__ __align__(16) T Ys[BK * LDC];
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  T* Os = reinterpret_cast<T*>(dyn_smem);          // BN x LDO: the finished tile, centroid-major

  const int tid = threadIdx.x, tx = tid % NTX, ty = tid / NTX;
  const int64_t m0 = (int64_t)blockIdx.x * BM;
  const int j0 = blockIdx.y * BN;
  const int n_kchunks = (d + BK - 1) / BK;

  T acc[TM][TN];
#pragma unroll
  for (int r = 0; r < TM; ++r)
#pragma unroll
    for (int c = 0; c < TN; ++c) acc[r][c] = T(0);

  ChunkRegs<T, BM, BK> xr;
  ChunkRegs<T, BN, BK> yr;
  fetch_chunk<T, BM, BK>(xr, X, m0, n, d, 0, xvec);
  fetch_chunk<T, BN, BK>(yr, Y, j0, k, d, 0, yvec);
  for (int kc = 0; kc < n_kchunks; ++kc) {
    __syncthreads();
    store_chunk<T, BM, BK>(xr, Xs, LDX);
    store_chunk<T, BN, BK>(yr, Ys, LDC);
    __syncthreads();
    if (kc + 1 < n_kchunks) {
      fetch_chunk<T, BM, BK>(xr, X, m0, n, d, (kc + 1) * BK, xvec);
      fetch_chunk<T, BN, BK>(yr, Y, j0, k, d, (kc + 1) * BK, yvec);
    }
#pragma unroll(KK_UNROLL)
    for (int kk = 0; kk < BK; ++kk) {
      T av[TM], bv[TN];
#pragma unroll
      for (int g = 0; g < TM / V; ++g) load_vec<T, V>(&av[g * V], &Xs[kk * LDX + g * NTY * V + ty * V]);
#pragma unroll
      for (int g = 0; g < TN / V; ++g) load_vec<T, V>(&bv[g * V], &Ys[kk * LDC + g * NTX * V + tx * V]);
#pragma unroll
      for (int r = 0; r < TM; ++r)
#pragma unroll
        for (int c = 0; c < TN; ++c) {
          const T diff = bv[c] - av[r];
          acc[r][c] = fma(diff, diff, acc[r][c]);
        }
    }
  }

  // transpose through shared memory, then whole lines of 128 consecutive samples per centroid
#pragma unroll
  for (int c = 0; c < TN; ++c) {
    const int col = (c / V) * NTX * V + tx * V + (c % V);
#pragma unroll
    for (int r = 0; r < TM; ++r) {
      const int row = (r / V) * NTY * V + ty * V + (r % V);
      Os[col * LDO + row] = sqrt(acc[r][c]);
    }
  }
  __syncthreads();
  const int rows = (int)((n - m0 < BM) ? (n - m0) : BM);
  const int cols = (k - j0 < BN) ? (k - j0) : BN;
  for (int e = tid; e < cols * BM; e += CC_THREADS) {
    const int col = e / BM, row = e % BM;
    if (row < rows) out_t[(int64_t)(j0 + col) * ldo + m0 + row] = Os[col * LDO + row];
  }
}

}  // namespace kmb

using namespace kmb;

extern "C" int kmb_euclidean_distances(int dtype, const void* X, const void* Y, void* out_t,
                                       int64_t n, int d, int k, int64_t ldo, void* stream) {
  KMB_REQUIRE(X && Y && out_t, "kmb_euclidean_distances: NULL argument");
  KMB_REQUIRE(n >= 0 && d > 0 && k > 0 && ldo >= n, "kmb_euclidean_distances: bad sizes");
  if (n == 0) return KMB_OK;
  KMB_DISPATCH_DTYPE(dtype, {
    using Cfg = CcTile<T>;
    const int64_t gy = ceil_div(k, Cfg::BN);
    KMB_REQUIRE(gy <= 65535, "kmb_euclidean_distances: too many centroid tiles (k=%d)", k);
    const size_t dyn = (size_t)Cfg::BN * (Cfg::BM + 1) * sizeof(T);
    auto kern = distances_tile_kernel<T>;
    KMB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    dim3 grid((unsigned)ceil_div(n, Cfg::BM), (unsigned)gy);
    kern<<<grid, CC_THREADS, dyn, (cudaStream_t)stream>>>((const T*)X, (const T*)Y, (T*)out_t, n, d, k,
                                                        ldo, cc_vec_width<T>(X, d),
                                                        cc_vec_width<T>(Y, d));
    KMB_CHECK_LAUNCH();
  });
  return KMB_OK;
}
