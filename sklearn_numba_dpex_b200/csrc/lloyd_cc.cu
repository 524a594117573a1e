// Fused Lloyd step and label assignment on the CUDA cores (fp32 and fp64).
//
// One CTA owns a tile of BM samples and walks the centroids BN at a time; every thread
// keeps a TM x TN register tile of dot products, folds it into a running
// (min pseudo-inertia, index) pair per sample, and the 16 threads that share a sample row
// merge their pairs with warp shuffles.  The update step then adds w*x into centroid sums
// held in shared memory (one private copy per CTA, flushed once at the end) when
// k*(d+1) elements fit, otherwise straight into a few global copies.
//
// Stands for fused_lloyd_single_step / assignment of the reference
// (sklearn_numba_dpex/kmeans/kernels/lloyd_single_step.py:149-414,
//  kmeans/kernels/compute_labels.py:75-168); the argmin rule (strict '<' from +inf in
// ascending centroid order, so the lowest index wins ties and NaN never wins) follows
// kmeans/kernels/_base_kmeans_kernel_funcs.py:351-366.
#include "kmb_common.cuh"

namespace kmb {

template <typename T>
struct CcTile;
template <>
struct CcTile<float> {
  static constexpr int BM = 128, BN = 128, BK = 16, TM = 8, TN = 8, V = 4, PAD = 4;
};
template <>
struct CcTile<double> {
  static constexpr int BM = 128, BN = 64, BK = 16, TM = 8, TN = 4, V = 2, PAD = 2;
};

constexpr int CC_THREADS = 256;
// Largest private accumulator (bytes) kept in shared memory by the update step.
constexpr size_t CC_PRIV_SMEM_MAX = 64 * 1024;

template <typename T>
struct CcArgs {
  const T* X;
  const T* w;
  const T* C;
  const T* h;
  const uint32_t* prev;
  uint32_t* labels;
  T* acc;
  int n_copies;
  int64_t acc_len;
  int64_t n;
  int d;
  int k;
  int smem_priv;
};

template <typename T, int V>
__device__ __forceinline__ void load_vec(T* dst, const T* src) {
  if constexpr (sizeof(T) == 4 && V == 4) {
    float4 v = *reinterpret_cast<const float4*>(src);
    dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
  } else {
    double2 v = *reinterpret_cast<const double2*>(src);
    dst[0] = v.x; dst[1] = v.y;
  }
}

template <typename T, bool UPDATE>
__global__ void __launch_bounds__(CC_THREADS, 2) lloyd_cc_kernel(CcArgs<T> a) {
  using Cfg = CcTile<T>;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, TM = Cfg::TM, TN = Cfg::TN;
  constexpr int V = Cfg::V, PAD = Cfg::PAD;
  constexpr int NTX = BN / TN, NTY = BM / TM;
  static_assert(NTX == 16 && NTY * NTX == CC_THREADS, "thread layout");

  __shared__ __align__(16) T Xs[BK][BM + PAD];
  __shared__ __align__(16) T Cs[BK][BN + PAD];
  __shared__ T hs[BN];
  __shared__ uint32_t lab_s[BM];
  __shared__ double red_s[32];
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  T* ssum = reinterpret_cast<T*>(dyn_smem);

  const int tid = threadIdx.x, tx = tid % NTX, ty = tid / NTX;
  const int d = a.d, k = a.k;
  const int64_t n = a.n;
  const int64_t n_tiles = (n + BM - 1) / BM;
  const int n_kchunks = (d + BK - 1) / BK;
  const int priv_len = k * d + k;
  T* acc_copy = UPDATE ? a.acc + (int64_t)(blockIdx.x % a.n_copies) * a.acc_len : nullptr;

  if (UPDATE && a.smem_priv) {
    for (int e = tid; e < priv_len; e += CC_THREADS) ssum[e] = T(0);
  }
  unsigned my_changed = 0;

  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int64_t m0 = tile * BM;
    const int rows = (int)((n - m0 < BM) ? (n - m0) : BM);
    T best[TM];
    uint32_t bi[TM];
#pragma unroll
    for (int r = 0; r < TM; ++r) {
      best[r] = inf_value<T>();
      bi[r] = 0u;
    }

    for (int cn = 0; cn < k; cn += BN) {
      T acc[TM][TN];
#pragma unroll
      for (int r = 0; r < TM; ++r)
#pragma unroll
        for (int c = 0; c < TN; ++c) acc[r][c] = T(0);

      for (int kc = 0; kc < n_kchunks; ++kc) {
        const int k0 = kc * BK;
        __syncthreads();
        if (!(n_kchunks == 1 && cn > 0)) {
#pragma unroll
          for (int i = 0; i < BM * BK / CC_THREADS; ++i) {
            const int e = tid + i * CC_THREADS;
            const int kk = e % BK, m = e / BK;
            T v = T(0);
            if (m < rows && k0 + kk < d) v = a.X[(m0 + m) * (int64_t)d + k0 + kk];
            Xs[kk][m] = v;
          }
        }
#pragma unroll
        for (int i = 0; i < BN * BK / CC_THREADS; ++i) {
          const int e = tid + i * CC_THREADS;
          const int kk = e % BK, j = e / BK;
          T v = T(0);
          if (cn + j < k && k0 + kk < d) v = a.C[(int64_t)(cn + j) * d + k0 + kk];
          Cs[kk][j] = v;
        }
        if (kc == 0 && tid < BN) hs[tid] = (cn + tid < k) ? a.h[cn + tid] : inf_value<T>();
        __syncthreads();

#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
          T av[TM], bv[TN];
#pragma unroll
          for (int g = 0; g < TM / V; ++g) load_vec<T, V>(&av[g * V], &Xs[kk][g * NTY * V + ty * V]);
#pragma unroll
          for (int g = 0; g < TN / V; ++g) load_vec<T, V>(&bv[g * V], &Cs[kk][g * NTX * V + tx * V]);
#pragma unroll
          for (int r = 0; r < TM; ++r)
#pragma unroll
            for (int c = 0; c < TN; ++c) acc[r][c] = fma(av[r], bv[c], acc[r][c]);
        }
      }

      // Fold this centroid tile into the running minimum, columns in ascending order.
#pragma unroll
      for (int c = 0; c < TN; ++c) {
        const int col = (c / V) * NTX * V + tx * V + (c % V);
        const T hj = hs[col];
#pragma unroll
        for (int r = 0; r < TM; ++r) {
          const T q = hj - acc[r][c];
          if (q < best[r]) {
            best[r] = q;
            bi[r] = (uint32_t)(cn + col);
          }
        }
      }
    }

    // Merge the 16 threads of a sample row: smaller value wins, then smaller index.
#pragma unroll
    for (int r = 0; r < TM; ++r) {
#pragma unroll
      for (int o = NTX / 2; o > 0; o >>= 1) {
        const T oq = __shfl_xor_sync(0xffffffffu, best[r], o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi[r], o);
        if (oq < best[r] || (oq == best[r] && oi < bi[r])) {
          best[r] = oq;
          bi[r] = oi;
        }
      }
    }
    if (tx == 0) {
#pragma unroll
      for (int r = 0; r < TM; ++r) lab_s[(r / V) * NTY * V + ty * V + (r % V)] = bi[r];
    }
    __syncthreads();

    if (tid < rows) {
      const uint32_t lab = lab_s[tid];
      a.labels[m0 + tid] = lab;
      if (UPDATE) {
        my_changed += (a.prev == nullptr) ? 1u : (a.prev[m0 + tid] != lab ? 1u : 0u);
        const T wi = a.w ? a.w[m0 + tid] : T(1);
        if (a.smem_priv) atomicAdd(&ssum[k * d + lab], wi);
        else atomicAdd(&acc_copy[(int64_t)k * d + lab], wi);
      }
    }
    if (UPDATE) {
      const int total = rows * d;
      const T* xt = a.X + m0 * (int64_t)d;
      // element e = tid + i * CC_THREADS of the tile is (row, f): two divisions per tile, then
      // both are advanced by increments
      const int upd_drow = CC_THREADS / d, upd_df = CC_THREADS - upd_drow * d;
      int row = tid / d, f = tid - row * d;
      for (int e = tid; e < total; e += CC_THREADS) {
        const T wi = a.w ? a.w[m0 + row] : T(1);
        const T v = xt[e] * wi;
        const uint32_t lab = lab_s[row];
        if (a.smem_priv) atomicAdd(&ssum[lab * d + f], v);
        else atomicAdd(&acc_copy[(int64_t)lab * d + f], v);
        row += upd_drow;
        f += upd_df;
        if (f >= d) {
          f -= d;
          ++row;
        }
      }
    }
  }

  if (UPDATE) {
    __syncthreads();
    if (a.smem_priv) {
      for (int e = tid; e < priv_len; e += CC_THREADS) {
        const T v = ssum[e];
        if (v != T(0)) atomicAdd(&acc_copy[e], v);
      }
    }
    const double tot = block_sum((double)my_changed, red_s);
    if (tid == 0 && tot != 0.0) atomicAdd(&acc_copy[(int64_t)k * d + k], (T)tot);
  }
}

template <typename T>
bool cc_can_privatise(int d, int k) {
  return (size_t)((int64_t)k * d + k) * sizeof(T) <= CC_PRIV_SMEM_MAX;
}

template <typename T, bool UPDATE>
int launch_lloyd_cc(const CcArgs<T>& args_in, cudaStream_t stream) {
  CcArgs<T> args = args_in;
  using Cfg = CcTile<T>;
  const int64_t n_tiles = ceil_div(args.n, Cfg::BM);
  if (n_tiles == 0) return KMB_OK;
  args.smem_priv = (UPDATE && cc_can_privatise<T>(args.d, args.k)) ? 1 : 0;
  size_t dyn = args.smem_priv ? (size_t)((int64_t)args.k * args.d + args.k) * sizeof(T) : 0;
  auto kern = lloyd_cc_kernel<T, UPDATE>;
  KMB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)CC_PRIV_SMEM_MAX));
  int64_t grid = (int64_t)sm_count() * 2;
  if (grid > n_tiles) grid = n_tiles;
  kern<<<(unsigned)grid, CC_THREADS, dyn, stream>>>(args);
  KMB_CHECK_LAUNCH();
  return KMB_OK;
}

// Entry points used by lloyd_api.cu
int lloyd_cc_step(int dtype, const void* X, const void* w, const void* C, const void* h,
                  const uint32_t* prev, uint32_t* labels, void* acc, int n_copies,
                  int64_t acc_len, int64_t n, int d, int k, cudaStream_t stream) {
  KMB_DISPATCH_DTYPE(dtype, {
    CcArgs<T> a{(const T*)X, (const T*)w, (const T*)C, (const T*)h, prev, labels, (T*)acc,
                n_copies, acc_len, n, d, k, 0};
    return launch_lloyd_cc<T, true>(a, stream);
  });
}

int lloyd_cc_assign(int dtype, const void* X, const void* C, const void* h, uint32_t* labels,
                    int64_t n, int d, int k, cudaStream_t stream) {
  KMB_DISPATCH_DTYPE(dtype, {
    CcArgs<T> a{(const T*)X, nullptr, (const T*)C, (const T*)h, nullptr, labels, nullptr,
                1, 0, n, d, k, 0};
    return launch_lloyd_cc<T, false>(a, stream);
  });
}

bool lloyd_cc_privatises(int dtype, int d, int k) {
  return dtype == KMB_F32 ? cc_can_privatise<float>(d, k) : cc_can_privatise<double>(d, k);
}

}  // namespace kmb
