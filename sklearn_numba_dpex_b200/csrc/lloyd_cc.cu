// Fused Lloyd step and label assignment on the CUDA cores (fp32 and fp64).
//
// One CTA owns a tile of 128 samples and walks the centroids BN at a time; every thread
// keeps a 4 x TN register tile of dot products (32 x 8 threads), folds it into a running
// (min pseudo-inertia, index) pair per sample, and the 8 threads that share a sample row
// merge their pairs with warp shuffles.
//
// Operand staging.  Sample chunks (16 features of the 128 rows) are fetched from global
// memory with 16-byte (or the widest aligned) vector loads into registers one chunk AHEAD of
// the arithmetic and stored feature-major into shared memory, so the loads of chunk c + 1 fly
// while chunk c is multiplied.  The centroids stay resident in shared memory for the whole
// kernel when they fit (32 KB), otherwise their chunks are staged like the samples.
//
// Update.  When k (d + 1) sums fit in 64 KB they live in shared memory, one private copy per
// CTA that is flushed once at the end.  Rows are added WITHOUT atomics: the clusters are
// dealt out to "owner groups" of G lanes (cluster j belongs to group j mod NG), every row of
// the tile is put on the list of the group that owns its label, and each group then adds its
// rows into its own clusters' sums, lane = feature.  No two groups ever touch the same sum,
// so plain loads and stores do, in fp64 as well (shared memory has no native fp64 atomic add).
// Otherwise the rows are added into a few global copies with atomics.
//
// Stands for fused_lloyd_single_step / assignment of the reference
// (sklearn_numba_dpex/kmeans/kernels/lloyd_single_step.py:149-414,
//  kmeans/kernels/compute_labels.py:75-168); the argmin rule (strict '<' from +inf in
// ascending centroid order, so the lowest index wins ties and NaN never wins) follows
// kmeans/kernels/_base_kmeans_kernel_funcs.py:351-366.
#include "cc_tile.cuh"

namespace kmb {

// Largest private accumulator (bytes) kept in shared memory by the update step.
constexpr size_t CC_PRIV_SMEM_MAX = 64 * 1024;
// Largest centroid set (bytes, padded to whole tiles and chunks) kept resident in shared memory.
constexpr size_t CC_RES_SMEM_MAX = 32 * 1024;

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
  int resident;
  int xvec;          // widest vector (elements) the rows of X can be loaded with: 4, 2 or 1
  int cvec;          // same for C
};

template <typename T, bool UPDATE, bool RESIDENT>
__global__ void __launch_bounds__(CC_THREADS, 2) lloyd_cc_kernel(CcArgs<T> a) {
  using Cfg = CcTile<T>;
  constexpr int BM = Cfg::BM, BN = Cfg::BN, BK = Cfg::BK, TM = Cfg::TM, TN = Cfg::TN;
  constexpr int V = Cfg::V, PAD = Cfg::PAD;
  constexpr int NTX = BN / TN, NTY = BM / TM;
  constexpr int LDX = BM + PAD, LDC = BN + PAD;
  constexpr int KK_UNROLL = sizeof(T) == 8 ? 1 : 2;
  static_assert(NTX == 8 && NTY * NTX == CC_THREADS, "thread layout");
  static_assert(BK % 4 == 0 && CC_THREADS % (BK / 4) == 0, "chunk shares");

  __shared__ __align__(16) T Xs[BK * LDX];
  __shared__ __align__(16) T Cs[BK * LDC];
  __shared__ T hs[BN];
  __shared__ uint32_t lab_s[BM];
  __shared__ double red_s[32];
  __shared__ int grp_cnt[CC_MAX_GROUPS];
  __shared__ unsigned char grp_rows[CC_MAX_GROUPS * BM];
  extern __shared__ __align__(16) unsigned char dyn_smem[];

  const int tid = threadIdx.x, tx = tid % NTX, ty = tid / NTX;
  const int d = a.d, k = a.k;
  const int64_t n = a.n;
  const int64_t n_tiles = (n + BM - 1) / BM;
  const int n_kchunks = (d + BK - 1) / BK;
  const int n_ctiles = (k + BN - 1) / BN;
  const int priv_len = k * d + k;
  T* acc_copy = UPDATE ? a.acc + (int64_t)(blockIdx.x % a.n_copies) * a.acc_len : nullptr;

  // dynamic shared memory: [private sums | resident centroids (feature-major, tile by tile)]
  T* ssum = reinterpret_cast<T*>(dyn_smem);
  const size_t priv_bytes = (UPDATE && a.smem_priv) ? (((size_t)priv_len * sizeof(T) + 15) / 16 * 16) : 0;
  T* Cres = reinterpret_cast<T*>(dyn_smem + priv_bytes);
  T* hres = Cres + (size_t)n_ctiles * n_kchunks * BK * LDC;

  if (UPDATE && a.smem_priv) {
    for (int e = tid; e < priv_len; e += CC_THREADS) ssum[e] = T(0);
  }
  if (tid < CC_MAX_GROUPS) grp_cnt[tid] = 0;
  if (RESIDENT) {
    // every centroid chunk goes to its place once: chunk (ct, kc) at Cres[(ct * n_kchunks + kc) * BK * LDC]
    for (int ct = 0; ct < n_ctiles; ++ct) {
      for (int kc = 0; kc < n_kchunks; ++kc) {
        ChunkRegs<T, BN, BK> cr;
        fetch_chunk<T, BN, BK>(cr, a.C, (int64_t)ct * BN, k, d, kc * BK, a.cvec);
        store_chunk<T, BN, BK>(cr, Cres + (size_t)(ct * n_kchunks + kc) * BK * LDC, LDC);
      }
      for (int j = tid; j < BN; j += CC_THREADS)
        hres[ct * BN + j] = (ct * BN + j < k) ? a.h[ct * BN + j] : inf_value<T>();
    }
  }
  unsigned my_changed = 0;

  // update geometry: groups of G lanes, group og owns the clusters j with j % NG == og
  const int G = owner_group_lanes(d);
  const int NG = (CC_THREADS / 32) * (32 / G);
  const int og = (tid >> 5) * (32 / G) + (tid & 31) / G;
  const int gl = (tid & 31) % G;

  ChunkRegs<T, BM, BK> xr;
  ChunkRegs<T, BN, BK> cr;
  if (blockIdx.x < n_tiles) {
    fetch_chunk<T, BM, BK>(xr, a.X, (int64_t)blockIdx.x * BM, n, d, 0, a.xvec);
    if (!RESIDENT) fetch_chunk<T, BN, BK>(cr, a.C, 0, k, d, 0, a.cvec);
  }

  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int64_t m0 = tile * BM;
    const int rows = (int)((n - m0 < BM) ? (n - m0) : BM);
    // previous label of the row this thread will write: fetched now, compared after the argmin
    uint32_t prev_lab = 0xffffffffu;
    if (UPDATE && a.prev != nullptr && tid < rows) prev_lab = __ldg(a.prev + m0 + tid);
    const bool has_next = tile + gridDim.x < n_tiles;
    T best[TM];
    uint32_t bi[TM];
#pragma unroll
    for (int r = 0; r < TM; ++r) {
      best[r] = inf_value<T>();
      bi[r] = 0u;
    }

    for (int ct = 0; ct < n_ctiles; ++ct) {
      const int cn = ct * BN;
      T acc[TM][TN];
#pragma unroll
      for (int r = 0; r < TM; ++r)
#pragma unroll
        for (int c = 0; c < TN; ++c) acc[r][c] = T(0);

      for (int kc = 0; kc < n_kchunks; ++kc) {
        // With a single feature chunk the sample chunk in shared memory serves every centroid
        // tile of this sample tile; otherwise it is staged again for each of them.
        const bool stage_x = !(n_kchunks == 1 && ct > 0);
        __syncthreads();          // everybody is done reading the previous chunk
        if (stage_x) store_chunk<T, BM, BK>(xr, Xs, LDX);
        if (!RESIDENT) {
          store_chunk<T, BN, BK>(cr, Cs, LDC);
          if (kc == 0 && tid < BN) hs[tid] = (cn + tid < k) ? a.h[cn + tid] : inf_value<T>();
        }
        __syncthreads();
        // fetch what the NEXT staging step will store, while this chunk is multiplied
        {
          int nkc = kc + 1, nct = ct;
          int64_t ntile = tile;
          if (nkc == n_kchunks) {
            nkc = 0;
            if (++nct == n_ctiles) {
              nct = 0;
              ntile = tile + gridDim.x;
            }
          }
          const bool more = ntile < n_tiles;
          const bool next_stage_x = !(n_kchunks == 1 && nct > 0);
          if (more && next_stage_x) fetch_chunk<T, BM, BK>(xr, a.X, ntile * BM, n, d, nkc * BK, a.xvec);
          if (more && !RESIDENT) fetch_chunk<T, BN, BK>(cr, a.C, (int64_t)nct * BN, k, d, nkc * BK, a.cvec);
        }
        const T* Cc = RESIDENT ? Cres + (size_t)(ct * n_kchunks + kc) * BK * LDC : Cs;
        // a short unroll keeps the 64 accumulators, the prefetched chunk and the operand vectors
        // inside 128 registers (two CTAs per SM); the tile itself supplies the parallelism
#pragma unroll(KK_UNROLL)
        for (int kk = 0; kk < BK; ++kk) {
          T av[TM], bv[TN];
#pragma unroll
          for (int g = 0; g < TM / V; ++g) load_vec<T, V>(&av[g * V], &Xs[kk * LDX + g * NTY * V + ty * V]);
#pragma unroll
          for (int g = 0; g < TN / V; ++g) load_vec<T, V>(&bv[g * V], &Cc[kk * LDC + g * NTX * V + tx * V]);
#pragma unroll
          for (int r = 0; r < TM; ++r)
#pragma unroll
            for (int c = 0; c < TN; ++c) acc[r][c] = fma(av[r], bv[c], acc[r][c]);
        }
      }

      // Fold this centroid tile into the running minimum, columns in ascending order.
      const T* hc = RESIDENT ? hres + cn : hs;
#pragma unroll
      for (int c = 0; c < TN; ++c) {
        const int col = (c / V) * NTX * V + tx * V + (c % V);
        const T hj = hc[col];
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

    // Merge the 8 threads of a sample row: smaller value wins, then smaller index.
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
        my_changed += (prev_lab != lab) ? 1u : 0u;
        if (a.smem_priv) {
          // hand the row to the group that owns its cluster
          const int owner = (int)(lab % (uint32_t)NG);
          const int pos = atomicAdd(&grp_cnt[owner], 1);
          grp_rows[owner * BM + pos] = (unsigned char)tid;
        } else {
          const T wi = a.w ? a.w[m0 + tid] : T(1);
          atomicAdd(&acc_copy[(int64_t)k * d + lab], wi);
        }
      }
    }
    if (UPDATE && a.smem_priv) {
      __syncthreads();
      // each owner group adds its rows into its own clusters: no other group touches them
      owner_group_update<T>(ssum, a.X + m0 * (int64_t)d, a.w ? a.w + m0 : nullptr, lab_s,
                            grp_rows + og * BM, grp_cnt[og], d, k, G, gl);
      __syncwarp();
      if (gl == 0) grp_cnt[og] = 0;     // next written after the barriers of the next tile
    } else if (UPDATE) {
      const int total = rows * d;
      const T* xt = a.X + m0 * (int64_t)d;
      // element e = tid + i * CC_THREADS of the tile is (row, f): two divisions per tile, then
      // both are advanced by increments
      const int upd_drow = CC_THREADS / d, upd_df = CC_THREADS - upd_drow * d;
      int row = tid / d, f = tid - row * d;
      for (int e = tid; e < total; e += CC_THREADS) {
        const T wi = a.w ? a.w[m0 + row] : T(1);
        const T v = xt[e] * wi;
        atomicAdd(&acc_copy[(int64_t)lab_s[row] * d + f], v);
        row += upd_drow;
        f += upd_df;
        if (f >= d) {
          f -= d;
          ++row;
        }
      }
    }
    (void)has_next;
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

template <typename T>
size_t cc_resident_bytes(int d, int k) {
  using Cfg = CcTile<T>;
  const size_t n_ctiles = (size_t)ceil_div(k, Cfg::BN), n_kchunks = (size_t)ceil_div(d, Cfg::BK);
  return (n_ctiles * n_kchunks * Cfg::BK * (Cfg::BN + Cfg::PAD) + n_ctiles * Cfg::BN) * sizeof(T);
}

template <typename T, bool UPDATE>
int launch_lloyd_cc(const CcArgs<T>& args_in, cudaStream_t stream) {
  CcArgs<T> args = args_in;
  using Cfg = CcTile<T>;
  const int64_t n_tiles = ceil_div(args.n, Cfg::BM);
  if (n_tiles == 0) return KMB_OK;
  args.smem_priv = (UPDATE && cc_can_privatise<T>(args.d, args.k)) ? 1 : 0;
  const size_t res_bytes = cc_resident_bytes<T>(args.d, args.k);
  args.resident = res_bytes <= CC_RES_SMEM_MAX ? 1 : 0;
  args.xvec = cc_vec_width<T>(args.X, args.d);
  args.cvec = cc_vec_width<T>(args.C, args.d);
  size_t dyn = args.smem_priv ? (((size_t)((int64_t)args.k * args.d + args.k) * sizeof(T) + 15) / 16 * 16) : 0;
  if (args.resident) dyn += res_bytes;
  auto kern = args.resident ? lloyd_cc_kernel<T, UPDATE, true> : lloyd_cc_kernel<T, UPDATE, false>;
  KMB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)(CC_PRIV_SMEM_MAX + CC_RES_SMEM_MAX + 16)));
  int64_t grid = (int64_t)sm_count() * 2;
  if (grid > n_tiles) grid = n_tiles;
  kern<<<(unsigned)grid, CC_THREADS, dyn, stream>>>(args);
  KMB_CHECK_LAUNCH();
  return KMB_OK;
}

// float64 on the double-precision MMA path (lloyd_f64.cu)
bool lloyd_f64_mma_enabled();
int lloyd_f64_step(const double* X, const double* w, const double* C, const double* h,
                   const uint32_t* prev, uint32_t* labels, double* acc, int n_copies,
                   int64_t acc_len, int64_t n, int d, int k, cudaStream_t stream);
int lloyd_f64_assign(const double* X, const double* C, const double* h, uint32_t* labels, int64_t n,
                     int d, int k, cudaStream_t stream);

// Entry points used by lloyd_api.cu
int lloyd_cc_step(int dtype, const void* X, const void* w, const void* C, const void* h,
                  const uint32_t* prev, uint32_t* labels, void* acc, int n_copies,
                  int64_t acc_len, int64_t n, int d, int k, cudaStream_t stream) {
  if (dtype == KMB_F64 && lloyd_f64_mma_enabled())
    return lloyd_f64_step((const double*)X, (const double*)w, (const double*)C, (const double*)h, prev,
                          labels, (double*)acc, n_copies, acc_len, n, d, k, stream);
  KMB_DISPATCH_DTYPE(dtype, {
    CcArgs<T> a{(const T*)X, (const T*)w, (const T*)C, (const T*)h, prev, labels, (T*)acc,
                n_copies, acc_len, n, d, k, 0, 0, 1, 1};
    return launch_lloyd_cc<T, true>(a, stream);
  });
}

int lloyd_cc_assign(int dtype, const void* X, const void* C, const void* h, uint32_t* labels,
                    int64_t n, int d, int k, cudaStream_t stream) {
  if (dtype == KMB_F64 && lloyd_f64_mma_enabled())
    return lloyd_f64_assign((const double*)X, (const double*)C, (const double*)h, labels, n, d, k,
                            stream);
  KMB_DISPATCH_DTYPE(dtype, {
    CcArgs<T> a{(const T*)X, nullptr, (const T*)C, (const T*)h, nullptr, labels, nullptr,
                1, 0, n, d, k, 0, 0, 1, 1};
    return launch_lloyd_cc<T, false>(a, stream);
  });
}

bool lloyd_cc_privatises(int dtype, int d, int k) {
  return dtype == KMB_F32 ? cc_can_privatise<float>(d, k) : cc_can_privatise<double>(d, k);
}

}  // namespace kmb
