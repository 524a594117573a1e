// Fused Lloyd step and label assignment in float64 on the double-precision tensor-core path
// (mma.sync m8n8k4 f64: tcgen05 has no float64 kind, so this is the tensor path fp64 has).
//
// With plain DFMAs a 4 x 8 register tile needs six 16-byte shared-memory loads per 32 FMAs, and
// the shared-memory pipe, not the FP64 pipe, bounds the step (measured: FP64 pipe 33 % busy).
// An 8x8x4 MMA takes one 8-byte operand load per thread for 256 FMAs of the warp, so a
// 32 x 32 warp tile needs 8 loads per 16 MMAs (4 096 FMAs): six times less shared-memory
// traffic and eight times fewer issue slots per FMA.
//
// One CTA of NW warps owns 16 NW samples and walks the centroids 64 at a time; warp w owns rows
// 16 w .. +15 and ALL 64 columns of the score tile as 2 x 8 MMA tiles, so a sample row belongs to
// one warp (four lanes) and its argmin needs no exchange between warps.  Both operands are
// staged ROW-major (feature index fastest, the layout they have in global memory) with a row
// pitch of BK + 4 doubles, which makes the fragment loads (8 rows x 4 consecutive features per
// warp) free of bank conflicts.  Chunks of 16 features are fetched with vector loads into
// registers one chunk ahead of the arithmetic; the centroids stay resident in shared memory for
// the whole kernel when they fit.
//
// Argmin and update are those of the CUDA-core kernel: strict '<' in ascending centroid order
// (lowest index wins ties, NaN never wins; kmeans/kernels/_base_kmeans_kernel_funcs.py:351-366
// of the reference), sums privatised in shared memory and added without atomics by owner groups
// when they fit, else global atomics.
//
// Stands for fused_lloyd_single_step / assignment of the reference
// (sklearn_numba_dpex/kmeans/kernels/lloyd_single_step.py:149-414,
//  kmeans/kernels/compute_labels.py:75-168) for float64 data.
#include <stdlib.h>

#include "cc_tile.cuh"

namespace kmb {

constexpr int F64_BN = 64, F64_BK = 16, F64_LD = F64_BK + 4;
constexpr size_t F64_PRIV_SMEM_MAX = 64 * 1024;
constexpr size_t F64_RES_SMEM_MAX = 48 * 1024;
constexpr int F64_MAX_GROUPS = CC_MAX_GROUPS;

struct F64Args {
  const double* X;
  const double* w;
  const double* C;
  const double* h;
  const uint32_t* prev;
  uint32_t* labels;
  double* acc;
  int n_copies;
  int64_t acc_len;
  int64_t n;
  int d;
  int k;
  int smem_priv;
  int resident;
  int xvec;
  int cvec;
};

__device__ __forceinline__ void dmma884(double (&c)[2], double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
               : "+d"(c[0]), "+d"(c[1])
               : "d"(a), "d"(b));
}

// Stores a fetched (ROWS x 16) chunk row-major with pitch `ld` doubles: each thread holds quads
// of 4 consecutive features, written as two 16-byte stores.
template <int ROWS, int THREADS>
__device__ __forceinline__ void store_chunk_rows(const ChunkRegs<double, ROWS, F64_BK, THREADS>& r,
                                                 double* __restrict__ S, int ld) {
  using R = ChunkRegs<double, ROWS, F64_BK, THREADS>;
  const int q = threadIdx.x % R::QPR;
#pragma unroll
  for (int i = 0; i < R::N; ++i) {
    const int m = threadIdx.x / R::QPR + i * R::RSTEP;
    if (m < ROWS) {
      double2* dst = reinterpret_cast<double2*>(S + (size_t)m * ld + q * 4);
      dst[0] = make_double2(r.v[i][0], r.v[i][1]);
      dst[1] = make_double2(r.v[i][2], r.v[i][3]);
    }
  }
}

// NW = warps of the CTA, each on a 16 x 64 score tile.  NW = 4 (128 threads, 64 samples) lets four
// CTAs share an SM, so that the serial phases of a tile (label write, update) of one CTA overlap
// the contractions of three others.
template <bool UPDATE, bool RESIDENT, int NW>
__global__ void __launch_bounds__(32 * NW, 16 / NW) lloyd_f64_kernel(F64Args a) {
  constexpr int BM = 16 * NW, THREADS = 32 * NW, BN = F64_BN, BK = F64_BK, LD = F64_LD;
  __shared__ __align__(16) double Xs[BM * LD];
  __shared__ uint32_t lab_s[BM];
  __shared__ double red_s[32];
  __shared__ int grp_cnt[F64_MAX_GROUPS];
  __shared__ unsigned char grp_rows[F64_MAX_GROUPS * BM];
  extern __shared__ __align__(16) unsigned char dyn_smem[];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gid = lane >> 2, tig = lane & 3;       // fragment coordinates inside an 8x8x4 MMA
  const int d = a.d, k = a.k;
  const int64_t n = a.n;
  const int64_t n_tiles = (n + BM - 1) / BM;
  const int n_kchunks = (d + BK - 1) / BK;
  const int n_ctiles = (k + BN - 1) / BN;
  const int priv_len = k * d + k;
  double* acc_copy = UPDATE ? a.acc + (int64_t)(blockIdx.x % a.n_copies) * a.acc_len : nullptr;

  // dynamic shared memory: [private sums | resident centroids, chunk (ct, kc) by chunk | half norms],
  // or, when the centroids are streamed, [private sums | one staged centroid chunk | its half norms]
  double* ssum = reinterpret_cast<double*>(dyn_smem);
  const size_t priv_bytes = (UPDATE && a.smem_priv) ? (((size_t)priv_len * sizeof(double) + 15) / 16 * 16) : 0;
  double* Cres = reinterpret_cast<double*>(dyn_smem + priv_bytes);
  double* hres = Cres + (size_t)n_ctiles * n_kchunks * BN * LD;
  double* Cs = Cres;                               // streamed form only
  double* hs = Cres + (size_t)BN * LD;

  if (UPDATE && a.smem_priv) {
    for (int e = tid; e < priv_len; e += THREADS) ssum[e] = 0.0;
  }
  if (tid < F64_MAX_GROUPS) grp_cnt[tid] = 0;
  if (RESIDENT) {
    for (int ct = 0; ct < n_ctiles; ++ct) {
      for (int kc = 0; kc < n_kchunks; ++kc) {
        ChunkRegs<double, BN, BK, THREADS> cr;
        fetch_chunk<double, BN, BK, THREADS>(cr, a.C, (int64_t)ct * BN, k, d, kc * BK, a.cvec);
        store_chunk_rows<BN, THREADS>(cr, Cres + (size_t)(ct * n_kchunks + kc) * BN * LD, LD);
      }
      for (int j = tid; j < BN; j += THREADS)
        hres[ct * BN + j] = (ct * BN + j < k) ? a.h[ct * BN + j] : inf_value<double>();
    }
  }
  unsigned my_changed = 0;

  // update geometry: groups of G lanes, group og owns the clusters j with j % NG == og
  const int G = owner_group_lanes(d);
  const int NG = (THREADS / 32) * (32 / G);
  const int og = warp * (32 / G) + lane / G;
  const int gl = lane % G;

  ChunkRegs<double, BM, BK, THREADS> xr;
  ChunkRegs<double, BN, BK, THREADS> cr;
  if (blockIdx.x < n_tiles) {
    fetch_chunk<double, BM, BK, THREADS>(xr, a.X, (int64_t)blockIdx.x * BM, n, d, 0, a.xvec);
    if (!RESIDENT) fetch_chunk<double, BN, BK, THREADS>(cr, a.C, 0, k, d, 0, a.cvec);
  }

  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int64_t m0 = tile * BM;
    const int rows = (int)((n - m0 < BM) ? (n - m0) : BM);
    // previous label of the row this thread will write: fetched now, compared after the argmin
    uint32_t prev_lab = 0xffffffffu;
    if (UPDATE && a.prev != nullptr && tid < rows) prev_lab = __ldg(a.prev + m0 + tid);
    double best[2];
    uint32_t bi[2];
#pragma unroll
    for (int mi = 0; mi < 2; ++mi) {
      best[mi] = inf_value<double>();
      bi[mi] = 0u;
    }

    for (int ct = 0; ct < n_ctiles; ++ct) {
      const int cn = ct * BN;
      double acc[2][8][2];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int ni = 0; ni < 8; ++ni) acc[mi][ni][0] = acc[mi][ni][1] = 0.0;

      for (int kc = 0; kc < n_kchunks; ++kc) {
        const bool stage_x = !(n_kchunks == 1 && ct > 0);
        __syncthreads();
        if (stage_x) store_chunk_rows<BM, THREADS>(xr, Xs, LD);
        if (!RESIDENT) {
          store_chunk_rows<BN, THREADS>(cr, Cs, LD);
          if (kc == 0 && tid < BN) hs[tid] = (cn + tid < k) ? a.h[cn + tid] : inf_value<double>();
        }
        __syncthreads();
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
          if (more && next_stage_x) fetch_chunk<double, BM, BK, THREADS>(xr, a.X, ntile * BM, n, d, nkc * BK, a.xvec);
          if (more && !RESIDENT) fetch_chunk<double, BN, BK, THREADS>(cr, a.C, (int64_t)nct * BN, k, d, nkc * BK, a.cvec);
        }
        const double* Cc = RESIDENT ? Cres + (size_t)(ct * n_kchunks + kc) * BN * LD : Cs;
        const double* xa = Xs + (size_t)(warp * 16 + gid) * LD + tig;
        const double* cb = Cc + (size_t)gid * LD + tig;
#pragma unroll
        for (int k4 = 0; k4 < BK / 4; ++k4) {
          double af[2], bf[8];
#pragma unroll
          for (int mi = 0; mi < 2; ++mi) af[mi] = xa[mi * 8 * LD + k4 * 4];
#pragma unroll
          for (int ni = 0; ni < 8; ++ni) bf[ni] = cb[ni * 8 * LD + k4 * 4];
#pragma unroll
          for (int ni = 0; ni < 8; ++ni)
#pragma unroll
            for (int mi = 0; mi < 2; ++mi) dmma884(acc[mi][ni], af[mi], bf[ni]);
        }
      }

      // fold this centroid tile into the running minimum, columns in ascending order
      const double* hc = RESIDENT ? hres + cn : hs;
#pragma unroll
      for (int ni = 0; ni < 8; ++ni) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int col = ni * 8 + 2 * tig + e;
          const double hj = hc[col];
#pragma unroll
          for (int mi = 0; mi < 2; ++mi) {
            const double q = hj - acc[mi][ni][e];
            if (q < best[mi]) {
              best[mi] = q;
              bi[mi] = (uint32_t)(cn + col);
            }
          }
        }
      }
    }

    // merge the 4 lanes that share a row; lane tig == 0 then holds the row's label
#pragma unroll
    for (int mi = 0; mi < 2; ++mi) {
#pragma unroll
      for (int o = 1; o <= 2; o <<= 1) {
        const double oq = __shfl_xor_sync(0xffffffffu, best[mi], o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi[mi], o);
        if (oq < best[mi] || (oq == best[mi] && oi < bi[mi])) {
          best[mi] = oq;
          bi[mi] = oi;
        }
      }
      if (tig == 0) lab_s[warp * 16 + mi * 8 + gid] = bi[mi];
    }
    __syncthreads();

    if (tid < rows) {
      const uint32_t lab = lab_s[tid];
      a.labels[m0 + tid] = lab;
      if (UPDATE) {
        my_changed += (prev_lab != lab) ? 1u : 0u;
        if (a.smem_priv) {
          const int owner = (int)(lab % (uint32_t)NG);
          const int pos = atomicAdd(&grp_cnt[owner], 1);
          grp_rows[owner * BM + pos] = (unsigned char)tid;
        } else {
          const double wi = a.w ? a.w[m0 + tid] : 1.0;
          atomicAdd(&acc_copy[(int64_t)k * d + lab], wi);
        }
      }
    }
    if (UPDATE && a.smem_priv) {
      __syncthreads();
      owner_group_update<double>(ssum, a.X + m0 * (int64_t)d, a.w ? a.w + m0 : nullptr, lab_s,
                                 grp_rows + og * BM, grp_cnt[og], d, k, G, gl);
      __syncwarp();
      if (gl == 0) grp_cnt[og] = 0;
    } else if (UPDATE) {
      const int total = rows * d;
      const double* xt = a.X + m0 * (int64_t)d;
      const int upd_drow = THREADS / d, upd_df = THREADS - upd_drow * d;
      int row = tid / d, f = tid - row * d;
      for (int e = tid; e < total; e += THREADS) {
        const double wi = a.w ? a.w[m0 + row] : 1.0;
        atomicAdd(&acc_copy[(int64_t)lab_s[row] * d + f], xt[e] * wi);
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
      for (int e = tid; e < priv_len; e += THREADS) {
        const double v = ssum[e];
        if (v != 0.0) atomicAdd(&acc_copy[e], v);
      }
    }
    const double tot = block_sum((double)my_changed, red_s);
    if (tid == 0 && tot != 0.0) atomicAdd(&acc_copy[(int64_t)k * d + k], tot);
  }
}

static size_t f64_resident_bytes(int d, int k) {
  const size_t n_ctiles = (size_t)ceil_div(k, F64_BN), n_kchunks = (size_t)ceil_div(d, F64_BK);
  return (n_ctiles * n_kchunks * F64_BN * F64_LD + n_ctiles * F64_BN) * sizeof(double);
}

// KMB_F64_WM=4 in the environment selects the 256-thread, 128-sample CTA of eight warps (A/B
// runs); the default is the 128-thread, 64-sample CTA of four warps, four to an SM.
static int f64_wm() {
  static int cached = -1;
  if (cached < 0) {
    const char* e = getenv("KMB_F64_WM");
    cached = (e != nullptr && e[0] == '4') ? 4 : 2;
  }
  return cached;
}

template <bool UPDATE, int NW>
static int launch_lloyd_f64_wm(F64Args args, cudaStream_t stream) {
  constexpr int BM = 16 * NW, THREADS = 32 * NW;
  const int64_t n_tiles = ceil_div(args.n, BM);
  if (n_tiles == 0) return KMB_OK;
  const size_t priv = (size_t)((int64_t)args.k * args.d + args.k) * sizeof(double);
  args.smem_priv = (UPDATE && priv <= F64_PRIV_SMEM_MAX) ? 1 : 0;
  const size_t res_bytes = f64_resident_bytes(args.d, args.k);
  args.resident = res_bytes <= F64_RES_SMEM_MAX ? 1 : 0;
  args.xvec = cc_vec_width<double>(args.X, args.d);
  args.cvec = cc_vec_width<double>(args.C, args.d);
  size_t dyn = args.smem_priv ? (priv + 15) / 16 * 16 : 0;
  dyn += args.resident ? res_bytes : (size_t)(F64_BN * F64_LD + F64_BN) * sizeof(double);
  auto kern = args.resident ? lloyd_f64_kernel<UPDATE, true, NW> : lloyd_f64_kernel<UPDATE, false, NW>;
  KMB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)(F64_PRIV_SMEM_MAX + F64_RES_SMEM_MAX + 16)));
  int64_t grid = (int64_t)sm_count() * (16 / NW);
  if (grid > n_tiles) grid = n_tiles;
  kern<<<(unsigned)grid, THREADS, dyn, stream>>>(args);
  KMB_CHECK_LAUNCH();
  return KMB_OK;
}

template <bool UPDATE>
static int launch_lloyd_f64(F64Args args, cudaStream_t stream) {
  return f64_wm() == 4 ? launch_lloyd_f64_wm<UPDATE, 8>(args, stream)
                       : launch_lloyd_f64_wm<UPDATE, 4>(args, stream);
}

// KMB_F64_MMA=0 in the environment sends float64 back to the DFMA kernel (A/B runs).
bool lloyd_f64_mma_enabled() {
  static int cached = -1;
  if (cached < 0) {
    const char* e = getenv("KMB_F64_MMA");
    cached = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return cached == 1;
}

int lloyd_f64_step(const double* X, const double* w, const double* C, const double* h,
                   const uint32_t* prev, uint32_t* labels, double* acc, int n_copies,
                   int64_t acc_len, int64_t n, int d, int k, cudaStream_t stream) {
  F64Args a{X, w, C, h, prev, labels, acc, n_copies, acc_len, n, d, k, 0, 0, 1, 1};
  return launch_lloyd_f64<true>(a, stream);
}

int lloyd_f64_assign(const double* X, const double* C, const double* h, uint32_t* labels, int64_t n,
                     int d, int k, cudaStream_t stream) {
  F64Args a{X, nullptr, C, h, nullptr, labels, nullptr, 1, 0, n, d, k, 0, 0, 1, 1};
  return launch_lloyd_f64<false>(a, stream);
}

}  // namespace kmb
