// k-means++ seeding kernels.  One round = sample (t CTAs) -> gather candidate rows ->
// step (one pass over X) -> select (1 CTA); nothing returns to the host inside a round.
//
// Every pass over the samples also leaves float64 sums of blocks of KPP_BLOCK rows, so the
// next round's sampler only has to walk the block sums and then one block of elements.
// Stands for the kernels of sklearn_numba_dpex/kmeans/kernels/kmeans_plusplus.py and the
// host loop of kmeans/drivers.py:847-908.
#include "kmb_common.cuh"

namespace kmb {

constexpr int KPP_BLOCK = 512;    // rows per partial-sum block (one CTA each)
constexpr int KPP_THREADS = 128;
constexpr int KPP_MAX_T = 16;     // 2 + ln(k) stays below 16 for k < 1.2e6

// One pass over the samples for up to TT candidates at once:
//   M_out[tau, i] = min(w_i * ||cand_tau - x_i||^2, closest_i)     (no min when closest == NULL)
//   bsum_out[tau, block] = float64 sum of the block's values.
// A CTA owns KPP_BLOCK consecutive rows and streams them through shared memory in tiles of
// KPP_THREADS / G rows with 16-byte asynchronous copies (KPP_STAGES tiles in flight), so the
// bytes outstanding per SM do not depend on the register budget of the arithmetic.  One row
// belongs to G adjacent threads (G = 1 unless rows are long); every thread walks its 16-byte
// chunks in ascending feature order (the tile's odd row pitch keeps these reads free of bank
// conflicts, the candidate reads are broadcasts) and keeps one running sum per candidate in
// registers: no reduction across lanes for G = 1, one or two shuffles otherwise.
constexpr int KPP_STAGES = 2;

// Threads per row: rows longer than 256 bytes are split over 2 or 4 threads so that a tile
// of KPP_THREADS / G rows stays around 32 KB.
inline int kpp_threads_per_row(int d, size_t esize) {
  const size_t row_bytes = (size_t)d * esize;
  return row_bytes <= 256 ? 1 : (row_bytes <= 512 ? 2 : 4);
}

// One aligned 16-byte load of VEC consecutive features (no bounds or alignment test).
template <typename T>
__device__ __forceinline__ void load16(const T* __restrict__ p, T (&v)[RowVec<T>::VEC]) {
  if constexpr (sizeof(T) == 4) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  } else {
    const double2 q = *reinterpret_cast<const double2*>(p);
    v[0] = q.x; v[1] = q.y;
  }
}

// Copies rows [r0, r0 + rows) of X (rows x d) into a tile whose rows are dp = d rounded up to
// whole 16-byte chunks, pitch ld.  Aligned rows go as 16-byte asynchronous copies; other rows
// element by element (4- or 8-byte asynchronous copies), the padding features of the tile
// having been zeroed once by zero_tile_padding.  Either way the arithmetic that follows reads
// whole aligned chunks and needs no bounds test.  One commit group per call.
template <typename T, int THREADS>
__device__ __forceinline__ void issue_padded_tile(T* __restrict__ dst, const T* __restrict__ X,
                                                  int64_t r0, int rows, int d, int ld, bool vec) {
  if (vec || rows <= 0) {
    issue_row_tile<T, THREADS>(dst, X, r0, rows, d, ld, true);
    return;
  }
  const T* src = X + r0 * (int64_t)d;
  const int total = rows * d;
  for (int e = threadIdx.x; e < total; e += THREADS) {
    const int row = e / d, f = e - row * d;
    __pipeline_memcpy_async(dst + (size_t)row * ld + f, src + e, sizeof(T));
  }
  __pipeline_commit();
}

template <typename T, int THREADS>
__device__ __forceinline__ void zero_tile_padding(T* __restrict__ tile, int tile_rows, int d, int dp,
                                                  int ld) {
  const int pad = dp - d;
  for (int e = threadIdx.x; e < tile_rows * pad; e += THREADS)
    tile[(size_t)(e / pad) * ld + d + e % pad] = T(0);
}

// The inner loop is free of bounds tests, and of the `tau < t` test as well: rows are staged
// as whole 16-byte chunks (zero padding features) and candidates t..TT-1 are zero rows whose
// sums are computed and dropped.  (A form with those tests costs three times the instructions.)
template <typename T, int TT>
__global__ void __launch_bounds__(KPP_THREADS)
kpp_scan_kernel(const T* __restrict__ X, const T* __restrict__ w, const T* __restrict__ cand_rows,
                const T* __restrict__ M_prev, const int32_t* __restrict__ best_prev,
                T* __restrict__ M_out, double* __restrict__ bsum_out, T* __restrict__ centers0,
                int64_t n, int d, int t, int64_t nb, int G, int aligned, int c_elems) {
  constexpr int VEC = RowVec<T>::VEC;
  __shared__ double red[32];
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  T* c = reinterpret_cast<T*>(dyn_smem);              // TT x dp candidates, zero padded
  T* tiles = c + c_elems;                             // KPP_STAGES x (R x ld)
  const int R = KPP_THREADS / G;                      // rows per tile
  const bool vec_ok = aligned != 0;                   // 16-byte copies usable for X rows
  const int dp = (d + VEC - 1) / VEC * VEC;           // row length in shared memory
  const int ld = tile_row_pitch<T>(dp, true);
  const size_t tile_elems = (size_t)R * ld;
  const int64_t b0 = (int64_t)blockIdx.x * KPP_BLOCK;
  const int n_tiles = KPP_BLOCK / R;

  if (dp != d) zero_tile_padding<T, KPP_THREADS>(tiles, KPP_STAGES * R, d, dp, ld);
#pragma unroll
  for (int sidx = 0; sidx < KPP_STAGES; ++sidx) {
    const int64_t r0 = b0 + (int64_t)sidx * R;
    const int rows = (sidx < n_tiles && r0 < n) ? (int)((n - r0 < R) ? (n - r0) : R) : 0;
    issue_padded_tile<T, KPP_THREADS>(tiles + sidx * tile_elems, X, r0, rows, d, ld, vec_ok);
  }
  for (int e = threadIdx.x; e < TT * dp; e += KPP_THREADS) {
    const int tau = e / dp, f = e - tau * dp;
    c[e] = (tau < t && f < d) ? cand_rows[tau * d + f] : T(0);
  }
  if (centers0 != nullptr && blockIdx.x == 0)
    for (int f = threadIdx.x; f < d; f += KPP_THREADS) centers0[f] = cand_rows[f];
  const T* closest = M_prev ? M_prev + (int64_t)(best_prev ? *best_prev : 0) * n : nullptr;
  const int r = threadIdx.x / G, li = threadIdx.x % G;   // row in the tile, part of the row
  const int nq = dp / VEC;                                // 16-byte chunks per row
  double acc[TT];
#pragma unroll
  for (int tau = 0; tau < TT; ++tau) acc[tau] = 0.0;

  for (int tix = 0; tix < n_tiles; ++tix) {
    __pipeline_wait_prior(KPP_STAGES - 1);
    __syncthreads();
    const T* row = tiles + (tix % KPP_STAGES) * tile_elems + (size_t)r * ld;
    const int64_t i = b0 + (int64_t)tix * R + r;
    const bool valid = i < n;
    // fetched first, so that their latency hides behind the distance arithmetic
    const T wi = (valid && w) ? w[i] : T(1);
    const T cl = (valid && closest) ? closest[i] : inf_value<T>();
    T s[TT];
#pragma unroll
    for (int tau = 0; tau < TT; ++tau) s[tau] = T(0);
    if constexpr (sizeof(T) == 4) {
      // packed fp32x2 arithmetic: one instruction subtracts or multiply-adds two features, so
      // the even features of a row accumulate in the low half and the odd ones in the high half
      unsigned long long s2[TT];
#pragma unroll
      for (int tau = 0; tau < TT; ++tau) s2[tau] = 0ull;
      for (int q = li; q < nq; q += G) {
        const ulonglong2 xq = *reinterpret_cast<const ulonglong2*>(row + q * VEC);
        const T* cq = c + q * VEC;
#pragma unroll
        for (int tau = 0; tau < TT; ++tau) {
          const ulonglong2 cv = *reinterpret_cast<const ulonglong2*>(cq + tau * dp);
          unsigned long long d0, d1;
          asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d0) : "l"(cv.x), "l"(xq.x));
          asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d1) : "l"(cv.y), "l"(xq.y));
          asm("fma.rn.f32x2 %0, %1, %1, %2;" : "=l"(s2[tau]) : "l"(d0), "l"(s2[tau]));
          asm("fma.rn.f32x2 %0, %1, %1, %2;" : "=l"(s2[tau]) : "l"(d1), "l"(s2[tau]));
        }
      }
#pragma unroll
      for (int tau = 0; tau < TT; ++tau)
        s[tau] = (T)(__uint_as_float((unsigned)(s2[tau] & 0xffffffffull)) +
                     __uint_as_float((unsigned)(s2[tau] >> 32)));
    } else {
      for (int q = li; q < nq; q += G) {
        T xv[VEC];
        load16<T>(row + q * VEC, xv);
        const T* cq = c + q * VEC;
#pragma unroll
        for (int tau = 0; tau < TT; ++tau) {
          T cv[VEC];
          load16<T>(cq + tau * dp, cv);
#pragma unroll
          for (int jj = 0; jj < VEC; ++jj) {
            const T diff = cv[jj] - xv[jj];
            s[tau] = fma(diff, diff, s[tau]);
          }
        }
      }
    }
    if (G > 1) {
#pragma unroll
      for (int tau = 0; tau < TT; ++tau) {
        if (tau < t) {
          s[tau] += __shfl_xor_sync(0xffffffffu, s[tau], 1);
          if (G > 2) s[tau] += __shfl_xor_sync(0xffffffffu, s[tau], 2);
        }
      }
    }
    if (valid && li == 0) {
      T* out = M_out + i;
#pragma unroll
      for (int tau = 0; tau < TT; ++tau) {
        if (tau < t) {
          T v = s[tau] * wi;
          v = (v < cl) ? v : cl;
          *out = v;
          out += n;
          acc[tau] += (double)v;
        }
      }
    }
    __syncthreads();
    const int nxt = tix + KPP_STAGES;
    const int64_t rn = b0 + (int64_t)nxt * R;
    const int rows = (nxt < n_tiles && rn < n) ? (int)((n - rn < R) ? (n - rn) : R) : 0;
    issue_padded_tile<T, KPP_THREADS>(tiles + (nxt % KPP_STAGES) * tile_elems, X, rn, rows, d, ld, vec_ok);
  }
  __pipeline_wait_prior(0);
#pragma unroll
  for (int tau = 0; tau < TT; ++tau) {
    if (tau < t) {
      const double tot = block_sum(acc[tau], red);
      if (threadIdx.x == 0) bsum_out[(int64_t)tau * nb + blockIdx.x] = tot;
    }
  }
}

// The same pass for fp32 rows and several candidates, with TWO
// rows per thread: every broadcast read of a candidate chunk from shared memory then serves two
// rows, which halves the shared-memory reads and the instructions per row (with ten candidates
// the one-row form spends 46 % of the shared-memory pipe on those reads).  A tile of
// 2 * KPP_THREADS / G rows is as large as both stages of the one-row form, so there is one
// buffer per CTA and the three resident CTAs of a SM overlap each other's copies.  Per-row
// arithmetic is identical to the one-row form (same chunk order, same packed accumulators).
template <int TT>
__global__ void __launch_bounds__(KPP_THREADS)
kpp_scan2_kernel(const float* __restrict__ X, const float* __restrict__ w,
                 const float* __restrict__ cand_rows, const float* __restrict__ M_prev,
                 const int32_t* __restrict__ best_prev, float* __restrict__ M_out,
                 double* __restrict__ bsum_out, int64_t n, int d, int t, int64_t nb, int G,
                 int aligned, int c_elems) {
  __shared__ double red[32];
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  float* c = reinterpret_cast<float*>(dyn_smem);     // TT x dp candidates, zero padded
  float* tile = c + c_elems;                         // R x ld
  const int Rh = KPP_THREADS / G;                    // rows per half tile
  const int R = 2 * Rh;
  const int dp = (d + 3) / 4 * 4;
  const int ld = tile_row_pitch<float>(dp, true);
  const int64_t b0 = (int64_t)blockIdx.x * KPP_BLOCK;
  const int n_tiles = KPP_BLOCK / R;
  if (dp != d) zero_tile_padding<float, KPP_THREADS>(tile, R, d, dp, ld);
  for (int e = threadIdx.x; e < TT * dp; e += KPP_THREADS) {
    const int tau = e / dp, f = e - tau * dp;
    c[e] = (tau < t && f < d) ? cand_rows[tau * d + f] : 0.f;
  }
  const float* closest = M_prev ? M_prev + (int64_t)(best_prev ? *best_prev : 0) * n : nullptr;
  const int r = threadIdx.x / G, li = threadIdx.x % G;
  const int nq = dp / 4;
  double acc[TT];
#pragma unroll
  for (int tau = 0; tau < TT; ++tau) acc[tau] = 0.0;

  for (int tix = 0; tix < n_tiles; ++tix) {
    const int64_t r0 = b0 + (int64_t)tix * R;
    const int rows = (r0 < n) ? (int)((n - r0 < R) ? (n - r0) : R) : 0;
    issue_padded_tile<float, KPP_THREADS>(tile, X, r0, rows, d, ld, aligned != 0);
    const int64_t i0 = r0 + r, i1 = i0 + Rh;
    const bool valid0 = i0 < n, valid1 = i1 < n;
    // fetched first, so that their latency hides behind the copy and the arithmetic
    const float w0 = (valid0 && w) ? w[i0] : 1.f, w1 = (valid1 && w) ? w[i1] : 1.f;
    const float cl0 = (valid0 && closest) ? closest[i0] : inf_value<float>();
    const float cl1 = (valid1 && closest) ? closest[i1] : inf_value<float>();
    __pipeline_wait_prior(0);
    __syncthreads();
    const float* row0 = tile + (size_t)r * ld;
    const float* row1 = tile + (size_t)(r + Rh) * ld;
    unsigned long long sa[TT], sb[TT];
#pragma unroll
    for (int tau = 0; tau < TT; ++tau) sa[tau] = sb[tau] = 0ull;
    for (int q = li; q < nq; q += G) {
      const ulonglong2 xa = *reinterpret_cast<const ulonglong2*>(row0 + q * 4);
      const ulonglong2 xb = *reinterpret_cast<const ulonglong2*>(row1 + q * 4);
      const float* cq = c + q * 4;
#pragma unroll
      for (int tau = 0; tau < TT; ++tau) {
        const ulonglong2 cv = *reinterpret_cast<const ulonglong2*>(cq + tau * dp);
        unsigned long long d0, d1, e0, e1;
        asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d0) : "l"(cv.x), "l"(xa.x));
        asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d1) : "l"(cv.y), "l"(xa.y));
        asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(e0) : "l"(cv.x), "l"(xb.x));
        asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(e1) : "l"(cv.y), "l"(xb.y));
        asm("fma.rn.f32x2 %0, %1, %1, %2;" : "=l"(sa[tau]) : "l"(d0), "l"(sa[tau]));
        asm("fma.rn.f32x2 %0, %1, %1, %2;" : "=l"(sb[tau]) : "l"(e0), "l"(sb[tau]));
        asm("fma.rn.f32x2 %0, %1, %1, %2;" : "=l"(sa[tau]) : "l"(d1), "l"(sa[tau]));
        asm("fma.rn.f32x2 %0, %1, %1, %2;" : "=l"(sb[tau]) : "l"(e1), "l"(sb[tau]));
      }
    }
#pragma unroll
    for (int tau = 0; tau < TT; ++tau) {
      if (tau < t) {
        float s0 = __uint_as_float((unsigned)(sa[tau] & 0xffffffffull)) +
                   __uint_as_float((unsigned)(sa[tau] >> 32));
        float s1 = __uint_as_float((unsigned)(sb[tau] & 0xffffffffull)) +
                   __uint_as_float((unsigned)(sb[tau] >> 32));
        if (G > 1) {
          s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
          s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
          if (G > 2) {
            s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
            s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
          }
        }
        if (li == 0) {
          if (valid0) {
            float v = s0 * w0;
            v = (v < cl0) ? v : cl0;
            M_out[(int64_t)tau * n + i0] = v;
            acc[tau] += (double)v;
          }
          if (valid1) {
            float v = s1 * w1;
            v = (v < cl1) ? v : cl1;
            M_out[(int64_t)tau * n + i1] = v;
            acc[tau] += (double)v;
          }
        }
      }
    }
    __syncthreads();   // the tile is overwritten by the next copy
  }
#pragma unroll
  for (int tau = 0; tau < TT; ++tau) {
    if (tau < t) {
      const double tot = block_sum(acc[tau], red);
      if (threadIdx.x == 0) bsum_out[(int64_t)tau * nb + blockIdx.x] = tot;
    }
  }
}

// One CTA per trial.  r = u * total; walk the block sums, then the elements of the block
// where the float64 inclusive prefix first reaches r.
template <typename T>
__global__ void __launch_bounds__(KPP_THREADS)
kpp_sample_kernel(const T* __restrict__ M, const double* __restrict__ bsum,
                  const int32_t* __restrict__ best, const T* __restrict__ total,
                  const T* __restrict__ u, const double* __restrict__ offset,
                  int32_t* __restrict__ cand, int64_t n, int64_t nb) {
  __shared__ double scan_s[KPP_THREADS];
  __shared__ double carry_s;
  __shared__ unsigned long long found_s;  // smallest matching index, ~0 = none
  const int tid = threadIdx.x;
  const int b = best ? *best : 0;
  const T* closest = M + (int64_t)b * n;
  const double* bs = bsum + (int64_t)b * nb;
  const T r_t = u[blockIdx.x] * total[0];
  // on a row shard the threshold is taken relative to the potential held by earlier shards
  const double r = (double)r_t - (offset ? offset[0] : 0.0);
  if (!(r > 0.0)) {
    if (tid == 0) cand[blockIdx.x] = 0;
    return;
  }
  if (tid == 0) {
    carry_s = 0.0;
    found_s = ~0ull;
  }
  __syncthreads();
  // --- level 1: first block whose inclusive prefix >= r.  Every thread sums one contiguous
  // segment of the block sums, one scan of the KPP_THREADS segment totals finds the segment in
  // which the prefix first reaches r, and its thread walks that segment.
  const int64_t seg = (nb + KPP_THREADS - 1) / KPP_THREADS;
  const int64_t s0 = (int64_t)tid * seg, s1 = (s0 + seg < nb) ? s0 + seg : nb;
  double mine = 0.0;
  for (int64_t j = s0; j < s1; ++j) mine += bs[j];
  scan_s[tid] = mine;
  __syncthreads();
  for (int o = 1; o < KPP_THREADS; o <<= 1) {
    const double add = (tid >= o) ? scan_s[tid - o] : 0.0;
    __syncthreads();
    scan_s[tid] += add;
    __syncthreads();
  }
  unsigned long long my_hit = ~0ull;
  double my_before = 0.0;
  {
    const double incl = scan_s[tid];
    const double excl = (tid == 0) ? 0.0 : scan_s[tid - 1];
    if (s0 < s1 && incl >= r && !(excl >= r)) {
      // this thread's segment: walk it from the prefix before it
      double run = excl;
      int64_t hit = s1 - 1;                        // rounding can leave r just past the last prefix
      for (int64_t j = s0; j < s1; ++j) {
        if (run + bs[j] >= r) {
          hit = j;
          break;
        }
        run += bs[j];
      }
      my_hit = (unsigned long long)hit;
      my_before = run;                             // prefix before block `hit`
      // with non-monotone prefixes (negative weights) several segments can qualify: lowest wins
      atomicMin(&found_s, my_hit);
    }
  }
  __syncthreads();
  if (my_hit != ~0ull && found_s == my_hit) carry_s = my_before;
  __syncthreads();
  if (found_s == ~0ull) {  // r beyond the last prefix: the running sum never reaches it
    if (tid == 0) cand[blockIdx.x] = (int32_t)(n - 1);
    return;
  }
  const int64_t blk = (int64_t)found_s;
  const double before = carry_s;                   // prefix before the block
  __syncthreads();
  // --- level 2: elements of block blk, KPP_THREADS at a time
  const int64_t e0 = blk * KPP_BLOCK;
  const int64_t e1 = (e0 + KPP_BLOCK < n) ? (e0 + KPP_BLOCK) : n;
  if (tid == 0) {
    carry_s = before;
    found_s = ~0ull;
  }
  __syncthreads();
  for (int64_t c0 = e0; c0 < e1; c0 += KPP_THREADS) {
    const int64_t i = c0 + tid;
    scan_s[tid] = (i < e1) ? (double)closest[i] : 0.0;
    __syncthreads();
    for (int o = 1; o < KPP_THREADS; o <<= 1) {
      const double add = (tid >= o) ? scan_s[tid - o] : 0.0;
      __syncthreads();
      scan_s[tid] += add;
      __syncthreads();
    }
    const double incl = carry_s + scan_s[tid];
    const double excl = (tid == 0) ? carry_s : carry_s + scan_s[tid - 1];
    if (i < e1 && incl >= r && !(excl >= r)) atomicMin(&found_s, (unsigned long long)i);
    __syncthreads();
    if (found_s != ~0ull) break;
    if (tid == 0) carry_s += scan_s[KPP_THREADS - 1];
    __syncthreads();
  }
  if (tid == 0) {
    // rounding between the two levels can leave r just past the block's last prefix
    const int64_t res = (found_s != ~0ull) ? (int64_t)found_s : (e1 - 1);
    cand[blockIdx.x] = (int32_t)res;
  }
}

template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ X, const int32_t* __restrict__ ids, int d,
                                   T* __restrict__ out) {
  const int64_t row = ids[blockIdx.x];
  for (int f = threadIdx.x; f < d; f += blockDim.x)
    out[(int64_t)blockIdx.x * d + f] = X[row * (int64_t)d + f];
}

// Single CTA: potentials in fixed order, argmin (lowest trial on ties), commit the centre.
template <typename T>
__global__ void __launch_bounds__(KPP_THREADS)
kpp_select_kernel(const double* __restrict__ bsum, const double* __restrict__ pots_in, int t,
                  int64_t nb, T* __restrict__ pots,
                  int32_t* __restrict__ best, T* __restrict__ total,
                  const T* __restrict__ cand_rows, const int32_t* __restrict__ cand,
                  T* __restrict__ centers, int32_t* __restrict__ indices, int c, int d) {
  __shared__ double red[32];
  __shared__ T pots_s[KPP_MAX_T];
  __shared__ int best_s;
  for (int tau = 0; tau < t; ++tau) {
    double tot;
    if (pots_in != nullptr) {
      tot = pots_in[tau];
    } else {
      double s = 0.0;
      for (int64_t b = threadIdx.x; b < nb; b += KPP_THREADS) s += bsum[(int64_t)tau * nb + b];
      tot = block_sum(s, red);
    }
    if (threadIdx.x == 0) pots_s[tau] = (T)tot;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    int bi = 0;
    T bv = pots_s[0];
    for (int tau = 1; tau < t; ++tau)
      if (pots_s[tau] < bv) {
        bv = pots_s[tau];
        bi = tau;
      }
    best_s = bi;
    *best = bi;
    *total = bv;
    if (pots)
      for (int tau = 0; tau < t; ++tau) pots[tau] = pots_s[tau];
    if (indices && cand) indices[c] = cand[bi];
  }
  __syncthreads();
  if (centers && cand_rows)
    for (int f = threadIdx.x; f < d; f += KPP_THREADS)
      centers[(int64_t)c * d + f] = cand_rows[(int64_t)best_s * d + f];
}

// Row shards: one block per trial picks the owner shard's candidate out of the gathered ones.
template <typename T>
__global__ void __launch_bounds__(KPP_THREADS)
kpp_pick_owned_kernel(const T* __restrict__ gathered, int n_shards, int t, int d,
                      const double* __restrict__ ends, const T* __restrict__ u,
                      const T* __restrict__ total, const int64_t* __restrict__ rows_offset,
                      int32_t* __restrict__ cand_global, T* __restrict__ rows_global) {
  const int tau = blockIdx.x;
  const double r = (double)(u[tau] * total[0]);
  int owner = 0;
  for (int w = 0; w < n_shards; ++w) owner += (ends[w] < r) ? 1 : 0;
  if (owner > n_shards - 1) owner = n_shards - 1;
  const T* src = gathered + ((int64_t)owner * t + tau) * (d + 1);
  for (int f = threadIdx.x; f < d; f += KPP_THREADS) rows_global[(int64_t)tau * d + f] = src[f];
  if (threadIdx.x == 0) {
    int32_t id;
    if (sizeof(T) == 4) {
      id = __float_as_int((float)src[d]);          // the column carries the id's bit pattern
    } else {
      id = (int32_t)src[d];
    }
    cand_global[tau] = (int32_t)((int64_t)id + rows_offset[owner]);
  }
}

// Row shards, single CTA: potentials summed over the shards in ascending order, argmin (lowest
// trial on ties), commit of the centre, and the prefix of the chosen candidate's shares.
template <typename T>
__global__ void __launch_bounds__(KPP_THREADS)
kpp_select_shards_kernel(const double* __restrict__ shard_pots, int n_shards, int shard, int t,
                         T* __restrict__ pots, int32_t* __restrict__ best, T* __restrict__ total,
                         const T* __restrict__ cand_rows, const int32_t* __restrict__ cand,
                         T* __restrict__ centers, int32_t* __restrict__ indices, int c, int d,
                         double* __restrict__ ends_out, double* __restrict__ offset_out) {
  __shared__ int best_s;
  if (threadIdx.x == 0) {
    int bi = 0;
    T bv = T(0);
    for (int tau = 0; tau < t; ++tau) {
      double tot = 0.0;
      for (int w = 0; w < n_shards; ++w) tot += shard_pots[(int64_t)w * t + tau];
      const T pv = (T)tot;
      if (pots) pots[tau] = pv;
      if (tau == 0 || pv < bv) {
        bv = pv;
        bi = tau;
      }
    }
    best_s = bi;
    *best = bi;
    *total = bv;
    if (indices && cand) indices[c] = cand[bi];
    double run = 0.0, mine = 0.0;
    for (int w = 0; w < n_shards; ++w) {
      if (w == shard) mine = run;
      run += shard_pots[(int64_t)w * t + bi];
      if (ends_out) ends_out[w] = run;
    }
    if (offset_out) *offset_out = mine;
  }
  __syncthreads();
  if (centers && cand_rows)
    for (int f = threadIdx.x; f < d; f += KPP_THREADS)
      centers[(int64_t)c * d + f] = cand_rows[(int64_t)best_s * d + f];
}

// pots[tau] = sum_b bsum[tau, b] in float64, fixed order; one block per trial.
__global__ void __launch_bounds__(KPP_THREADS)
kpp_potentials_kernel(const double* __restrict__ bsum, int64_t nb, double* __restrict__ pots) {
  __shared__ double red[32];
  double s = 0.0;
  for (int64_t b = threadIdx.x; b < nb; b += KPP_THREADS) s += bsum[(int64_t)blockIdx.x * nb + b];
  const double tot = block_sum(s, red);
  if (threadIdx.x == 0) pots[blockIdx.x] = tot;
}

// Launches kpp_scan_kernel with the instantiation that fits t and the dtype.
template <typename T>
static int launch_kpp_scan(const T* X, const T* w, const T* cand_rows, const T* M_prev,
                           const int32_t* best_prev, T* M_out, double* bsum_out, T* centers0,
                           int64_t n, int d, int t, cudaStream_t stream) {
  constexpr int VEC = RowVec<T>::VEC;
  const int G = kpp_threads_per_row(d, sizeof(T));
  const int R = KPP_THREADS / G;
  const int64_t nb = ceil_div(n, KPP_BLOCK);
  const int aligned = ((d % VEC == 0) && (((uintptr_t)X & 15) == 0)) ? 1 : 0;
  // shared memory holds TT candidate rows (zero rows beyond t) of dp = d rounded up to whole
  // 16-byte chunks, and tiles whose rows are dp long as well
  const int tt = t <= 1 ? 1 : (t <= 4 ? 4 : (t <= 6 ? 6 : (t <= 8 ? 8 : (t <= 10 ? 10 : (t <= 12 ? 12 : KPP_MAX_T)))));
  const int dp = (d + VEC - 1) / VEC * VEC;
  const int c_elems = tt * dp;
  const int ld = tile_row_pitch<T>(dp, true);
  const size_t dyn = ((size_t)c_elems + (size_t)KPP_STAGES * R * ld) * sizeof(T);
  KMB_REQUIRE(dyn <= 200 * 1024, "k-means++ pass: rows too long for the staged tiles (d=%d, t=%d)", d, t);
  auto run = [&](auto kern) -> int {
    if (dyn > 48 * 1024)
      KMB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    kern<<<(unsigned)nb, KPP_THREADS, dyn, stream>>>(X, w, cand_rows, M_prev, best_prev, M_out,
                                                     bsum_out, centers0, n, d, t, nb, G, aligned,
                                                     c_elems);
    KMB_CHECK_LAUNCH();
    return KMB_OK;
  };
  if constexpr (sizeof(T) == 4) {
    // several candidates: two rows per thread, one tile buffer (see kpp_scan2_kernel)
    const size_t dyn2 = ((size_t)c_elems + (size_t)2 * R * ld) * sizeof(T);
    if (tt >= 6 && centers0 == nullptr && dyn2 <= 74 * 1024) {
      auto run2 = [&](auto kern) -> int {
        if (dyn2 > 48 * 1024)
          KMB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn2));
        kern<<<(unsigned)nb, KPP_THREADS, dyn2, stream>>>(X, w, cand_rows, M_prev, best_prev, M_out,
                                                          bsum_out, n, d, t, nb, G, aligned, c_elems);
        KMB_CHECK_LAUNCH();
        return KMB_OK;
      };
      switch (tt) {
        case 6: return run2(kpp_scan2_kernel<6>);
        case 8: return run2(kpp_scan2_kernel<8>);
        case 10: return run2(kpp_scan2_kernel<10>);
        case 12: return run2(kpp_scan2_kernel<12>);
        default: return run2(kpp_scan2_kernel<KPP_MAX_T>);
      }
    }
  }
  switch (tt) {
    case 1: return run(kpp_scan_kernel<T, 1>);
    case 4: return run(kpp_scan_kernel<T, 4>);
    case 6: return run(kpp_scan_kernel<T, 6>);
    case 8: return run(kpp_scan_kernel<T, 8>);
    case 10: return run(kpp_scan_kernel<T, 10>);
    case 12: return run(kpp_scan_kernel<T, 12>);
    default: return run(kpp_scan_kernel<T, KPP_MAX_T>);
  }
}

}  // namespace kmb

using namespace kmb;

extern "C" {

int kmb_kpp_block_rows(void) { return KPP_BLOCK; }

int kmb_kpp_init(int dtype, const void* X, const void* w, int64_t first, const void* first_row,
                 void* closest, double* bsum, void* centers, int32_t* indices, int64_t n, int d,
                 void* stream) {
  KMB_REQUIRE(X && closest && bsum && centers && indices, "kmb_kpp_init: NULL argument");
  KMB_REQUIRE(n > 0 && d > 0 && first >= 0 && (first_row != nullptr || first < n),
              "kmb_kpp_init: bad sizes");
  KMB_REQUIRE(n < (1ll << 31), "kmb_kpp_init: n must be below 2^31 (int32 candidate ids)");
  const int32_t first32 = (int32_t)first;
  KMB_CHECK_CUDA(cudaMemcpyAsync(indices, &first32, sizeof(int32_t), cudaMemcpyHostToDevice,
                                 (cudaStream_t)stream));
  KMB_DISPATCH_DTYPE(dtype, {
    const T* row = first_row ? (const T*)first_row : (const T*)X + first * (int64_t)d;
    return launch_kpp_scan<T>((const T*)X, (const T*)w, row, nullptr, nullptr, (T*)closest, bsum,
                              (T*)centers, n, d, 1, (cudaStream_t)stream);
  });
}

int kmb_kpp_sample(int dtype, const void* M, const double* bsum, const int32_t* best,
                   const void* total, const void* u, const double* offset, int t, int32_t* cand,
                   int64_t n, void* stream) {
  KMB_REQUIRE(M && bsum && total && u && cand, "kmb_kpp_sample: NULL argument");
  KMB_REQUIRE(n > 0 && t > 0 && t <= KPP_MAX_T, "kmb_kpp_sample: bad sizes");
  const int64_t nb = ceil_div(n, KPP_BLOCK);
  KMB_DISPATCH_DTYPE(dtype, {
    kpp_sample_kernel<T><<<t, KPP_THREADS, 0, (cudaStream_t)stream>>>(
        (const T*)M, bsum, best, (const T*)total, (const T*)u, offset, cand, n, nb);
    KMB_CHECK_LAUNCH();
  });
  return KMB_OK;
}

int kmb_gather_rows(int dtype, const void* X, const int32_t* ids, int t, int d, void* out,
                    void* stream) {
  KMB_REQUIRE(X && ids && out && t > 0 && d > 0, "kmb_gather_rows: bad arguments");
  KMB_DISPATCH_DTYPE(dtype, {
    gather_rows_kernel<T><<<t, 128, 0, (cudaStream_t)stream>>>((const T*)X, ids, d, (T*)out);
    KMB_CHECK_LAUNCH();
  });
  return KMB_OK;
}

int kmb_kpp_step(int dtype, const void* X, const void* w, const void* cand_rows, const void* M_prev,
                 const int32_t* best_prev, void* M_out, double* bsum_out, int64_t n, int d, int t,
                 void* stream) {
  KMB_REQUIRE(X && cand_rows && M_prev && M_out && bsum_out, "kmb_kpp_step: NULL argument");
  KMB_REQUIRE(n > 0 && d > 0 && t > 0 && t <= KPP_MAX_T, "kmb_kpp_step: bad sizes (t <= %d)",
              KPP_MAX_T);
  KMB_DISPATCH_DTYPE(dtype, {
    return launch_kpp_scan<T>((const T*)X, (const T*)w, (const T*)cand_rows, (const T*)M_prev,
                              best_prev, (T*)M_out, bsum_out, (T*)nullptr, n, d, t,
                              (cudaStream_t)stream);
  });
}

int kmb_kpp_potentials(const double* bsum, int t, int64_t nb, double* pots, void* stream) {
  KMB_REQUIRE(bsum && pots && t > 0 && nb > 0, "kmb_kpp_potentials: bad arguments");
  kpp_potentials_kernel<<<t, KPP_THREADS, 0, (cudaStream_t)stream>>>(bsum, nb, pots);
  KMB_CHECK_LAUNCH();
  return KMB_OK;
}

int kmb_kpp_select(int dtype, const double* bsum, const double* pots_in, int t, int64_t nb,
                   void* pots, int32_t* best, void* total, const void* cand_rows,
                   const int32_t* cand, void* centers, int32_t* indices, int c, int d,
                   void* stream) {
  KMB_REQUIRE((bsum || pots_in) && best && total, "kmb_kpp_select: NULL argument");
  KMB_REQUIRE(t > 0 && t <= KPP_MAX_T && nb > 0 && c >= 0 && d > 0, "kmb_kpp_select: bad sizes");
  KMB_DISPATCH_DTYPE(dtype, {
    kpp_select_kernel<T><<<1, KPP_THREADS, 0, (cudaStream_t)stream>>>(
        bsum, pots_in, t, nb, (T*)pots, best, (T*)total, (const T*)cand_rows, cand, (T*)centers,
        indices, c, d);
    KMB_CHECK_LAUNCH();
  });
  return KMB_OK;
}

int kmb_kpp_pick_owned(int dtype, const void* gathered, int n_shards, int t, int d,
                       const double* ends, const void* u, const void* total,
                       const int64_t* rows_offset, int32_t* cand_global, void* rows_global,
                       void* stream) {
  KMB_REQUIRE(gathered && ends && u && total && rows_offset && cand_global && rows_global,
              "kmb_kpp_pick_owned: NULL argument");
  KMB_REQUIRE(n_shards > 0 && t > 0 && t <= KPP_MAX_T && d > 0, "kmb_kpp_pick_owned: bad sizes");
  KMB_DISPATCH_DTYPE(dtype, {
    kpp_pick_owned_kernel<T><<<t, KPP_THREADS, 0, (cudaStream_t)stream>>>(
        (const T*)gathered, n_shards, t, d, ends, (const T*)u, (const T*)total, rows_offset,
        cand_global, (T*)rows_global);
    KMB_CHECK_LAUNCH();
  });
  return KMB_OK;
}

int kmb_kpp_select_shards(int dtype, const double* shard_pots, int n_shards, int shard, int t,
                          void* pots, int32_t* best, void* total, const void* cand_rows,
                          const int32_t* cand, void* centers, int32_t* indices, int c, int d,
                          double* ends_out, double* offset_out, void* stream) {
  KMB_REQUIRE(shard_pots && best && total, "kmb_kpp_select_shards: NULL argument");
  KMB_REQUIRE(n_shards > 0 && shard >= 0 && shard < n_shards && t > 0 && t <= KPP_MAX_T && c >= 0 && d > 0,
              "kmb_kpp_select_shards: bad sizes");
  KMB_DISPATCH_DTYPE(dtype, {
    kpp_select_shards_kernel<T><<<1, KPP_THREADS, 0, (cudaStream_t)stream>>>(
        shard_pots, n_shards, shard, t, (T*)pots, best, (T*)total, (const T*)cand_rows, cand,
        (T*)centers, indices, c, d, ends_out, offset_out);
    KMB_CHECK_LAUNCH();
  });
  return KMB_OK;
}

}  // extern "C"
