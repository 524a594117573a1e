// Building blocks of the register-tiled CUDA-core kernels (fused Lloyd step, euclidean
// distances): tile shapes per dtype, and the staging of a (rows x BK) chunk of a row-major
// matrix through registers into feature-major shared memory.
#pragma once
#include "kmb_common.cuh"

namespace kmb {

constexpr int CC_THREADS = 256;

template <typename T>
struct CcTile;
template <>
struct CcTile<float> {
  static constexpr int BM = 128, BN = 128, BK = 16, TM = 4, TN = 16, V = 4, PAD = 4;
};
template <>
struct CcTile<double> {
  static constexpr int BM = 128, BN = 64, BK = 8, TM = 4, TN = 8, V = 2, PAD = 2;
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

// Registers that hold one thread's share of a (ROWS x BK) chunk.  A row of the chunk is BK / 4
// quads of 4 consecutive features; thread t takes quad t % QPR of rows t / QPR, t / QPR + RSTEP, ...
template <typename T, int ROWS, int BK, int THREADS = CC_THREADS>
struct ChunkRegs {
  static constexpr int QPR = BK / 4;
  static constexpr int RSTEP = THREADS / QPR;
  static constexpr int N = (ROWS + RSTEP - 1) / RSTEP;
  T v[N][4];
};

// Fetches the chunk [row0, row0 + ROWS) x [k0, k0 + BK) of the row-major matrix M (n_rows x d)
// into registers, zero beyond the matrix.  `vec` is the widest aligned vector width.
template <typename T, int ROWS, int BK, int THREADS = CC_THREADS>
__device__ __forceinline__ void fetch_chunk(ChunkRegs<T, ROWS, BK, THREADS>& r, const T* __restrict__ M,
                                            int64_t row0, int64_t n_rows, int d, int k0, int vec) {
  using R = ChunkRegs<T, ROWS, BK, THREADS>;
  const int q = threadIdx.x % R::QPR;
  const int f0 = k0 + q * 4;
#pragma unroll
  for (int i = 0; i < R::N; ++i) {
    const int lr = threadIdx.x / R::QPR + i * R::RSTEP;
    const int64_t row = row0 + lr;
    T* v = r.v[i];
    v[0] = v[1] = v[2] = v[3] = T(0);
    if (lr < ROWS && row < n_rows && f0 < d) {
      const T* p = M + row * (int64_t)d + f0;
      if (f0 + 4 <= d && vec == 4) {
        if constexpr (sizeof(T) == 4) {
          const float4 t = __ldg(reinterpret_cast<const float4*>(p));
          v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        } else {
          const double2 a = __ldg(reinterpret_cast<const double2*>(p));
          const double2 b = __ldg(reinterpret_cast<const double2*>(p + 2));
          v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
        }
      } else if (vec >= 2 && f0 + 2 <= d) {
        if constexpr (sizeof(T) == 4) {
          const float2 a = __ldg(reinterpret_cast<const float2*>(p));
          v[0] = a.x; v[1] = a.y;
          if (f0 + 4 <= d) {
            const float2 b = __ldg(reinterpret_cast<const float2*>(p + 2));
            v[2] = b.x; v[3] = b.y;
          } else if (f0 + 3 <= d) {
            v[2] = __ldg(p + 2);
          }
        } else {
          const double2 a = __ldg(reinterpret_cast<const double2*>(p));
          v[0] = a.x; v[1] = a.y;
          if (f0 + 4 <= d) {
            const double2 b = __ldg(reinterpret_cast<const double2*>(p + 2));
            v[2] = b.x; v[3] = b.y;
          } else if (f0 + 3 <= d) {
            v[2] = __ldg(p + 2);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (f0 + j < d) v[j] = __ldg(p + j);
      }
    }
  }
}

// Stores the fetched chunk feature-major: S[kk][m], row pitch `ld`.
template <typename T, int ROWS, int BK, int THREADS = CC_THREADS>
__device__ __forceinline__ void store_chunk(const ChunkRegs<T, ROWS, BK, THREADS>& r, T* __restrict__ S, int ld) {
  using R = ChunkRegs<T, ROWS, BK, THREADS>;
  const int q = threadIdx.x % R::QPR;
#pragma unroll
  for (int i = 0; i < R::N; ++i) {
    const int m = threadIdx.x / R::QPR + i * R::RSTEP;
    if (m < ROWS) {
#pragma unroll
      for (int j = 0; j < 4; ++j) S[(q * 4 + j) * ld + m] = r.v[i][j];
    }
  }
}

// Widest vector width (elements: 4, 2 or 1) with which rows of a (rows x d) matrix at `base`
// can be loaded: every row start and every quad inside a row must be aligned to it.
template <typename T>
int cc_vec_width(const void* base, int d) {
  const uintptr_t p = (uintptr_t)base;
  if (d % 4 == 0 && p % (4 * sizeof(T) > 16 ? 16 : 4 * sizeof(T)) == 0) return 4;
  if (d % 2 == 0 && p % (2 * sizeof(T)) == 0) return 2;
  return 1;
}

// ---- atomics-free centroid update through owner groups ------------------------------------
// The clusters are dealt out to NG groups of G lanes (cluster j belongs to group j % NG); every
// row of the tile is on the list of the group that owns its label, and a group adds its rows
// into its own clusters' sums: no two groups ever touch the same sum, so plain shared-memory
// loads and stores do.  A lane serves 4 consecutive features; rows are taken two at a time so
// that the global loads of both are in flight together (the loads are the latency of the loop;
// four rows at a time with strided lanes measured 6 - 13 % slower).
constexpr int CC_MAX_GROUPS = 64;

__host__ __device__ inline int owner_group_lanes(int d) {
  int G = 4;
  while (G * 4 < d && G < 32) G <<= 1;
  return G;
}

template <typename T>
__device__ __forceinline__ void owner_group_update(T* __restrict__ ssum, const T* __restrict__ xt,
                                                   const T* __restrict__ wt,
                                                   const uint32_t* __restrict__ lab_s,
                                                   const unsigned char* __restrict__ rows, int cnt,
                                                   int d, int k, int G, int gl) {
  for (int i = 0; i < cnt; i += 2) {
    const bool two = i + 1 < cnt;
    const int r0 = rows[i], r1 = two ? rows[i + 1] : r0;
    const uint32_t l0 = lab_s[r0], l1 = lab_s[r1];
    const T w0 = wt ? wt[r0] : T(1), w1 = wt ? wt[r1] : T(1);
    for (int f = gl * 4; f < d; f += G * 4) {
      T x0[4], x1[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        x0[e] = (f + e < d) ? xt[(int64_t)r0 * d + f + e] : T(0);
        x1[e] = (two && f + e < d) ? xt[(int64_t)r1 * d + f + e] : T(0);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (f + e < d) ssum[l0 * d + f + e] += x0[e] * w0;
      if (two) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (f + e < d) ssum[l1 * d + f + e] += x1[e] * w1;
      }
    }
    if (gl == 0) {
      ssum[k * d + l0] += w0;
      if (two) ssum[k * d + l1] += w1;
    }
  }
}

}  // namespace kmb
