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
template <typename T, int ROWS, int BK>
struct ChunkRegs {
  static constexpr int QPR = BK / 4;
  static constexpr int RSTEP = CC_THREADS / QPR;
  static constexpr int N = (ROWS + RSTEP - 1) / RSTEP;
  T v[N][4];
};

// Fetches the chunk [row0, row0 + ROWS) x [k0, k0 + BK) of the row-major matrix M (n_rows x d)
// into registers, zero beyond the matrix.  `vec` is the widest aligned vector width.
template <typename T, int ROWS, int BK>
__device__ __forceinline__ void fetch_chunk(ChunkRegs<T, ROWS, BK>& r, const T* __restrict__ M,
                                            int64_t row0, int64_t n_rows, int d, int k0, int vec) {
  using R = ChunkRegs<T, ROWS, BK>;
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
template <typename T, int ROWS, int BK>
__device__ __forceinline__ void store_chunk(const ChunkRegs<T, ROWS, BK>& r, T* __restrict__ S, int ld) {
  using R = ChunkRegs<T, ROWS, BK>;
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
// loads and stores do.  A lane serves 4 features (strided by the group width); rows are taken
// four at a time so that their global loads are in flight together (the loads are the latency
// of the loop).
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
  // lane gl serves features gl, gl + G, gl + 2 G, gl + 3 G of a block of 4 G features:
  // consecutive lanes touch consecutive addresses (coalesced loads, conflict-free banks)
  for (int i = 0; i < cnt; i += 4) {
    int r[4];
    uint32_t l[4];
    T w[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      r[u] = rows[(i + u < cnt) ? i + u : i];
      l[u] = lab_s[r[u]];
      w[u] = wt ? wt[r[u]] : T(1);
    }
    for (int f0 = 0; f0 < d; f0 += G * 4) {
      T x[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int f = f0 + gl + e * G;
          x[u][e] = (i + u < cnt && f < d) ? xt[(int64_t)r[u] * d + f] : T(0);
        }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (i + u < cnt) {            // in list order: two rows of one cluster add one after the other
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int f = f0 + gl + e * G;
            if (f < d) ssum[l[u] * d + f] += x[u][e] * w[u];
          }
        }
      }
    }
    if (gl == 0) {
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i + u < cnt) ssum[k * d + l[u]] += w[u];
    }
  }
}

}  // namespace kmb
