// Single-pass row kernels, all bound by HBM bandwidth: inertia, euclidean distances,
// column sums / sums of squares, row-vector add (centring), relocation, label utilities.
//
// Row kernels give each sample row to a group of G lanes (G = smallest power of two >= d,
// at most 32): lane l of the group reads features l, l+G, ... so a warp reads whole rows
// back to back, and the group folds its partial sums with shuffles in a fixed order.
#include "kmb_common.cuh"

namespace kmb {

constexpr int RS_THREADS = 256;
constexpr int RS_MAX_BLOCKS = 2048;  // fixed-order partial sums: one float64 per block

__device__ __forceinline__ double group_sum(double v, int G) {
  for (int o = G >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// per_sample[i] = w_i * sum_f (x - c[label])^2 ; partial[b] = float64 block sum.
// Rows stream through shared memory in tiles (two in flight, 16-byte asynchronous copies);
// one row belongs to G adjacent threads, each walking its 16-byte chunks in ascending feature
// order (the tile's odd row pitch keeps the reads conflict-free); the row's centroid is
// gathered from L2.
constexpr int IN_THREADS = 128;
constexpr int IN_STAGES = 2;

inline int inertia_threads_per_row(int d, size_t esize) {
  const size_t row_bytes = (size_t)d * esize;
  return row_bytes <= 256 ? 1 : (row_bytes <= 512 ? 2 : 4);
}

// FAST = rows of X and of C are whole, aligned 16-byte chunks: no bounds tests in the loop.
template <typename T, bool FAST>
__global__ void __launch_bounds__(IN_THREADS)
inertia_kernel(const T* __restrict__ X, const T* __restrict__ w, const T* __restrict__ C,
               const uint32_t* __restrict__ labels, T* __restrict__ per_sample,
               double* __restrict__ partial, int64_t n, int d, int k, int G, int aligned,
               int64_t n_tiles_total) {
  constexpr int VEC = RowVec<T>::VEC;
  __shared__ double red[32];
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  T* tiles = reinterpret_cast<T*>(dyn_smem);          // IN_STAGES x (R x d)
  const int R = IN_THREADS / G;
  const bool vec_ok = aligned != 0;                   // 16-byte chunks usable for X rows
  const int ld = tile_row_pitch<T>(d, vec_ok);
  const size_t tile_elems = (size_t)R * ld;
  const int r = threadIdx.x / G, li = threadIdx.x % G;
  const int nq = (d + VEC - 1) / VEC;
  double block_acc = 0.0;

  // this CTA's tiles: blockIdx, blockIdx + gridDim, ...
  auto tile_rows = [&](int64_t tile) -> int {
    const int64_t r0 = tile * R;
    return (tile < n_tiles_total && r0 < n) ? (int)((n - r0 < R) ? (n - r0) : R) : 0;
  };
#pragma unroll
  for (int sidx = 0; sidx < IN_STAGES; ++sidx) {
    const int64_t tile = (int64_t)blockIdx.x + (int64_t)sidx * gridDim.x;
    issue_row_tile<T, IN_THREADS>(tiles + sidx * tile_elems, X, tile * R, tile_rows(tile), d, ld,
                                  vec_ok);
  }
  int slot = 0;
  for (int64_t tile = blockIdx.x; tile < n_tiles_total; tile += gridDim.x) {
    __pipeline_wait_prior(IN_STAGES - 1);
    __syncthreads();
    const T* row = tiles + slot * tile_elems + (size_t)r * ld;
    const int64_t i = tile * R + r;
    const bool valid = i < n;
    const uint32_t lab = valid ? labels[i] : 0u;
    const T wi = (valid && w) ? w[i] : T(1);
    const T* crow = C + (int64_t)(lab < (uint32_t)k ? lab : 0u) * d;
    const bool c_vec = ((d % VEC) == 0) && ((((uintptr_t)C) & 15) == 0);
    T s = T(0);
    if constexpr (FAST) {
#pragma unroll 4
      for (int q = li; q < nq; q += G) {
        T xv[VEC], cv[VEC];
        load_row_vec<T>(row, q * VEC, q * VEC + VEC, true, xv);
        load_row_vec<T>(crow, q * VEC, q * VEC + VEC, true, cv);
#pragma unroll
        for (int jj = 0; jj < VEC; ++jj) {
          const T diff = xv[jj] - cv[jj];
          s = fma(diff, diff, s);
        }
      }
    } else {
      for (int q = li; q < nq; q += G) {
        const int f0 = q * VEC;
        T xv[VEC], cv[VEC];
        load_row_vec<T>(row, f0, d, vec_ok, xv);
        load_row_vec<T>(crow, f0, d, c_vec, cv);
#pragma unroll
        for (int jj = 0; jj < VEC; ++jj) {
          const T diff = xv[jj] - cv[jj];
          s = fma(diff, diff, s);
        }
      }
    }
    if (G > 1) {
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      if (G > 2) s += __shfl_xor_sync(0xffffffffu, s, 2);
    }
    if (valid && li == 0) {
      const T v = s * wi;
      if (per_sample) per_sample[i] = v;
      block_acc += (double)v;
    }
    __syncthreads();
    const int64_t nxt = tile + (int64_t)IN_STAGES * gridDim.x;
    issue_row_tile<T, IN_THREADS>(tiles + slot * tile_elems, X, nxt * R, tile_rows(nxt), d, ld,
                                  vec_ok);
    slot = (slot + 1) % IN_STAGES;
  }
  __pipeline_wait_prior(0);
  const double tot = block_sum(block_acc, red);
  if (threadIdx.x == 0 && partial) partial[blockIdx.x] = tot;
}

// out[q] = sum_b partial[q * stride + b] in ascending b, one block per q; written as T
// when out_t is given, as float64 when out_d is given.
template <typename T>
__global__ void sum_partials_kernel(const double* __restrict__ partial, int count, int stride,
                                    T* __restrict__ out_t, double* __restrict__ out_d) {
  __shared__ double red[32];
  const double* p = partial + (int64_t)blockIdx.x * stride;
  double s = 0.0;
  for (int b = threadIdx.x; b < count; b += blockDim.x) s += p[b];
  const double tot = block_sum(s, red);
  if (threadIdx.x == 0) {
    if (out_t) out_t[blockIdx.x] = (T)tot;
    if (out_d) out_d[blockIdx.x] = tot;
  }
}

// partial[b*d + f] = float64 sum over the block's rows of X[i, f].
template <typename T>
__global__ void __launch_bounds__(RS_THREADS)
col_sums_kernel(const T* __restrict__ X, double* __restrict__ partial, int64_t n, int d,
                int64_t rows_per_block) {
  // thread t owns features t, t+blockDim, ...; consecutive threads read consecutive floats.
  const int64_t r0 = (int64_t)blockIdx.x * rows_per_block;
  const int64_t r1 = (r0 + rows_per_block < n) ? (r0 + rows_per_block) : n;
  for (int f = threadIdx.x; f < d; f += RS_THREADS) {
    double s = 0.0;
    for (int64_t i = r0; i < r1; ++i) s += (double)X[i * (int64_t)d + f];
    partial[(int64_t)f * gridDim.x + blockIdx.x] = s;
  }
}

// Narrow rows (d < 32): flat sweep, each thread strides by a multiple of d so that it
// always meets the same feature.
template <typename T>
__global__ void __launch_bounds__(RS_THREADS)
col_sums_flat_kernel(const T* __restrict__ X, double* __restrict__ partial, int64_t n, int d,
                     int slots) {
  // slots = largest multiple of d that is <= RS_THREADS; threads >= slots idle.
  __shared__ double sh[RS_THREADS];
  const int t = threadIdx.x;
  double s = 0.0;
  const int64_t total = n * (int64_t)d;
  if (t < slots) {
    for (int64_t e = (int64_t)blockIdx.x * slots + t; e < total; e += (int64_t)gridDim.x * slots)
      s += (double)X[e];
  }
  sh[t] = s;
  __syncthreads();
  if (t < d) {
    double acc = 0.0;
    for (int u = t; u < slots; u += d) acc += sh[u];
    partial[(int64_t)t * gridDim.x + blockIdx.x] = acc;
  }
}

// One aligned 16-byte read-only load: four floats or two doubles.
__device__ __forceinline__ void load_vec16(float (&dst)[4], const float* src) {
  const float4 v = __ldg(reinterpret_cast<const float4*>(src));
  dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
}
__device__ __forceinline__ void load_vec16(double (&dst)[2], const double* src) {
  const double2 v = __ldg(reinterpret_cast<const double2*>(src));
  dst[0] = v.x; dst[1] = v.y;
}

// Inertia for rows that are whole aligned 16-byte chunks, at most 32 of them: G lanes (the
// power of two >= chunks per row) share a row, each with one chunk of the row and the same chunk
// of the row's centroid, so both reads are coalesced, nothing is staged, and a warp has
// 4 x 32 / G rows in flight.  The squared differences are summed over the lane's chunk in
// ascending feature order and then over the lanes by a shuffle tree.
constexpr int INL_THREADS = 256;
constexpr int INL_UNROLL = 4;
template <typename T>
__global__ void __launch_bounds__(INL_THREADS)
inertia_lanes_kernel(const T* __restrict__ X, const T* __restrict__ w, const T* __restrict__ C,
                     const uint32_t* __restrict__ labels, T* __restrict__ per_sample,
                     double* __restrict__ partial, int64_t n, int d, int k, int G) {
  constexpr int VEC = 16 / (int)sizeof(T);
  __shared__ double red[32];
  const int cpr = d / VEC;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int li = lane & (G - 1), sub = lane / G, rpw = 32 / G;
  const int64_t n_warps = (int64_t)gridDim.x * (INL_THREADS / 32);
  const int64_t rows_per_step = (int64_t)rpw * INL_UNROLL;
  double acc = 0.0;
  for (int64_t r0 = ((int64_t)blockIdx.x * (INL_THREADS / 32) + warp) * rows_per_step; r0 < n;
       r0 += n_warps * rows_per_step) {
    T xv[INL_UNROLL][VEC], cv[INL_UNROLL][VEC];
    bool valid[INL_UNROLL];
    uint32_t lab[INL_UNROLL];
#pragma unroll
    for (int u = 0; u < INL_UNROLL; ++u) {
      const int64_t i = r0 + (int64_t)u * rpw + sub;
      valid[u] = i < n;
      lab[u] = valid[u] ? __ldg(labels + i) : 0u;
      if (lab[u] >= (uint32_t)k) lab[u] = 0u;
    }
#pragma unroll
    for (int u = 0; u < INL_UNROLL; ++u) {
      const int64_t i = r0 + (int64_t)u * rpw + sub;
      if (valid[u] && li < cpr) {
        load_vec16(xv[u], X + i * (int64_t)d + li * VEC);
        load_vec16(cv[u], C + (int64_t)lab[u] * d + li * VEC);
      } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j) xv[u][j] = cv[u][j] = T(0);
      }
    }
#pragma unroll
    for (int u = 0; u < INL_UNROLL; ++u) {
      T sq = T(0);
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const T diff = xv[u][j] - cv[u][j];
        sq = fma(diff, diff, sq);
      }
      for (int o = G >> 1; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
      const int64_t i = r0 + (int64_t)u * rpw + sub;
      if (valid[u] && li == 0) {
        const T v = sq * (w ? w[i] : T(1));
        if (per_sample) per_sample[i] = v;
        acc += (double)v;
      }
    }
  }
  const double tot = block_sum(acc, red);
  if (threadIdx.x == 0 && partial) partial[blockIdx.x] = tot;
}

// The same loads from memory that the kernel also writes (no read-only path).
__device__ __forceinline__ void load_vec16_rw(float (&dst)[4], const float* src) {
  const float4 v = *reinterpret_cast<const float4*>(src);
  dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
}
__device__ __forceinline__ void load_vec16_rw(double (&dst)[2], const double* src) {
  const double2 v = *reinterpret_cast<const double2*>(src);
  dst[0] = v.x; dst[1] = v.y;
}

// Rows that are whole 16-byte chunks (d a multiple of VEC = 16 / sizeof(T), at most RS_THREADS
// chunks per row, aligned base): the same flat sweep with 16-byte loads.  A thread strides by a
// multiple of the row length in chunks, so it always meets the same VEC features, and keeps one
// float64 sum for each of them; two loads are in flight per thread.
template <typename T>
__global__ void __launch_bounds__(RS_THREADS)
col_sums_vec_kernel(const T* __restrict__ X, double* __restrict__ partial, int64_t n, int d, int slots) {
  constexpr int VEC = 16 / (int)sizeof(T);
  __shared__ double sh[VEC][RS_THREADS];
  const int t = threadIdx.x;
  const int cpr = d / VEC;                         // chunks per row
  double s[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) s[v] = 0.0;
  const int64_t total = n * (int64_t)cpr;
  if (t < slots) {
    const int64_t step = (int64_t)gridDim.x * slots;
    int64_t e = (int64_t)blockIdx.x * slots + t;
    for (; e + step < total; e += 2 * step) {
      T a[VEC], b[VEC];
      load_vec16(a, X + e * VEC);
      load_vec16(b, X + (e + step) * VEC);
#pragma unroll
      for (int v = 0; v < VEC; ++v) s[v] += (double)a[v];
#pragma unroll
      for (int v = 0; v < VEC; ++v) s[v] += (double)b[v];
    }
    if (e < total) {
      T a[VEC];
      load_vec16(a, X + e * VEC);
#pragma unroll
      for (int v = 0; v < VEC; ++v) s[v] += (double)a[v];
    }
  }
#pragma unroll
  for (int v = 0; v < VEC; ++v) sh[v][t] = s[v];
  __syncthreads();
  if (t < d) {
    const int c = t / VEC, v = t % VEC;            // feature t = chunk c of a row, component v
    double acc = 0.0;
    for (int u = c; u < slots; u += cpr) acc += sh[v][u];
    partial[(int64_t)t * gridDim.x + blockIdx.x] = acc;
  }
}

template <typename T>
__global__ void __launch_bounds__(RS_THREADS)
sum_kernel(const T* __restrict__ v, int64_t len, int square, double* __restrict__ partial) {
  __shared__ double red[32];
  double s = 0.0;
  for (int64_t e = (int64_t)blockIdx.x * RS_THREADS + threadIdx.x; e < len;
       e += (int64_t)gridDim.x * RS_THREADS) {
    const double x = (double)v[e];
    s += square == 1 ? x * x : (square == 2 ? x - x : x);   // x - x: 0 when finite, else NaN
  }
  const double tot = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = tot;
}

template <typename T>
__global__ void __launch_bounds__(RS_THREADS)
add_row_vector_kernel(T* __restrict__ X, int64_t total, int d, const T* __restrict__ vec, T sign) {
  for (int64_t e = (int64_t)blockIdx.x * RS_THREADS + threadIdx.x; e < total;
       e += (int64_t)gridDim.x * RS_THREADS)
    X[e] = X[e] + sign * vec[e % d];
}

__device__ __forceinline__ void store_vec16(float* dst, const float (&v)[4]) {
  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store_vec16(double* dst, const double (&v)[2]) {
  *reinterpret_cast<double2*>(dst) = make_double2(v[0], v[1]);
}

// The same update for rows that are whole 16-byte chunks: a thread strides by a multiple of the
// row length in chunks, so it always meets the same features, whose part of the vector it keeps
// in registers; 16-byte loads and stores, two chunks in flight, no division in the loop.
template <typename T>
__global__ void __launch_bounds__(RS_THREADS)
add_row_vector_vec_kernel(T* __restrict__ X, int64_t n, int d, const T* __restrict__ vec, T sign, int slots) {
  constexpr int VEC = 16 / (int)sizeof(T);
  const int t = threadIdx.x;
  if (t >= slots) return;
  const int cpr = d / VEC;
  const int64_t total = n * (int64_t)cpr;
  T add[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) add[v] = sign * vec[(t % cpr) * VEC + v];
  const int64_t step = (int64_t)gridDim.x * slots;
  int64_t e = (int64_t)blockIdx.x * slots + t;
  for (; e + step < total; e += 2 * step) {
    T a[VEC], b[VEC];
    load_vec16_rw(a, X + e * VEC);
    load_vec16_rw(b, X + (e + step) * VEC);
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      a[v] = a[v] + add[v];
      b[v] = b[v] + add[v];
    }
    store_vec16(X + e * VEC, a);
    store_vec16(X + (e + step) * VEC, b);
  }
  if (e < total) {
    T a[VEC];
    load_vec16_rw(a, X + e * VEC);
#pragma unroll
    for (int v = 0; v < VEC; ++v) a[v] = a[v] + add[v];
    store_vec16(X + e * VEC, a);
  }
}

// One block per relocated cluster (kmeans/kernels/utils.py:21-76 of the reference).
template <typename T>
__global__ void relocate_kernel(const T* __restrict__ X, const T* __restrict__ w,
                                const uint32_t* __restrict__ labels,
                                const int64_t* __restrict__ far_idx,
                                const uint32_t* __restrict__ empty_list, T* __restrict__ per_sample,
                                T* __restrict__ acc, int d, int k, int64_t n_rows) {
  const int r = blockIdx.x;
  const uint32_t j = empty_list[r];
  const int64_t q = far_idx[r];
  if (q < 0 || q >= n_rows || j >= (uint32_t)k) return;
  const uint32_t donor = labels[q];
  if (donor >= (uint32_t)k) return;
  const T wq = w ? w[q] : T(1);
  for (int f = threadIdx.x; f < d; f += blockDim.x) {
    const T addend = X[q * (int64_t)d + f] * wq;
    atomicAdd(&acc[(int64_t)donor * d + f], -addend);
    acc[(int64_t)j * d + f] = addend;
  }
  if (threadIdx.x == 0) {
    if (per_sample) per_sample[q] = T(0);
    atomicAdd(&acc[(int64_t)k * d + donor], -wq);
    acc[(int64_t)k * d + j] = wq;
  }
}

__global__ void fill_i32_kernel(int32_t* p, int len, int32_t v) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e < len) p[e] = v;
}

__global__ void build_mapping_kernel(const uint32_t* __restrict__ l1,
                                     const uint32_t* __restrict__ l2, int64_t n, int k,
                                     int32_t* __restrict__ mapping) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t a = l1[i];
    if (a < (uint32_t)k) mapping[a] = (int32_t)l2[i];
  }
}

__global__ void check_mapping_kernel(const uint32_t* __restrict__ l1,
                                     const uint32_t* __restrict__ l2, int64_t n, int k,
                                     const int32_t* __restrict__ mapping,
                                     int32_t* __restrict__ result) {
  bool bad = false;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t a = l1[i];
    if (a >= (uint32_t)k || mapping[a] != (int32_t)l2[i]) bad = true;
  }
  if (bad) *result = 0;
}

__global__ void mark_seen_kernel(const uint32_t* __restrict__ labels, int64_t n, int k,
                                 int32_t* __restrict__ seen) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t a = labels[i];
    if (a < (uint32_t)k && seen[a] == 0) seen[a] = 1;
  }
}

__global__ void count_seen_kernel(const int32_t* __restrict__ seen, int k, int32_t* out) {
  __shared__ double red[32];
  double s = 0.0;
  for (int j = threadIdx.x; j < k; j += blockDim.x) s += seen[j] ? 1.0 : 0.0;
  const double tot = block_sum(s, red);
  if (threadIdx.x == 0) *out = (int32_t)tot;
}

static inline int scan_grid(int64_t items_per_block_unit, int64_t n_units) {
  int64_t g = ceil_div(n_units, items_per_block_unit);
  const int64_t cap = (int64_t)sm_count() * 8;
  if (g > cap) g = cap;
  if (g > RS_MAX_BLOCKS) g = RS_MAX_BLOCKS;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace kmb

using namespace kmb;

extern "C" {

int kmb_inertia(int dtype, const void* X, const void* w, const void* C, const uint32_t* labels,
                void* per_sample, void* total, int64_t n, int d, int k, void* workspace,
                size_t workspace_bytes, void* stream) {
  KMB_REQUIRE(X && C && labels, "kmb_inertia: NULL argument");
  KMB_REQUIRE(n >= 0 && d > 0 && k > 0, "kmb_inertia: bad sizes");
  cudaStream_t s = (cudaStream_t)stream;
  const size_t esize = dtype == KMB_F32 ? 4 : 8;
  const int G = inertia_threads_per_row(d, esize);
  const int R = IN_THREADS / G;
  const int64_t n_tiles = ceil_div(n > 0 ? n : 1, R);
  const bool vec = (d % (int)(16 / esize) == 0) && (((uintptr_t)X & 15) == 0);
  const int vecn = (int)(16 / esize);
  const int ld = vec ? ((((d + vecn - 1) / vecn) | 1) * vecn) : (d | 1);
  const size_t dyn = (size_t)IN_STAGES * R * ld * esize;
  KMB_REQUIRE(dyn <= 200 * 1024, "kmb_inertia: rows too long for the staged tiles (d=%d)", d);
  int per_sm = (int)((220 * 1024) / (dyn + 1024));   // CTAs that fit one SM's shared memory
  if (per_sm > 8) per_sm = 8;
  if (per_sm < 1) per_sm = 1;
  int64_t grid = (int64_t)sm_count() * per_sm;
  if (grid > n_tiles) grid = n_tiles;
  if (grid > RS_MAX_BLOCKS) grid = RS_MAX_BLOCKS;
  if (total) {
    if (workspace == nullptr || workspace_bytes < (size_t)grid * sizeof(double)) {
      set_error("kmb_inertia: workspace of %zu bytes needed, %zu given",
                (size_t)grid * sizeof(double), workspace_bytes);
      return KMB_ERR_WORKSPACE;
    }
  }
  // rows of whole aligned chunks, at most 32 of them: the lanes-per-row kernel, nothing staged
  if (vec && (((uintptr_t)C & 15) == 0) && d / vecn <= 32 && n > 0) {
    int GL = 1;
    while (GL < d / vecn) GL <<= 1;
    const int64_t rows_per_cta = (int64_t)(INL_THREADS / 32) * (32 / GL) * INL_UNROLL;
    int64_t g2 = ceil_div(n, rows_per_cta);
    const int64_t cap = (int64_t)sm_count() * 8;
    if (g2 > cap) g2 = cap;
    if (g2 > RS_MAX_BLOCKS) g2 = RS_MAX_BLOCKS;
    if (total && (workspace == nullptr || workspace_bytes < (size_t)g2 * sizeof(double))) {
      set_error("kmb_inertia: workspace of %zu bytes needed, %zu given", (size_t)g2 * sizeof(double),
                workspace_bytes);
      return KMB_ERR_WORKSPACE;
    }
    KMB_DISPATCH_DTYPE(dtype, {
      inertia_lanes_kernel<T><<<(unsigned)g2, INL_THREADS, 0, s>>>(
          (const T*)X, (const T*)w, (const T*)C, labels, (T*)per_sample,
          total ? (double*)workspace : nullptr, n, d, k, GL);
      KMB_CHECK_LAUNCH();
      if (total) {
        sum_partials_kernel<T><<<1, 256, 0, s>>>((const double*)workspace, (int)g2, (int)g2, (T*)total,
                                                 nullptr);
        KMB_CHECK_LAUNCH();
      }
    });
    return KMB_OK;
  }
  KMB_DISPATCH_DTYPE(dtype, {
    const int aligned = vec ? 1 : 0;
    const bool fast = vec && (((uintptr_t)C & 15) == 0);
    auto kern = fast ? inertia_kernel<T, true> : inertia_kernel<T, false>;
    if (dyn > 48 * 1024)
      KMB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    kern<<<(unsigned)grid, IN_THREADS, dyn, s>>>((const T*)X, (const T*)w, (const T*)C, labels,
                                                 (T*)per_sample, total ? (double*)workspace : nullptr,
                                                 n, d, k, G, aligned, n_tiles);
    KMB_CHECK_LAUNCH();
    if (total) {
      sum_partials_kernel<T><<<1, 256, 0, s>>>((const double*)workspace, (int)grid, (int)grid,
                                               (T*)total, nullptr);
      KMB_CHECK_LAUNCH();
    }
  });
  return KMB_OK;
}

int kmb_col_sums(int dtype, const void* X, int64_t n, int d, double* out, void* workspace,
                 size_t workspace_bytes, void* stream) {
  KMB_REQUIRE(X && out && n >= 0 && d > 0, "kmb_col_sums: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  int grid;
  const int vec = dtype == KMB_F32 ? 4 : 2;
  const bool vec_ok = d % vec == 0 && d / vec <= RS_THREADS && d <= RS_THREADS && ((uintptr_t)X & 15) == 0;
  const int vslots = vec_ok ? (RS_THREADS / (d / vec)) * (d / vec) : 0;
  const bool flat = !vec_ok && d <= 32;
  const int slots = flat ? (RS_THREADS / d) * d : 0;
  if (vec_ok) {
    grid = scan_grid((int64_t)vslots * 8, n * (int64_t)(d / vec) > 0 ? n * (int64_t)(d / vec) : 1);
  } else if (flat) {
    grid = scan_grid(slots, n * (int64_t)d > 0 ? n * (int64_t)d : 1);
  } else {
    grid = scan_grid(64, n > 0 ? n : 1);
  }
  const size_t need = (size_t)grid * d * sizeof(double);
  if (workspace == nullptr || workspace_bytes < need) {
    set_error("kmb_col_sums: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    return KMB_ERR_WORKSPACE;
  }
  KMB_DISPATCH_DTYPE(dtype, {
    if (vec_ok) {
      col_sums_vec_kernel<T><<<grid, RS_THREADS, 0, s>>>((const T*)X, (double*)workspace, n, d, vslots);
    } else if (flat) {
      col_sums_flat_kernel<T><<<grid, RS_THREADS, 0, s>>>((const T*)X, (double*)workspace, n, d, slots);
    } else {
      const int64_t rpb = ceil_div(n > 0 ? n : 1, grid);
      col_sums_kernel<T><<<grid, RS_THREADS, 0, s>>>((const T*)X, (double*)workspace, n, d, rpb);
    }
    KMB_CHECK_LAUNCH();
    sum_partials_kernel<T><<<d, 256, 0, s>>>((const double*)workspace, grid, grid, nullptr, out);
    KMB_CHECK_LAUNCH();
  });
  return KMB_OK;
}

int kmb_sum(int dtype, const void* v, int64_t len, int square, double* out, void* workspace,
            size_t workspace_bytes, void* stream) {
  KMB_REQUIRE(out && len >= 0 && (v || len == 0) && square >= 0 && square <= 2, "kmb_sum: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = scan_grid(RS_THREADS * 8, len > 0 ? len : 1);
  const size_t need = (size_t)grid * sizeof(double);
  if (workspace == nullptr || workspace_bytes < need) {
    set_error("kmb_sum: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    return KMB_ERR_WORKSPACE;
  }
  KMB_DISPATCH_DTYPE(dtype, {
    sum_kernel<T><<<grid, RS_THREADS, 0, s>>>((const T*)v, len, square, (double*)workspace);
    KMB_CHECK_LAUNCH();
    sum_partials_kernel<T><<<1, 256, 0, s>>>((const double*)workspace, grid, grid, nullptr, out);
    KMB_CHECK_LAUNCH();
  });
  return KMB_OK;
}

int kmb_add_row_vector(int dtype, void* X, int64_t n, int d, const void* vec, double sign,
                       void* stream) {
  KMB_REQUIRE(X && vec && n >= 0 && d > 0, "kmb_add_row_vector: bad arguments");
  if (n == 0) return KMB_OK;
  const int64_t total = n * (int64_t)d;
  const int vw = dtype == KMB_F32 ? 4 : 2;
  const bool vec_ok = d % vw == 0 && d / vw <= RS_THREADS && ((uintptr_t)X & 15) == 0;
  KMB_DISPATCH_DTYPE(dtype, {
    if (vec_ok) {
      const int cpr = d / vw, slots = (RS_THREADS / cpr) * cpr;
      const int grid = scan_grid((int64_t)slots * 8, n * (int64_t)cpr);
      add_row_vector_vec_kernel<T><<<grid, RS_THREADS, 0, (cudaStream_t)stream>>>((T*)X, n, d, (const T*)vec,
                                                                                  (T)sign, slots);
    } else {
      const int grid = scan_grid(RS_THREADS * 4, total);
      add_row_vector_kernel<T><<<grid, RS_THREADS, 0, (cudaStream_t)stream>>>((T*)X, total, d,
                                                                              (const T*)vec, (T)sign);
    }
    KMB_CHECK_LAUNCH();
  });
  return KMB_OK;
}

int kmb_relocate_empty_clusters(int dtype, const void* X, const void* w, const uint32_t* labels,
                                int64_t n_rows, const int64_t* far_idx, const uint32_t* empty_list, int n_reloc,
                                void* per_sample, void* acc, int d, int k, void* stream) {
  KMB_REQUIRE(X && labels && far_idx && empty_list && acc, "kmb_relocate_empty_clusters: NULL argument");
  KMB_REQUIRE(n_reloc >= 0 && n_reloc <= k && d > 0 && n_rows >= 0, "kmb_relocate_empty_clusters: bad sizes");
  if (n_reloc == 0) return KMB_OK;
  KMB_DISPATCH_DTYPE(dtype, {
    relocate_kernel<T><<<n_reloc, 128, 0, (cudaStream_t)stream>>>(
        (const T*)X, (const T*)w, labels, far_idx, empty_list, (T*)per_sample, (T*)acc, d, k, n_rows);
    KMB_CHECK_LAUNCH();
  });
  return KMB_OK;
}

int kmb_same_clustering(const uint32_t* labels1, const uint32_t* labels2, int64_t n, int k,
                        int32_t* map_scratch, int32_t* result, void* stream) {
  KMB_REQUIRE(labels1 && labels2 && map_scratch && result && k > 0 && n >= 0,
              "kmb_same_clustering: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  fill_i32_kernel<<<(unsigned)ceil_div(k, 256), 256, 0, s>>>(map_scratch, k, -1);
  fill_i32_kernel<<<1, 32, 0, s>>>(result, 1, 1);
  KMB_CHECK_LAUNCH();
  if (n == 0) return KMB_OK;
  const int grid = scan_grid(256 * 4, n);
  build_mapping_kernel<<<grid, 256, 0, s>>>(labels1, labels2, n, k, map_scratch);
  check_mapping_kernel<<<grid, 256, 0, s>>>(labels1, labels2, n, k, map_scratch, result);
  KMB_CHECK_LAUNCH();
  return KMB_OK;
}

int kmb_count_distinct(const uint32_t* labels, int64_t n, int k, int32_t* seen_scratch,
                       int32_t* out, void* stream) {
  KMB_REQUIRE(labels && seen_scratch && out && k > 0 && n >= 0, "kmb_count_distinct: bad arguments");
  cudaStream_t s = (cudaStream_t)stream;
  fill_i32_kernel<<<(unsigned)ceil_div(k, 256), 256, 0, s>>>(seen_scratch, k, 0);
  if (n > 0) {
    const int grid = scan_grid(256 * 4, n);
    mark_seen_kernel<<<grid, 256, 0, s>>>(labels, n, k, seen_scratch);
  }
  count_seen_kernel<<<1, 256, 0, s>>>(seen_scratch, k, out);
  KMB_CHECK_LAUNCH();
  return KMB_OK;
}

}  // extern "C"
