// Row-wise top-k by MSB-first radix select (8-bit digits, shared-memory histograms).
//
// The key of element i is (order-preserving unsigned image of the value) followed by the
// 32-bit complement of i, so all keys of a row are distinct: the select needs no tie
// budget, and "largest value first, lowest index first among equals" falls out of the
// key order.  Stands for topk / topk_idx of sklearn_numba_dpex/common/topk.py:112-270
// (histogram kernel :621-771, threshold search :1003-1093, gather :1143-1365), which leave
// the order of the output and the choice among ties undefined.
#include <mutex>

#include "kmb_common.cuh"

namespace kmb {

typedef unsigned __int128 u128;

constexpr int TK_THREADS = 256;
constexpr int TK_RADIX_BITS = 8;
constexpr int TK_BINS = 1 << TK_RADIX_BITS;

struct TkState {          // per row
  unsigned long long prefix_hi, prefix_lo;  // digits decided so far (right-aligned)
  unsigned long long kth_hi, kth_lo;        // smallest key that is still among the k largest
  long long k_rem;                          // how many of the matching items are wanted
  unsigned long long cursor;                // gather cursor
  unsigned int ticket;                      // CTAs of the current histogram pass that are done
  int done;                                 // the threshold is final: later passes return at once
};

template <typename T>
struct TkKey;
template <>
struct TkKey<float> {
  static constexpr int BITS = 64;
  __device__ static __forceinline__ u128 make(float v, int64_t i) {
    uint32_t b = __float_as_uint(v);
    b ^= (b >> 31) ? 0xffffffffu : 0x80000000u;
    return ((u128)b << 32) | (u128)(0xffffffffu - (uint32_t)i);
  }
};
template <>
struct TkKey<double> {
  static constexpr int BITS = 96;
  __device__ static __forceinline__ u128 make(double v, int64_t i) {
    unsigned long long b = (unsigned long long)__double_as_longlong(v);
    b ^= (b >> 63) ? 0xffffffffffffffffull : 0x8000000000000000ull;
    return ((u128)b << 32) | (u128)(0xffffffffu - (uint32_t)i);
  }
};

__global__ void topk_init_kernel(TkState* st, unsigned int* hist, int n_rows, int k,
                                 size_t hist_len) {
  const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e < hist_len) hist[e] = 0u;
  if (e < (size_t)n_rows) {
    st[e].prefix_hi = 0ull;
    st[e].prefix_lo = 0ull;
    st[e].kth_hi = 0ull;
    st[e].kth_lo = 0ull;
    st[e].k_rem = k;
    st[e].cursor = 0ull;
    st[e].ticket = 0u;
    st[e].done = 0;
  }
}

// Histogram of the digit at `shift` over the items whose higher digits equal the prefix; the
// CTA of a row that finishes last then walks the bins from the top until k_rem items are
// covered and appends that digit to the prefix.  When the chosen bin holds exactly the number of
// items still wanted, everything at or above it is the answer: the row is marked done and the
// remaining passes return without reading it (the reference stops its passes the same way,
// common/topk.py:1059-1061).  With continuous data that happens after two or three of the
// eight (fp64: twelve) passes.
template <typename T>
__global__ void __launch_bounds__(TK_THREADS)
topk_hist_kernel(const T* __restrict__ values, int64_t n_cols, TkState* __restrict__ st,
                 unsigned int* __restrict__ hist, int shift, int first_pass) {
  __shared__ unsigned int sh[TK_BINS];
  __shared__ int last_s;
  const int row = blockIdx.y;
  if (*((volatile int*)&st[row].done)) return;
  const T* v = values + (int64_t)row * n_cols;
  sh[threadIdx.x] = 0u;
  __syncthreads();
  const u128 prefix = ((u128)st[row].prefix_hi << 64) | (u128)st[row].prefix_lo;
  for (int64_t i = (int64_t)blockIdx.x * TK_THREADS + threadIdx.x; i < n_cols;
       i += (int64_t)gridDim.x * TK_THREADS) {
    const u128 key = TkKey<T>::make(v[i], i);
    if (first_pass || (key >> (shift + TK_RADIX_BITS)) == prefix)
      atomicAdd(&sh[(unsigned)(key >> shift) & (TK_BINS - 1)], 1u);
  }
  __syncthreads();
  unsigned int* h = hist + (size_t)row * TK_BINS;
  const unsigned int c = sh[threadIdx.x];
  if (c) atomicAdd(&h[threadIdx.x], c);

  // ---- the last CTA of the row advances the prefix
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last_s = (atomicAdd(&st[row].ticket, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  sh[threadIdx.x] = __ldcg(&h[threadIdx.x]);
  __syncthreads();
  if (threadIdx.x == 0) {
    long long k_rem = st[row].k_rem;
    int digit = 0;
    for (int b = TK_BINS - 1; b >= 0; --b) {
      const long long cb = (long long)sh[b];
      if (cb >= k_rem) {
        digit = b;
        break;
      }
      k_rem -= cb;
    }
    const u128 np = (prefix << TK_RADIX_BITS) | (u128)digit;
    const u128 kth = np << shift;
    st[row].prefix_hi = (unsigned long long)(np >> 64);
    st[row].prefix_lo = (unsigned long long)np;
    st[row].kth_hi = (unsigned long long)(kth >> 64);
    st[row].kth_lo = (unsigned long long)kth;
    st[row].k_rem = k_rem;
    st[row].ticket = 0u;
    if ((long long)sh[digit] == k_rem || shift == 0) st[row].done = 1;
  }
}

// Emit the items whose key is >= the k-th largest key (exactly k per row), unordered.
template <typename T>
__global__ void __launch_bounds__(TK_THREADS)
topk_gather_kernel(const T* __restrict__ values, int64_t n_cols, TkState* __restrict__ st, int k,
                   int64_t* __restrict__ tmp_idx) {
  const int row = blockIdx.y;
  const T* v = values + (int64_t)row * n_cols;
  const u128 kth = ((u128)st[row].kth_hi << 64) | (u128)st[row].kth_lo;
  for (int64_t i = (int64_t)blockIdx.x * TK_THREADS + threadIdx.x; i < n_cols;
       i += (int64_t)gridDim.x * TK_THREADS) {
    const u128 key = TkKey<T>::make(v[i], i);
    if (key >= kth) {
      const unsigned long long pos = atomicAdd(&st[row].cursor, 1ull);
      if (pos < (unsigned long long)k) tmp_idx[(int64_t)row * k + pos] = i;
    }
  }
}

// Rank sort of the k winners of a row: position = number of winners with a larger key.  The
// keys are staged in shared memory when all k of them fit (`staged`), else read from global.
constexpr int TK_SORT_SMEM_MAX_K = 4096;

template <typename T>
__global__ void __launch_bounds__(TK_THREADS)
topk_sort_kernel(const T* __restrict__ values, int64_t n_cols, int k,
                 const int64_t* __restrict__ tmp_idx, T* __restrict__ out_values,
                 int64_t* __restrict__ out_idx, int staged) {
  extern __shared__ __align__(16) unsigned char tk_dyn[];
  u128* keys_s = reinterpret_cast<u128*>(tk_dyn);
  const int row = blockIdx.y;
  const int e = blockIdx.x * TK_THREADS + threadIdx.x;
  const T* v = values + (int64_t)row * n_cols;
  const int64_t* mine = tmp_idx + (int64_t)row * k;
  if (staged) {
    for (int o = threadIdx.x; o < k; o += TK_THREADS) {
      const int64_t j = mine[o];
      keys_s[o] = TkKey<T>::make(v[j], j);
    }
    __syncthreads();
  }
  if (e >= k) return;
  const int64_t i = mine[e];
  const T vi = v[i];
  const u128 key = TkKey<T>::make(vi, i);
  int rank = 0;
  if (staged) {
    for (int o = 0; o < k; ++o) rank += (keys_s[o] > key) ? 1 : 0;
  } else {
    for (int o = 0; o < k; ++o) {
      const int64_t j = mine[o];
      rank += (TkKey<T>::make(v[j], j) > key) ? 1 : 0;
    }
  }
  if (out_values) out_values[(int64_t)row * k + rank] = vi;
  if (out_idx) out_idx[(int64_t)row * k + rank] = i;
}

template <typename T>
int topk_run(const T* values, int n_rows, int64_t n_cols, int k, T* out_values, int64_t* out_idx,
             void* workspace, cudaStream_t s) {
  unsigned char* ws = (unsigned char*)workspace;
  constexpr int n_passes = TkKey<T>::BITS / TK_RADIX_BITS;
  TkState* st = (TkState*)ws;
  size_t off = ((size_t)n_rows * sizeof(TkState) + 255) / 256 * 256;
  unsigned int* hist = (unsigned int*)(ws + off);
  const size_t hist_len = (size_t)n_passes * n_rows * TK_BINS;
  off += (hist_len * sizeof(unsigned int) + 255) / 256 * 256;
  int64_t* tmp_idx = (int64_t*)(ws + off);

  const size_t init_items = hist_len > (size_t)n_rows ? hist_len : (size_t)n_rows;
  topk_init_kernel<<<(unsigned)ceil_div((int64_t)init_items, 256), 256, 0, s>>>(st, hist, n_rows, k,
                                                                               hist_len);
  KMB_CHECK_LAUNCH();
  int64_t gx = ceil_div(n_cols, (int64_t)TK_THREADS * 8);
  const int64_t cap = ceil_div((int64_t)sm_count() * 8, n_rows);
  if (gx > cap) gx = cap;
  if (gx < 1) gx = 1;
  dim3 grid((unsigned)gx, (unsigned)n_rows);
  for (int p = 0; p < n_passes; ++p) {
    const int shift = TkKey<T>::BITS - (p + 1) * TK_RADIX_BITS;
    unsigned int* h = hist + (size_t)p * n_rows * TK_BINS;
    topk_hist_kernel<T><<<grid, TK_THREADS, 0, s>>>(values, n_cols, st, h, shift, p == 0);
    KMB_CHECK_LAUNCH();
  }
  topk_gather_kernel<T><<<grid, TK_THREADS, 0, s>>>(values, n_cols, st, k, tmp_idx);
  KMB_CHECK_LAUNCH();
  dim3 sgrid((unsigned)ceil_div(k, TK_THREADS), (unsigned)n_rows);
  const int staged = k <= TK_SORT_SMEM_MAX_K ? 1 : 0;
  const size_t sort_smem = staged ? (size_t)k * sizeof(u128) : 0;
  if (sort_smem > 48 * 1024)
    KMB_CHECK_CUDA(cudaFuncSetAttribute(topk_sort_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)(TK_SORT_SMEM_MAX_K * sizeof(u128))));
  topk_sort_kernel<T><<<sgrid, TK_THREADS, sort_smem, s>>>(values, n_cols, k, tmp_idx, out_values,
                                                          out_idx, staged);
  KMB_CHECK_LAUNCH();
  return KMB_OK;
}

// ---- scratch for kmb_topk_idx_static: lives in the library image, one instance per GPU that
// loads the library, until the process exits.  48 KB covers one row and k <= 4096.
constexpr int TK_STATIC_MAX_K = 4096;
constexpr size_t TK_STATIC_BYTES = 48 * 1024;
static __device__ __align__(256) unsigned char g_topk_static_scratch[TK_STATIC_BYTES];

// In host code the symbol above is only a handle; the device address has to be asked for,
// once per device, with that device current.
static int topk_static_scratch_ptr(void** out) {
  static std::mutex mu;
  static void* cached[64] = {nullptr};
  int dev = 0;
  KMB_CHECK_CUDA(cudaGetDevice(&dev));
  KMB_REQUIRE(dev >= 0 && dev < 64, "kmb_topk_idx_static: device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    KMB_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_topk_static_scratch));
    KMB_REQUIRE(ptr != nullptr, "kmb_topk_idx_static: the scratch symbol has no device address");
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return KMB_OK;
}

}  // namespace kmb

using namespace kmb;

extern "C" {

size_t kmb_topk_workspace_bytes(int n_rows, int64_t n_cols, int k) {
  (void)n_cols;
  if (n_rows < 1) n_rows = 1;
  if (k < 1) k = 1;
  const size_t n_passes = 96 / TK_RADIX_BITS;
  size_t b = ((size_t)n_rows * sizeof(TkState) + 255) / 256 * 256;
  b += (n_passes * (size_t)n_rows * TK_BINS * sizeof(unsigned int) + 255) / 256 * 256;
  b += (size_t)n_rows * (size_t)k * sizeof(int64_t);
  return b + 256;
}

int kmb_topk(int dtype, const void* values, int n_rows, int64_t n_cols, int k, void* out_values,
             int64_t* out_idx, void* workspace, size_t workspace_bytes, void* stream) {
  KMB_REQUIRE(values && (out_values || out_idx), "kmb_topk: NULL argument");
  KMB_REQUIRE(n_rows >= 1 && n_rows <= 65535, "kmb_topk: n_rows must be in [1, 65535]");
  KMB_REQUIRE(k >= 1, "kmb_topk: k must be >= 1");
  if (n_cols < k) {
    set_error("Expected k to be greater than or equal to the number of items in the search space, "
              "but got k=%d and %lld items in the search space.", k, (long long)n_cols);
    return KMB_ERR_INVALID;
  }
  KMB_REQUIRE(n_cols < (1ll << 32), "kmb_topk: n_cols must be below 2^32");
  const size_t need = kmb_topk_workspace_bytes(n_rows, n_cols, k);
  if (workspace == nullptr || workspace_bytes < need) {
    set_error("kmb_topk: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    return KMB_ERR_WORKSPACE;
  }
  KMB_REQUIRE(((uintptr_t)workspace & 15) == 0, "kmb_topk: workspace must be 16-byte aligned");
  KMB_DISPATCH_DTYPE(dtype, {
    return topk_run<T>((const T*)values, n_rows, n_cols, k, (T*)out_values, out_idx, workspace,
                       (cudaStream_t)stream);
  });
}

int kmb_topk_idx_static(int dtype, const void* values, int64_t n_cols, int k, int64_t* out_idx,
                        void* stream) {
  KMB_REQUIRE(values && out_idx, "kmb_topk_idx_static: NULL argument");
  KMB_REQUIRE(k >= 1, "kmb_topk_idx_static: k must be >= 1");
  if (k > TK_STATIC_MAX_K) {
    set_error("kmb_topk_idx_static: k=%d is beyond the built-in scratch, which holds k <= %d; use "
              "kmb_topk with a workspace instead", k, TK_STATIC_MAX_K);
    return KMB_ERR_INVALID;
  }
  if (n_cols < k) {
    set_error("Expected k to be greater than or equal to the number of items in the search space, "
              "but got k=%d and %lld items in the search space.", k, (long long)n_cols);
    return KMB_ERR_INVALID;
  }
  KMB_REQUIRE(n_cols < (1ll << 32), "kmb_topk_idx_static: n_cols must be below 2^32");
  if (kmb_topk_workspace_bytes(1, n_cols, k) > TK_STATIC_BYTES) {
    set_error("kmb_topk_idx_static: built-in scratch of %zu bytes is too small for k=%d",
              TK_STATIC_BYTES, k);
    return KMB_ERR_INVALID;
  }
  void* scratch = nullptr;
  const int rc = topk_static_scratch_ptr(&scratch);
  if (rc != KMB_OK) return rc;
  // topk_run begins by clearing the histograms, the prefix state and the gather cursor, so
  // whatever the previous call left in the scratch does not matter.
  KMB_DISPATCH_DTYPE(dtype, {
    return topk_run<T>((const T*)values, 1, n_cols, k, (T*)nullptr, out_idx, scratch,
                       (cudaStream_t)stream);
  });
}

}  // extern "C"
