// Small per-iteration kernels around the fused step: half norms, merge of accumulator
// copies, and the finalize pair (division, shifts, next half norms, empty list, status).
#include "kmb_common.cuh"

namespace kmb {

// One warp per centroid.
template <typename T>
__global__ void half_norm_kernel(const T* __restrict__ C, T* __restrict__ h, int k, int d) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= k) return;
  double s = 0.0;
  for (int f = lane; f < d; f += 32) {
    const double v = (double)C[(int64_t)warp * d + f];
    s += v * v;
  }
  s = warp_sum(s);
  if (lane == 0) h[warp] = (T)(s * 0.5);
}

template <typename T>
__global__ void merge_copies_kernel(const T* __restrict__ acc, int n_copies, int64_t len,
                                    T* __restrict__ out) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= len) return;
  T s = acc[e];
  for (int c = 1; c < n_copies; ++c) s += acc[(int64_t)c * len + e];
  out[e] = s;
}

// One warp per cluster: C_new = sums / count, squared shift, half norm of C_new.
template <typename T>
__global__ void finalize_rows_kernel(const T* __restrict__ acc, const T* __restrict__ C_old,
                                     T* __restrict__ C_new, T* __restrict__ h_new,
                                     T* __restrict__ shifts, int k, int d) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= k) return;
  const T cnt = acc[(int64_t)k * d + warp];
  double shift = 0.0, norm = 0.0;
  for (int f = lane; f < d; f += 32) {
    const int64_t e = (int64_t)warp * d + f;
    const T cn = acc[e] / cnt;
    C_new[e] = cn;
    const T diff = C_old[e] - cn;
    shift += (double)diff * (double)diff;
    norm += (double)cn * (double)cn;
  }
  shift = warp_sum(shift);
  norm = warp_sum(norm);
  if (lane == 0) {
    shifts[warp] = (T)shift;
    h_new[warp] = (T)(norm * 0.5);
  }
}

// Single CTA: fixed-order total of the shifts, ascending empty-cluster list, status.
template <typename T>
__global__ void finalize_status_kernel(const T* __restrict__ acc, const T* __restrict__ shifts,
                                       uint32_t* __restrict__ empty_list,
                                       kmb_lloyd_status* __restrict__ st, int k, int d) {
  __shared__ double red[32];
  __shared__ int warp_counts[32];
  __shared__ int base_s;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  double s = 0.0;
  for (int j = tid; j < k; j += blockDim.x) s += (double)shifts[j];
  const double total = block_sum(s, red);

  if (tid == 0) base_s = 0;
  __syncthreads();
  const T* counts = acc + (int64_t)k * d;
  for (int j0 = 0; j0 < k; j0 += blockDim.x) {
    const int j = j0 + tid;
    const bool empty = (j < k) && (counts[j] == T(0));
    const unsigned ballot = __ballot_sync(0xffffffffu, empty);
    if (lane == 0) warp_counts[wid] = __popc(ballot);
    __syncthreads();
    int offset = base_s;
    for (int w = 0; w < wid; ++w) offset += warp_counts[w];
    if (empty) empty_list[offset + __popc(ballot & ((1u << lane) - 1u))] = (uint32_t)j;
    __syncthreads();
    if (tid == 0) {
      int add = 0;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) add += warp_counts[w];
      base_s += add;
    }
    __syncthreads();
  }
  if (tid == 0) {
    st->n_empty = base_s;
    st->changed = (acc[(int64_t)k * d + k] != T(0)) ? 1 : 0;
    st->shift_total = total;
    st->inertia = 0.0;
    st->reserved = 0.0;
  }
}

}  // namespace kmb

using namespace kmb;

extern "C" {

int64_t kmb_lloyd_acc_len(int d, int k) {
  int64_t len = (int64_t)k * d + k + 1;
  return (len + 63) / 64 * 64;
}

int kmb_half_l2_norm(int dtype, const void* C, void* half_norms, int k, int d, void* stream) {
  KMB_REQUIRE(C && half_norms && k > 0 && d > 0, "kmb_half_l2_norm: bad arguments");
  KMB_DISPATCH_DTYPE(dtype, {
    const int threads = 256, warps = threads / 32;
    half_norm_kernel<T><<<(unsigned)ceil_div(k, warps), threads, 0, (cudaStream_t)stream>>>(
        (const T*)C, (T*)half_norms, k, d);
    KMB_CHECK_LAUNCH();
  });
  return KMB_OK;
}

int kmb_lloyd_merge_copies(int dtype, const void* acc, int n_copies, int64_t acc_len, void* out,
                           void* stream) {
  KMB_REQUIRE(acc && out && n_copies >= 1 && acc_len > 0, "kmb_lloyd_merge_copies: bad arguments");
  KMB_DISPATCH_DTYPE(dtype, {
    merge_copies_kernel<T><<<(unsigned)ceil_div(acc_len, 256), 256, 0, (cudaStream_t)stream>>>(
        (const T*)acc, n_copies, acc_len, (T*)out);
    KMB_CHECK_LAUNCH();
  });
  return KMB_OK;
}

int kmb_lloyd_finalize(int dtype, const void* acc, const void* C_old, void* C_new,
                       void* half_norms_new, void* shifts, uint32_t* empty_list,
                       kmb_lloyd_status* status, int k, int d, void* stream) {
  KMB_REQUIRE(acc && C_old && C_new && half_norms_new && shifts && empty_list && status,
              "kmb_lloyd_finalize: NULL argument");
  KMB_REQUIRE(k > 0 && d > 0, "kmb_lloyd_finalize: k and d must be positive");
  KMB_DISPATCH_DTYPE(dtype, {
    const int threads = 256, warps = threads / 32;
    finalize_rows_kernel<T><<<(unsigned)ceil_div(k, warps), threads, 0, (cudaStream_t)stream>>>(
        (const T*)acc, (const T*)C_old, (T*)C_new, (T*)half_norms_new, (T*)shifts, k, d);
    KMB_CHECK_LAUNCH();
    finalize_status_kernel<T><<<1, 1024, 0, (cudaStream_t)stream>>>(
        (const T*)acc, (const T*)shifts, empty_list, status, k, d);
    KMB_CHECK_LAUNCH();
  });
  return KMB_OK;
}

}  // extern "C"
