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
__global__ void merge_copies_kernel(T* __restrict__ acc, int n_copies, int64_t len,
                                    T* __restrict__ out, int clear) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= len) return;
  T s = acc[e];
  for (int c = 1; c < n_copies; ++c) s += acc[(int64_t)c * len + e];
  out[e] = s;
  if (clear)
    for (int c = 0; c < n_copies; ++c) acc[(int64_t)c * len + e] = T(0);
}

template <typename T>
struct FinArgs {
  T* acc;                // n_copies x acc_len, or NULL
  T* merged;             // acc_len
  const T* C_old;
  T* C_new;
  T* h_new;
  T* shifts;
  uint32_t* empty_list;
  kmb_lloyd_status* st;
  LloydControl* ctl;
  float* chi;            // operands of the next tensor-core step (k_pad x d_pad each), or NULL
  float* clo;
  float* h_pad;
  int64_t acc_len;
  int n_copies;
  int merge;             // merged is computed from the copies (else it is the input)
  int clear;             // the copies are zeroed once read
  int k, d, k_pad, d_pad;
  int fold_at;           // first of the two fold features of the operands, or -1 (lloyd_tc_fold_at)
};

// One warp per cluster: (merge of the accumulator copies), C_new = sums / count, squared shift,
// half norm of C_new, and the hi / lo split of C_new for the next tensor-core step.  The CTA
// that finishes last then writes the status record: fixed-order total of the shifts and the
// ascending list of empty clusters.
template <typename T>
__global__ void __launch_bounds__(256) finalize_fused_kernel(FinArgs<T> a) {
  __shared__ double red[32];
  __shared__ int warp_counts[32];
  __shared__ int base_s;
  __shared__ int is_last_s;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int k = a.k, d = a.d;
  const int j = blockIdx.x * (blockDim.x >> 5) + wid;
  const int64_t kd = (int64_t)k * d;

  if (j < k) {
    T cnt;
    if (a.merge) {
      cnt = a.acc[kd + j];
      for (int c = 1; c < a.n_copies; ++c) cnt += a.acc[(int64_t)c * a.acc_len + kd + j];
    } else {
      cnt = a.merged[kd + j];
    }
    double shift = 0.0, norm = 0.0;
    for (int f = lane; f < d; f += 32) {
      const int64_t e = (int64_t)j * d + f;
      T s;
      if (a.merge) {
        s = a.acc[e];
        for (int c = 1; c < a.n_copies; ++c) s += a.acc[(int64_t)c * a.acc_len + e];
        a.merged[e] = s;
      } else {
        s = a.merged[e];
      }
      const T cn = s / cnt;
      a.C_new[e] = cn;
      const T diff = a.C_old[e] - cn;
      shift += (double)diff * (double)diff;
      norm += (double)cn * (double)cn;
      if (a.chi != nullptr) {
        const float hi = tf32_rna((float)cn);
        a.chi[(int64_t)j * a.d_pad + f] = hi;
        a.clo[(int64_t)j * a.d_pad + f] = tf32_rna((float)cn - hi);
      }
    }
    shift = warp_sum(shift);
    norm = warp_sum(norm);
    __syncwarp();
    if (a.clear && a.acc != nullptr) {
      for (int c = 0; c < a.n_copies; ++c) {
        T* copy = a.acc + (int64_t)c * a.acc_len;
        for (int f = lane; f < d; f += 32) copy[(int64_t)j * d + f] = T(0);
        if (lane == 0) copy[kd + j] = T(0);
      }
    }
    if (lane == 0) {
      if (a.merge) a.merged[kd + j] = cnt;
      a.shifts[j] = (T)shift;
      a.h_new[j] = (T)(norm * 0.5);
      if (a.h_pad != nullptr) a.h_pad[j] = (float)(norm * 0.5);
    }
    if (a.chi != nullptr) {
      for (int f = d + lane; f < a.d_pad; f += 32) {
        a.chi[(int64_t)j * a.d_pad + f] = 0.f;
        a.clo[(int64_t)j * a.d_pad + f] = 0.f;
      }
      __syncwarp();
      if (lane == 0 && a.fold_at >= 0) {
        // after the data features: the fold features may sit in zero padding INSIDE the rows
        float fhi[2], flo[2];
        lloyd_tc_fold_values((float)(norm * 0.5), fhi, flo);
        a.chi[(int64_t)j * a.d_pad + a.fold_at] = fhi[0];
        a.clo[(int64_t)j * a.d_pad + a.fold_at] = flo[0];
        a.chi[(int64_t)j * a.d_pad + a.fold_at + 1] = fhi[1];
        a.clo[(int64_t)j * a.d_pad + a.fold_at + 1] = flo[1];
      }
    }
  } else if (a.chi != nullptr && j < a.k_pad) {
    // padding centroids of the tensor-core operands: zero rows that can never win (half norm
    // +inf; with folded half norms a NaN in the fold feature, which makes their scores NaN)
    for (int f = lane; f < a.d_pad; f += 32) {
      a.chi[(int64_t)j * a.d_pad + f] = 0.f;
      a.clo[(int64_t)j * a.d_pad + f] = 0.f;
    }
    __syncwarp();
    if (lane == 0) {
      a.h_pad[j] = __int_as_float(0x7f800000);
      if (a.fold_at >= 0) a.chi[(int64_t)j * a.d_pad + a.fold_at] = __int_as_float(0x7fc00000);
    }
  }
  if (blockIdx.x == 0 && tid == 0) {
    // the "labels changed" counter follows the counts
    if (a.merge) {
      T ch = a.acc[kd + k];
      for (int c = 1; c < a.n_copies; ++c) ch += a.acc[(int64_t)c * a.acc_len + kd + k];
      a.merged[kd + k] = ch;
    }
    if (a.clear && a.acc != nullptr)
      for (int c = 0; c < a.n_copies; ++c) a.acc[(int64_t)c * a.acc_len + kd + k] = T(0);
  }

  // ---- the CTA that arrives last writes the status record
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int t = atomicAdd(&a.ctl->ticket, 1u);
    is_last_s = (t == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!is_last_s) return;
  __threadfence();

  double s = 0.0;
  for (int c = tid; c < k; c += blockDim.x) s += (double)__ldcg(&a.shifts[c]);
  const double total = block_sum(s, red);

  if (tid == 0) base_s = 0;
  __syncthreads();
  const T* counts = a.merged + kd;
  for (int j0 = 0; j0 < k; j0 += blockDim.x) {
    const int c = j0 + tid;
    const bool empty = (c < k) && (__ldcg(&counts[c]) == T(0));
    const unsigned ballot = __ballot_sync(0xffffffffu, empty);
    if (lane == 0) warp_counts[wid] = __popc(ballot);
    __syncthreads();
    int offset = base_s;
    for (int w = 0; w < wid; ++w) offset += warp_counts[w];
    if (empty) a.empty_list[offset + __popc(ballot & ((1u << lane) - 1u))] = (uint32_t)c;
    __syncthreads();
    if (tid == 0) {
      int add = 0;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) add += warp_counts[w];
      base_s += add;
    }
    __syncthreads();
  }
  if (tid == 0) {
    a.st->n_empty = base_s;
    a.st->changed = (__ldcg(&a.merged[kd + k]) != T(0)) ? 1 : 0;
    a.st->shift_total = total;
    a.st->inertia = 0.0;
    a.st->wait_error = *((volatile int*)&a.ctl->wait_error);
    a.st->reserved = 0;
    a.ctl->ticket = 0u;
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

int kmb_lloyd_merge_copies(int dtype, void* acc, int n_copies, int64_t acc_len, void* out,
                           int clear_acc, void* stream) {
  KMB_REQUIRE(acc && out && n_copies >= 1 && acc_len > 0, "kmb_lloyd_merge_copies: bad arguments");
  KMB_REQUIRE(acc != out || !clear_acc, "kmb_lloyd_merge_copies: cannot clear acc when out aliases it");
  KMB_DISPATCH_DTYPE(dtype, {
    merge_copies_kernel<T><<<(unsigned)ceil_div(acc_len, 256), 256, 0, (cudaStream_t)stream>>>(
        (T*)acc, n_copies, acc_len, (T*)out, clear_acc);
    KMB_CHECK_LAUNCH();
  });
  return KMB_OK;
}

int kmb_lloyd_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
  KMB_REQUIRE(workspace != nullptr, "kmb_lloyd_workspace_init: workspace is NULL");
  LloydWorkspace ws = lloyd_carve(workspace, 1, 1);
  if (ws.bytes > workspace_bytes) {
    set_error("kmb_lloyd_workspace_init: workspace of %zu bytes needed, %zu given", ws.bytes,
              workspace_bytes);
    return KMB_ERR_WORKSPACE;
  }
  KMB_CHECK_CUDA(cudaMemsetAsync(ws.ctl, 0, sizeof(LloydControl), (cudaStream_t)stream));
  return KMB_OK;
}

int kmb_lloyd_finalize(int dtype, void* acc, int n_copies, void* merged, int flags,
                       const void* C_old, void* C_new, void* half_norms_new, void* shifts,
                       uint32_t* empty_list, kmb_lloyd_status* status, int k, int d,
                       void* workspace, size_t workspace_bytes, void* stream) {
  KMB_REQUIRE(merged && C_old && C_new && half_norms_new && shifts && empty_list && status,
              "kmb_lloyd_finalize: NULL argument");
  KMB_REQUIRE(k > 0 && d > 0, "kmb_lloyd_finalize: k and d must be positive");
  KMB_REQUIRE((flags & ~(KMB_FIN_MERGE | KMB_FIN_CLEAR_ACC | KMB_FIN_PREPARE_TF32X3 | KMB_LLOYD_PAD_MASK)) == 0,
              "kmb_lloyd_finalize: unknown flag bits %d", flags);
  const int pad = (flags & KMB_LLOYD_PAD_MASK) >> 8;
  KMB_REQUIRE(pad < d, "kmb_lloyd_finalize: %d padding features in rows of %d", pad, d);
  const bool merge = flags & KMB_FIN_MERGE, clear = flags & KMB_FIN_CLEAR_ACC;
  const bool prepare = flags & KMB_FIN_PREPARE_TF32X3;
  KMB_REQUIRE(!(merge || clear) || (acc != nullptr && n_copies >= 1),
              "kmb_lloyd_finalize: KMB_FIN_MERGE / KMB_FIN_CLEAR_ACC need the accumulator copies");
  KMB_REQUIRE(!(clear && acc == merged), "kmb_lloyd_finalize: cannot clear acc when merged aliases it");
  KMB_REQUIRE(!prepare || dtype == KMB_F32, "kmb_lloyd_finalize: KMB_FIN_PREPARE_TF32X3 is fp32 only");
  KMB_REQUIRE(workspace != nullptr, "kmb_lloyd_finalize: workspace is NULL");
  LloydWorkspace ws = lloyd_carve(workspace, prepare ? d : 1, prepare ? k : 1);
  if (ws.bytes > workspace_bytes) {
    set_error("kmb_lloyd_finalize: workspace of %zu bytes needed, %zu given", ws.bytes,
              workspace_bytes);
    return KMB_ERR_WORKSPACE;
  }
  KMB_DISPATCH_DTYPE(dtype, {
    FinArgs<T> a;
    a.acc = (T*)acc; a.merged = (T*)merged; a.C_old = (const T*)C_old; a.C_new = (T*)C_new;
    a.h_new = (T*)half_norms_new; a.shifts = (T*)shifts; a.empty_list = empty_list;
    a.st = status; a.ctl = ws.ctl;
    a.chi = prepare ? ws.chi : nullptr; a.clo = prepare ? ws.clo : nullptr;
    a.h_pad = prepare ? ws.h_pad : nullptr;
    a.acc_len = kmb_lloyd_acc_len(d, k); a.n_copies = n_copies; a.merge = merge; a.clear = clear;
    a.k = k; a.d = d; a.k_pad = ws.k_pad; a.d_pad = ws.d_pad;
    a.fold_at = prepare ? lloyd_tc_fold_at(d, pad) : -1;
    const int threads = 256, warps = threads / 32;
    const int rows = prepare ? ws.k_pad : k;
    finalize_fused_kernel<T><<<(unsigned)ceil_div(rows, warps), threads, 0, (cudaStream_t)stream>>>(a);
    KMB_CHECK_LAUNCH();
  });
  return KMB_OK;
}

}  // extern "C"
