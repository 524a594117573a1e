// C entry points of the fused Lloyd step and label assignment: argument checks and the
// choice between the CUDA-core kernel and the tcgen05 3xTF32 kernel.
#include "kmb_common.cuh"

namespace kmb {
int lloyd_cc_step(int dtype, const void* X, const void* w, const void* C, const void* h,
                  const uint32_t* prev, uint32_t* labels, void* acc, int n_copies,
                  int64_t acc_len, int64_t n, int d, int k, cudaStream_t stream);
int lloyd_cc_assign(int dtype, const void* X, const void* C, const void* h, uint32_t* labels,
                    int64_t n, int d, int k, cudaStream_t stream);
bool lloyd_cc_privatises(int dtype, int d, int k);

bool lloyd_tc_supported(int dtype, int64_t n, int d, int k);
bool lloyd_tc_preferred(int dtype, int64_t n, int d, int k);
int lloyd_tc_run(const float* X, const float* w, const float* C, const float* h,
                 const uint32_t* prev, uint32_t* labels, float* acc, int n_copies,
                 int64_t acc_len, int64_t n, int d, int k, int pad, bool update, bool operands_ready,
                 void* workspace, size_t workspace_bytes, cudaStream_t stream);
int lloyd_tc_acc_copies(int d, int k);
}  // namespace kmb

using namespace kmb;

static int resolve_algo(int dtype, int algo, int64_t n, int d, int k) {
  if (algo == KMB_ALGO_CUDA_CORE) return KMB_ALGO_CUDA_CORE;
  if (algo == KMB_ALGO_TF32X3) return lloyd_tc_supported(dtype, n, d, k) ? KMB_ALGO_TF32X3 : -1;
  return lloyd_tc_preferred(dtype, n, d, k) ? KMB_ALGO_TF32X3 : KMB_ALGO_CUDA_CORE;
}

extern "C" {

int kmb_lloyd_resolve_algo(int dtype, int algo, int64_t n, int d, int k) {
  if (dtype != KMB_F32 && dtype != KMB_F64) {
    set_error("dtype must be KMB_F32 or KMB_F64, got %d", dtype);
    return KMB_ERR_INVALID;
  }
  if (algo < KMB_ALGO_AUTO || algo > KMB_ALGO_TF32X3) {
    set_error("unknown algo %d", algo);
    return KMB_ERR_INVALID;
  }
  const int r = resolve_algo(dtype, algo, n, d, k);
  if (r < 0) {
    set_error("KMB_ALGO_TF32X3 does not support dtype=%d n=%lld d=%d k=%d (fp32 only, "
              "d a multiple of 4 and <= 128, k <= 65536)", dtype, (long long)n, d, k);
    return KMB_ERR_UNSUPPORTED;
  }
  return r;
}

int kmb_lloyd_acc_copies(int dtype, int algo, int64_t n, int d, int k) {
  const int r = kmb_lloyd_resolve_algo(dtype, algo, n, d, k);
  if (r < 0) return r;
  if (r == KMB_ALGO_TF32X3) return lloyd_tc_acc_copies(d, k);
  return lloyd_cc_privatises(dtype, d, k) ? 1 : 8;
}

int kmb_lloyd_wait_error(const void* workspace, int* host_flag, void* stream) {
  KMB_REQUIRE(workspace && host_flag, "kmb_lloyd_wait_error: bad arguments");
  LloydWorkspace ws = lloyd_carve(const_cast<void*>(workspace), 1, 1);
  KMB_CHECK_CUDA(cudaMemcpyAsync(host_flag, &ws.ctl->wait_error, sizeof(int),
                                 cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  KMB_CHECK_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  if (*host_flag != 0) {
    set_error("a bounded wait inside the tcgen05 Lloyd kernel ran out; results computed on this "
              "workspace since its last kmb_lloyd_workspace_init are invalid");
    return KMB_ERR_CUDA;
  }
  return KMB_OK;
}

int kmb_lloyd_step(int dtype, int algo, const void* X, const void* w, const void* C,
                   const void* half_norms, const uint32_t* prev_labels, uint32_t* labels,
                   void* acc, int n_copies, int64_t n, int d, int k, int flags, void* workspace,
                   size_t workspace_bytes, void* stream) {
  KMB_REQUIRE(X && C && half_norms && labels && acc, "kmb_lloyd_step: NULL argument");
  KMB_REQUIRE(n >= 0 && d > 0 && k > 0 && n_copies >= 1, "kmb_lloyd_step: bad sizes");
  KMB_REQUIRE((int64_t)k * d < (1ll << 31), "kmb_lloyd_step: k*d must be below 2^31");
  const int r = kmb_lloyd_resolve_algo(dtype, algo, n, d, k);
  if (r < 0) return r;
  KMB_REQUIRE((flags & ~(KMB_STEP_ACC_CLEARED | KMB_STEP_OPERANDS_READY | KMB_LLOYD_PAD_MASK)) == 0,
              "kmb_lloyd_step: unknown flag bits %d", flags);
  const int pad = (flags & KMB_LLOYD_PAD_MASK) >> 8;
  KMB_REQUIRE(pad < d, "kmb_lloyd_step: %d padding features in rows of %d", pad, d);
  const int64_t acc_len = kmb_lloyd_acc_len(d, k);
  const size_t esize = dtype == KMB_F32 ? 4 : 8;
  if (!(flags & KMB_STEP_ACC_CLEARED))
    KMB_CHECK_CUDA(cudaMemsetAsync(acc, 0, (size_t)n_copies * acc_len * esize, (cudaStream_t)stream));
  if (n == 0) return KMB_OK;
  if (r == KMB_ALGO_TF32X3)
    return lloyd_tc_run((const float*)X, (const float*)w, (const float*)C,
                        (const float*)half_norms, prev_labels, labels, (float*)acc, n_copies,
                        acc_len, n, d, k, pad, true, (flags & KMB_STEP_OPERANDS_READY) != 0, workspace,
                        workspace_bytes, (cudaStream_t)stream);
  return lloyd_cc_step(dtype, X, w, C, half_norms, prev_labels, labels, acc, n_copies, acc_len, n,
                       d, k, (cudaStream_t)stream);
}

int kmb_lloyd_plan_launch(const kmb_lloyd_plan* plan, int64_t it, int flags, void* event_before_step,
                          void* event_after_step, void* event_done, void* stream) {
  KMB_REQUIRE(plan != nullptr && it >= 0, "kmb_lloyd_plan_launch: bad arguments");
  KMB_REQUIRE((flags & ~(KMB_PLAN_HAVE_PREV | KMB_PLAN_OPERANDS_READY | KMB_LLOYD_PAD_MASK)) == 0,
              "kmb_lloyd_plan_launch: unknown flag bits %d", flags);
  const int pad_bits = flags & KMB_LLOYD_PAD_MASK;
  KMB_REQUIRE(plan->algo == KMB_ALGO_CUDA_CORE || plan->algo == KMB_ALGO_TF32X3,
              "kmb_lloyd_plan_launch: the plan must hold a resolved algo");
  cudaStream_t s = (cudaStream_t)stream;
  const int c = (int)(it % 3), cn = (int)((it + 1) % 3), l = (int)(it % 2), lp = (int)((it + 1) % 2);
  const bool tc = plan->algo == KMB_ALGO_TF32X3;
  if (event_before_step) KMB_CHECK_CUDA(cudaEventRecord((cudaEvent_t)event_before_step, s));
  int rc = kmb_lloyd_step(plan->dtype, plan->algo, plan->X, plan->w, plan->C[c], plan->h[c],
                          (flags & KMB_PLAN_HAVE_PREV) ? plan->labels[lp] : nullptr, plan->labels[l],
                          plan->acc, plan->n_copies, plan->n, plan->d, plan->k,
                          KMB_STEP_ACC_CLEARED | pad_bits |
                              ((flags & KMB_PLAN_OPERANDS_READY) ? KMB_STEP_OPERANDS_READY : 0),
                          plan->workspace, plan->workspace_bytes, stream);
  if (rc != KMB_OK) return rc;
  if (event_after_step) KMB_CHECK_CUDA(cudaEventRecord((cudaEvent_t)event_after_step, s));
  rc = kmb_lloyd_finalize(plan->dtype, plan->acc, plan->n_copies, plan->merged[l],
                          KMB_FIN_MERGE | KMB_FIN_CLEAR_ACC | pad_bits | (tc ? KMB_FIN_PREPARE_TF32X3 : 0),
                          plan->C[c], plan->C[cn], plan->h[cn], plan->shifts, plan->empty_list[l],
                          plan->status[l], plan->k, plan->d, plan->workspace, plan->workspace_bytes,
                          stream);
  if (rc != KMB_OK) return rc;
  if (event_done) KMB_CHECK_CUDA(cudaEventRecord((cudaEvent_t)event_done, s));
  return KMB_OK;
}

int kmb_assign_labels(int dtype, int algo, const void* X, const void* C, const void* half_norms,
                      uint32_t* labels, int64_t n, int d, int k, int flags, void* workspace,
                      size_t workspace_bytes, void* stream) {
  KMB_REQUIRE(X && C && half_norms && labels, "kmb_assign_labels: NULL argument");
  KMB_REQUIRE(n >= 0 && d > 0 && k > 0, "kmb_assign_labels: bad sizes");
  KMB_REQUIRE((flags & ~KMB_LLOYD_PAD_MASK) == 0, "kmb_assign_labels: unknown flag bits %d", flags);
  const int pad = (flags & KMB_LLOYD_PAD_MASK) >> 8;
  KMB_REQUIRE(pad < d, "kmb_assign_labels: %d padding features in rows of %d", pad, d);
  KMB_REQUIRE((int64_t)k * d < (1ll << 31), "kmb_assign_labels: k*d must be below 2^31");
  const int r = kmb_lloyd_resolve_algo(dtype, algo, n, d, k);
  if (r < 0) return r;
  if (n == 0) return KMB_OK;
  if (r == KMB_ALGO_TF32X3)
    return lloyd_tc_run((const float*)X, nullptr, (const float*)C, (const float*)half_norms,
                        nullptr, labels, nullptr, 1, 0, n, d, k, pad, false, false, workspace,
                        workspace_bytes, (cudaStream_t)stream);
  return lloyd_cc_assign(dtype, X, C, half_norms, labels, n, d, k, (cudaStream_t)stream);
}

}  // extern "C"
