// tcgen05 3xTF32 fused Lloyd step (placeholder until the kernel lands: reports
// "not supported" so that KMB_ALGO_AUTO resolves to the CUDA-core kernel).
#include "kmb_common.cuh"

namespace kmb {

bool lloyd_tc_supported(int, int64_t, int, int) { return false; }
bool lloyd_tc_preferred(int, int64_t, int, int) { return false; }
int lloyd_tc_acc_copies(int, int) { return 8; }

int lloyd_tc_run(const float*, const float*, const float*, const float*, const uint32_t*,
                 uint32_t*, float*, int, int64_t, int64_t, int, int, bool, void*, size_t,
                 cudaStream_t) {
  set_error("the tcgen05 step is not built into this library");
  return KMB_ERR_UNSUPPORTED;
}

int lloyd_tc_matmul(const float*, const float*, float*, int64_t, int, int, void*, size_t,
                    cudaStream_t) {
  set_error("the tcgen05 step is not built into this library");
  return KMB_ERR_UNSUPPORTED;
}

}  // namespace kmb
