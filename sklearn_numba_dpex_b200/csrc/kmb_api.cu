// Library-wide entry points: error string, device query, workspace sizing, host RNG.
#include "kmb_common.cuh"

namespace kmb {
static thread_local char g_err[1024] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
}  // namespace kmb

extern "C" {

const char* kmb_last_error(void) { return kmb::g_err; }

int kmb_version(void) { return 100; }

int kmb_device_info(int device, int* sm_count, int* cc_major, int* cc_minor) {
  KMB_REQUIRE(sm_count && cc_major && cc_minor, "kmb_device_info: NULL output");
  KMB_CHECK_CUDA(cudaDeviceGetAttribute(sm_count, cudaDevAttrMultiProcessorCount, device));
  KMB_CHECK_CUDA(cudaDeviceGetAttribute(cc_major, cudaDevAttrComputeCapabilityMajor, device));
  KMB_CHECK_CUDA(cudaDeviceGetAttribute(cc_minor, cudaDevAttrComputeCapabilityMinor, device));
  return KMB_OK;
}

int kmb_host_device_pointer(void* host, void** device) {
  KMB_REQUIRE(host && device, "kmb_host_device_pointer: NULL argument");
  KMB_CHECK_CUDA(cudaHostGetDevicePointer(device, host, 0));
  return KMB_OK;
}

size_t kmb_workspace_bytes(int64_t n, int d, int k) {
  // Fixed-order reductions use <= 4096 float64 partials per reduced quantity and at most
  // max(d, 64) quantities; the tensor-core step keeps hi/lo copies of the centroids.
  size_t partials = (size_t)4096 * sizeof(double) * (size_t)(d > 64 ? d : 64);
  size_t centroid_split = (size_t)2 * (size_t)(k + 256) * (size_t)(d + 32) * sizeof(float) +
                          (size_t)(k + 256) * sizeof(float) + 8192;
  size_t topk = kmb_topk_workspace_bytes(1, n, k);
  return partials + centroid_split + topk + 65536;
}

/* ---- xoroshiro128++ on the host.  Follows sklearn_numba_dpex/common/random.py:188-292. */
static inline uint64_t rotl64(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }

static inline uint64_t splitmix64(uint64_t* state) {
  uint64_t z = (*state += 0x9E3779B97F4A7C15ull);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

uint64_t kmb_xoroshiro_next(uint64_t* states, int idx) {
  uint64_t s0 = states[2 * idx], s1 = states[2 * idx + 1];
  uint64_t result = rotl64(s0 + s1, 17) + s0;
  s1 ^= s0;
  states[2 * idx] = rotl64(s0, 49) ^ s1 ^ (s1 << 21);
  states[2 * idx + 1] = rotl64(s1, 28);
  return result;
}

static void xoroshiro_jump(uint64_t* states, int idx) {
  static const uint64_t JUMP[2] = {0x2BD7A6A6E99C2DDCull, 0x0992CCAF6A6FCA05ull};
  uint64_t a0 = 0, a1 = 0;
  for (int i = 0; i < 2; ++i)
    for (int b = 0; b < 64; ++b) {
      if (JUMP[i] & (1ull << b)) {
        a0 ^= states[2 * idx];
        a1 ^= states[2 * idx + 1];
      }
      kmb_xoroshiro_next(states, idx);
    }
  states[2 * idx] = a0;
  states[2 * idx + 1] = a1;
}

int kmb_xoroshiro_init(uint64_t* states, int n_states, uint64_t seed, int subsequence_start) {
  KMB_REQUIRE(states != nullptr && n_states >= 0 && subsequence_start >= 0,
              "kmb_xoroshiro_init: bad arguments");
  if (n_states < 1) return KMB_OK;
  uint64_t sm = seed;
  states[0] = splitmix64(&sm);
  states[1] = splitmix64(&sm);
  for (int i = 0; i < subsequence_start; ++i) xoroshiro_jump(states, 0);
  for (int i = 1; i < n_states; ++i) {
    states[2 * i] = states[2 * (i - 1)];
    states[2 * i + 1] = states[2 * (i - 1) + 1];
    xoroshiro_jump(states, i);
  }
  return KMB_OK;
}

float kmb_u64_to_unit_f32(uint64_t x) { return (float)(x >> 40) * (1.0f / 16777216.0f); }

double kmb_u64_to_unit_f64(uint64_t x) {
  return (double)(x >> 11) * (1.0 / 9007199254740992.0);
}

}  // extern "C"
