/*
 * TEST INFRASTRUCTURE ONLY — plain C restatement of one Lloyd iteration of the reference,
 * threaded with OpenMP so that it can serve as the CPU baseline of the benchmark and check
 * mid-sized cases in seconds.  Nothing in the shipped package links or loads this file.
 *
 * Arithmetic follows the reference's fused kernel
 * (sklearn_numba_dpex/kmeans/kernels/lloyd_single_step.py:149-414 and
 *  kmeans/kernels/_base_kmeans_kernel_funcs.py:266-301, 351-366):
 *   dot_j accumulates x_f * c_jf feature by feature in the compute type (multiply, then
 *   add: compiled with -ffp-contract=off), q_j = h_j - dot_j, label = first j with the
 *   strictly smallest q_j scanning upward from +inf; then w*x and w are added into one
 *   private copy of the centroid sums / counts per thread, merged in thread order (the
 *   reference merges its private copies in copy order, kmeans/kernels/utils.py:148-157).
 * Centroids are passed feature-major, Ct (d, k), the reference's own layout.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ROWS 4

#define DEFINE_ORACLE(T, SUFFIX)                                                               \
  int oracle_lloyd_iter_##SUFFIX(const T* X, const T* w, const T* Ct, const T* h, int64_t n,   \
                                 int d, int k, uint32_t* labels, T* sums, T* counts,          \
                                 int do_update) {                                              \
    int nthreads = 1;                                                                          \
    _Pragma("omp parallel")                                                                    \
    {                                                                                          \
      _Pragma("omp single") nthreads = omp_get_num_threads();                                  \
    }                                                                                          \
    T* psums = NULL;                                                                           \
    T* pcnt = NULL;                                                                            \
    if (do_update) {                                                                           \
      psums = (T*)calloc((size_t)nthreads * k * d, sizeof(T));                                 \
      pcnt = (T*)calloc((size_t)nthreads * k, sizeof(T));                                      \
      if (!psums || !pcnt) return -1;                                                          \
    }                                                                                          \
    _Pragma("omp parallel")                                                                    \
    {                                                                                          \
      const int tid = omp_get_thread_num();                                                    \
      T* dots = (T*)malloc((size_t)ROWS * k * sizeof(T));                                      \
      T* my_sums = do_update ? psums + (size_t)tid * k * d : NULL;                             \
      T* my_cnt = do_update ? pcnt + (size_t)tid * k : NULL;                                   \
      _Pragma("omp for schedule(static)")                                                      \
      for (int64_t i0 = 0; i0 < n; i0 += ROWS) {                                               \
        const int rows = (int)((n - i0 < ROWS) ? (n - i0) : ROWS);                             \
        for (int r = 0; r < ROWS; ++r)                                                         \
          for (int j = 0; j < k; ++j) dots[r * k + j] = (T)0;                                  \
        for (int f = 0; f < d; ++f) {                                                          \
          const T* c = Ct + (size_t)f * k;                                                     \
          T xv[ROWS];                                                                          \
          for (int r = 0; r < ROWS; ++r) xv[r] = (r < rows) ? X[(i0 + r) * d + f] : (T)0;      \
          for (int j = 0; j < k; ++j) {                                                        \
            const T cv = c[j];                                                                 \
            for (int r = 0; r < ROWS; ++r) dots[r * k + j] += xv[r] * cv;                      \
          }                                                                                    \
        }                                                                                      \
        for (int r = 0; r < rows; ++r) {                                                       \
          T best = (T)INFINITY;                                                                \
          uint32_t bi = 0;                                                                     \
          for (int j = 0; j < k; ++j) {                                                        \
            const T q = h[j] - dots[r * k + j];                                                \
            if (q < best) {                                                                    \
              best = q;                                                                        \
              bi = (uint32_t)j;                                                                \
            }                                                                                  \
          }                                                                                    \
          labels[i0 + r] = bi;                                                                 \
          if (do_update) {                                                                     \
            const T wi = w ? w[i0 + r] : (T)1;                                                 \
            my_cnt[bi] += wi;                                                                  \
            for (int f = 0; f < d; ++f) my_sums[(size_t)bi * d + f] += X[(i0 + r) * d + f] * wi; \
          }                                                                                    \
        }                                                                                      \
      }                                                                                        \
      free(dots);                                                                              \
    }                                                                                          \
    if (do_update) {                                                                           \
      memset(sums, 0, (size_t)k * d * sizeof(T));                                              \
      memset(counts, 0, (size_t)k * sizeof(T));                                                \
      for (int t = 0; t < nthreads; ++t) {                                                     \
        for (size_t e = 0; e < (size_t)k * d; ++e) sums[e] += psums[(size_t)t * k * d + e];    \
        for (int j = 0; j < k; ++j) counts[j] += pcnt[(size_t)t * k + j];                      \
      }                                                                                        \
      free(psums);                                                                             \
      free(pcnt);                                                                              \
    }                                                                                          \
    return nthreads;                                                                           \
  }

DEFINE_ORACLE(float, f32)
DEFINE_ORACLE(double, f64)

void oracle_set_num_threads(int count) {
#ifdef _OPENMP
  if (count > 0) omp_set_num_threads(count);
#else
  (void)count;
#endif
}

int oracle_num_threads(void) {
  int n = 1;
#pragma omp parallel
  {
#pragma omp single
    n = omp_get_num_threads();
  }
  return n;
}
