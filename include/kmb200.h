/*
 * kmb200 — C ABI of the B200 (sm_100a) KMeans kernels.
 *
 * The reference (soda-inria/sklearn-numba-dpex) has no foreign-function boundary:
 * its drivers call numba_dpex kernel objects directly.  Each entry point below
 * replaces one such kernel (or a fixed short sequence of them) and cites the
 * reference kernel factory it stands for, path relative to the reference root.
 *
 * Conventions
 *  - every function returns KMB_OK (0) or a negative kmb_status; it never throws,
 *    never exits; kmb_last_error() gives the message of the calling thread's last
 *    failure;
 *  - all array arguments are DEVICE pointers owned by the caller unless a comment
 *    says "host"; nothing is allocated or freed inside the library; scratch comes
 *    from a caller-provided workspace (see kmb_workspace_bytes);
 *  - `dtype` is KMB_F32 or KMB_F64 and names the type of every `void*` array of
 *    floating-point data in that call;
 *  - `stream` is a cudaStream_t passed as void*; work is enqueued, not awaited;
 *  - layout: samples are rows.  X is (n, d) row-major, centroids C are (k, d)
 *    row-major (the reference holds the transposes X_t (d, n), centroids_t (d, k));
 *    labels are uint32 (n); weights (n) may be NULL, meaning all ones.
 */
#ifndef KMB200_H
#define KMB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { KMB_F32 = 0, KMB_F64 = 1 } kmb_dtype;

typedef enum {
  KMB_OK = 0,
  KMB_ERR_INVALID = -1,     /* bad argument (shape, dtype, NULL, alignment)          */
  KMB_ERR_CUDA = -2,        /* a CUDA runtime / driver call failed                   */
  KMB_ERR_UNSUPPORTED = -3, /* valid request this build / device cannot serve        */
  KMB_ERR_WORKSPACE = -4    /* caller's workspace is too small                       */
} kmb_status;

/* Which contraction the fused step / label assignment uses. */
typedef enum {
  KMB_ALGO_AUTO = 0,      /* tensor cores when the shape qualifies, else CUDA cores  */
  KMB_ALGO_CUDA_CORE = 1, /* register-tiled FMA kernel (fp32 and fp64)               */
  KMB_ALGO_TF32X3 = 2     /* tcgen05 kind::tf32, 3 products per pair (fp32 only)     */
} kmb_algo;

/* Record written by kmb_lloyd_finalize (32 bytes of device memory, or of page-locked host
 * memory through its device address, see kmb_host_device_pointer). */
typedef struct {
  int32_t n_empty;     /* clusters whose weight sum is exactly 0                      */
  int32_t changed;     /* 1 if any label differs from the previous labels, else 0     */
  double shift_total;  /* sum_j sum_f (C_old - C_new)^2                               */
  double inertia;      /* reserved (0)                                                */
  int32_t wait_error;  /* copy of the workspace's time-out flag (see kmb_lloyd_wait_error) */
  int32_t reserved;
} kmb_lloyd_status;

/* Flags of kmb_lloyd_step. */
enum {
  KMB_STEP_ACC_CLEARED = 1,    /* every copy of `acc` is already zero: skip the clearing     */
  KMB_STEP_OPERANDS_READY = 2  /* KMB_ALGO_TF32X3: the split operands of C already sit in the
                                  workspace (written by kmb_lloyd_finalize with
                                  KMB_FIN_PREPARE_TF32X3 on the same workspace, C being that
                                  call's C_new): skip the split kernel                       */
};
/* Flags of kmb_lloyd_finalize. */
enum {
  KMB_FIN_MERGE = 1,          /* merged[e] = sum over copies of acc[c][e] is computed here;
                                 without it `merged` is the input (e.g. after an all-reduce)  */
  KMB_FIN_CLEAR_ACC = 2,      /* zero every copy of `acc` once it has been read               */
  KMB_FIN_PREPARE_TF32X3 = 4  /* also write the tensor-core operands of C_new into the
                                 workspace for the next kmb_lloyd_step (fp32 only)           */
};

/* Bits 8-9 of the `flags` of kmb_lloyd_step, kmb_assign_labels, kmb_lloyd_finalize and
 * kmb_lloyd_plan_launch: how many TRAILING features of X and of the centroids are zero padding
 * added by the caller (0..3; a caller that rounded d up to a multiple of 4 so that
 * KMB_ALGO_TF32X3 accepts it).  The tensor-core step then keeps its two extra contraction
 * features (the folded half norms) in those slots instead of widening the rows: d = 14 padded to
 * 16 contracts over 16 features instead of 18 -> 24.  The same value must be given to the
 * finalize call that prepares the operands and to the step that uses them; the padding features
 * of X and of every centroid must really be zero.  No counterpart in the reference. */
#define KMB_LLOYD_PAD_FEATURES(n) (((n) & 3) << 8)
#define KMB_LLOYD_PAD_MASK (3 << 8)

const char* kmb_last_error(void);
int kmb_version(void);
/* SM count and compute capability of `device` (host outputs). */
int kmb_device_info(int device, int* sm_count, int* cc_major, int* cc_minor);

/* Device address of page-locked host memory (`host` must be pinned, e.g. cudaHostAlloc), so
 * that a kernel can write a small result record straight into host memory: *device receives
 * the pointer to hand to e.g. kmb_lloyd_finalize as `status`.  No counterpart in the reference,
 * which reads its per-iteration scalars with blocking device-to-host copies
 * (kmeans/drivers.py:238, 329, 341). */
int kmb_host_device_pointer(void* host, void** device);

/* Bytes of scratch that is enough for ANY call below on these sizes. */
size_t kmb_workspace_bytes(int64_t n, int d, int k);

/* Length, in elements of `dtype`, of one accumulator copy used by kmb_lloyd_step:
 * [ sums k*d | counts k | changed 1 | padding ] rounded up to a multiple of 64. */
int64_t kmb_lloyd_acc_len(int d, int k);
/* Number of accumulator copies kmb_lloyd_step wants for this shape and algo. */
int kmb_lloyd_acc_copies(int dtype, int algo, int64_t n, int d, int k);
/* The algo KMB_ALGO_AUTO resolves to for this shape. */
int kmb_lloyd_resolve_algo(int dtype, int algo, int64_t n, int d, int k);

/* half_norms[j] = (sum_f C[j,f]^2) / 2.
 * Replaces make_half_l2_norm_2d_axis0_kernel, sklearn_numba_dpex/common/kernels.py:117-145. */
int kmb_half_l2_norm(int dtype, const void* C, void* half_norms, int k, int d, void* stream);

/* Lloyd workspace.  kmb_lloyd_step, kmb_assign_labels, kmb_lloyd_finalize and
 * kmb_matmul_nt keep a small control block (a sticky time-out flag of the tensor-core kernel
 * and a counter of the finalize kernel) at the start of the workspace they are given, and the
 * tensor-core operands behind it.  Clear the control block ONCE after allocating a
 * workspace, and again to acknowledge a reported time-out; the calls themselves never clear
 * it.  A workspace that also serves other entry points (kmb_inertia, kmb_sum, ...) must be
 * re-initialised before it is handed to the Lloyd calls again.  No counterpart in the
 * reference. */
int kmb_lloyd_workspace_init(void* workspace, size_t workspace_bytes, void* stream);

/* One fused Lloyd step over n samples: label_i = argmin_j (half_norms[j] - x_i.c_j)
 * (lowest j on ties), labels written, number of labels differing from prev_labels
 * counted (prev_labels may be NULL: counts n), and w_i*x_i / w_i accumulated into
 * copy (blockIdx % n_copies) of `acc` (n_copies x kmb_lloyd_acc_len).  `acc` is
 * cleared by this call unless KMB_STEP_ACC_CLEARED is given.
 * Replaces make_lloyd_single_step_fixed_window_kernel,
 * sklearn_numba_dpex/kmeans/kernels/lloyd_single_step.py:35-424, and the two
 * make_initialize_to_zeros_kernel launches of kmeans/drivers.py:195-196. */
int kmb_lloyd_step(int dtype, int algo, const void* X, const void* w, const void* C,
                   const void* half_norms, const uint32_t* prev_labels, uint32_t* labels,
                   void* acc, int n_copies, int64_t n, int d, int k, int flags, void* workspace,
                   size_t workspace_bytes, void* stream);

/* Copies the workspace's time-out flag to *host_flag (host memory), waits for the stream,
 * and returns KMB_ERR_CUDA if a bounded wait inside a KMB_ALGO_TF32X3 kernel ran out on this
 * workspace since its last kmb_lloyd_workspace_init (outputs computed since are invalid).
 * The same flag travels in kmb_lloyd_status.wait_error.  No counterpart in the reference,
 * whose kernels have no device-side waits. */
int kmb_lloyd_wait_error(const void* workspace, int* host_flag, void* stream);

/* out[e] = sum over copies of acc[c][e], copies added in ascending order; with clear_acc
 * the copies are zeroed afterwards.  Replaces the private-copy summation of
 * make_reduce_centroid_data_kernel, sklearn_numba_dpex/kmeans/kernels/utils.py:130-157. */
int kmb_lloyd_merge_copies(int dtype, void* acc, int n_copies, int64_t acc_len, void* out,
                           int clear_acc, void* stream);

/* From the accumulator (its copies merged here with KMB_FIN_MERGE, or `merged` given):
 * C_new = sums / counts, half norms of C_new, total squared shift against C_old, ascending
 * list of empty clusters, and the status record; one kernel.  `merged` holds
 * kmb_lloyd_acc_len elements, `shifts` k elements of scratch, both in `dtype`; `acc` may be
 * NULL when neither KMB_FIN_MERGE nor KMB_FIN_CLEAR_ACC is given.  The workspace must have
 * been initialised with kmb_lloyd_workspace_init.
 * Replaces make_reduce_centroid_data_kernel (kmeans/kernels/utils.py:114-195),
 * make_broadcast_division_1d_2d_axis0_kernel (common/kernels.py:61-82),
 * make_centroid_shifts_kernel (kmeans/kernels/utils.py:80-110) with its sum reduction, the
 * make_half_l2_norm_2d_axis0_kernel of the next iteration, and (KMB_FIN_CLEAR_ACC) the
 * make_initialize_to_zeros_kernel launches of the next iteration. */
int kmb_lloyd_finalize(int dtype, void* acc, int n_copies, void* merged, int flags,
                       const void* C_old, void* C_new, void* half_norms_new, void* shifts,
                       uint32_t* empty_list, kmb_lloyd_status* status, int k, int d,
                       void* workspace, size_t workspace_bytes, void* stream);

/* One whole single-GPU iteration in one call, for hosts whose per-call overhead matters (a
 * Python loop on a 30 us kernel): the buffers of the loop are described ONCE in a plan, and
 * kmb_lloyd_plan_launch(plan, it, ...) enqueues iteration `it` on them: kmb_lloyd_step reading
 * centroids C[it % 3], half norms h[it % 3] and previous labels labels[(it + 1) % 2], writing
 * labels[it % 2]; then kmb_lloyd_finalize (merge + clear + operands of the next step) writing
 * merged[it % 2], C[(it + 1) % 3], h[(it + 1) % 3], empty_list[it % 2] and status[it % 2].
 * The three-deep centroid ring lets a caller enqueue iteration it + 1 before it has read the
 * status of iteration it and still find everything iteration it produced.  `acc` must be zero
 * before the first launch (every launch leaves it zero again).  flags: KMB_PLAN_HAVE_PREV when
 * labels[(it + 1) % 2] hold previous labels, KMB_PLAN_OPERANDS_READY as KMB_STEP_OPERANDS_READY.
 * The three events (cudaEvent_t as void*, each may be NULL) are recorded before the fused
 * kernel, after it, and after the finalize kernel.  The caller owns the plan's memory; the
 * library keeps no reference to it after the call returns.  No counterpart in the reference,
 * whose loop issues one Python call per kernel (kmeans/drivers.py:188-343). */
typedef struct {
  int32_t dtype, algo;              /* algo resolved: KMB_ALGO_CUDA_CORE or KMB_ALGO_TF32X3 */
  int32_t d, k, n_copies, reserved;
  int64_t n;
  const void* X;
  const void* w;                    /* may be NULL */
  void* C[3];
  void* h[3];
  uint32_t* labels[2];
  void* acc;
  void* merged[2];
  void* shifts;
  uint32_t* empty_list[2];
  kmb_lloyd_status* status[2];
  void* workspace;
  size_t workspace_bytes;
} kmb_lloyd_plan;
enum { KMB_PLAN_HAVE_PREV = 1, KMB_PLAN_OPERANDS_READY = 2 };
int kmb_lloyd_plan_launch(const kmb_lloyd_plan* plan, int64_t it, int flags, void* event_before_step,
                          void* event_after_step, void* event_done, void* stream);

/* labels only.  flags: 0 or KMB_LLOYD_PAD_FEATURES(n_pad).  Replaces
 * make_label_assignment_fixed_window_kernel,
 * sklearn_numba_dpex/kmeans/kernels/compute_labels.py:19-185. */
int kmb_assign_labels(int dtype, int algo, const void* X, const void* C,
                      const void* half_norms, uint32_t* labels, int64_t n, int d, int k,
                      int flags, void* workspace, size_t workspace_bytes, void* stream);

/* per_sample[i] = w_i * sum_f (X[i,f] - C[labels[i],f])^2 (per_sample may be NULL);
 * total (may be NULL) receives the sum over i as one element of `dtype`, summed in
 * float64 in a fixed order.
 * Replaces make_compute_inertia_kernel, kmeans/kernels/compute_inertia.py:9-42, and the
 * make_sum_reduction_2d_kernel that follows it (kmeans/drivers.py:379-391). */
int kmb_inertia(int dtype, const void* X, const void* w, const void* C,
                const uint32_t* labels, void* per_sample, void* total, int64_t n, int d,
                int k, void* workspace, size_t workspace_bytes, void* stream);

/* out_t[j*ldo + i] = sqrt(sum_f (Y[j,f] - X[i,f])^2) for i < n, j < k: the (k, n) array whose
 * transpose the reference returns.  ldo >= n is the pitch of out_t in elements, so that a block
 * of rows can be written into a larger (k, n_total) array (pass out_t + first_row and
 * ldo = n_total).  Squared differences are accumulated directly, as in the reference.
 * Replaces make_compute_euclidean_distances_fixed_window_kernel,
 * kmeans/kernels/compute_euclidean_distances.py:16-161. */
int kmb_euclidean_distances(int dtype, const void* X, const void* Y, void* out_t,
                            int64_t n, int d, int k, int64_t ldo, void* stream);

/* Empty-cluster relocation on un-normalised sums: for i < n_reloc, j = empty_list[i],
 * q = far_idx[i]: sums[label_q] -= w_q x_q; sums[j] = w_q x_q; counts likewise;
 * per_sample[q] = 0 (per_sample may be NULL).  `acc` is one merged accumulator; X, w and
 * labels hold n_rows rows, and pairs whose q or label falls outside are skipped.
 * Replaces make_relocate_empty_clusters_kernel, kmeans/kernels/utils.py:12-76. */
int kmb_relocate_empty_clusters(int dtype, const void* X, const void* w,
                                const uint32_t* labels, int64_t n_rows, const int64_t* far_idx,
                                const uint32_t* empty_list, int n_reloc, void* per_sample,
                                void* acc, int d, int k, void* stream);

/* Row-wise k largest of `values` (n_rows, n_cols) by radix select.  out_values
 * (n_rows, k) and/or out_idx (n_rows, k) int64 may be NULL.  Output is ordered by
 * descending value, ties by ascending index (the reference leaves both undefined).
 * Replaces topk / topk_idx, sklearn_numba_dpex/common/topk.py:112-270 and the kernels
 * at :621-771, :1003-1093, :1143-1365. */
int kmb_topk(int dtype, const void* values, int n_rows, int64_t n_cols, int k,
             void* out_values, int64_t* out_idx, void* workspace, size_t workspace_bytes,
             void* stream);
size_t kmb_topk_workspace_bytes(int n_rows, int64_t n_cols, int k);

/* kmb_topk for callers that can hand over no scratch memory: int64 indices of the k largest
 * of ONE row of n_cols values, same order as kmb_topk.  Some hosts of this library cannot
 * allocate device memory at the point where they need a top-k: a process that gave the whole
 * GPU to its own arena at start-up has nothing left for cudaMalloc, and a latency-critical
 * loop cannot afford the device-wide synchronisation cudaMalloc/cudaFree imply.  For them the
 * scratch (radix histograms, select state, gather list) is a 48 KB array built into the
 * library image; it exists once on every GPU that loads the library and stays until the
 * process ends.  Limits: one row, k <= 4096 (larger k is rejected with KMB_ERR_INVALID; use
 * kmb_topk).  The call allocates and frees nothing.  The first call on each device looks up
 * the array's device address (cudaGetSymbolAddress, with that device current); later calls
 * only launch kernels.  The array is chosen by the CURRENT device of the calling thread, so
 * `stream` and `values` must belong to that device: a stream of another GPU would be handed
 * the wrong GPU's array, and nothing here can detect that.  All calls on a
 * device share the one array: each call clears the parts that must start at zero, but two
 * calls whose kernels overlap on the GPU (different streams, or different host threads) race
 * on it and must be serialised by the caller.  It has no counterpart in the reference. */
int kmb_topk_idx_static(int dtype, const void* values, int64_t n_cols, int k, int64_t* out_idx,
                        void* stream);

/* ---- k-means++ (kmeans/drivers.py:735-910) ---------------------------------------- */
/* Rows per partial-sum block used by the k-means++ kernels. */
int kmb_kpp_block_rows(void);

/* closest[i] = w_i * ||X[i] - X[first]||^2, bsum[b] = float64 sum of block b,
 * centers row 0 = X[first], indices[0] = first.  When first_row (d elements) is given it is
 * used instead of X[first] (row shards: the first centre may live on another rank).
 * Replaces make_kmeansplusplus_init_kernel, kmeans/kernels/kmeans_plusplus.py:16-58, and
 * the potential sum of drivers.py:844. */
int kmb_kpp_init(int dtype, const void* X, const void* w, int64_t first, const void* first_row,
                 void* closest, double* bsum, void* centers, int32_t* indices, int64_t n, int d,
                 void* stream);

/* For each trial tau < t: r = u[tau] * total, cand[tau] = first i whose inclusive prefix
 * sum of closest reaches r (0 if r <= 0, n-1 if never).  closest is row *best of
 * M (.., n) and its block sums row *best of bsum (.., nb); the prefix is taken in
 * float64.  offset (one float64, may be NULL) is subtracted from r: the potential held by
 * the row shards before this one.  Replaces make_sample_center_candidates_kernel,
 * kmeans/kernels/kmeans_plusplus.py:61-103 (a sequential running sum there). */
int kmb_kpp_sample(int dtype, const void* M, const double* bsum, const int32_t* best,
                   const void* total, const void* u, const double* offset, int t, int32_t* cand,
                   int64_t n, void* stream);

/* out[tau, :] = X[ids[tau], :]  (ids on device). */
int kmb_gather_rows(int dtype, const void* X, const int32_t* ids, int t, int d, void* out,
                    void* stream);

/* M_out[tau, i] = min(w_i * ||cand_rows[tau] - X[i]||^2, closest[i]) and
 * bsum_out[tau, b] = float64 block sums, closest = row *best of M_prev.
 * Replaces make_kmeansplusplus_single_step_fixed_window_kernel,
 * kmeans/kernels/kmeans_plusplus.py:106-262, and the row sums of drivers.py:895. */
int kmb_kpp_step(int dtype, const void* X, const void* w, const void* cand_rows,
                 const void* M_prev, const int32_t* best_prev, void* M_out,
                 double* bsum_out, int64_t n, int d, int t, void* stream);

/* pots[tau] = sum_b bsum[tau, b] in float64, fixed order (the row sums of drivers.py:895,
 * kept in float64 so that shards can be all-reduced before the argmin). */
int kmb_kpp_potentials(const double* bsum, int t, int64_t nb, double* pots, void* stream);

/* pots[tau] = pots_in[tau] if given, else sum_b bsum[tau, b] (rounded to dtype); *best = argmin (lowest
 * tau on ties); *total = pots[*best]; centers row c = cand_rows[*best];
 * indices[c] = cand[*best].  Replaces make_argmin_reduction_1d_kernel
 * (common/reductions.py:18-209) and the host steps of drivers.py:897-908. */
int kmb_kpp_select(int dtype, const double* bsum, const double* pots_in, int t, int64_t nb,
                   void* pots, int32_t* best, void* total, const void* cand_rows,
                   const int32_t* cand, void* centers, int32_t* indices, int c, int d,
                   void* stream);

/* Row-sharded seeding, two glue kernels of a round (the reference seeds on one device: no
 * counterpart; they stand where drivers.py:897-908 picks candidates and potentials on the host).
 *
 * kmb_kpp_pick_owned: every shard searched its own rows for each of the t thresholds
 * r[tau] = u[tau] * total (product in dtype, compared in float64); the valid answer is that of
 * the OWNER, the first shard whose inclusive prefix ends[w] reaches r (the last shard when
 * rounding leaves none).  `gathered` is the all-gather over the shards of (t, d + 1) blocks: a
 * candidate row followed by its LOCAL row id (the int32's bit pattern in a float32 column, its
 * value in a float64 one).  Writes cand_global[tau] = id + rows_offset[owner] and
 * rows_global (t, d).
 *
 * kmb_kpp_select_shards: kmb_kpp_select on shard_pots (n_shards, t), the all-gather of every
 * shard's float64 potentials: pots[tau] = sum over the shards in ascending order; the choice is
 * committed as kmb_kpp_select commits it; ends_out[w] = inclusive prefix over the shards of the
 * chosen candidate's potentials and *offset_out = the exclusive prefix of shard `shard`, which
 * is what the next round's kmb_kpp_sample and kmb_kpp_pick_owned take. */
int kmb_kpp_pick_owned(int dtype, const void* gathered, int n_shards, int t, int d,
                       const double* ends, const void* u, const void* total,
                       const int64_t* rows_offset, int32_t* cand_global, void* rows_global,
                       void* stream);
int kmb_kpp_select_shards(int dtype, const double* shard_pots, int n_shards, int shard, int t,
                          void* pots, int32_t* best, void* total, const void* cand_rows,
                          const int32_t* cand, void* centers, int32_t* indices, int c, int d,
                          double* ends_out, double* offset_out, void* stream);

/* ---- data preparation (kmeans/drivers.py:436-589) --------------------------------- */
/* out[f] = sum_i X[i,f] in float64 (d doubles). Replaces make_sum_reduction_2d_kernel
 * axis=1 (common/reductions.py:214-393) at drivers.py:478. */
int kmb_col_sums(int dtype, const void* X, int64_t n, int d, double* out, void* workspace,
                 size_t workspace_bytes, void* stream);
/* *out = sum_i v[i] (square=0), sum_i v[i]^2 (square=1) or sum_i (v[i] - v[i]) (square=2:
 * 0 when every element is finite, NaN otherwise -- the finiteness test of the input
 * validation, sklearn_numba_dpex/kmeans/engine.py:319-331), float64, fixed order.
 * Replaces the 1-D make_sum_reduction_2d_kernel uses at drivers.py:470-476, 516-524,
 * 533-540. */
int kmb_sum(int dtype, const void* v, int64_t len, int square, double* out, void* workspace,
            size_t workspace_bytes, void* stream);
/* X[i,f] += sign * vec[f].  Replaces make_broadcast_ops_1d_2d_axis1_kernel,
 * common/kernels.py:86-113. */
int kmb_add_row_vector(int dtype, void* X, int64_t n, int d, const void* vec, double sign,
                       void* stream);

/* ---- label utilities (kmeans/kernels/utils.py:199-279) ---------------------------- */
/* *result = 1 if the two labelings are equal up to a permutation of label values.
 * map_scratch: k int32.  Replaces make_is_same_clustering_kernel. */
int kmb_same_clustering(const uint32_t* labels1, const uint32_t* labels2, int64_t n, int k,
                        int32_t* map_scratch, int32_t* result, void* stream);
/* *out = number of distinct label values. seen_scratch: k int32.
 * Replaces make_get_nb_distinct_clusters_kernel. */
int kmb_count_distinct(const uint32_t* labels, int64_t n, int k, int32_t* seen_scratch,
                       int32_t* out, void* stream);

/* ---- RNG, host only (sklearn_numba_dpex/common/random.py:29-292) ------------------- */
/* states: host uint64[n_states][2].  SplitMix64 seeding then 2^64 jumps. */
int kmb_xoroshiro_init(uint64_t* states, int n_states, uint64_t seed, int subsequence_start);
/* next raw value of states[idx]; advances that state. */
uint64_t kmb_xoroshiro_next(uint64_t* states, int idx);
/* uint64 -> [0,1): (x>>40)*2^-24 as float, (x>>11)*2^-53 as double. */
float kmb_u64_to_unit_f32(uint64_t x);
double kmb_u64_to_unit_f64(uint64_t x);

/* Test hook for the distance contraction alone: out[i,j] = sum_f X[i,f]*Y[j,f] with the
 * named algo's arithmetic (m, n multiples of nothing in particular).  Stands for
 * make_matmul_2d_kernel, sklearn_numba_dpex/common/matmul.py:13-489, which the KMeans
 * path itself never calls. */
int kmb_matmul_nt(int dtype, int algo, const void* X, const void* Y, void* out, int64_t m,
                  int n, int kdim, void* workspace, size_t workspace_bytes, void* stream);

/* Measurement hook for the benchmark: best-of-`repeats` FMA rate (TFLOP/s, 2 flops per FMA) of
 * the CUDA cores in `dtype`, from a register-resident kernel timed with CUDA events; it is the
 * roofline denominator of the KMB_ALGO_CUDA_CORE step.  `scratch` is any device buffer of at
 * least 8 * 256 * (SM count) elements of `dtype` (never written in practice).  Waits for the
 * stream.  No counterpart in the reference. */
int kmb_measure_fma_peak(int dtype, int repeats, double* tflops, void* scratch, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KMB200_H */
