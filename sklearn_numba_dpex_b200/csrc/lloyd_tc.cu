// Fused Lloyd step on the 5th-generation tensor cores: tcgen05.mma kind::tf32 with the
// 3xTF32 split (x = xh + xl, c = ch + cl, x.c ~ xl.ch + xh.cl + xh.ch, fp32 accumulation in
// tensor memory), TMA-staged operand tiles, an argmin epilogue fed by tcgen05.ld, and a
// centroid update with 16-byte vector reductions.
//
// One persistent CTA per SM, 12 warps:
//   warp 0       TMA producer of the raw fp32 sample tile (128 rows x d, 128B-swizzled)
//   warp 1       TMA producer of the centroid stages (hi and lo parts, 128 centroids x 32
//                features each, five stages = 160 KB in flight)
//   warps 2, 3   issue the MMAs, one accumulator buffer each (warp 2 also allocates tensor
//                memory); the whole warp walks the loop so that descriptors stay in the uniform
//                datapath, one elected lane issues
//   warps 4..7   split the staged sample tile into hi / lo parts held in TENSOR MEMORY (the A
//                operand is read from TMEM), then run the argmin epilogue on columns 0..63 of
//                every accumulator: one sample row per thread = one TMEM lane, a min-tree per 32
//                accumulator columns; they merge the two halves into the labels
//   warps 8..11  argmin epilogue on columns 64..127 of every accumulator
//   warps 4..11  centroid update of the tile, 16 rows per warp: 16-byte vector reductions
//                (red.global.add.v4.f32) into an L2-resident accumulator copy
// Tensor memory (512 columns): A_hi [0,128) | A_lo [128,256) | accumulator 0 [256,384) |
// accumulator 1 [384,512).  Accumulators are double-buffered, so the epilogue of centroid
// tile j overlaps the MMAs of tile j+1, and the next sample tile is split into TMEM as soon
// as the last accumulator of the current tile has completed.  Rows of at most 64 features
// leave room for two sample tiles in tensor memory (A_hi | A_lo of 64 columns each, twice), and
// then the split of tile t + 1 overlaps the MMAs of tile t as well.
//
// CTAs walk the centroid tiles (and the feature chunks inside a tile) in rotated orders
// that depend on blockIdx, so that the 148 SMs do not all pull the same L2 lines at the same
// moment; the argmin stays "lowest index wins ties" by merging per-tile minima
// lexicographically.
//
// Every wait on an mbarrier is bounded: on time-out the CTA raises a flag in global memory and
// all roles leave their loops.  On the way out the producers wait (again bounded) for the bulk
// copies they still have in flight and the MMA warps for their last MMAs, then tensor memory is
// released and the kernel returns; the flag is sticky and reaches the host through the status
// record and kmb_lloyd_wait_error.
//
// Stands for fused_lloyd_single_step / assignment of the reference
// (sklearn_numba_dpex/kmeans/kernels/lloyd_single_step.py:149-414,
//  kmeans/kernels/compute_labels.py:75-168) when the contraction is GEMM-sized.
#include <cuda.h>
#include <stdlib.h>

#include "kmb_common.cuh"

namespace kmb {

constexpr int TC_BM = 128;          // samples per tile = TMEM lanes
constexpr int TC_BN = 128;          // centroids per MMA / accumulator buffer
constexpr int TC_KC = 32;           // features per 128-byte swizzle atom
constexpr int TC_STAGES = 5;        // centroid stages in flight
constexpr int TC_MAX_D = 128;       // d_pad <= 128: hi and lo parts take 2 x 128 TMEM columns
constexpr int TC_WARPS = 12;
constexpr int TC_THREADS = TC_WARPS * 32;
constexpr int TC_EPI_WARP0 = 4;
constexpr int TC_UPD_WARP0 = 8;
constexpr int TC_ATOM_BYTES = TC_BM * TC_KC * 4;  // 16 KB: 128 rows x 128 B
constexpr int TC_A_HI_COL = 0, TC_A_LO_COL = 128, TC_ACC_COL = 256, TC_TMEM_COLS = 512;
constexpr long long TC_TIMEOUT_CYCLES = 4000000000LL;  // ~2 s at 2 GHz

struct TcSmem {
  // all tiles 1024-byte aligned (128B swizzle atoms repeat every 1024 bytes)
  unsigned char xstage[TC_MAX_D / TC_KC][TC_ATOM_BYTES];
  unsigned char bhi[TC_STAGES][TC_ATOM_BYTES];
  unsigned char blo[TC_STAGES][TC_ATOM_BYTES];
  // k <= 65536, so labels fit 16 bits here (shared memory is full to the last kilobyte)
  uint16_t lab_s[2][TC_BM];       // labels of a finished tile, read by the centroid update
  float part_v[TC_BM];            // group 1's minimum and index per row, merged by group 0
  uint16_t part_i[TC_BM];
  unsigned long long x_full[2], x_conv[2], x_stage_free[2];
  unsigned long long b_full[TC_STAGES], b_empty[TC_STAGES];
  unsigned long long acc_full[2], acc_empty[2];
  unsigned long long part_full[2], lab_ready[2];
  unsigned long long drain[2];      // [MMA warp]: its last MMAs have completed (aborting CTA only)
  long long timeout_cycles;
  unsigned int tmem_base;
  volatile int abort_flag;
};

static_assert(sizeof(TcSmem) + 1024 <= 232448, "TcSmem exceeds the 227 KB a CTA may use");

struct TcParams {
  const float* X;
  const float* w;
  const float* h_pad;       // k_pad entries, +inf beyond k
  const uint32_t* prev;
  uint32_t* labels;
  float* acc;               // n_copies x acc_len, or NULL (labels only)
  float* dots;              // optional (n, ldd) raw dot products (test hook), or NULL
  int* error_flag;
  int64_t acc_len;
  int64_t n;
  int ldd;
  int n_copies;
  int d;
  int d_pad;
  int k;
  int k_pad;
  uint32_t sleep_ns;        // > 0: barrier waits may sleep this long between polls (see mbar_try_wait_sleep)
  int round_lo;             // general kernel: round the low parts of the sample split (else truncated)
  int acc_bufs;             // quads kernel: accumulators to use when three fit (2 or 3)
  int mma_warps;            // quads kernel: warps that issue MMAs (1..TQ_MMA_WARPS)
  float fone;               // 1.0f, opaque to the compiler (see take_if_equal)
  int fold_at;              // first of the two fold features (lloyd_tc_fold_at), or -1
  long long timeout_cycles; // limit of every barrier wait
  int test_stall;           // test hook: the sample-tile producer stops after its first tile
};

// ---------------------------------------------------------------------------- PTX
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(void* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(void* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(void* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(void* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same test, but the hardware may keep the thread asleep for up to `hint_ns` nanoseconds
// while the phase is incomplete: a waiting warp then costs no issue slots (a spinning one
// competes with the epilogue warps for the integer pipe).
__device__ __forceinline__ bool mbar_try_wait_sleep(void* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}

// Bounded wait: false when the CTA is aborting or the time limit ran out.
__device__ __forceinline__ bool mbar_wait(void* bar, uint32_t parity, TcSmem* sm, int* error_flag,
                                          uint32_t sleep_ns = 0u) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (sleep_ns != 0u) {
      if (mbar_try_wait_sleep(bar, parity, sleep_ns)) return true;
    } else {
      for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    }
    if (sm->abort_flag) return false;
    if (clock64() - t0 > sm->timeout_cycles) {
      sm->abort_flag = 1;
      atomicExch(error_flag, 1);
      return false;
    }
  }
}

// Leaving an aborting CTA: wait, for about a millisecond at most, until phase `parity` of a
// barrier has completed.
__device__ __forceinline__ void drain_wait(void* bar, uint32_t parity) {
  for (int i = 0; i < 4096; ++i) {
    if (mbar_try_wait(bar, parity)) return;
    __nanosleep(256);
  }
}
// A producer that armed the `full` barriers of a ring of n_slots slots for items 0 .. issued - 1
// (item i -> slot i mod n_slots, phase (i / n_slots) & 1) waits for the last copy into every slot,
// so that no bulk copy is still writing this CTA's shared memory when the CTA exits.
__device__ __forceinline__ void drain_ring(unsigned long long* bars, uint32_t n_slots, uint32_t issued) {
  for (uint32_t s = 0; s < n_slots && s < issued; ++s) {
    const uint32_t last = s + ((issued - 1u - s) / n_slots) * n_slots;
    drain_wait(&bars[s], (last / n_slots) & 1u);
  }
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y,
                                            void* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(void* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void umma_commit(void* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
      "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]),
      "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]),
      "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// A operand read from tensor memory (lane = row, one 32-bit column per tf32 element).
__device__ __forceinline__ void umma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Round-to-nearest (ties away) to the 10-bit tf32 mantissa with integer ops only: the split
// of a whole sample tile then runs on the ALU instead of the conversion unit.
__device__ __forceinline__ float tf32_round_alu(float x) {
  return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u);
}

// One lane of a converged warp (warp-uniform predicate).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
// Aborting CTA: the elected lane of an MMA warp commits once more, to a barrier nobody else uses,
// and waits (bounded) for it: all MMAs it issued have then completed.
__device__ __forceinline__ void mma_drain(void* bar) {
  if (elect_one()) {
    umma_commit(bar);
    drain_wait(bar, 0u);
  }
  __syncwarp();
}

// Shared-memory matrix descriptor of a K-major, 128B-swizzled tile whose rows are 128 bytes
// apart and whose 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t make_sdesc(uint32_t saddr) {
  uint64_t desc = 0;
  desc |= (uint64_t)((saddr & 0x3FFFF) >> 4);   // start address, 16-byte units
  desc |= (uint64_t)1 << 16;                    // leading byte offset (unused with swizzle)
  desc |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset between 8-row groups
  desc |= (uint64_t)1 << 46;                    // descriptor version of sm_100
  desc |= (uint64_t)2 << 61;                    // SWIZZLE_128B
  return desc;
}

// kind::tf32, fp32 accumulate, both operands K-major, M = 128, N = 128.
constexpr uint32_t TC_IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TC_BN >> 3) << 17) |
                              ((uint32_t)(TC_BM >> 4) << 24);


// Build with -DKMB_TC_PROFILE to make CTA 0 print how long its MMA warp waited on each barrier.
#ifdef KMB_TC_PROFILE
#define KMB_PROF(...) __VA_ARGS__
#else
#define KMB_PROF(...)
#endif

// ------------------------------------------------------------------------- the kernel
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Maximum of 32 scores with three-input maxima (NaNs are dropped; 32 NaNs give NaN).
__device__ __forceinline__ float max32(const float (&q)[32]) {
  float a[11];
#pragma unroll
  for (int j = 0; j < 10; ++j) a[j] = fmax3(q[3 * j], q[3 * j + 1], q[3 * j + 2]);
  a[10] = fmaxf(q[30], q[31]);
  const float b0 = fmax3(a[0], a[1], a[2]), b1 = fmax3(a[3], a[4], a[5]);
  const float b2 = fmax3(a[6], a[7], a[8]), b3 = fmaxf(a[9], a[10]);
  return fmaxf(fmax3(b0, b1, b2), b3);
}

// LOWEST index j with q[j] == m, m being the maximum of the 32 scores; (-inf, base) when m is
// NaN: one equality scan from the top index down, so that the lowest equal index is written
// last.  (A variant that searched on the FMA pipe, e_j = (m - q[j]) * 2^126 + j reduced with
// three-input minima, executed 25 % more instructions and measured 6 % slower on short rows:
// the epilogue is bound by issue slots, not by the integer pipe.)
__device__ __forceinline__ void index_of_max32(const float (&q)[32], float m, uint32_t base,
                                               float& out_v, uint32_t& out_i) {
  uint32_t idx = 0;
#pragma unroll
  for (int j = 31; j >= 1; --j) idx = (q[j] == m) ? (uint32_t)j : idx;
  idx = (q[0] == m) ? 0u : idx;
  out_v = (m == m) ? m : __int_as_float(0xff800000);
  out_i = base + idx;
}

// Maximum of the scores s[j] of 32 consecutive centroids and the LOWEST index that attains it.
// The score is acc[j] - h[j] (the negated pseudo-inertia), or acc[j] itself when the half norms
// were folded into the contraction.  A NaN score never wins; 32 NaNs give (-inf, base).
template <bool FOLD>
__device__ __forceinline__ void argmax32(const uint32_t (&v)[32], const float4 (&h4)[8],
                                         uint32_t base, float& out_v, uint32_t& out_i) {
  float q[32];
  if (FOLD) {
#pragma unroll
    for (int j = 0; j < 32; ++j) q[j] = __uint_as_float(v[j]);
  } else {
#pragma unroll
    for (int j4 = 0; j4 < 8; ++j4) {
      const float4 hv = h4[j4];
      q[4 * j4 + 0] = __uint_as_float(v[4 * j4 + 0]) - hv.x;
      q[4 * j4 + 1] = __uint_as_float(v[4 * j4 + 1]) - hv.y;
      q[4 * j4 + 2] = __uint_as_float(v[4 * j4 + 2]) - hv.z;
      q[4 * j4 + 3] = __uint_as_float(v[4 * j4 + 3]) - hv.w;
    }
  }
  index_of_max32(q, max32(q), base, out_v, out_i);
}

// acc = (qj == m) ? one * J + basef : acc with the select done by a PREDICATED FMA: the comparison
// runs on the integer pipe, the conditional write on the FMA pipe.  `one` is 1.0f passed at run
// time, so that the compiler cannot turn the FMA back into a move or a select; J is an immediate
// (HEX = its float32 bit pattern) and basef changes with every group of 32 scores, so that
// nothing of it can be computed ahead of the loop and kept in registers.
#define KMB_TAKE_IF_EQUAL(acc, qj, HEX)                                                        \
  asm("{\n\t.reg .pred p;\n\tsetp.eq.f32 p, %1, %2;\n\t@p fma.rn.f32 %0, %3, 0f" HEX ", %4;\n\t}" \
      : "+f"(acc)                                                                                       \
      : "f"(qj), "f"(m), "f"(one), "f"(basef))

// argmax32 for folded half norms with the index carried as a float (exact: indices < 2^24) and
// the index search split between the pipes: per score one comparison on the integer pipe (half
// rate) and one predicated multiply on the FMA pipe, instead of a comparison and a select both on
// the integer pipe.  Four independent chains (scores 0..7, 8..15, 16..23, 24..31) walk down from
// their top index so that the lowest equal index of each is written last; 32 NaNs give (-inf, some index), which
// never wins a strict comparison.
__device__ __forceinline__ void argmax32_fidx(const uint32_t (&v)[32], float basef, float one,
                                              float& out_v, float& out_if) {
  float q[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) q[j] = __uint_as_float(v[j]);
  const float m = max32(q);
  float i0 = 3.0e38f, i1 = 3.0e38f, i2 = 3.0e38f, i3 = 3.0e38f;
  KMB_TAKE_IF_EQUAL(i3, q[31], "41F80000");
  KMB_TAKE_IF_EQUAL(i2, q[23], "41B80000");
  KMB_TAKE_IF_EQUAL(i1, q[15], "41700000");
  KMB_TAKE_IF_EQUAL(i0, q[7], "40E00000");
  KMB_TAKE_IF_EQUAL(i3, q[30], "41F00000");
  KMB_TAKE_IF_EQUAL(i2, q[22], "41B00000");
  KMB_TAKE_IF_EQUAL(i1, q[14], "41600000");
  KMB_TAKE_IF_EQUAL(i0, q[6], "40C00000");
  KMB_TAKE_IF_EQUAL(i3, q[29], "41E80000");
  KMB_TAKE_IF_EQUAL(i2, q[21], "41A80000");
  KMB_TAKE_IF_EQUAL(i1, q[13], "41500000");
  KMB_TAKE_IF_EQUAL(i0, q[5], "40A00000");
  KMB_TAKE_IF_EQUAL(i3, q[28], "41E00000");
  KMB_TAKE_IF_EQUAL(i2, q[20], "41A00000");
  KMB_TAKE_IF_EQUAL(i1, q[12], "41400000");
  KMB_TAKE_IF_EQUAL(i0, q[4], "40800000");
  KMB_TAKE_IF_EQUAL(i3, q[27], "41D80000");
  KMB_TAKE_IF_EQUAL(i2, q[19], "41980000");
  KMB_TAKE_IF_EQUAL(i1, q[11], "41300000");
  KMB_TAKE_IF_EQUAL(i0, q[3], "40400000");
  KMB_TAKE_IF_EQUAL(i3, q[26], "41D00000");
  KMB_TAKE_IF_EQUAL(i2, q[18], "41900000");
  KMB_TAKE_IF_EQUAL(i1, q[10], "41200000");
  KMB_TAKE_IF_EQUAL(i0, q[2], "40000000");
  KMB_TAKE_IF_EQUAL(i3, q[25], "41C80000");
  KMB_TAKE_IF_EQUAL(i2, q[17], "41880000");
  KMB_TAKE_IF_EQUAL(i1, q[9], "41100000");
  KMB_TAKE_IF_EQUAL(i0, q[1], "3F800000");
  KMB_TAKE_IF_EQUAL(i3, q[24], "41C00000");
  KMB_TAKE_IF_EQUAL(i2, q[16], "41800000");
  KMB_TAKE_IF_EQUAL(i1, q[8], "41000000");
  KMB_TAKE_IF_EQUAL(i0, q[0], "00000000");
  out_v = (m == m) ? m : __int_as_float(0xff800000);
  out_if = fminf(fminf(i0, i1), fminf(i2, i3));
}
#undef KMB_TAKE_IF_EQUAL

// The sample side of the folded half norms: 1.0 in the two fold features, which are components
// off and off + 1 (off = fold_at mod 4 = 0, 1 or 2) of one 16-byte chunk of the row.
__device__ __forceinline__ void set_fold_ones(float4& x, int off) {
  if (off == 0) {
    x.x = 1.f;
    x.y = 1.f;
  } else if (off == 1) {
    x.y = 1.f;
    x.z = 1.f;
  } else {
    x.z = 1.f;
    x.w = 1.f;
  }
}

template <bool FOLD>
__global__ void __launch_bounds__(TC_THREADS, 1)
lloyd_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_chi,
                const __grid_constant__ CUtensorMap map_clo, TcParams p) {
  // FOLD: features fold_at and fold_at + 1 of the operands carry the half norms (see lloyd_tc_fold_at)
  const int d_eff = FOLD ? (p.fold_at + 2 > p.d ? p.fold_at + 2 : p.d) : p.d;
  const int fold_chunk = FOLD ? p.fold_at / 4 : -1;   // 16-byte chunk of a row that holds them
  const int fold_off = FOLD ? p.fold_at % 4 : 0;
  extern __shared__ unsigned char smem_raw[];
  TcSmem* sm = reinterpret_cast<TcSmem*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_kc = p.d_pad / TC_KC;
  const int n_nt = p.k_pad / TC_BN;
  const int64_t n_tiles = (p.n + TC_BM - 1) / TC_BM;
  const bool update = p.acc != nullptr;
  // rotated walk orders of this CTA
  const int nt0 = (int)(blockIdx.x % (unsigned)n_nt);
  // Rows of at most 64 (padded) features leave room for TWO sample tiles, both in the staging
  // buffers (2 atoms each) and in tensor memory (hi | lo in 64 + 64 columns each): tile t + 1 is
  // then split while the MMAs of tile t run, and the MMA warp never waits between tiles.
  const bool two_tiles = p.d_pad <= 64;
  // When all centroid stages of a sample tile fit the ring at once they are loaded ONCE per CTA
  // and stay: stage (i, j) of this CTA's walk order then lives in slot i * n_kc + j for good.
  const uint32_t n_st = (uint32_t)(n_nt * n_kc);
  const bool resident = n_st <= (uint32_t)TC_STAGES;
  const int kc0 = (int)((blockIdx.x / (unsigned)n_nt) % (unsigned)n_kc);

  if (threadIdx.x == 0) {
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sm->x_full[a], 1);
      // both worker groups split the tile when it has more than one 32-feature chunk
      mbar_init(&sm->x_conv[a], n_kc > 1 ? 8 : 4);
      mbar_init(&sm->x_stage_free[a], n_kc > 1 ? 8 : 4);
    }
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(&sm->b_full[s], 1);
      mbar_init(&sm->b_empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sm->acc_full[a], 1);
      mbar_init(&sm->acc_empty[a], 8);
      mbar_init(&sm->part_full[a], 4);
      mbar_init(&sm->lab_ready[a], 4);
      mbar_init(&sm->drain[a], 1);
    }
    sm->timeout_cycles = p.timeout_cycles;
    sm->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 2) {
    tmem_alloc(&sm->tmem_base, TC_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm->tmem_base;

  if (warp == 0) {
    // ---------------------------------------------------------------- sample tiles
    if (lane == 0) {
      uint32_t t = 0;
      for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++t) {
        const uint32_t xs = two_tiles ? (t & 1) : 0, xu = two_tiles ? (t >> 1) : t;
        if (p.test_stall != 0 && t >= 1) break;    // test hook: a sample tile that never arrives
        if (!mbar_wait(&sm->x_stage_free[xs], (xu & 1) ^ 1, sm, p.error_flag, p.sleep_ns)) break;
        mbar_expect_tx(&sm->x_full[xs], (uint32_t)n_kc * TC_ATOM_BYTES);
        for (int kc = 0; kc < n_kc; ++kc)
          tma_load_2d(sm->xstage[xs * 2 + kc], &map_x, kc * TC_KC, (int)(tile * TC_BM), &sm->x_full[xs]);
      }
      if (sm->abort_flag) drain_ring(sm->x_full, two_tiles ? 2u : 1u, t);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- centroid stages
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        if (resident && it != 0) break;     // everything is in shared memory already
        for (int i = 0; i < n_nt && ok; ++i) {
          const int nt = (nt0 + i < n_nt) ? nt0 + i : nt0 + i - n_nt;
          for (int j = 0; j < n_kc; ++j, ++it) {
            const int kc = (kc0 + j) % n_kc;
            const uint32_t s = it % TC_STAGES, u = it / TC_STAGES;
            if (!mbar_wait(&sm->b_empty[s], (u & 1) ^ 1, sm, p.error_flag, p.sleep_ns)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&sm->b_full[s], 2 * TC_ATOM_BYTES);
            tma_load_2d(sm->bhi[s], &map_chi, kc * TC_KC, nt * TC_BN, &sm->b_full[s]);
            tma_load_2d(sm->blo[s], &map_clo, kc * TC_KC, nt * TC_BN, &sm->b_full[s]);
          }
        }
      }
      if (sm->abort_flag) drain_ring(sm->b_full, (uint32_t)TC_STAGES, it);
    }
  } else if (warp < TC_EPI_WARP0) {
    // ------------------------------------------------------------------------ MMA
    // Two issuing warps: warp 2 owns accumulator 0, warp 3 accumulator 1, i.e. they take the
    // centroid tiles of a sample tile in turn.  One thread cannot prepare and issue twelve MMAs
    // per stage in the 768 cycles the tensor pipe needs for them; two can.  Counters are kept
    // by increment-and-wrap: every instruction in this loop is on the critical path.
    const uint32_t mw = (uint32_t)warp - 2u;
    const uint32_t ring = resident ? n_st : (uint32_t)TC_STAGES;
    const uint32_t lap_flip = resident ? 0u : 1u;   // resident stages complete one phase only
    const int ks_last = ((d_eff - 1) % TC_KC) / 8 + 1;   // k-steps of the last chunk that hold data
    uint32_t t = 0, g = 0, s = 0, lap = 0;
    bool ok = true;
    KMB_PROF(long long w_conv = 0, w_acc = 0, w_b = 0, t_all = clock64(), tw;)
    const uint64_t b_hi0 = make_sdesc(smem_u32(sm->bhi[0]));
    const uint64_t b_lo0 = make_sdesc(smem_u32(sm->blo[0]));
    const uint32_t d_tmem = tmem_base + TC_ACC_COL + mw * TC_BN;
    for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++t) {
      const uint32_t xs = two_tiles ? (t & 1) : 0, xu = two_tiles ? (t >> 1) : t;
      const uint32_t a_hi0 = tmem_base + (two_tiles ? xs * 128 : TC_A_HI_COL);
      const uint32_t a_lo0 = tmem_base + (two_tiles ? xs * 128 + 64 : TC_A_LO_COL);
      KMB_PROF(tw = clock64();)
      if (!__all_sync(0xffffffffu, mbar_wait(&sm->x_conv[xs], xu & 1, sm, p.error_flag, p.sleep_ns))) break;
      KMB_PROF(w_conv += clock64() - tw;)
      tc_fence_after();
      for (int i = 0; i < n_nt && ok; ++i, ++g) {
        if ((g & 1u) != mw) {                 // the other warp's centroid tile: skip its stages
          s += (uint32_t)n_kc;
          if (s >= ring) {
            s -= ring;
            lap ^= lap_flip;
          }
          continue;
        }
        KMB_PROF(tw = clock64();)
        if (!__all_sync(0xffffffffu, mbar_wait(&sm->acc_empty[mw], ((g >> 1) & 1) ^ 1, sm, p.error_flag, p.sleep_ns))) {
          ok = false;
          break;
        }
        KMB_PROF(w_acc += clock64() - tw;)
        tc_fence_after();
        int kc = kc0;
        for (int j = 0; j < n_kc; ++j) {
          KMB_PROF(tw = clock64();)
          if (!__all_sync(0xffffffffu, mbar_wait(&sm->b_full[s], lap, sm, p.error_flag, p.sleep_ns))) {
            ok = false;
            break;
          }
          KMB_PROF(w_b += clock64() - tw;)
          tc_fence_after();
          const uint64_t b_hi = b_hi0 + (uint64_t)(s * (TC_ATOM_BYTES >> 4));
          const uint64_t b_lo = b_lo0 + (uint64_t)(s * (TC_ATOM_BYTES >> 4));
          const uint32_t a_hi = a_hi0 + kc * TC_KC;
          const uint32_t a_lo = a_lo0 + kc * TC_KC;
          // k-steps whose 8 features all lie in the zero padding are skipped
          const int ks_n = (kc == n_kc - 1) ? ks_last : TC_KC / 8;
          if (elect_one()) {
#pragma unroll
            for (int ks = 0; ks < TC_KC / 8; ++ks) {
              if (ks < ks_n) {
                const uint64_t adv = (uint64_t)(ks * 2);  // 8 tf32 = 32 bytes = 2 x 16-byte units
                umma_tf32_ts(d_tmem, a_lo + ks * 8, b_hi + adv, TC_IDESC, (j | ks) != 0);
                umma_tf32_ts(d_tmem, a_hi + ks * 8, b_lo + adv, TC_IDESC, 1);
                umma_tf32_ts(d_tmem, a_hi + ks * 8, b_hi + adv, TC_IDESC, 1);
              }
            }
            if (!resident) umma_commit(&sm->b_empty[s]);
            if (j == n_kc - 1) umma_commit(&sm->acc_full[mw]);
          }
          __syncwarp();
          if (++kc == n_kc) kc = 0;
          if (++s == ring) {
            s = 0;
            lap ^= lap_flip;
          }
        }
      }
    }
    if (sm->abort_flag) mma_drain(&sm->drain[mw]);
    KMB_PROF(if (blockIdx.x == 0 && lane == 0) printf("[tc prof] mma warp %d: total %lld cyc, wait x_conv %lld, acc_empty %lld, b_full %lld, tiles %u\n", warp, clock64() - t_all, w_conv, w_acc, w_b, t);)
  } else {
    // ------------------------------------- workers: split into TMEM, argmin, centroid update
    // Two groups of four warps; warp w of a group owns TMEM lanes 32 * (w % 4) .. + 31, i.e. one
    // sample row per thread.  Both groups read every accumulator: group 0 folds columns 0..63
    // of the centroid tile, group 1 columns 64..127, so an accumulator is drained (and handed
    // back to the MMA warp) in half the time.  At the end of a sample tile group 1 passes its
    // (minimum, index) pairs through shared memory, group 0 merges them into the labels, and
    // all eight warps add the tile's rows (16 rows per warp) into the centroid sums.
    const int grp = warp >= TC_UPD_WARP0 ? 1 : 0;
    const int lane_base = (warp & 3) * 32;
    const int row = lane_base + lane;
    float* acc_copy = update ? p.acc + (int64_t)(blockIdx.x % p.n_copies) * p.acc_len : nullptr;
    uint32_t t = 0, g = 0, changed = 0;
    bool ok = true;
    // update geometry: G lanes (a power of two) of 16 bytes serve one row
    const int urow0 = (warp - TC_EPI_WARP0) * 16;     // first of the 16 rows this warp adds
    int G = 1;
    while (G * 4 < p.d) G <<= 1;
    const int rpi = 32 / G;                      // rows per warp instruction
    const int sub = lane / G;                    // which of those rows this lane serves
    const int col = (lane % G) * 4;              // first feature of this lane
    const bool col_ok = col < p.d;
    const int n_instr = (16 + rpi - 1) / rpi;

    // Splits the staged tile (row `row`, 128B-swizzled atoms) into TMEM: hi -> columns
    // [0, d_pad), lo -> [128, 128 + d_pad) of this thread's lane; with two tiles in flight tile
    // tt goes to columns (tt & 1) * 128 + [0, d_pad) and + 64 + [0, d_pad).  False on time-out.
    auto convert_tile = [&](uint32_t tt) -> bool {
      const uint32_t xs = two_tiles ? (tt & 1) : 0, xu = two_tiles ? (tt >> 1) : tt;
      const uint32_t hi_col = two_tiles ? xs * 128 : TC_A_HI_COL;
      const uint32_t lo_col = two_tiles ? xs * 128 + 64 : TC_A_LO_COL;
      if (!__all_sync(0xffffffffu, mbar_wait(&sm->x_full[xs], xu & 1, sm, p.error_flag, p.sleep_ns))) return false;
      for (int kc = 0; kc < n_kc; ++kc) {
        if (n_kc > 1 && (kc & 1) != grp) continue;     // the other group's chunk
        uint32_t hi[32], lo[32];
        const unsigned char* rowp = sm->xstage[xs * 2 + kc] + row * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float4 x = *reinterpret_cast<const float4*>(rowp + ((c ^ (row & 7)) << 4));
          if (FOLD && kc * 8 + c == fold_chunk) set_fold_ones(x, fold_off);
          // the tensor core reads the top 19 bits of each word: round the low part as well
          // instead of letting it be truncated
          const float h0 = tf32_round_alu(x.x), h1 = tf32_round_alu(x.y);
          const float h2 = tf32_round_alu(x.z), h3 = tf32_round_alu(x.w);
          float l0 = x.x - h0, l1 = x.y - h1, l2 = x.z - h2, l3 = x.w - h3;
          if (p.round_lo) {
            l0 = tf32_round_alu(l0); l1 = tf32_round_alu(l1);
            l2 = tf32_round_alu(l2); l3 = tf32_round_alu(l3);
          }
          hi[4 * c + 0] = __float_as_uint(h0); lo[4 * c + 0] = __float_as_uint(l0);
          hi[4 * c + 1] = __float_as_uint(h1); lo[4 * c + 1] = __float_as_uint(l1);
          hi[4 * c + 2] = __float_as_uint(h2); lo[4 * c + 2] = __float_as_uint(l2);
          hi[4 * c + 3] = __float_as_uint(h3); lo[4 * c + 3] = __float_as_uint(l3);
        }
        const uint32_t lane_addr = tmem_base + ((uint32_t)lane_base << 16) + kc * TC_KC;
        tmem_st32(lane_addr + hi_col, hi);
        tmem_st32(lane_addr + lo_col, lo);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&sm->x_conv[xs]);
        mbar_arrive(&sm->x_stage_free[xs]);
      }
      return true;
    };

    KMB_PROF(long long w_acc = 0, w_part = 0, w_lab = 0, c_conv = 0, c_upd = 0, t_all = clock64(), tw;)
    const bool converts = grp == 0 || n_kc > 1;
    if (converts) ok = convert_tile(0);
    for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++t) {
      const int64_t m0 = tile * TC_BM;
      const bool has_next = tile + gridDim.x < n_tiles;
      const uint32_t buf = t & 1, ub = t >> 1;
      float best = __int_as_float(0xff800000);      // scores: larger is nearer
      uint32_t bi = 0;
      // Two tiles in flight: the other tensor-memory half was last read by tile t - 1, whose
      // accumulators this warp has already consumed, so it is free now.
      // Short rows (d <= 32): the rows this warp will add into the centroid sums are fetched
      // now, so that their latency is hidden behind the epilogues instead of following them.
      const float* xbase = p.X + (m0 + urow0) * (int64_t)p.d + col;
      const bool pre = update && n_instr <= 4;
      float4 xpre[4];
      auto pre_ok = [&](int j) -> bool {
        const int r = j * rpi + sub;
        return pre && j < n_instr && r < 16 && col_ok && (m0 + urow0 + r < p.n);
      };
#pragma unroll
      for (int j = 0; j < 4; ++j)
        xpre[j] = pre_ok(j) ? __ldg(reinterpret_cast<const float4*>(xbase + (int64_t)(j * rpi + sub) * p.d))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
      KMB_PROF(tw = clock64();)
      if (converts && two_tiles && has_next && !convert_tile(t + 1)) break;
      KMB_PROF(c_conv += clock64() - tw;)
      for (int i = 0; i < n_nt && ok; ++i, ++g) {
        const uint32_t ab = g & 1, ug = g >> 1;
        const int nt_w = (nt0 + i < n_nt) ? nt0 + i : nt0 + i - n_nt;   // nt0, i < n_nt: no division
        const int cn = nt_w * TC_BN + grp * 64;   // first centroid of this half
        KMB_PROF(tw = clock64();)
        if (!__all_sync(0xffffffffu, mbar_wait(&sm->acc_full[ab], ug & 1, sm, p.error_flag, p.sleep_ns))) {
          ok = false;
          break;
        }
        KMB_PROF(w_acc += clock64() - tw;)
        tc_fence_after();
        // The last accumulator of a tile completing means every MMA of the tile has read its
        // A operand: split the next tile into TMEM first, so that the MMA warp can go on
        // while this tile's last epilogue runs.
        if (converts && !two_tiles && i == n_nt - 1 && has_next) {
          if (!convert_tile(t + 1)) {
            ok = false;
            break;
          }
        }
        const uint32_t taddr =
            tmem_base + ((uint32_t)lane_base << 16) + TC_ACC_COL + ab * TC_BN + grp * 64;
        // half norms of this half (unless folded into the contraction): same address in every
        // lane (broadcast loads), issued ahead of the tensor-memory loads so that both
        // latencies overlap
        const float4* hp = reinterpret_cast<const float4*>(p.h_pad + cn);
        float4 ha[8], hb[8];
        if (!FOLD) {
#pragma unroll
          for (int j = 0; j < 8; ++j) ha[j] = __ldg(hp + j);
        }
        uint32_t va[32], vb[32];
        tmem_ld32(taddr, va);
        tmem_ld32(taddr + 32, vb);
        tmem_ld_wait();
        // the accumulator is in registers now: hand the buffer back before the argmax
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->acc_empty[ab]);
        if (p.dots != nullptr && m0 + row < p.n) {
          float* drow = p.dots + (m0 + row) * (int64_t)p.ldd;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (cn + j < p.k) drow[cn + j] = __uint_as_float(va[j]);
            if (cn + 32 + j < p.k) drow[cn + 32 + j] = __uint_as_float(vb[j]);
          }
        }
        float qa, qb;
        uint32_t ia, ib;
        argmax32<FOLD>(va, ha, (uint32_t)cn, qa, ia);
        if (!FOLD) {
#pragma unroll
          for (int j = 0; j < 8; ++j) hb[j] = __ldg(hp + 8 + j);
        }
        argmax32<FOLD>(vb, hb, (uint32_t)(cn + 32), qb, ib);
        if (qb > qa) { qa = qb; ia = ib; }            // ascending inside the half: strict '>'
        // halves arrive in rotated order: larger score wins, equal scores -> smaller index
        if (qa > best || (qa == best && ia < bi)) {
          best = qa;
          bi = ia;
        }
      }
      if (!ok) break;

      if (grp == 1) {
        sm->part_v[row] = best;
        sm->part_i[row] = (uint16_t)bi;
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->part_full[buf]);
      } else {
        KMB_PROF(tw = clock64();)
        if (!__all_sync(0xffffffffu, mbar_wait(&sm->part_full[buf], ub & 1, sm, p.error_flag, p.sleep_ns))) break;
        KMB_PROF(w_part += clock64() - tw;)
        const float ov = sm->part_v[row];
        const uint32_t oi = sm->part_i[row];
        if (ov > best || (ov == best && oi < bi)) {
          best = ov;
          bi = oi;
        }
        if (m0 + row < p.n) {
          p.labels[m0 + row] = bi;
          if (update) changed += (p.prev == nullptr) ? 1u : (p.prev[m0 + row] != bi ? 1u : 0u);
        }
        sm->lab_s[buf][row] = (uint16_t)bi;
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->lab_ready[buf]);
      }
      // Every warp waits for the merged labels of the tile (also when nothing is updated, so
      // that group 1 never runs a whole tile ahead of group 0: part_* have one buffer, read by
      // group 0 before it arrives here).  lab_s[buf] is reused two tiles later; by then every
      // warp has passed this point of tile t + 1, which it reaches only after finishing the
      // update of tile t.
      KMB_PROF(tw = clock64();)
      if (!__all_sync(0xffffffffu, mbar_wait(&sm->lab_ready[buf], ub & 1, sm, p.error_flag, p.sleep_ns))) break;
      KMB_PROF(w_lab += clock64() - tw;)
      if (!update) continue;
      KMB_PROF(tw = clock64();)

      // ---- centroid update of rows urow0 .. urow0 + 15 of this tile
      const int my = urow0 + (lane & 15);
      const uint32_t ubi = sm->lab_s[buf][my];
      const bool uvalid = m0 + my < p.n;
      float uwi = 0.f;
      if (uvalid) uwi = p.w ? p.w[m0 + my] : 1.f;
      if (uvalid && lane < 16) atomicAdd(&acc_copy[(int64_t)p.k * p.d + ubi], uwi);
      // The tile's rows come back from L2 (they were streamed through it moments ago).  One
      // warp instruction adds 32 / G rows; eight instructions are in flight.
      if (pre) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const bool okj = pre_ok(j);
          const int src = okj ? j * rpi + sub : 0;
          const uint32_t lab = __shfl_sync(0xffffffffu, ubi, src);
          const float wr = __shfl_sync(0xffffffffu, uwi, src);
          if (okj) {
            float4 v;
            v.x = xpre[j].x * wr; v.y = xpre[j].y * wr; v.z = xpre[j].z * wr; v.w = xpre[j].w * wr;
            atomicAdd(reinterpret_cast<float4*>(acc_copy + (int64_t)lab * p.d + col), v);
          }
        }
      }
#pragma unroll 1
      for (int i0 = 0; i0 < (pre ? 0 : n_instr); i0 += 8) {
        float4 xs[8];
        bool oks[8];
        int rs[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          rs[j] = (i0 + j) * rpi + sub;                      // row of this lane, 0..15 when in range
          const bool in_range = (i0 + j) < n_instr && rs[j] < 16;
          const int src = in_range ? rs[j] : 0;
          // every lane takes part in the shuffle: it must not sit behind a short-circuit '&&'
          const int row_valid = __shfl_sync(0xffffffffu, (int)uvalid, src);
          oks[j] = in_range && col_ok && (row_valid != 0);
          xs[j] = oks[j] ? __ldg(reinterpret_cast<const float4*>(xbase + (int64_t)rs[j] * p.d))
                         : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int src = oks[j] ? rs[j] : 0;
          const uint32_t lab = __shfl_sync(0xffffffffu, ubi, src);
          const float wr = __shfl_sync(0xffffffffu, uwi, src);
          if (oks[j]) {
            float4 v;
            v.x = xs[j].x * wr; v.y = xs[j].y * wr; v.z = xs[j].z * wr; v.w = xs[j].w * wr;
            atomicAdd(reinterpret_cast<float4*>(acc_copy + (int64_t)lab * p.d + col), v);
          }
        }
      }
      KMB_PROF(c_upd += clock64() - tw;)
    }
    KMB_PROF(if (blockIdx.x == 0 && lane == 0 && (warp == TC_EPI_WARP0 || warp == TC_UPD_WARP0)) printf("[tc prof] worker warp %d: total %lld cyc, wait acc_full %lld, part_full %lld, lab_ready %lld, convert(top) %lld, update %lld, tiles %u\n", warp, clock64() - t_all, w_acc, w_part, w_lab, c_conv, c_upd, t);)
    if (update && grp == 0) {
      for (int o = 16; o > 0; o >>= 1) changed += __shfl_xor_sync(0xffffffffu, changed, o);
      if (lane == 0 && changed != 0) atomicAdd(&acc_copy[(int64_t)p.k * p.d + p.k], (float)changed);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TC_TMEM_COLS);
  }
}

// ------------------------------------------------------- the kernel for short rows
// Rows of at most 28 features (one 32-feature chunk including the two fold features).  With so
// little contraction per accumulator element the step is bound by the epilogue, not by the
// tensor pipe: per 128-row tile the MMAs need 64 cycles per k-step and centroid tile, the
// argmax about 2.5 instructions per accumulator element.  So this kernel spends its warps
// there: 20 warps, of which 16 are workers (four per scheduler).
//   warp 0       TMA producer of the sample tiles (two in flight)
//   warp 1       TMA producer of the centroid stages (resident when all of them fit)
//   warps 2, 3   issue the MMAs, one accumulator buffer each (warp 2 owns tensor memory)
//   warps 4..19  worker (lq, cq) = (warp % 4, (warp - 4) / 4): TMEM lanes 32 lq .. 32 lq + 31,
//                i.e. one sample row per thread.  It splits features 8 cq .. 8 cq + 7 of its row
//                into hi / lo parts in tensor memory (the slice that holds features d, d + 1
//                writes the ones of the folded half norms), folds columns 32 cq .. 32 cq + 31 of
//                every accumulator into a running (score, index), and adds 8 of the tile's rows
//                into the centroid sums.  Quarter 0 merges the four partial results of a row.
// Tensor memory: sample tile slot s (s = 0, 1): hi at columns 64 s, lo at 64 s + 32;
// accumulators at 256 and 384.
constexpr int TS_WARPS = 20;
constexpr int TS_THREADS = TS_WARPS * 32;
constexpr int TS_WORKER0 = 4;
constexpr int TS_WORKERS = 16;

struct TsSmem {
  unsigned char xstage[2][TC_ATOM_BYTES];
  unsigned char bhi[TC_STAGES][TC_ATOM_BYTES];
  unsigned char blo[TC_STAGES][TC_ATOM_BYTES];
  uint16_t lab_s[2][TC_BM];
  float part_v[3][TC_BM];         // quarters 1..3: best score and index per row, merged by quarter 0
  uint16_t part_i[3][TC_BM];
  unsigned long long x_full[2], x_conv[2], x_stage_free[2];
  unsigned long long b_full[TC_STAGES], b_empty[TC_STAGES];
  unsigned long long acc_full[2], acc_empty[2];
  unsigned long long part_full[2], lab_ready[2];
  unsigned long long drain[2];      // [MMA warp]: its last MMAs have completed (aborting CTA only)
  long long timeout_cycles;
  unsigned int tmem_base;
  volatile int abort_flag;
};
static_assert(sizeof(TsSmem) + 1024 <= 232448, "TsSmem exceeds the 227 KB a CTA may use");

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
      : "memory");
}

// Bounded wait on a barrier of the short-row kernel (same rule as mbar_wait).
__device__ __forceinline__ bool ts_wait(void* bar, uint32_t parity, TsSmem* sm, int* error_flag,
                                        uint32_t sleep_ns = 0u) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (sleep_ns != 0u) {
      if (mbar_try_wait_sleep(bar, parity, sleep_ns)) return true;
    } else {
      for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    }
    if (sm->abort_flag) return false;
    if (clock64() - t0 > sm->timeout_cycles) {
      sm->abort_flag = 1;
      atomicExch(error_flag, 1);
      return false;
    }
  }
}

__global__ void __launch_bounds__(TS_THREADS, 1)
lloyd_tc_small_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_chi,
                      const __grid_constant__ CUtensorMap map_clo, TcParams p) {
  extern __shared__ unsigned char smem_raw[];
  TsSmem* sm = reinterpret_cast<TsSmem*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_nt = p.k_pad / TC_BN;
  const int64_t n_tiles = (p.n + TC_BM - 1) / TC_BM;
  const bool update = p.acc != nullptr;
  const int nt0 = (int)(blockIdx.x % (unsigned)n_nt);
  const bool resident = n_nt <= TC_STAGES;
  const int d_eff = p.fold_at + 2 > p.d ? p.fold_at + 2 : p.d;   // data features and the two fold features
  const int n_ks = (d_eff + 7) / 8;                // k-steps (of 8 features) that hold data: 1..4
  const int fold_chunk = p.fold_at / 4;            // 16-byte chunk of a row holding the fold features
  const int fold_off = p.fold_at % 4;

  if (threadIdx.x == 0) {
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sm->x_full[a], 1);
      mbar_init(&sm->x_conv[a], 4 * n_ks);         // one arrival per converting warp
      mbar_init(&sm->x_stage_free[a], 4 * n_ks);
      mbar_init(&sm->acc_full[a], 1);
      mbar_init(&sm->acc_empty[a], TS_WORKERS);
      mbar_init(&sm->part_full[a], 12);
      mbar_init(&sm->lab_ready[a], 4);
      mbar_init(&sm->drain[a], 1);
    }
    sm->timeout_cycles = p.timeout_cycles;
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(&sm->b_full[s], 1);
      mbar_init(&sm->b_empty[s], 1);
    }
    sm->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 2) {
    tmem_alloc(&sm->tmem_base, TC_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm->tmem_base;

  if (warp == 0) {
    // ---------------------------------------------------------------- sample tiles
    if (lane == 0) {
      uint32_t t = 0;
      for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++t) {
        const uint32_t xs = t & 1, xu = t >> 1;
        if (p.test_stall != 0 && t >= 1) break;    // test hook: a sample tile that never arrives
        if (!ts_wait(&sm->x_stage_free[xs], (xu & 1) ^ 1, sm, p.error_flag, p.sleep_ns)) break;
        mbar_expect_tx(&sm->x_full[xs], TC_ATOM_BYTES);
        tma_load_2d(sm->xstage[xs], &map_x, 0, (int)(tile * TC_BM), &sm->x_full[xs]);
      }
      if (sm->abort_flag) drain_ring(sm->x_full, 2u, t);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- centroid stages
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        if (resident && it != 0) break;            // everything is in shared memory already
        for (int i = 0; i < n_nt; ++i, ++it) {
          const int nt = (nt0 + i < n_nt) ? nt0 + i : nt0 + i - n_nt;
          const uint32_t s = it % TC_STAGES, u = it / TC_STAGES;
          if (!ts_wait(&sm->b_empty[s], (u & 1) ^ 1, sm, p.error_flag, p.sleep_ns)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&sm->b_full[s], 2 * TC_ATOM_BYTES);
          tma_load_2d(sm->bhi[s], &map_chi, 0, nt * TC_BN, &sm->b_full[s]);
          tma_load_2d(sm->blo[s], &map_clo, 0, nt * TC_BN, &sm->b_full[s]);
        }
      }
      if (sm->abort_flag) drain_ring(sm->b_full, (uint32_t)TC_STAGES, it);
    }
  } else if (warp < TS_WORKER0) {
    // ------------------------------------------------------------------------ MMA
    const uint32_t mw = (uint32_t)warp - 2u;
    const uint32_t ring = resident ? (uint32_t)n_nt : (uint32_t)TC_STAGES;
    const uint32_t lap_flip = resident ? 0u : 1u;
    uint32_t t = 0, g = 0, s = 0, lap = 0;
    bool ok = true;
    const uint64_t b_hi0 = make_sdesc(smem_u32(sm->bhi[0]));
    const uint64_t b_lo0 = make_sdesc(smem_u32(sm->blo[0]));
    const uint32_t d_tmem = tmem_base + TC_ACC_COL + mw * TC_BN;
    for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++t) {
      const uint32_t xs = t & 1, xu = t >> 1;
      const uint32_t a_hi = tmem_base + xs * 64, a_lo = a_hi + 32;
      if (!__all_sync(0xffffffffu, ts_wait(&sm->x_conv[xs], xu & 1, sm, p.error_flag, p.sleep_ns))) break;
      tc_fence_after();
      for (int i = 0; i < n_nt && ok; ++i, ++g) {
        if ((g & 1u) == mw) {
          if (!__all_sync(0xffffffffu, ts_wait(&sm->acc_empty[mw], ((g >> 1) & 1) ^ 1, sm, p.error_flag, p.sleep_ns)) ||
              !__all_sync(0xffffffffu, ts_wait(&sm->b_full[s], lap, sm, p.error_flag, p.sleep_ns))) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t b_hi = b_hi0 + (uint64_t)(s * (TC_ATOM_BYTES >> 4));
          const uint64_t b_lo = b_lo0 + (uint64_t)(s * (TC_ATOM_BYTES >> 4));
          if (elect_one()) {
#pragma unroll
            for (int ks = 0; ks < TC_KC / 8; ++ks) {
              if (ks < n_ks) {
                const uint64_t adv = (uint64_t)(ks * 2);
                umma_tf32_ts(d_tmem, a_lo + ks * 8, b_hi + adv, TC_IDESC, ks != 0);
                umma_tf32_ts(d_tmem, a_hi + ks * 8, b_lo + adv, TC_IDESC, 1);
                umma_tf32_ts(d_tmem, a_hi + ks * 8, b_hi + adv, TC_IDESC, 1);
              }
            }
            if (!resident) umma_commit(&sm->b_empty[s]);
            umma_commit(&sm->acc_full[mw]);
          }
          __syncwarp();
        }
        if (++s == ring) {
          s = 0;
          lap ^= lap_flip;
        }
      }
    }
    if (sm->abort_flag) mma_drain(&sm->drain[mw]);
  } else {
    // -------------------------------------------------------------------- workers
    const int wk = warp - TS_WORKER0;
    const int lq = warp & 3, cq = wk >> 2;
    const int lane_base = lq * 32;
    const int row = lane_base + lane;
    const bool converts = cq < n_ks;
    float* acc_copy = update ? p.acc + (int64_t)(blockIdx.x % p.n_copies) * p.acc_len : nullptr;
    uint32_t t = 0, g = 0, changed = 0;
    bool ok = true;
    // update geometry: G lanes (a power of two) of 16 bytes serve one row; a warp adds 8 rows
    const int urow0 = wk * 8;
    int G = 1;
    while (G * 4 < p.d) G <<= 1;
    const int rpi = 32 / G;                        // rows per warp instruction: 4 .. 32
    const int sub = lane / G;
    const int col = (lane % G) * 4;
    const bool col_ok = col < p.d;
    const int n_instr = (8 + rpi - 1) / rpi;       // 1 or 2

    auto convert_tile = [&](uint32_t tt) -> bool {
      const uint32_t xs = tt & 1, xu = tt >> 1;
      if (!__all_sync(0xffffffffu, ts_wait(&sm->x_full[xs], xu & 1, sm, p.error_flag, p.sleep_ns))) return false;
      uint32_t hi[8], lo[8];
      const unsigned char* rowp = sm->xstage[xs] + row * 128;
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        const int c = cq * 2 + c2;
        float4 x = *reinterpret_cast<const float4*>(rowp + ((c ^ (row & 7)) << 4));
        if (c == fold_chunk) set_fold_ones(x, fold_off);
        const float h0 = tf32_round_alu(x.x), h1 = tf32_round_alu(x.y);
        const float h2 = tf32_round_alu(x.z), h3 = tf32_round_alu(x.w);
        hi[4 * c2 + 0] = __float_as_uint(h0); lo[4 * c2 + 0] = __float_as_uint(tf32_round_alu(x.x - h0));
        hi[4 * c2 + 1] = __float_as_uint(h1); lo[4 * c2 + 1] = __float_as_uint(tf32_round_alu(x.y - h1));
        hi[4 * c2 + 2] = __float_as_uint(h2); lo[4 * c2 + 2] = __float_as_uint(tf32_round_alu(x.z - h2));
        hi[4 * c2 + 3] = __float_as_uint(h3); lo[4 * c2 + 3] = __float_as_uint(tf32_round_alu(x.w - h3));
      }
      const uint32_t lane_addr = tmem_base + ((uint32_t)lane_base << 16) + xs * 64 + cq * 8;
      tmem_st8(lane_addr, hi);
      tmem_st8(lane_addr + 32, lo);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&sm->x_conv[xs]);
        mbar_arrive(&sm->x_stage_free[xs]);
      }
      return true;
    };

    KMB_PROF(long long c_conv = 0, w_acc = 0, c_arg = 0, w_part = 0, w_lab = 0, c_upd = 0, t_all = clock64(), tw;)
    if (converts) ok = convert_tile(0);
    for (int64_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++t) {
      const int64_t m0 = tile * TC_BM;
      const bool has_next = tile + gridDim.x < n_tiles;
      const uint32_t buf = t & 1, ub = t >> 1;
      float best = __int_as_float(0xff800000);
      uint32_t bi = 0;
      // previous label of this thread's row: fetched now, compared once the new one is known
      uint32_t prev_lab = 0xffffffffu;
      if (update && cq == 0 && p.prev != nullptr && m0 + row < p.n) prev_lab = __ldg(p.prev + m0 + row);
      // the rows this warp will add into the centroid sums are fetched now, so that their
      // latency hides behind the epilogues
      const float* xbase = p.X + (m0 + urow0) * (int64_t)p.d + col;
      float4 xpre[2];
      auto pre_ok = [&](int j) -> bool {
        const int r = j * rpi + sub;
        return update && j < n_instr && r < 8 && col_ok && (m0 + urow0 + r < p.n);
      };
#pragma unroll
      for (int j = 0; j < 2; ++j)
        xpre[j] = pre_ok(j) ? __ldg(reinterpret_cast<const float4*>(xbase + (int64_t)(j * rpi + sub) * p.d))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
      // the other tensor-memory slot was last read by the MMAs of tile t - 1, all of whose
      // accumulators this warp has consumed: it is free for tile t + 1
      KMB_PROF(tw = clock64();)
      if (converts && has_next && !convert_tile(t + 1)) break;
      KMB_PROF(c_conv += clock64() - tw;)
      for (int i = 0; i < n_nt; ++i, ++g) {
        const uint32_t ab = g & 1, ug = g >> 1;
        const int nt_w = (nt0 + i < n_nt) ? nt0 + i : nt0 + i - n_nt;   // nt0, i < n_nt: no division
        const int cn = nt_w * TC_BN + cq * 32;
        KMB_PROF(tw = clock64();)
        if (!__all_sync(0xffffffffu, ts_wait(&sm->acc_full[ab], ug & 1, sm, p.error_flag, p.sleep_ns))) {
          ok = false;
          break;
        }
        KMB_PROF(w_acc += clock64() - tw; tw = clock64();)
        tc_fence_after();
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)lane_base << 16) + TC_ACC_COL + ab * TC_BN + cq * 32, v);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->acc_empty[ab]);
        float qa;
        uint32_t ia;
        const float4 unused[8] = {};
        argmax32<true>(v, unused, (uint32_t)cn, qa, ia);
        // centroid tiles arrive in rotated order: larger score wins, equal scores -> smaller index
        if (qa > best || (qa == best && ia < bi)) {
          best = qa;
          bi = ia;
        }
        KMB_PROF(c_arg += clock64() - tw;)
      }
      if (!ok) break;

      if (cq != 0) {
        sm->part_v[cq - 1][row] = best;
        sm->part_i[cq - 1][row] = (uint16_t)bi;
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->part_full[buf]);
      } else {
        KMB_PROF(tw = clock64();)
        if (!__all_sync(0xffffffffu, ts_wait(&sm->part_full[buf], ub & 1, sm, p.error_flag, p.sleep_ns))) break;
        KMB_PROF(w_part += clock64() - tw;)
#pragma unroll
        for (int q = 0; q < 3; ++q) {
          const float ov = sm->part_v[q][row];
          const uint32_t oi = sm->part_i[q][row];
          if (ov > best || (ov == best && oi < bi)) {
            best = ov;
            bi = oi;
          }
        }
        sm->lab_s[buf][row] = (uint16_t)bi;
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->lab_ready[buf]);
        if (m0 + row < p.n) {
          p.labels[m0 + row] = bi;
          if (update) changed += (prev_lab != bi) ? 1u : 0u;
        }
      }
      // Every warp waits for the merged labels (also when nothing is updated): part_* have one
      // buffer, which quarter 0 has read before it arrives here, so no quarter can overwrite
      // it a tile early.  lab_s[buf] is reused two tiles later; by then every warp has passed
      // this point of tile t + 1, which it reaches only after finishing the update of tile t.
      KMB_PROF(tw = clock64();)
      if (!__all_sync(0xffffffffu, ts_wait(&sm->lab_ready[buf], ub & 1, sm, p.error_flag, p.sleep_ns))) break;
      KMB_PROF(w_lab += clock64() - tw;)
      if (!update) continue;
      KMB_PROF(tw = clock64();)

      // ---- centroid update of rows urow0 .. urow0 + 7 of this tile
      const int my = urow0 + (lane & 7);
      const uint32_t ubi = sm->lab_s[buf][my];
      const bool uvalid = m0 + my < p.n;
      float uwi = 0.f;
      if (uvalid) uwi = p.w ? p.w[m0 + my] : 1.f;
      if (uvalid && lane < 8) atomicAdd(&acc_copy[(int64_t)p.k * p.d + ubi], uwi);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const bool okj = pre_ok(j);
        const int src = okj ? j * rpi + sub : 0;
        const uint32_t lab = __shfl_sync(0xffffffffu, ubi, src);
        const float wr = __shfl_sync(0xffffffffu, uwi, src);
        if (okj) {
          float4 u;
          u.x = xpre[j].x * wr; u.y = xpre[j].y * wr; u.z = xpre[j].z * wr; u.w = xpre[j].w * wr;
          atomicAdd(reinterpret_cast<float4*>(acc_copy + (int64_t)lab * p.d + col), u);
        }
      }
      KMB_PROF(c_upd += clock64() - tw;)
    }
    KMB_PROF(if (blockIdx.x == 0 && lane == 0 && (warp & 3) == 0) printf("[ts prof] worker warp %d (cq %d): total %lld cyc, convert %lld, wait acc_full %lld, ld+argmax %lld, wait part %lld, wait labels %lld, update %lld, tiles %u\n", warp, cq, clock64() - t_all, c_conv, w_acc, c_arg, w_part, w_lab, c_upd, t);)
    if (update && cq == 0) {
      for (int o = 16; o > 0; o >>= 1) changed += __shfl_xor_sync(0xffffffffu, changed, o);
      if (lane == 0 && changed != 0) atomicAdd(&acc_copy[(int64_t)p.k * p.d + p.k], (float)changed);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TC_TMEM_COLS);
  }
}

}  // namespace kmb

#include "lloyd_tc_quads.cuh"
#include "lloyd_tc_quads_ss.cuh"

namespace kmb {

static int tc_env_int(const char* name, int dflt) {
  const char* e = getenv(name);
  return e != nullptr ? atoi(e) : dflt;
}

// KMB_TC_SLEEP_NS=<n> in the environment makes the barrier waits sleep up to n ns between
// polls (A/B runs); the default polls without sleeping.
static uint32_t tc_sleep_ns() {
  static long cached = -1;
  if (cached < 0) {
    const char* e = getenv("KMB_TC_SLEEP_NS");
    cached = (e != nullptr) ? atol(e) : 0;
    if (cached < 0) cached = 0;
  }
  return (uint32_t)cached;
}

// Which kernel takes short rows: the four-quad kernel (default, KMB_TC_SMALL=3); 0 selects the
// general kernel, 1 the sixteen-worker kernel (A/B runs: on n = 5 M, d = 14, k = 256 they
// measured 0.37 ms, 0.77 ms and 0.56 ms per step).
static int tc_small_mode() {
  static int cached = -1;
  if (cached < 0) {
    const char* e = getenv("KMB_TC_SMALL");
    cached = (e == nullptr) ? 3 : ((e[0] == '0' || e[0] == '1') ? e[0] - '0' : 3);
  }
  return cached;
}

// Centroids -> zero-padded hi / lo parts (both rounded to tf32) and +inf-padded half norms.
// With fold_at >= 0 the features fold_at and fold_at + 1 carry -h (see lloyd_tc_fold_at); padding
// centroids get a NaN there, so that their scores are NaN and never win.
__global__ void tc_split_centroids_kernel(const float* __restrict__ C, const float* __restrict__ h,
                                          float* __restrict__ chi, float* __restrict__ clo,
                                          float* __restrict__ h_pad, int k, int d, int k_pad,
                                          int d_pad, int fold_at) {
  const int64_t total = (int64_t)k_pad * d_pad;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (int64_t)gridDim.x * blockDim.x) {
    const int j = (int)(e / d_pad), f = (int)(e % d_pad);
    float hi = 0.f, lo = 0.f;
    if (fold_at >= 0 && (f == fold_at || f == fold_at + 1)) {
      // the fold features: after the data, or in the caller's zero padding inside the rows
      if (j < k) {
        float fhi[2], flo[2];
        lloyd_tc_fold_values(h[j], fhi, flo);
        hi = fhi[f - fold_at];
        lo = flo[f - fold_at];
      } else if (f == fold_at) {
        hi = __int_as_float(0x7fc00000);
      }
    } else if (j < k && f < d) {
      const float c = C[(int64_t)j * d + f];
      hi = tf32_rna(c);
      lo = tf32_rna(c - hi);
    }
    chi[e] = hi;
    clo[e] = lo;
    if (f == 0) h_pad[j] = (j < k && h != nullptr) ? h[j] : (j < k ? 0.f : __int_as_float(0x7f800000));
  }
}

// ------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  }
  return fn;
}

// (rows, cols) fp32 row-major tensor with row stride ld (elements); box = 32 cols x 128 rows.
static int make_map(CUtensorMap* map, const float* base, int64_t rows, int cols, int64_t ld) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return KMB_ERR_CUDA;
  }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
  cuuint32_t box[2] = {(cuuint32_t)TC_KC, (cuuint32_t)TC_BM};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld cols=%d ld=%lld)", (int)r,
              (long long)rows, cols, (long long)ld);
    return KMB_ERR_CUDA;
  }
  return KMB_OK;
}

static inline int round_up(int v, int m) { return (v + m - 1) / m * m; }

bool lloyd_tc_supported(int dtype, int64_t n, int d, int k) {
  return dtype == KMB_F32 && n >= 0 && n < (1ll << 31) - TC_BM && d >= 4 && d % 4 == 0 &&
         d <= TC_MAX_D && k >= 1 && k <= 65536;
}

bool lloyd_tc_preferred(int dtype, int64_t n, int d, int k) {
  // Measured on B200: with k >= 128 and tens of thousands of samples the tensor-core step
  // wins even at d = 16 (n=5M, d=14 padded to 16, k=256: 0.84 ms against 1.61 ms on the CUDA
  // cores); for small problems its fixed cost per launch and per 128-row tile loses
  // (n=50k, k=127: 52 us against 32 us).
  return lloyd_tc_supported(dtype, n, d, k) && d >= 8 && k >= 128 && n >= 32768;
}

int lloyd_tc_acc_copies(int, int) { return 16; }

static int tc_launch(const float* X, const float* w, const float* C, const float* h,
                     const uint32_t* prev, uint32_t* labels, float* acc, int n_copies,
                     int64_t acc_len, float* dots, int ldd, int64_t n, int d, int k, int pad,
                     bool operands_ready, void* workspace, size_t workspace_bytes,
                     cudaStream_t stream) {
  KMB_REQUIRE(lloyd_tc_supported(KMB_F32, n, d, k), "tcgen05 step: unsupported shape n=%lld d=%d k=%d",
              (long long)n, d, k);
  KMB_REQUIRE(((uintptr_t)X & 15) == 0 && ((uintptr_t)C & 15) == 0,
              "tcgen05 step: X and C must be 16-byte aligned");
  KMB_REQUIRE(acc == nullptr || ((uintptr_t)acc & 15) == 0, "tcgen05 step: acc must be 16-byte aligned");
  const int d_pad = round_up(d, TC_KC), k_pad = round_up(k, TC_BN);
  KMB_REQUIRE(workspace != nullptr, "tcgen05 step: workspace is NULL");
  LloydWorkspace ws = lloyd_carve(workspace, d, k);
  if (ws.bytes > workspace_bytes) {
    set_error("tcgen05 step: workspace of %zu bytes needed, %zu given", ws.bytes, workspace_bytes);
    return KMB_ERR_WORKSPACE;
  }
  // The time-out flag in the control block is sticky: only kmb_lloyd_workspace_init clears it.
  // The raw-product hook (dots) must see plain dot products, so it never folds.
  const int fold_at = (dots == nullptr && h != nullptr) ? lloyd_tc_fold_at(d, pad) : -1;
  const bool fold = fold_at >= 0;
  if (!operands_ready) {
    const int64_t total = (int64_t)k_pad * d_pad;
    int grid = (int)ceil_div(total, 256);
    if (grid > 1184) grid = 1184;
    tc_split_centroids_kernel<<<grid, 256, 0, stream>>>(C, h, ws.chi, ws.clo, ws.h_pad, k, d, k_pad,
                                                        d_pad, fold_at);
    KMB_CHECK_LAUNCH();
  }
  CUtensorMap map_x, map_chi, map_clo;
  int rc;
  if ((rc = make_map(&map_x, X, n, d, d)) != KMB_OK) return rc;
  if ((rc = make_map(&map_chi, ws.chi, k_pad, d_pad, d_pad)) != KMB_OK) return rc;
  if ((rc = make_map(&map_clo, ws.clo, k_pad, d_pad, d_pad)) != KMB_OK) return rc;

  TcParams p;
  p.X = X; p.w = w; p.h_pad = ws.h_pad; p.prev = prev; p.labels = labels; p.acc = acc;
  p.dots = dots; p.error_flag = &ws.ctl->wait_error; p.acc_len = acc_len; p.n = n; p.ldd = ldd;
  p.n_copies = n_copies; p.d = d; p.d_pad = d_pad; p.k = k; p.k_pad = k_pad;
  p.sleep_ns = tc_sleep_ns();
  p.round_lo = tc_env_int("KMB_TC_ROUND_LO", 1);
  p.acc_bufs = tc_env_int("KMB_TQ_ACC", 3);
  p.mma_warps = tc_env_int("KMB_TQ_MMA", TQ_MMA_WARPS);
  if (p.mma_warps != 1) p.mma_warps = TQ_MMA_WARPS;
  p.fone = 1.0f;
  p.fold_at = fold_at;
  // KMB_TC_TIMEOUT_MS: limit of every barrier wait (default 2 s at 2 GHz); KMB_TC_TEST_STALL=1
  // makes every CTA's sample-tile producer stop after its first tile, which is how the tests make
  // a wait run out without faulting anything.
  const int timeout_ms = tc_env_int("KMB_TC_TIMEOUT_MS", 0);
  p.timeout_cycles = timeout_ms > 0 ? (long long)timeout_ms * 2000000LL : TC_TIMEOUT_CYCLES;
  p.test_stall = tc_env_int("KMB_TC_TEST_STALL", 0);

  const int64_t n_tiles = ceil_div(n, TC_BM);
  int64_t grid = sm_count();
  if (grid > n_tiles) grid = n_tiles;
  if (fold && d_pad == TC_KC && tc_small_mode() == 3 && (fold_at + 2 > d ? fold_at + 2 : d) <= 16 &&
      k_pad / TC_BN <= TS2_STAGES && tc_env_int("KMB_TQ_SS", 0) != 0) {
    // KMB_TQ_SS=1: rows of at most 16 contraction features with all centroid stages resident go
    // to the kernel that reads the sample operand from shared memory (two sample stages per
    // quad); it measured 2 % slower than the kernel below
    const size_t smem = sizeof(Ts2Smem) + 1024;
    KMB_CHECK_CUDA(cudaFuncSetAttribute(lloyd_tc_quads_ss_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
    lloyd_tc_quads_ss_kernel<<<(unsigned)grid, tq_threads(4), smem, stream>>>(map_x, map_chi, map_clo, p);
    KMB_CHECK_LAUNCH();
    return KMB_OK;
  }
  if (fold && d_pad == TC_KC && tc_small_mode() == 3) {
    // short rows: four quads, each owning whole sample tiles
    const size_t smem = sizeof(TqSmem) + 1024;
    // KMB_TQ_FIDX=0 keeps the whole index search on the integer pipe (A/B runs)
    const bool fidx = tc_env_int("KMB_TQ_FIDX", 1) != 0;
    auto kern = fidx ? lloyd_tc_quads_kernel<true, 4> : lloyd_tc_quads_kernel<false, 4>;
    KMB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<(unsigned)grid, tq_threads(4), smem, stream>>>(map_x, map_chi, map_clo, p);
    KMB_CHECK_LAUNCH();
    return KMB_OK;
  }
  if (fold && d_pad == TC_KC && tc_small_mode() == 1) {
    // short rows: the kernel with sixteen epilogue warps on every tile
    const size_t smem = sizeof(TsSmem) + 1024;
    KMB_CHECK_CUDA(cudaFuncSetAttribute(lloyd_tc_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
    lloyd_tc_small_kernel<<<(unsigned)grid, TS_THREADS, smem, stream>>>(map_x, map_chi, map_clo, p);
    KMB_CHECK_LAUNCH();
    return KMB_OK;
  }
  const size_t smem = sizeof(TcSmem) + 1024;
  if (fold) {
    KMB_CHECK_CUDA(cudaFuncSetAttribute(lloyd_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
    lloyd_tc_kernel<true><<<(unsigned)grid, TC_THREADS, smem, stream>>>(map_x, map_chi, map_clo, p);
  } else {
    KMB_CHECK_CUDA(cudaFuncSetAttribute(lloyd_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)smem));
    lloyd_tc_kernel<false><<<(unsigned)grid, TC_THREADS, smem, stream>>>(map_x, map_chi, map_clo, p);
  }
  KMB_CHECK_LAUNCH();
  return KMB_OK;
}

int lloyd_tc_run(const float* X, const float* w, const float* C, const float* h,
                 const uint32_t* prev, uint32_t* labels, float* acc, int n_copies, int64_t acc_len,
                 int64_t n, int d, int k, int pad, bool update, bool operands_ready, void* workspace,
                 size_t workspace_bytes, cudaStream_t stream) {
  return tc_launch(X, w, C, h, prev, labels, update ? acc : nullptr, n_copies, acc_len, nullptr, 0, n,
                   d, k, pad, operands_ready, workspace, workspace_bytes, stream);
}

// out[i, j] = X[i, :] . Y[j, :] with the 3xTF32 pipeline; labels go to scratch in the workspace.
int lloyd_tc_matmul(const float* X, const float* Y, float* out, int64_t m, int n, int kdim,
                    void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  LloydWorkspace ws = lloyd_carve(workspace, kdim, n);
  const size_t lab_bytes = ((size_t)m * sizeof(uint32_t) + 255) / 256 * 256;
  if (workspace == nullptr || ws.bytes + lab_bytes > workspace_bytes) {
    set_error("kmb_matmul_nt: workspace of %zu bytes needed, %zu given", ws.bytes + lab_bytes,
              workspace_bytes);
    return KMB_ERR_WORKSPACE;
  }
  uint32_t* labels = (uint32_t*)((unsigned char*)workspace + ws.bytes);
  return tc_launch(X, nullptr, Y, nullptr, nullptr, labels, nullptr, 1, 0, out, n, m, kdim, n, 0, false,
                   workspace, workspace_bytes, stream);
}

}  // namespace kmb
