// Short-row form of the tensor-core Lloyd step in which every sample tile belongs to ONE quad of
// warps from start to finish.  Included by lloyd_tc.cu (PTX wrappers, TcParams, argmax32).
//
// Rows of at most 28 features (one 32-feature chunk including the two fold features, see
// lloyd_tc_folds).  At this size the step is bound by the instructions of the epilogue warps, and
// two thirds of those are per-tile bookkeeping that EVERY warp touching a tile repeats (barrier
// waits, tensor-memory loads, label exchange, update addressing).  Here only four warps touch a
// tile, and they never talk to each other:
//   warp 0        TMA producer of the sample tiles (one slot per quad)
//   warp 1        TMA producer of the centroid stages (resident when all of them fit)
//   warps 2, 3    issue the MMAs in tile order, alternate accumulators each (TQ_MMA_WARPS; four
//                 issuing warps measured 4 % faster by themselves, but 22 warps leave 88
//                 registers per thread instead of 96 and the argmax then loses 13 %)
//   warps 4 + 4 Q .. 7 + 4 Q   quad Q (Q = 0..3) owns the CTA's tiles t with t mod 4 = Q.  Warp lq of a
//                 quad owns TMEM lanes 32 lq .. 32 lq + 31, i.e. ONE THREAD OWNS ONE SAMPLE ROW of
//                 the tile: it splits the row into hi / lo parts in the quad's tensor-memory slot,
//                 reduces ALL columns of every accumulator of the tile (32 at a time) to its
//                 (score, index), writes the label, and adds its own row into the centroid sums
//                 with 16-byte vector reductions.  No partial results, no label exchange.
// Four tiles are in flight, one per quad, each at a different stage (split, MMA, argmax, update),
// so the quads hide each other's latencies and spread the argmax bursts over time.
// Tensor memory (512 columns): the sample slot of quad Q holds the hi part and then the lo part
// of its tile, 8 columns per k-step each.  Rows of at most 16 features (two k-steps) need 32
// columns per quad, which leaves room for THREE 128-column accumulators behind the slots; longer
// rows take 64 columns per quad and two accumulators.  The accumulators are used in turn by the
// CTA-wide sequence g = 0, 1, 2, ... of (tile, centroid tile) pairs: buffer g mod n_acc.
#pragma once

namespace kmb {

constexpr int TQ_MMA_WARPS = 2;     // the issuing loops assume one or two warps (parity of g)
constexpr int TQ_WORKER0 = 2 + TQ_MMA_WARPS;
constexpr int TQ_MAX_QUADS = 4;
constexpr int tq_threads(int nq) { return (TQ_WORKER0 + 4 * nq) * 32; }
constexpr int TQ_STAGES = 4;        // centroid stages (hi + lo = 32 KB each)

struct TqSmem {
  unsigned char xstage[TQ_MAX_QUADS][TC_ATOM_BYTES];          // [quad]
  unsigned char bhi[TQ_STAGES][TC_ATOM_BYTES];
  unsigned char blo[TQ_STAGES][TC_ATOM_BYTES];
  unsigned long long x_full[TQ_MAX_QUADS], x_conv[TQ_MAX_QUADS], x_stage_free[TQ_MAX_QUADS];   // [quad]
  // [quad][buffer]: an accumulator of the quad's tile is complete.  One barrier per quad AND buffer:
  // a waiter may be at most one phase ahead of its barrier, which holds for the accumulators of
  // one quad (consumed in order) but not for a barrier shared by quads working on different tiles.
  unsigned long long acc_full[TQ_MAX_QUADS][3];
  // [buffer][MMA warp that fills it next]: its four readers have it in registers
  unsigned long long acc_empty[3][TQ_MMA_WARPS];
  unsigned long long b_full[TQ_STAGES], b_empty[TQ_STAGES];
  unsigned long long drain[TQ_MMA_WARPS];          // [MMA warp]: its last MMAs have completed (aborting CTA only)
  long long timeout_cycles;
  unsigned int tmem_base;
  volatile int abort_flag;
  KMB_PROF(long long ts[16];)                      // time line of one tile (profiling build)
};
static_assert(sizeof(TqSmem) + 1024 <= 232448, "TqSmem exceeds the 227 KB a CTA may use");

// Bounded wait on a barrier of this kernel (same rule as mbar_wait).
__device__ __forceinline__ bool tq_wait(void* bar, uint32_t parity, TqSmem* sm, int* error_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (sm->abort_flag) return false;
    if (clock64() - t0 > sm->timeout_cycles) {
      sm->abort_flag = 1;
      atomicExch(error_flag, 1);
      return false;
    }
  }
}

// Profiling build: time stamps of CTA 0's tile TQ_PROBE_TILE (a tile of quad 0).
#define TQ_PROBE_TILE 40
#define TQ_STAMP(cond, slot) KMB_PROF(if (blockIdx.x == 0 && lane == 0 && (cond)) sm->ts[slot] = clock64();)
// FIDX: search the index of the maximum on the FMA pipe (see argmax32_fidx).  NQ: quads of worker
// warps = sample tiles in flight (4; five, which fit when the rows need at most two k-steps,
// measured 9 % slower).  Keeping the rows in shared memory from the split to the update instead
// of fetching them again from L2 measured no gain either: the update's time is its reductions.
template <bool FIDX, int NQ>
__global__ void __launch_bounds__(tq_threads(NQ), 1)
lloyd_tc_quads_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_chi,
                      const __grid_constant__ CUtensorMap map_clo, TcParams p) {
  extern __shared__ unsigned char smem_raw[];
  TqSmem* sm = reinterpret_cast<TqSmem*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_nt = p.k_pad / TC_BN;
  // n < 2^31 - 128 (checked by the host), so tile and row indices fit 32 bits
  const int n_tiles = (int)((p.n + TC_BM - 1) / TC_BM);
  const int my_tiles = (n_tiles > (int)blockIdx.x) ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const bool update = p.acc != nullptr;
  const int nt0 = (int)(blockIdx.x % (unsigned)n_nt);
  const bool resident = n_nt <= TQ_STAGES;
  const int d_eff = p.fold_at + 2 > p.d ? p.fold_at + 2 : p.d;   // data features and the two fold features
  const int n_ks = (d_eff + 7) / 8;                // k-steps / 8-feature slices that hold data: 1..4
  const int fold_chunk = p.fold_at / 4;            // 16-byte chunk of a row holding the fold features
  const int fold_off = p.fold_at % 4;
  // tensor-memory layout (see the head of this file)
  const uint32_t half_cols = (n_ks <= 2) ? 16u : 32u;          // columns of the hi (or lo) part of a slot
  const uint32_t acc_col0 = (uint32_t)NQ * 2u * half_cols;     // NQ slots of 2 * half_cols columns
  const uint32_t n_acc = (acc_col0 + 3u * TC_BN <= (uint32_t)TC_TMEM_COLS && p.acc_bufs >= 3) ? 3u : 2u;

  if (threadIdx.x == 0) {
    for (int a = 0; a < NQ; ++a) {
      mbar_init(&sm->x_full[a], 1);
      mbar_init(&sm->x_conv[a], 4);
      mbar_init(&sm->x_stage_free[a], 4);
    }
    for (int a = 0; a < 3; ++a) {
      for (int q = 0; q < NQ; ++q) mbar_init(&sm->acc_full[q][a], 1);
      for (int w = 0; w < TQ_MMA_WARPS; ++w) mbar_init(&sm->acc_empty[a][w], 4);
    }
    for (int s = 0; s < TQ_STAGES; ++s) {
      mbar_init(&sm->b_full[s], 1);
      mbar_init(&sm->b_empty[s], 1);
    }
    for (int w = 0; w < TQ_MMA_WARPS; ++w) mbar_init(&sm->drain[w], 1);
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

  // CTA-local tile t (global tile blockIdx.x + t * gridDim.x) belongs to quad t mod NQ and is the
  // (t / NQ)-th tile of that quad.
  if (warp == 0) {
    // ---------------------------------------------------------------- sample tiles
    if (lane == 0) {
      int t = 0;
      for (; t < my_tiles; ++t) {
        const int q = t % NQ;
        if (p.test_stall != 0 && t >= 1) break;    // test hook: a sample tile that never arrives
        if (!tq_wait(&sm->x_stage_free[q], ((uint32_t)(t / NQ) & 1u) ^ 1u, sm, p.error_flag)) break;
        mbar_expect_tx(&sm->x_full[q], TC_ATOM_BYTES);
        tma_load_2d(sm->xstage[q], &map_x, 0, ((int)blockIdx.x + t * (int)gridDim.x) * TC_BM, &sm->x_full[q]);
      }
      if (sm->abort_flag) drain_ring(sm->x_full, (uint32_t)NQ, (uint32_t)t);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- centroid stages
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = 0; t < my_tiles && ok; ++t) {
        if (resident && t != 0) break;             // everything is in shared memory already
        for (int i = 0; i < n_nt; ++i, ++it) {
          const int nt = (nt0 + i < n_nt) ? nt0 + i : nt0 + i - n_nt;
          const uint32_t s = it % TQ_STAGES, u = it / TQ_STAGES;
          if (!tq_wait(&sm->b_empty[s], (u & 1u) ^ 1u, sm, p.error_flag)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&sm->b_full[s], 2 * TC_ATOM_BYTES);
          tma_load_2d(sm->bhi[s], &map_chi, 0, nt * TC_BN, &sm->b_full[s]);
          tma_load_2d(sm->blo[s], &map_clo, 0, nt * TC_BN, &sm->b_full[s]);
        }
      }
      if (sm->abort_flag) drain_ring(sm->b_full, (uint32_t)TQ_STAGES, it);
    }
  } else if (warp < TQ_WORKER0) {
    // ------------------------------------------------------------------------ MMA
    // The issuing warps walk all tiles in order; warp mw issues the accumulators g = t * n_nt + i
    // with g mod n_mma == mw into buffer g mod n_acc and commits each to the (quad, buffer)
    // barrier of the tile's owner.  A buffer is handed back through the barrier of the warp that
    // fills it NEXT (accumulator g + n_acc), so every barrier has one waiter, which takes its
    // phases in order.  A warp waits for the split of a tile only when it issues for that tile.
    // (No runtime division in these loops: every cycle of an issuing warp delays all four quads.)
    const uint32_t mw = (uint32_t)warp - 2u;
    const uint32_t n_mma = (uint32_t)p.mma_warps;              // 1 or 2
    const uint32_t ring = resident ? (uint32_t)n_nt : (uint32_t)TQ_STAGES;
    const uint32_t lap_flip = resident ? 0u : 1u;
    uint32_t g = 0, s = 0, lap = 0;
    uint32_t ab = 0u;                              // g mod n_acc, kept by increment and wrap
    uint32_t e_seen = 0u;                          // bit b: parity of this warp's next wait on acc_empty[b][mw]
    uint32_t b_seen = 0u;                          // bit s: this warp has seen centroid stage s complete
    bool ok = true;
    KMB_PROF(long long m_conv = 0, m_empty = 0, m_b = 0, m_issue = 0, m_fence = 0, m_mma = 0, m_all = clock64(), mt, mt2;)
    const uint64_t b_hi0 = make_sdesc(smem_u32(sm->bhi[0]));
    const uint64_t b_lo0 = make_sdesc(smem_u32(sm->blo[0]));
    for (int t = 0; t < my_tiles && ok && mw < n_mma; ++t) {
      const uint32_t q = (uint32_t)(t % NQ);
      const uint32_t a_hi = tmem_base + q * 2u * half_cols, a_lo = a_hi + half_cols;
      if (n_nt == 1 && n_mma == 2u && (g & 1u) != mw) {
        // the tile's only accumulator is the other warp's: nothing to wait for here
        ++g;
        if (++ab == n_acc) ab = 0u;
        if (++s == ring) {
          s = 0;
          lap ^= lap_flip;
        }
        continue;
      }
      KMB_PROF(mt = clock64();)
      if (!__all_sync(0xffffffffu, tq_wait(&sm->x_conv[q], (uint32_t)(t / NQ) & 1u, sm, p.error_flag))) break;
      KMB_PROF(m_conv += clock64() - mt; mt2 = clock64();)
      TQ_STAMP(t == TQ_PROBE_TILE, mw == 0 ? 2 : 6)
      tc_fence_after();
      KMB_PROF(m_fence += clock64() - mt2;)
      for (int i = 0; i < n_nt && ok; ++i, ++g) {
        if (n_mma == 1u || (g & 1u) == mw) {
          const uint32_t d_tmem = tmem_base + acc_col0 + ab * TC_BN;
          KMB_PROF(mt = clock64();)
          if (g >= n_acc) {                                    // the buffer has been used before
            if (!__all_sync(0xffffffffu, tq_wait(&sm->acc_empty[ab][mw], (e_seen >> ab) & 1u, sm, p.error_flag))) {
              ok = false;
              break;
            }
            e_seen ^= 1u << ab;
          }
          KMB_PROF(m_empty += clock64() - mt; mt = clock64();)
          TQ_STAMP(t == TQ_PROBE_TILE, i == 0 ? 3 : 7)
          // resident centroid stages complete once: after this warp has seen a stage it skips the poll
          if (!(resident && ((b_seen >> s) & 1u))) {
            if (!__all_sync(0xffffffffu, tq_wait(&sm->b_full[s], lap, sm, p.error_flag))) {
              ok = false;
              break;
            }
            b_seen |= 1u << s;
          }
          KMB_PROF(m_b += clock64() - mt; mt = clock64();)
          TQ_STAMP(t == TQ_PROBE_TILE && i == 0, 4)
          tc_fence_after();
          KMB_PROF(m_fence += clock64() - mt; mt2 = clock64();)
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
            KMB_PROF(m_mma += clock64() - mt2;)
            umma_commit(&sm->acc_full[q][ab]);
          }
          __syncwarp();
          KMB_PROF(m_issue += clock64() - mt;)
          TQ_STAMP(t == TQ_PROBE_TILE, i == 0 ? 5 : 8)
        }
        if (++ab == n_acc) ab = 0u;
        if (++s == ring) {
          s = 0;
          lap ^= lap_flip;
        }
      }
    }
    KMB_PROF(if (blockIdx.x == 0 && lane == 0) printf("[tq prof] mma warp %u: total %lld cyc, wait x_conv %lld, acc_empty %lld, b_full %lld, issue %lld (fences %lld, elected lane's MMAs %lld), accumulators %u\n", mw, clock64() - m_all, m_conv, m_empty, m_b, m_issue, m_fence, m_mma, g);)
    if (sm->abort_flag) mma_drain(&sm->drain[mw]);
  } else {
    // -------------------------------------------------------------------- workers
    const int wk = warp - TQ_WORKER0;
    const int quad = wk >> 2, lq = warp & 3;
    const int lane_base = lq * 32;
    const int row = lane_base + lane;              // this thread's row of every tile of the quad
    float* acc_copy = update ? p.acc + (int64_t)(blockIdx.x % p.n_copies) * p.acc_len : nullptr;
    uint32_t changed = 0;
    uint32_t seen = 0u;                            // bit b: parity of this quad's next accumulator in buffer b
    bool ok = true;
    const int n_chunks = p.d / 4;                  // 16-byte chunks of a data row (d is a multiple of 4)
    const uint32_t slot_addr = tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)quad * 2u * half_cols;
    const int my_count = (my_tiles > quad) ? (my_tiles - 1 - quad) / NQ + 1 : 0;
    const uint32_t n_mma = (uint32_t)p.mma_warps;
    // buffer of the first accumulator of this quad's current tile: (t * n_nt) mod n_acc, advanced
    // by (4 * n_nt) mod n_acc from tile to tile
    uint32_t ab0 = ((uint32_t)quad * (uint32_t)n_nt) % n_acc;
    const uint32_t ab_step = ((uint32_t)NQ * (uint32_t)n_nt) % n_acc;
    KMB_PROF(long long w_x = 0, c_split = 0, w_acc = 0, c_arg = 0, c_upd = 0, t_all = clock64(), tw;)

    for (int jt = 0; jt < my_count && ok; ++jt) {
      const int t = quad + NQ * jt;
      const int m0 = ((int)blockIdx.x + t * (int)gridDim.x) * TC_BM;   // first row of the tile
      const bool valid = m0 + row < (int)p.n;
      // previous label and weight of this row: fetched now, used once the new label is known
      uint32_t prev_lab = 0xffffffffu;
      float wr = 1.f;
      if (update && valid) {
        if (p.prev != nullptr) prev_lab = __ldg(p.prev + m0 + row);
        if (p.w != nullptr) wr = __ldg(p.w + m0 + row);
      }

      // ---- split this thread's row into hi / lo parts in the quad's tensor-memory slot
      KMB_PROF(tw = clock64();)
      if (!__all_sync(0xffffffffu, tq_wait(&sm->x_full[quad], (uint32_t)jt & 1u, sm, p.error_flag))) break;
      KMB_PROF(w_x += clock64() - tw; tw = clock64();)
      TQ_STAMP(t == TQ_PROBE_TILE && lq == 0, 0)
      {
        const unsigned char* rowp = sm->xstage[quad] + row * 128;
#pragma unroll 1
        for (int sl = 0; sl < n_ks; ++sl) {        // 8 features per slice
          uint32_t hi[8], lo[8];
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {
            const int c = sl * 2 + c2;
            float4 x = *reinterpret_cast<const float4*>(rowp + ((c ^ (row & 7)) << 4));
            if (c == fold_chunk) set_fold_ones(x, fold_off);
            const float h0 = tf32_round_alu(x.x), h1 = tf32_round_alu(x.y);
            const float h2 = tf32_round_alu(x.z), h3 = tf32_round_alu(x.w);
            hi[4 * c2 + 0] = __float_as_uint(h0); lo[4 * c2 + 0] = __float_as_uint(tf32_round_alu(x.x - h0));
            hi[4 * c2 + 1] = __float_as_uint(h1); lo[4 * c2 + 1] = __float_as_uint(tf32_round_alu(x.y - h1));
            hi[4 * c2 + 2] = __float_as_uint(h2); lo[4 * c2 + 2] = __float_as_uint(tf32_round_alu(x.z - h2));
            hi[4 * c2 + 3] = __float_as_uint(h3); lo[4 * c2 + 3] = __float_as_uint(tf32_round_alu(x.w - h3));
          }
          tmem_st8(slot_addr + sl * 8, hi);
          tmem_st8(slot_addr + half_cols + sl * 8, lo);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&sm->x_conv[quad]);          // the MMAs of this tile may start
          mbar_arrive(&sm->x_stage_free[quad]);    // the staging buffer may take the quad's next tile
        }
      }
      KMB_PROF(c_split += clock64() - tw;)
      TQ_STAMP(t == TQ_PROBE_TILE && lq == 0, 1)

      // ---- reduce every accumulator of the tile to this row's (score, index)
      float best = __int_as_float(0xff800000);
      uint32_t bi = 0;
      float bif = 0.f;                             // FIDX: the index is carried as a float
      const uint32_t g0 = (uint32_t)t * (uint32_t)n_nt;
      uint32_t ab = ab0;
      ab0 += ab_step;
      if (ab0 >= n_acc) ab0 -= n_acc;
      for (int i = 0; i < n_nt; ++i, ab = (ab + 1u == n_acc) ? 0u : ab + 1u) {
        const uint32_t g = g0 + (uint32_t)i;
        const int nt_w = (nt0 + i < n_nt) ? nt0 + i : nt0 + i - n_nt;
        const int cn = nt_w * TC_BN;
        KMB_PROF(tw = clock64();)
        if (!__all_sync(0xffffffffu, tq_wait(&sm->acc_full[quad][ab], (seen >> ab) & 1u, sm, p.error_flag))) {
          ok = false;
          break;
        }
        KMB_PROF(w_acc += clock64() - tw; tw = clock64();)
        TQ_STAMP(t == TQ_PROBE_TILE && lq == 0 && i < 2, i == 0 ? 9 : 11)
        seen ^= 1u << ab;
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)lane_base << 16) + acc_col0 + ab * TC_BN;
        const float4 unused[8] = {};
        float qa = __int_as_float(0xff800000);
        uint32_t ia = 0;
        float iaf = 0.f;
#pragma unroll 1
        for (int c4 = 0; c4 < 4; ++c4) {
          uint32_t v[32];
          tmem_ld32(taddr + c4 * 32, v);
          tmem_ld_wait();
          if (c4 == 3) {
            // the whole accumulator has been read: hand the buffer back before the last argmax
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm->acc_empty[ab][n_mma == 2u ? ((g + n_acc) & 1u) : 0u]);
          }
          float qv;
          if (FIDX) {
            float ivf;
            argmax32_fidx(v, (float)(cn + c4 * 32), p.fone, qv, ivf);
            if (qv > qa) { qa = qv; iaf = ivf; }   // ascending inside the centroid tile: strict '>'
          } else {
            uint32_t iv;
            argmax32<true>(v, unused, (uint32_t)(cn + c4 * 32), qv, iv);
            if (qv > qa) { qa = qv; ia = iv; }
          }
        }
        // centroid tiles arrive in rotated order: larger score wins, equal scores -> smaller index
        if (FIDX) {
          if (qa > best || (qa == best && iaf < bif)) {
            best = qa;
            bif = iaf;
          }
        } else if (qa > best || (qa == best && ia < bi)) {
          best = qa;
          bi = ia;
        }
        KMB_PROF(c_arg += clock64() - tw;)
        TQ_STAMP(t == TQ_PROBE_TILE && lq == 0 && i < 2, i == 0 ? 10 : 12)
      }
      if (FIDX) bi = (uint32_t)bif;
      if (!ok) break;

      // ---- label and update of this thread's own row
      KMB_PROF(tw = clock64();)
      if (valid) {
        p.labels[m0 + row] = bi;
        if (update) {
          changed += (prev_lab != bi) ? 1u : 0u;
          const float4* xrow = reinterpret_cast<const float4*>(p.X + (int64_t)(m0 + row) * p.d);
          float* dst = acc_copy + (int64_t)bi * p.d;
          atomicAdd(&acc_copy[(int64_t)p.k * p.d + bi], wr);
          for (int c0 = 0; c0 < n_chunks; c0 += 4) {
            float4 x[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
              x[u] = (c0 + u < n_chunks) ? __ldg(xrow + c0 + u) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (c0 + u < n_chunks) {
                float4 a4;
                a4.x = x[u].x * wr; a4.y = x[u].y * wr; a4.z = x[u].z * wr; a4.w = x[u].w * wr;
                atomicAdd(reinterpret_cast<float4*>(dst + 4 * (c0 + u)), a4);
              }
            }
          }
        }
      }
      KMB_PROF(c_upd += clock64() - tw;)
      TQ_STAMP(t == TQ_PROBE_TILE && lq == 0, 13)
    }
    KMB_PROF(if (blockIdx.x == 0 && lane == 0 && lq == 0 && quad == 0 && my_tiles > TQ_PROBE_TILE) { const long long z = sm->ts[0]; printf("[tq prof] tile %d time line (cycles after its sample tile arrived): split done %lld | mma warp 0: saw split %lld, buffer free %lld, centroids ready %lld, issued %lld | mma warp 1: saw split %lld, buffer free %lld, issued %lld | worker: acc 0 complete %lld, read %lld, acc 1 complete %lld, read %lld, update done %lld\n", TQ_PROBE_TILE, sm->ts[1] - z, sm->ts[2] - z, sm->ts[3] - z, sm->ts[4] - z, sm->ts[5] - z, sm->ts[6] - z, sm->ts[7] - z, sm->ts[8] - z, sm->ts[9] - z, sm->ts[10] - z, sm->ts[11] - z, sm->ts[12] - z, sm->ts[13] - z); })
    KMB_PROF(if (blockIdx.x == 0 && lane == 0 && lq == 0) printf("[tq prof] quad %d: total %lld cyc, wait x_full %lld, split %lld, wait acc_full %lld, loads + argmax %lld, update %lld, tiles %d\n", quad, clock64() - t_all, w_x, c_split, w_acc, c_arg, c_upd, my_count);)
    if (update) {
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
