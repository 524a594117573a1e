// Short-row form of the tensor-core Lloyd step, organised as two independent TEAMS per CTA.
// Included by lloyd_tc.cu (it uses that file's PTX wrappers, TcParams and argmax32).
//
// Rows of at most 28 features (one 32-feature chunk including the two fold features, see
// lloyd_tc_folds).  With so little contraction per accumulator element the step is bound by the
// instructions of the epilogue warps, of which only a third is the argmax itself: the rest is
// the per-tile bookkeeping every warp repeats (barrier waits, tensor-memory loads, label
// exchange, update addressing).  So the work is cut to have as few warps as possible repeat it
// while sixteen warps stay resident to hide latencies: the sample tiles of a CTA alternate
// between two teams, and a team is a complete pipeline of its own:
//   warp 0        TMA producer of the sample tiles of both teams (two in flight per team)
//   warp 1        TMA producer of the centroid stages, shared: both teams walk the same stage
//                 sequence, one round per pair of sample tiles, and a stage is recycled when the
//                 MMA warps of BOTH teams have committed it
//   warp 2 + T    MMA issuer of team T (T = 0, 1), one accumulator buffer of its own
//   warps 4 + 8 T .. 11 + 8 T   the eight workers of team T: worker (lq, ch) owns TMEM lanes
//                 32 lq .. 32 lq + 31 (one sample row per thread) and columns 64 ch .. 64 ch + 63
//                 of every accumulator; it splits feature slices ch and ch + 2 (8 features each)
//                 of its row into tensor memory, keeps a running (score, index), and adds 16
//                 of the tile's rows into the centroid sums.  Half 0 merges the two halves.
// Tensor memory: sample-tile slot s = 2 T + (tile of the team & 1): hi at columns 64 s, lo at
// 64 s + 32 (256 columns); accumulator of team T at 256 + 128 T.
// While one team waits for a barrier or a load, the other one computes: the two run out of
// phase by construction, which also spreads the argmax bursts over time.
#pragma once

namespace kmb {

constexpr int TT_WARPS = 20;
constexpr int TT_THREADS = TT_WARPS * 32;
constexpr int TT_WORKER0 = 4;
constexpr int TT_TEAM_WARPS = 8;
constexpr int TT_STAGES = 4;        // centroid stages (hi + lo = 32 KB each)

struct TtSmem {
  unsigned char xstage[4][TC_ATOM_BYTES];          // [2 T + slot]
  unsigned char bhi[TT_STAGES][TC_ATOM_BYTES];
  unsigned char blo[TT_STAGES][TC_ATOM_BYTES];
  uint16_t lab_s[2][2][TC_BM];                     // [team][tile & 1]
  float part_v[2][TC_BM];                          // [team]: half 1's best score per row
  uint16_t part_i[2][TC_BM];
  unsigned long long x_full[4], x_conv[4], x_stage_free[4];
  unsigned long long b_full[TT_STAGES], b_empty[TT_STAGES];
  unsigned long long acc_full[2], acc_empty[2];    // [team]
  unsigned long long part_full[2], lab_ready[2];   // [team]
  unsigned int tmem_base;
  volatile int abort_flag;
};
static_assert(sizeof(TtSmem) + 1024 <= 232448, "TtSmem exceeds the 227 KB a CTA may use");

// Bounded wait on a barrier of this kernel (same rule as mbar_wait).
__device__ __forceinline__ bool tt_wait(void* bar, uint32_t parity, TtSmem* sm, int* error_flag,
                                        uint32_t sleep_ns) {
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
    if (clock64() - t0 > TC_TIMEOUT_CYCLES) {
      sm->abort_flag = 1;
      atomicExch(error_flag, 1);
      return false;
    }
  }
}

__global__ void __launch_bounds__(TT_THREADS, 1)
lloyd_tc_teams_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_chi,
                      const __grid_constant__ CUtensorMap map_clo, TcParams p) {
  extern __shared__ unsigned char smem_raw[];
  TtSmem* sm = reinterpret_cast<TtSmem*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_nt = p.k_pad / TC_BN;
  // n < 2^31 - 128 (checked by the host), so tile and row indices fit 32 bits
  const int n_tiles = (int)((p.n + TC_BM - 1) / TC_BM);
  const int my_tiles = (n_tiles > (int)blockIdx.x) ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const int n_rounds = (my_tiles + 1) >> 1;        // pairs of sample tiles of this CTA
  const bool update = p.acc != nullptr;
  const int nt0 = (int)(blockIdx.x % (unsigned)n_nt);
  const bool resident = n_nt <= TT_STAGES;
  const int d_eff = p.d + 2;                       // data features + the two fold features
  const int n_ks = (d_eff + 7) / 8;                // k-steps / feature slices that hold data: 1..4
  const int fold_chunk = p.d / 4;                  // 16-byte chunk of a row holding features d, d + 1
  const int n_conv = 4 * (n_ks < 2 ? n_ks : 2);    // warps of a team that split feature slices

  if (threadIdx.x == 0) {
    for (int a = 0; a < 4; ++a) {
      mbar_init(&sm->x_full[a], 1);
      mbar_init(&sm->x_conv[a], n_conv);
      mbar_init(&sm->x_stage_free[a], n_conv);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sm->acc_full[a], 1);
      mbar_init(&sm->acc_empty[a], TT_TEAM_WARPS);
      mbar_init(&sm->part_full[a], 4);
      mbar_init(&sm->lab_ready[a], 4);
    }
    for (int s = 0; s < TT_STAGES; ++s) {
      mbar_init(&sm->b_full[s], 1);
      mbar_init(&sm->b_empty[s], 2);               // both teams' MMA warps
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

  // CTA-local tile t (global tile blockIdx.x + t * gridDim.x) belongs to team t & 1; it is tile
  // jt = t >> 1 of that team and uses sample slot 2 * team + (jt & 1) for the (jt >> 1)-th time.
  if (warp == 0) {
    // ---------------------------------------------------------------- sample tiles
    if (lane == 0) {
      for (int t = 0; t < my_tiles; ++t) {
        const int jt = t >> 1, slot = 2 * (t & 1) + (jt & 1);
        if (!tt_wait(&sm->x_stage_free[slot], ((uint32_t)(jt >> 1) & 1u) ^ 1u, sm, p.error_flag, p.sleep_ns)) break;
        mbar_expect_tx(&sm->x_full[slot], TC_ATOM_BYTES);
        tma_load_2d(sm->xstage[slot], &map_x, 0, ((int)blockIdx.x + t * (int)gridDim.x) * TC_BM, &sm->x_full[slot]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------- centroid stages, one sequence per round
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int r = 0; r < n_rounds && ok; ++r) {
        if (resident && r != 0) break;             // everything is in shared memory already
        for (int i = 0; i < n_nt; ++i, ++it) {
          const int nt = (nt0 + i < n_nt) ? nt0 + i : nt0 + i - n_nt;
          const uint32_t s = it % TT_STAGES, u = it / TT_STAGES;
          if (!tt_wait(&sm->b_empty[s], (u & 1u) ^ 1u, sm, p.error_flag, p.sleep_ns)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&sm->b_full[s], 2 * TC_ATOM_BYTES);
          tma_load_2d(sm->bhi[s], &map_chi, 0, nt * TC_BN, &sm->b_full[s]);
          tma_load_2d(sm->blo[s], &map_clo, 0, nt * TC_BN, &sm->b_full[s]);
        }
      }
    }
  } else if (warp < TT_WORKER0) {
    // --------------------------------------------------------- MMA issuer of team mw
    const uint32_t mw = (uint32_t)warp - 2u;
    const uint32_t ring = resident ? (uint32_t)n_nt : (uint32_t)TT_STAGES;
    const uint32_t lap_flip = resident ? 0u : 1u;
    uint32_t s = 0, lap = 0, ga = 0;
    bool ok = true;
    const uint64_t b_hi0 = make_sdesc(smem_u32(sm->bhi[0]));
    const uint64_t b_lo0 = make_sdesc(smem_u32(sm->blo[0]));
    const uint32_t d_tmem = tmem_base + TC_ACC_COL + mw * TC_BN;
    for (int r = 0; r < n_rounds && ok; ++r) {
      const bool have = 2 * r + (int)mw < my_tiles;   // the last round may hold one tile only
      const uint32_t slot = 2u * mw + ((uint32_t)r & 1u);
      const uint32_t a_hi = tmem_base + slot * 64u, a_lo = a_hi + 32u;
      if (have) {
        if (!__all_sync(0xffffffffu, tt_wait(&sm->x_conv[slot], ((uint32_t)r >> 1) & 1u, sm, p.error_flag, p.sleep_ns))) break;
        tc_fence_after();
      }
      for (int i = 0; i < n_nt && ok; ++i) {
        if (have) {
          if (!__all_sync(0xffffffffu, tt_wait(&sm->acc_empty[mw], (ga & 1u) ^ 1u, sm, p.error_flag, p.sleep_ns)) ||
              !__all_sync(0xffffffffu, tt_wait(&sm->b_full[s], lap, sm, p.error_flag, p.sleep_ns))) {
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
          ++ga;
        } else if (!resident) {
          // no tile of this team in the last round: still hand the stage back on its behalf
          if (!__all_sync(0xffffffffu, tt_wait(&sm->b_full[s], lap, sm, p.error_flag, p.sleep_ns))) {
            ok = false;
            break;
          }
          if (lane == 0) mbar_arrive(&sm->b_empty[s]);
          __syncwarp();
        }
        if (++s == ring) {
          s = 0;
          lap ^= lap_flip;
        }
      }
    }
  } else {
    // -------------------------------------------------------------------- workers
    const int wk = warp - TT_WORKER0;
    const int team = wk >> 3;
    const int lq = warp & 3, ch = (wk >> 2) & 1;
    const int lane_base = lq * 32;
    const int row = lane_base + lane;
    const bool converts = ch < n_ks;               // slices ch and ch + 2, where they hold data
    float* acc_copy = update ? p.acc + (int64_t)(blockIdx.x % p.n_copies) * p.acc_len : nullptr;
    uint32_t ga = 0, changed = 0;
    bool ok = true;
    // update geometry: G lanes (a power of two) of 16 bytes serve one row; a warp adds 16 rows
    const int urow0 = (wk & 7) * 16;
    int G = 1;
    while (G * 4 < p.d) G <<= 1;
    const int rpi = 32 / G;                        // rows per warp instruction: 4 .. 32
    const int sub = lane / G;
    const int col = (lane % G) * 4;
    const bool col_ok = col < p.d;
    const int n_tiles_i = n_tiles;
    const int my_first = team, my_step = 2;        // CTA-local tiles of this team: team, team + 2, ...

    // Splits feature slices ch and ch + 2 of this thread's row of the team's tile jt into tensor
    // memory (hi at the slot's columns 8 s .., lo 32 further).  False on time-out.
    auto convert_tile = [&](int jt) -> bool {
      const uint32_t slot = 2u * (uint32_t)team + ((uint32_t)jt & 1u);
      if (!__all_sync(0xffffffffu, tt_wait(&sm->x_full[slot], ((uint32_t)jt >> 1) & 1u, sm, p.error_flag, p.sleep_ns)))
        return false;
      const unsigned char* rowp = sm->xstage[slot] + row * 128;
      const uint32_t lane_addr = tmem_base + ((uint32_t)lane_base << 16) + slot * 64u;
#pragma unroll 1
      for (int s2 = 0; s2 < 2; ++s2) {
        const int sl = ch + 2 * s2;                // feature slice: features 8 sl .. 8 sl + 7
        if (sl < n_ks) {
          uint32_t hi[8], lo[8];
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {
            const int c = sl * 2 + c2;
            float4 x = *reinterpret_cast<const float4*>(rowp + ((c ^ (row & 7)) << 4));
            if (c == fold_chunk) {
              x.x = 1.f;
              x.y = 1.f;
            }
            const float h0 = tf32_round_alu(x.x), h1 = tf32_round_alu(x.y);
            const float h2 = tf32_round_alu(x.z), h3 = tf32_round_alu(x.w);
            hi[4 * c2 + 0] = __float_as_uint(h0); lo[4 * c2 + 0] = __float_as_uint(tf32_round_alu(x.x - h0));
            hi[4 * c2 + 1] = __float_as_uint(h1); lo[4 * c2 + 1] = __float_as_uint(tf32_round_alu(x.y - h1));
            hi[4 * c2 + 2] = __float_as_uint(h2); lo[4 * c2 + 2] = __float_as_uint(tf32_round_alu(x.z - h2));
            hi[4 * c2 + 3] = __float_as_uint(h3); lo[4 * c2 + 3] = __float_as_uint(tf32_round_alu(x.w - h3));
          }
          tmem_st8(lane_addr + sl * 8, hi);
          tmem_st8(lane_addr + 32 + sl * 8, lo);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&sm->x_conv[slot]);
        mbar_arrive(&sm->x_stage_free[slot]);
      }
      return true;
    };

    const int my_count = (my_tiles > team) ? (my_tiles - 1 - team) / 2 + 1 : 0;   // tiles of this team
    if (converts && my_count > 0) ok = convert_tile(0);
    for (int jt = 0; jt < my_count && ok; ++jt) {
      const int t = my_first + jt * my_step;
      const int m0 = ((int)blockIdx.x + t * (int)gridDim.x) * TC_BM;   // first row of the tile
      const uint32_t buf = (uint32_t)jt & 1u;
      float best = __int_as_float(0xff800000);
      uint32_t bi = 0;
      // previous label of this thread's row: fetched now, compared once the new one is known
      uint32_t prev_lab = 0xffffffffu;
      if (update && ch == 0 && p.prev != nullptr && m0 + row < (int)p.n) prev_lab = __ldg(p.prev + m0 + row);
      // the rows this warp will add into the centroid sums are fetched now, so that their
      // latency hides behind the epilogues: instruction j serves rows j * rpi + sub (< 16)
      const float* xbase = p.X + (int64_t)(m0 + urow0) * p.d + col;
      // (rows of up to 16 features: two instructions cover the warp's 16 rows and are fetched
      // ahead; longer rows need four and are fetched when they are added)
      const bool pre = rpi >= 8;
      float4 xpre[2];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int r = j * rpi + sub;
        const bool okj = pre && update && r < 16 && col_ok && (m0 + urow0 + r < (int)p.n);
        xpre[j] = okj ? __ldg(reinterpret_cast<const float4*>(xbase + r * p.d)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
      // the team's other sample slot was last read by the MMAs of tile jt - 1, all of whose
      // accumulators this warp has consumed: it is free for tile jt + 1
      if (converts && jt + 1 < my_count && !convert_tile(jt + 1)) break;
      for (int i = 0; i < n_nt; ++i, ++ga) {
        const int nt_w = (nt0 + i < n_nt) ? nt0 + i : nt0 + i - n_nt;
        const int cn = nt_w * TC_BN + ch * 64;     // first centroid of this half
        if (!__all_sync(0xffffffffu, tt_wait(&sm->acc_full[team], ga & 1u, sm, p.error_flag, p.sleep_ns))) {
          ok = false;
          break;
        }
        tc_fence_after();
        // 32 columns at a time: the second load is issued once the first 32 scores have been
        // reduced, which keeps the two tiles of registers from being live together
        const uint32_t taddr = tmem_base + ((uint32_t)lane_base << 16) + TC_ACC_COL + team * TC_BN + ch * 64;
        const float4 unused[8] = {};
        float qa, qb;
        uint32_t ia, ib;
        {
          uint32_t va[32];
          tmem_ld32(taddr, va);
          tmem_ld_wait();
          argmax32<true>(va, unused, (uint32_t)cn, qa, ia);
        }
        {
          uint32_t vb[32];
          tmem_ld32(taddr + 32, vb);
          tmem_ld_wait();
          // the accumulator is in registers now: hand the buffer back before the second argmax
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm->acc_empty[team]);
          argmax32<true>(vb, unused, (uint32_t)(cn + 32), qb, ib);
        }
        if (qb > qa) { qa = qb; ia = ib; }         // ascending inside the half: strict '>'
        // centroid tiles arrive in rotated order: larger score wins, equal scores -> smaller index
        if (qa > best || (qa == best && ia < bi)) {
          best = qa;
          bi = ia;
        }
      }
      if (!ok) break;

      if (ch != 0) {
        sm->part_v[team][row] = best;
        sm->part_i[team][row] = (uint16_t)bi;
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->part_full[team]);
      } else {
        if (!__all_sync(0xffffffffu, tt_wait(&sm->part_full[team], (uint32_t)jt & 1u, sm, p.error_flag, p.sleep_ns))) break;
        const float ov = sm->part_v[team][row];
        const uint32_t oi = sm->part_i[team][row];
        if (ov > best || (ov == best && oi < bi)) {
          best = ov;
          bi = oi;
        }
        sm->lab_s[team][buf][row] = (uint16_t)bi;
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm->lab_ready[team]);
        if (m0 + row < (int)p.n) {
          p.labels[m0 + row] = bi;
          if (update) changed += (prev_lab != bi) ? 1u : 0u;
        }
      }
      // Every warp of the team waits for the merged labels (also when nothing is updated):
      // part_* have one buffer per team, which half 0 has read before it arrives here, so half 1
      // cannot overwrite it a tile early.  lab_s[team][buf] is reused two tiles later; by then
      // every warp has passed this point of tile jt + 1, which it reaches only after its update
      // of tile jt.
      if (!__all_sync(0xffffffffu, tt_wait(&sm->lab_ready[team], (uint32_t)jt & 1u, sm, p.error_flag, p.sleep_ns))) break;
      if (!update) continue;

      // ---- centroid update of rows urow0 .. urow0 + 15 of this tile
      const int my = urow0 + (lane & 15);
      const uint32_t ubi = sm->lab_s[team][buf][my];
      const bool uvalid = m0 + my < (int)p.n;
      float uwi = 0.f;
      if (uvalid) uwi = p.w ? p.w[m0 + my] : 1.f;
      if (uvalid && lane < 16) atomicAdd(&acc_copy[(int64_t)p.k * p.d + ubi], uwi);
      auto add_rows = [&](int j, const float4& x) {
        const int r = j * rpi + sub;
        const bool okj = r < 16 && col_ok && (m0 + urow0 + r < (int)p.n);
        const int src = okj ? r : 0;
        const uint32_t lab = __shfl_sync(0xffffffffu, ubi, src);
        const float wr = __shfl_sync(0xffffffffu, uwi, src);
        if (okj) {
          float4 u;
          u.x = x.x * wr; u.y = x.y * wr; u.z = x.z * wr; u.w = x.w * wr;
          atomicAdd(reinterpret_cast<float4*>(acc_copy + (int64_t)lab * p.d + col), u);
        }
      };
      if (pre) {
        add_rows(0, xpre[0]);
        add_rows(1, xpre[1]);
      } else {
#pragma unroll 1
        for (int j = 0; j < 4; ++j) {
          const int r = j * rpi + sub;
          const bool okj = r < 16 && col_ok && (m0 + urow0 + r < (int)p.n);
          add_rows(j, okj ? __ldg(reinterpret_cast<const float4*>(xbase + r * p.d))
                          : make_float4(0.f, 0.f, 0.f, 0.f));
        }
      }
    }
    (void)n_tiles_i;
    if (update && ch == 0) {
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
