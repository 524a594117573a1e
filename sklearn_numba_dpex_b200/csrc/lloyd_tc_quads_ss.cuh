// Short-row form of the tensor-core Lloyd step for rows of at most 16 contraction features
// (data + the two fold features), with the SAMPLE operand read from shared memory.  Included by
// lloyd_tc.cu after lloyd_tc_quads.cuh (PTX wrappers, TcParams, argmax32_fidx, tq_threads).
//
// Same division of labour as lloyd_tc_quads_kernel (one thread owns one sample row of a tile
// from its split to its update, four quads of worker warps), but the split of a row is done IN
// PLACE in the staged tile: a 128-byte row of the stage holds 32 floats of which at most 16 are
// contraction features, so the thread writes the rounded hi parts back over features 0..15 and
// the lo parts into the unused features 16..31, and the MMAs take both operands from shared
// memory (tcgen05.mma with two shared-memory descriptors).  Consequences:
//   * tensor memory holds nothing but accumulators: FOUR of 128 columns instead of two or three;
//   * a quad has TWO stages, so it splits tile j + 1 before it reduces the accumulators of tile
//     j: the MMAs of its next tile run under the argmax and the update of the current one, and
//     the chain split -> MMA -> argmax -> update is no longer exposed once per tile;
//   * no tensor-memory stores and no wait for them in the split.
// The price is shared-memory traffic of the MMAs (4 KB of samples per MMA on top of the 4 KB of
// centroids) and three centroid stages instead of four beside the eight sample stages.
// Measured on n = 5 M, d = 14, k = 256: 0.314 ms per step against 0.307 ms for
// lloyd_tc_quads_kernel.  The wait for accumulators does fall from a third of a worker's time to
// a ninth, but the MMAs now read 96 KB of operands per tile from shared memory (about 1 600
// cycles per tile at the rate measured with the argmax and the update switched off), and the
// argmax (37 %) and the update (19 %) of a worker are unchanged; so the kernel is kept as an
// alternative (KMB_TQ_SS=1), not as the default.  The host
// sends a shape here only when ALL centroid stages stay resident (k <= 384): with an odd number
// of streamed stages the two issuing warps would meet every stage on alternate laps and could
// not track its barrier by parity alone.
//
//   warp 0        TMA producer of the sample tiles (two stages per quad)
//   warp 1        TMA producer of the centroid stages (resident when all of them fit)
//   warps 2, 3    issue the MMAs in tile order, alternate accumulators each
//   warps 4 + 4 Q .. 7 + 4 Q   quad Q
#pragma once

namespace kmb {

constexpr int TS2_STAGES = 3;       // centroid stages (hi + lo = 32 KB each)
constexpr int TS2_ACC = 4;          // accumulators of 128 columns

struct Ts2Smem {
  unsigned char xstage[4][2][TC_ATOM_BYTES];       // [quad][stage]
  unsigned char bhi[TS2_STAGES][TC_ATOM_BYTES];
  unsigned char blo[TS2_STAGES][TC_ATOM_BYTES];
  unsigned long long x_full[4][2];                 // the tile has arrived
  unsigned long long x_conv[4][2];                 // its rows have been split in place
  unsigned long long x_free[4][2];                 // every MMA that reads the stage has completed
  // [quad][buffer]: an accumulator of one of the quad's tiles is complete (see TqSmem::acc_full)
  unsigned long long acc_full[4][TS2_ACC];
  // [buffer]: its four readers have it in registers.  Buffers alternate between the two issuing
  // warps like the accumulators do, so every barrier has one waiter.
  unsigned long long acc_empty[TS2_ACC];
  unsigned long long b_full[TS2_STAGES], b_empty[TS2_STAGES];
  unsigned long long drain[2];
  long long timeout_cycles;
  unsigned int tmem_base;
  volatile int abort_flag;
};
static_assert(sizeof(Ts2Smem) + 1024 <= 232448, "Ts2Smem exceeds the 227 KB a CTA may use");

// Bounded wait on a barrier of this kernel (same rule as mbar_wait).
__device__ __forceinline__ bool ts2_wait(void* bar, uint32_t parity, Ts2Smem* sm, int* error_flag) {
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

// D[tmem] (+)= A[smem] * B[smem]^T, kind::tf32, both operands K-major shared-memory descriptors.
__device__ __forceinline__ void umma_tf32_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Writes of this thread to shared memory become visible to the tensor core and to TMA.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__global__ void __launch_bounds__(tq_threads(4), 1)
lloyd_tc_quads_ss_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_chi,
                         const __grid_constant__ CUtensorMap map_clo, TcParams p) {
  extern __shared__ unsigned char smem_raw[];
  Ts2Smem* sm = reinterpret_cast<Ts2Smem*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_nt = p.k_pad / TC_BN;
  // n < 2^31 - 128 (checked by the host), so tile and row indices fit 32 bits
  const int n_tiles = (int)((p.n + TC_BM - 1) / TC_BM);
  const int my_tiles = (n_tiles > (int)blockIdx.x) ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  const bool update = p.acc != nullptr;
  const int nt0 = (int)(blockIdx.x % (unsigned)n_nt);
  const bool resident = n_nt <= TS2_STAGES;
  const int d_eff = p.fold_at + 2 > p.d ? p.fold_at + 2 : p.d;   // <= 16 (checked by the host)
  const int n_ks = (d_eff + 7) / 8;                // k-steps of 8 features that hold data: 1 or 2
  const int fold_chunk = p.fold_at / 4;            // 16-byte chunk of a row holding the fold features
  const int fold_off = p.fold_at % 4;

  if (threadIdx.x == 0) {
    for (int q = 0; q < 4; ++q) {
      for (int st = 0; st < 2; ++st) {
        mbar_init(&sm->x_full[q][st], 1);
        mbar_init(&sm->x_conv[q][st], 4);
        // both issuing warps read the stage, unless a tile has one accumulator only
        mbar_init(&sm->x_free[q][st], n_nt >= 2 ? 2 : 1);
      }
      for (int a = 0; a < TS2_ACC; ++a) mbar_init(&sm->acc_full[q][a], 1);
    }
    for (int a = 0; a < TS2_ACC; ++a) mbar_init(&sm->acc_empty[a], 4);
    for (int s = 0; s < TS2_STAGES; ++s) {
      mbar_init(&sm->b_full[s], 1);
      mbar_init(&sm->b_empty[s], 1);
    }
    mbar_init(&sm->drain[0], 1);
    mbar_init(&sm->drain[1], 1);
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

  // CTA-local tile t (global tile blockIdx.x + t * gridDim.x) belongs to quad t & 3, is the
  // (t >> 2)-th tile of that quad and uses the quad's stage (t >> 2) & 1 for the (t >> 3)-th time.
  if (warp == 0) {
    // ---------------------------------------------------------------- sample tiles
    if (lane == 0) {
      int t = 0;
      for (; t < my_tiles; ++t) {
        const int q = t & 3, st = (t >> 2) & 1;
        if (p.test_stall != 0 && t >= 1) break;    // test hook: a sample tile that never arrives
        if (!ts2_wait(&sm->x_free[q][st], ((uint32_t)(t >> 3) & 1u) ^ 1u, sm, p.error_flag)) break;
        mbar_expect_tx(&sm->x_full[q][st], TC_ATOM_BYTES);
        tma_load_2d(sm->xstage[q][st], &map_x, 0, ((int)blockIdx.x + t * (int)gridDim.x) * TC_BM,
                    &sm->x_full[q][st]);
      }
      // (quad, stage) pairs form a ring of eight slots in tile order
      if (sm->abort_flag) {
        for (int u = 0; u < 8 && u < t; ++u) {
          const int last = u + ((t - 1 - u) / 8) * 8;          // last tile that used slot u
          drain_wait(&sm->x_full[last & 3][(last >> 2) & 1], (uint32_t)(last >> 3) & 1u);
        }
      }
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
          const uint32_t s = it % TS2_STAGES, u = it / TS2_STAGES;
          if (!ts2_wait(&sm->b_empty[s], (u & 1u) ^ 1u, sm, p.error_flag)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&sm->b_full[s], 2 * TC_ATOM_BYTES);
          tma_load_2d(sm->bhi[s], &map_chi, 0, nt * TC_BN, &sm->b_full[s]);
          tma_load_2d(sm->blo[s], &map_clo, 0, nt * TC_BN, &sm->b_full[s]);
        }
      }
      if (sm->abort_flag) drain_ring(sm->b_full, (uint32_t)TS2_STAGES, it);
    }
  } else if (warp < TQ_WORKER0) {
    // ------------------------------------------------------------------------ MMA
    // Both warps walk all tiles in order; warp mw issues the accumulators g = t * n_nt + i with
    // g & 1 == mw into buffer g & 3 (its own two buffers) and commits each to the (quad, buffer)
    // barrier of the tile's owner; after its last accumulator of a tile it also commits to the
    // stage's `free` barrier.  (No division in these loops.)
    const uint32_t mw = (uint32_t)warp - 2u;
    const uint32_t ring = resident ? (uint32_t)n_nt : (uint32_t)TS2_STAGES;
    const uint32_t lap_flip = resident ? 0u : 1u;
    uint32_t g = 0, s = 0, lap = 0;
    uint32_t uses = 0u;                            // accumulators this warp has issued
    uint32_t e_seen = 0u;                          // bit b: parity of this warp's next wait on acc_empty[b]
    uint32_t b_seen = 0u;                          // bit s: this warp has seen centroid stage s complete
    bool ok = true;
    const uint64_t b_hi0 = make_sdesc(smem_u32(sm->bhi[0]));
    const uint64_t b_lo0 = make_sdesc(smem_u32(sm->blo[0]));
    const uint64_t a_0 = make_sdesc(smem_u32(sm->xstage[0][0]));
    for (int t = 0; t < my_tiles && ok; ++t) {
      const uint32_t q = (uint32_t)t & 3u, st = ((uint32_t)t >> 2) & 1u;
      if (n_nt == 1 && (g & 1u) != mw) {
        // the tile's only accumulator is the other warp's: nothing to wait for here
        ++g;
        if (++s == ring) {
          s = 0;
          lap ^= lap_flip;
        }
        continue;
      }
      if (!__all_sync(0xffffffffu, ts2_wait(&sm->x_conv[q][st], ((uint32_t)t >> 3) & 1u, sm, p.error_flag))) break;
      tc_fence_after();
      // hi parts: features 0..15 of the stage's rows, lo parts: features 16..31 (64 bytes further)
      const uint64_t a_hi = a_0 + (uint64_t)((q * 2u + st) * (TC_ATOM_BYTES >> 4));
      const uint64_t a_lo = a_hi + 4u;
      // index of this warp's last accumulator of the tile
      const int i_last = ((g + (uint32_t)n_nt - 1u) & 1u) == mw ? n_nt - 1 : n_nt - 2;
      for (int i = 0; i < n_nt && ok; ++i, ++g) {
        if ((g & 1u) == mw) {
          const uint32_t ab = g & 3u;                          // accumulator buffer
          const uint32_t d_tmem = tmem_base + ab * TC_BN;
          if (uses >= 2u) {                                    // the buffer has been used before
            if (!__all_sync(0xffffffffu, ts2_wait(&sm->acc_empty[ab], (e_seen >> ab) & 1u, sm, p.error_flag))) {
              ok = false;
              break;
            }
            e_seen ^= 1u << ab;
          }
          // resident centroid stages complete once: after this warp has seen a stage it skips the poll
          if (!(resident && ((b_seen >> s) & 1u))) {
            if (!__all_sync(0xffffffffu, ts2_wait(&sm->b_full[s], lap, sm, p.error_flag))) {
              ok = false;
              break;
            }
            b_seen |= 1u << s;
          }
          tc_fence_after();
          const uint64_t b_hi = b_hi0 + (uint64_t)(s * (TC_ATOM_BYTES >> 4));
          const uint64_t b_lo = b_lo0 + (uint64_t)(s * (TC_ATOM_BYTES >> 4));
          if (elect_one()) {
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
              if (ks < n_ks) {
                const uint64_t adv = (uint64_t)(ks * 2);       // 8 tf32 = 32 bytes = 2 x 16-byte units
                umma_tf32_ss(d_tmem, a_lo + adv, b_hi + adv, TC_IDESC, ks != 0);
                umma_tf32_ss(d_tmem, a_hi + adv, b_lo + adv, TC_IDESC, 1);
                umma_tf32_ss(d_tmem, a_hi + adv, b_hi + adv, TC_IDESC, 1);
              }
            }
            if (!resident) umma_commit(&sm->b_empty[s]);
            umma_commit(&sm->acc_full[q][ab]);
            if (i == i_last) umma_commit(&sm->x_free[q][st]);
          }
          __syncwarp();
          ++uses;
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
    const int wk = warp - TQ_WORKER0;
    const int quad = wk >> 2, lq = warp & 3;
    const int lane_base = lq * 32;
    const int row = lane_base + lane;              // this thread's row of every tile of the quad
    float* acc_copy = update ? p.acc + (int64_t)(blockIdx.x % p.n_copies) * p.acc_len : nullptr;
    uint32_t changed = 0;
    uint32_t seen = 0u;                            // bit b: parity of this quad's next accumulator in buffer b
    bool ok = true;
    const int n_chunks = p.d / 4;                  // 16-byte chunks of a data row (d is a multiple of 4)
    const int my_count = (my_tiles > quad) ? (my_tiles - 1 - quad) / 4 + 1 : 0;

    // Splits this thread's row of the quad's tile jt in place: hi parts over features 0..15, lo
    // parts into features 16..31 of the same 128-byte row (chunks are XOR-swizzled by the row).
    auto split_tile = [&](int jt) -> bool {
      const int st = jt & 1;
      if (!__all_sync(0xffffffffu, ts2_wait(&sm->x_full[quad][st], ((uint32_t)jt >> 1) & 1u, sm, p.error_flag)))
        return false;
      unsigned char* rowp = sm->xstage[quad][st] + row * 128;
      const int sw = row & 7;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (c < 2 * n_ks) {
          float4 x = *reinterpret_cast<const float4*>(rowp + ((c ^ sw) << 4));
          if (c == fold_chunk) set_fold_ones(x, fold_off);
          float4 h, l;
          h.x = tf32_round_alu(x.x); h.y = tf32_round_alu(x.y);
          h.z = tf32_round_alu(x.z); h.w = tf32_round_alu(x.w);
          l.x = tf32_round_alu(x.x - h.x); l.y = tf32_round_alu(x.y - h.y);
          l.z = tf32_round_alu(x.z - h.z); l.w = tf32_round_alu(x.w - h.w);
          *reinterpret_cast<float4*>(rowp + ((c ^ sw) << 4)) = h;
          *reinterpret_cast<float4*>(rowp + (((c + 4) ^ sw) << 4)) = l;
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm->x_conv[quad][st]);       // the MMAs of this tile may start
      return true;
    };

    KMB_PROF(long long c_split = 0, w_acc = 0, c_ld = 0, c_arg = 0, c_upd = 0, t_all = clock64(), tw;)
    if (my_count > 0 && !split_tile(0)) ok = false;
    for (int jt = 0; jt < my_count && ok; ++jt) {
      const int t = quad + 4 * jt;
      const int m0 = ((int)blockIdx.x + t * (int)gridDim.x) * TC_BM;   // first row of the tile
      const bool valid = m0 + row < (int)p.n;
      // previous label and weight of this row: fetched now, used once the new label is known
      uint32_t prev_lab = 0xffffffffu;
      float wr = 1.f;
      if (update && valid) {
        if (p.prev != nullptr) prev_lab = __ldg(p.prev + m0 + row);
        if (p.w != nullptr) wr = __ldg(p.w + m0 + row);
      }
      // the quad's next tile is split now, so that its MMAs run under the work below
      KMB_PROF(tw = clock64();)
      if (jt + 1 < my_count && !split_tile(jt + 1)) break;
      KMB_PROF(c_split += clock64() - tw;)

      // ---- reduce every accumulator of the tile to this row's (score, index)
      float best = __int_as_float(0xff800000);
      float bif = 0.f;                             // the index is carried as a float
      const uint32_t g0 = (uint32_t)t * (uint32_t)n_nt;
      for (int i = 0; i < n_nt; ++i) {
        const uint32_t ab = (g0 + (uint32_t)i) & 3u;
        const int nt_w = (nt0 + i < n_nt) ? nt0 + i : nt0 + i - n_nt;
        const int cn = nt_w * TC_BN;
        KMB_PROF(tw = clock64();)
        if (!__all_sync(0xffffffffu, ts2_wait(&sm->acc_full[quad][ab], (seen >> ab) & 1u, sm, p.error_flag))) {
          ok = false;
          break;
        }
        KMB_PROF(w_acc += clock64() - tw;)
        seen ^= 1u << ab;
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)lane_base << 16) + ab * TC_BN;
        float qa = __int_as_float(0xff800000);
        float iaf = 0.f;
#pragma unroll 1
        for (int c4 = 0; c4 < 4; ++c4) {
          uint32_t v[32];
          KMB_PROF(tw = clock64();)
          tmem_ld32(taddr + c4 * 32, v);
          tmem_ld_wait();
          KMB_PROF(c_ld += clock64() - tw; tw = clock64();)
          if (c4 == 3) {
            // the whole accumulator has been read: hand the buffer back before the last argmax
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm->acc_empty[ab]);
          }
          float qv, ivf;
          argmax32_fidx(v, (float)(cn + c4 * 32), p.fone, qv, ivf);
          if (qv > qa) { qa = qv; iaf = ivf; }     // ascending inside the centroid tile: strict '>'
          KMB_PROF(c_arg += clock64() - tw;)
        }
        // centroid tiles arrive in rotated order: larger score wins, equal scores -> smaller index
        if (qa > best || (qa == best && iaf < bif)) {
          best = qa;
          bif = iaf;
        }
      }
      if (!ok) break;
      const uint32_t bi = (uint32_t)bif;

      // ---- label and update of this thread's own row
      KMB_PROF(tw = clock64();)
      if (valid) {
        p.labels[m0 + row] = bi;
        if (update) {
          changed += (prev_lab != bi) ? 1u : 0u;
          const float4* xrow = reinterpret_cast<const float4*>(p.X + (int64_t)(m0 + row) * p.d);
          float* dst = acc_copy + (int64_t)bi * p.d;
          atomicAdd(&acc_copy[(int64_t)p.k * p.d + bi], wr);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (u < n_chunks) {
              const float4 x = __ldg(xrow + u);
              float4 a4;
              a4.x = x.x * wr; a4.y = x.y * wr; a4.z = x.z * wr; a4.w = x.w * wr;
              atomicAdd(reinterpret_cast<float4*>(dst + 4 * u), a4);
            }
          }
        }
      }
      KMB_PROF(c_upd += clock64() - tw;)
    }
    KMB_PROF(if (blockIdx.x == 0 && lane == 0 && lq == 0) printf("[ss prof] quad %d: total %lld cyc, split of the next tile (with its wait) %lld, wait acc_full %lld, tensor-memory loads %lld, argmax %lld, update %lld, tiles %d\n", quad, clock64() - t_all, c_split, w_acc, c_ld, c_arg, c_upd, my_count);)
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
