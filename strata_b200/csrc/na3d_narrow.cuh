// Neighbourhood-attention forward for key rows of up to 16 columns (kernel width <= 9): the
// variant that runs TWO CTAs per SM.
//
// Why a second kernel: with narrow key rows a block of two units is 128 keys, and S (128
// columns), P (64) and O (64) of one query tile fit in 256 TMEM columns - half an SM's TMEM.
// A CTA then needs only six warps (TMA, MMA, four softmax warps), half the shared memory
// (one Q tile, a three-stage K/V ring) and can be resident twice per SM. Each CTA runs a
// simple, strictly ordered pipeline per key block
//     Q K^T -> S   |   softmax: S -> P   |   P V -> O
// and the latencies of that chain (MMA issue and completion, tcgen05.ld / st round trips,
// barrier hand-offs) are hidden by the OTHER CTA on the SM rather than by deeper buffering
// inside one CTA. One softmax thread owns one query row for the whole key block, so a thread
// has 64-128 independent scores per block to keep the FMA and exponential units fed.
//
//   warp 0   TMA producer: Q tile (single buffer, re-filled as soon as the item's last Q K^T
//            has completed) and K / V units (one box of 4 rows x EWP keys per unit).
//   warp 1   MMA issuer. After P(i) is ready it issues P V of block i, then Q K^T of block
//            i+1; the S-full arrival of block i+1 therefore also says that P(i) has been
//            consumed and O is up to date. Barrier arrivals through tcgen05.commit are kept to
//            two per block (P V done, S full): a commit costs the issuing thread about as
//            much as three MMAs.
//   warps 2-5  softmax, one thread per query row (TMEM lane quarter = warp & 3).
//            First block of an item seen by a warp: masked maximum first, to fix the
//            reference. Afterwards a block is handled in ONE pass against the current
//            reference with no maximum at all: the block's row sum doubles as the overflow
//            detector (a sum beyond 2^16, infinite or NaN means some score outran the
//            reference); only then the block maximum is taken, the reference moved (TMEM
//            accumulator and running sum rescaled) and the block redone. S is not overwritten
//            by P, so a redo is always possible. The row loops are kept rolled: the per-block
//            code stays small enough for the instruction caches with two CTAs resident.
//   P        bf16 pairs, column j of the P region holds keys 2j, 2j+1 of the block; rows a
//            query cannot see hold zeros.
#pragma once

namespace strata {

template <int KW>
struct Na3dNarrowCfg {
  static constexpr int EW = NA_QW + KW - 1;
  static constexpr int EWP = (EW + 7) / 8 * 8;                  // 8 or 16
  static constexpr int NKEYS = 8 * EWP;                         // 64 or 128
  static constexpr int THREADS = 192;
  static constexpr int S_COL = 0, P_COL = 128, O_COL = 192, TMEM_COLS = 256;
  static constexpr int KV_BYTES = NKEYS * 128;
  static constexpr int UNIT_BYTES = 4 * EWP * 128;
  static constexpr int Q_BYTES = 128 * 128;
  static constexpr int STAGES = 3;
  static constexpr int KV_OFF = Q_BYTES;
  static constexpr int BAR_OFF = KV_OFF + STAGES * 2 * KV_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256;
  static constexpr int PCOLS_ROW = EWP / 2;
  static_assert(EWP <= 16, "narrow variant: key rows of at most 16 columns");
  static_assert(TOTAL <= 115712, "two CTAs per SM: at most half of the SM's shared memory");
};

template <int KW>
__global__ void __launch_bounds__(Na3dNarrowCfg<KW>::THREADS, 2)
na3d_fwd_narrow_kernel(const __grid_constant__ CUtensorMap tmQ,
                       const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const Na3dParams p) {
  using Cfg = Na3dNarrowCfg<KW>;
  constexpr int EW = Cfg::EW;
  constexpr int EWP = Cfg::EWP;
  constexpr int NKEYS = Cfg::NKEYS;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  if ((sbase & 1023u) != 0) {  // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(&g_status, 0, ST_BAD_TMEM);
    return;
  }
  const uint32_t q_smem = sbase;
  auto k_smem = [&](int st) { return sbase + Cfg::KV_OFF + st * 2 * Cfg::KV_BYTES; };
  auto v_smem = [&](int st) { return k_smem(st) + Cfg::KV_BYTES; };
  const uint32_t bar = sbase + Cfg::BAR_OFF;
  const uint32_t q_full = bar, q_empty = bar + 8, s_full = bar + 16, p_ready = bar + 24;
  auto kv_full = [&](int st) { return bar + 32u + 8u * st; };
  auto pv_done = [&](int st) { return bar + 64u + 8u * st; };   // K/V stage free, O updated
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::BAR_OFF + 128);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::BAR_OFF + 136);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nblk = p.nblk;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_ready, 4);   // one arrival per softmax warp
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(pv_done(s), 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      bool ok = true;
      int n = 0, st = 0;
      uint32_t ph = 0;
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, ++n) {
        const NaItem it = na_decode_item<KW>(item, p);
        if (!mbar_wait(q_empty, (n & 1u) ^ 1u, abort_flag, ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(q_full, Cfg::Q_BYTES);
        tma_load_5d(q_smem, &tmQ, it.head * 64, it.w0, it.h0, it.d0, it.b, q_full);
        for (int i = 0; i < nblk; ++i) {
          if (!mbar_wait(pv_done(st), ph ^ 1u, abort_flag, ST_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          mbar_expect_tx(kv_full(st), 2 * Cfg::KV_BYTES);
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const uint32_t u = p.blk[i][s];
            const int kh0 = it.bh0 + 4 * static_cast<int>(u & 15u);
            const int kd0 = it.bd0 + static_cast<int>((u >> 4) & 15u);
            tma_load_5d(k_smem(st) + s * Cfg::UNIT_BYTES, &tmK, it.head * 64, it.bw0, kh0, kd0,
                        it.b, kv_full(st));
            tma_load_5d(v_smem(st) + s * Cfg::UNIT_BYTES, &tmV, it.head * 64, it.bw0, kh0, kd0,
                        it.b, kv_full(st));
          }
          if (++st == STAGES) { st = 0; ph ^= 1u; }
        }
      }
      if (!ok)
#pragma unroll 1
        for (int i = 0; i < 2000; ++i) __nanosleep(100);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, NKEYS, false, false);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 64, false, true);
      constexpr int PV_STEPS = NKEYS / 16;
      constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t STAGE_UNITS = (2 * Cfg::KV_BYTES) >> 4;
      auto lo_of = [](uint32_t addr) { return ((addr & 0x3FFFFu) >> 4) | (1u << 16); };
      auto desc = [](uint32_t lo) { return (static_cast<uint64_t>(DESC_HI) << 32) | lo; };
      const uint32_t q_lo = lo_of(q_smem);
      const uint32_t k_lo0 = lo_of(k_smem(0));
      const uint32_t v_lo0 = lo_of(v_smem(0));
      const uint32_t s_tmem = tmem_base + Cfg::S_COL;
      const uint32_t p_tmem = tmem_base + Cfg::P_COL;
      const uint32_t o_tmem = tmem_base + Cfg::O_COL;

      int qk_st = 0;
      uint32_t qk_ph = 0;
      auto issue_qk = [&]() -> bool {
        if (!mbar_wait(kv_full(qk_st), qk_ph, abort_flag, ST_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint32_t klo = k_lo0 + qk_st * STAGE_UNITS;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_ss(s_tmem, desc(q_lo + 2u * k), desc(klo + 2u * k), idesc_qk, k != 0 ? 1u : 0u);
        umma_commit(s_full);
        if (++qk_st == STAGES) { qk_st = 0; qk_ph ^= 1u; }
        return true;
      };

      bool ok = true;
      int n = 0, pv_st = 0;
      uint32_t gb = 0;
      bool pre_issued = false;   // S of this item's block 0 was issued during the previous item
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, ++n) {
        if (!pre_issued) {
          if (!mbar_wait(q_full, n & 1u, abort_flag, ST_TIMEOUT_MMA)) break;
          if (!issue_qk()) break;
          if (nblk == 1) umma_commit(q_empty);
        }
        pre_issued = false;
        for (int i = 0; i < nblk; ++i, ++gb) {
          if (!mbar_wait(p_ready, gb & 1u, abort_flag, ST_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          // O += P V of this block ...
          const uint32_t vlo = v_lo0 + pv_st * STAGE_UNITS;
#pragma unroll
          for (int s = 0; s < PV_STEPS; ++s)
            umma_ts(o_tmem, p_tmem + 8 * s, desc(vlo + 128u * s), idesc_pv,
                    (s != 0 || i != 0) ? 1u : 0u);
          umma_commit(pv_done(pv_st));
          if (++pv_st == STAGES) pv_st = 0;
          // ... then the scores of the next block (of this item, or block 0 of the next item);
          // its S-full arrival also tells the softmax warps that P has been consumed
          if (i + 1 < nblk) {
            if (!issue_qk()) { ok = false; break; }
            if (i + 2 == nblk) umma_commit(q_empty);   // last Q K^T of this item issued
          } else if (item + static_cast<int>(gridDim.x) < p.n_items) {
            if (!mbar_wait(q_full, (n + 1) & 1u, abort_flag, ST_TIMEOUT_MMA)) {
              ok = false;
              break;
            }
            if (!issue_qk()) { ok = false; break; }
            if (nblk == 1) umma_commit(q_empty);
            pre_issued = true;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax warps
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;        // query row
    const int zw = r & 7;
    const int zh = (r >> 3) % p.QH;
    const int zd = (r >> 3) / p.QH;
    const uint32_t lane_taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_taddr = lane_taddr + Cfg::S_COL;
    const uint32_t p_taddr = lane_taddr + Cfg::P_COL;
    const uint32_t o_taddr = lane_taddr + Cfg::O_COL;
    const float c = p.scale_log2e;
    constexpr float SUM_LIMIT = 65536.0f;

    bool ok = true;
    uint32_t gb = 0;
    int st_prev = STAGES - 1;     // ring stage and phase of block gb-1 (for pv_done)
    uint32_t ph_prev = 1;
    for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
      const NaItem it = na_decode_item<KW>(item, p);
      const bool q_ok = (it.d0 + zd < p.D) && (it.h0 + zh < p.q_h0 + p.q_H) &&
                        (it.w0 + zw < p.q_w0 + p.q_W);
      const int id = min(it.d0 + zd, p.D - 1), ih = min(it.h0 + zh, p.H - 1),
                iw = min(it.w0 + zw, p.W - 1);
      const int wd = na_window_start(id, p.D, p.kd) - it.bd0;
      const int wh = na_window_start(ih, p.H, p.kh) - it.bh0;
      const int ww = na_window_start(iw, p.W, KW) - it.bw0;
      const uint32_t hmask_all = ((1u << p.kh) - 1u) << wh;   // bit = key row of the box

      // Scores are handled in scaled form t = s*c - mc (c = scale*log2 e, mc the scaled
      // reference). nb2 holds, per pair of key columns, the addend of that form: -mc inside
      // the query's window, -1e30 outside (the column mask).
      float mc = 0.f, l_run = 0.f;
      uint64_t nb2[EW / 2];
      auto set_nb = [&](float ref) {
#pragma unroll
        for (int k2 = 0; k2 < EW / 2; ++k2) {
          const float lo = (static_cast<unsigned>(2 * k2 - ww) < static_cast<unsigned>(KW)) ? -ref : -1e30f;
          const float hi = (static_cast<unsigned>(2 * k2 + 1 - ww) < static_cast<unsigned>(KW)) ? -ref : -1e30f;
          nb2[k2] = pack2(lo, hi);
        }
      };
      set_nb(0.f);
      const uint64_t c2 = pack2(c, c);

      for (int i = 0; i < nblk; ++i, ++gb) {
        // this thread's 8 key rows of the block: bit rr set = row rr lies in the query's window
        uint32_t rowmask = 0;
        {
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const uint32_t u = p.blk[i][s];
            const bool pl_ok = (u >> 15) == 0u &&
                               static_cast<unsigned>(static_cast<int>((u >> 4) & 15u) - wd) <
                                   static_cast<unsigned>(p.kd);
            const uint32_t m = pl_ok ? (hmask_all >> (4u * (u & 15u))) & 15u : 0u;
            rowmask |= m << (4 * s);
          }
        }
        const uint32_t warp_rows = __reduce_or_sync(0xffffffffu, rowmask);
        if (!mbar_wait(s_full, gb & 1u, abort_flag, ST_TIMEOUT_SOFTMAX)) {
          ok = false;
          break;
        }
        tc_fence_after();

        // The row loops below are deliberately not unrolled over rows: the whole per-block body
        // stays a few kilobytes of code, which two resident CTAs can keep in the instruction
        // caches; rows no query of the warp can see are skipped warp-uniformly.
        bool take_max = warp_rows != 0u && __any_sync(0xffffffffu, l_run == 0.f);
        bool settled = false;
        float rs_blk;
#pragma unroll 1
        while (true) {
          if (take_max) {
            // masked maximum of this thread's visible scores (scaled form) ...
            float bm = -1e30f;
#pragma unroll 1
            for (int rr = 0; rr < 8; ++rr) {
              if (!((warp_rows >> rr) & 1u)) continue;
              uint32_t a[EWP];
              tmem_ld_keyrow<EWP>(s_taddr + rr * EWP, a);
              tmem_ld_wait();
              float rm0 = -1e30f, rm1 = -1e30f;
#pragma unroll
              for (int k2 = 0; k2 < EW / 2; ++k2) {
                float t0, t1;
                unpack2(ffma2(pack2u(a[2 * k2], a[2 * k2 + 1]), c2, nb2[k2]), t0, t1);
                if (k2 & 1) rm1 = fmax3(rm1, t0, t1); else rm0 = fmax3(rm0, t0, t1);
              }
              bm = fmaxf(bm, ((rowmask >> rr) & 1u) ? fmaxf(rm0, rm1) : -1e30f);
            }
            // ... moves the reference up by bm where that is called for: always while nothing
            // has been accumulated yet (free), otherwise only beyond a margin of 2^8 - then the
            // TMEM accumulator and the running sum are rescaled (the previous block's P V has
            // completed: its commit precedes this block's S-full commit).
            const bool fresh = l_run == 0.f;
            const bool grow = fresh ? (bm > -1e29f) : (bm > 8.0f);
            const bool rescale = grow && !fresh;
            if (__any_sync(0xffffffffu, rescale)) {
              const float alpha = rescale ? fast_exp2(-bm) : 1.0f;
              l_run *= alpha;
#pragma unroll 1
              for (int hh = 0; hh < 4; ++hh) {
                uint32_t ob[16];
                tmem_ld_x16(o_taddr + 16 * hh, ob);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  ob[j] = __float_as_uint(__uint_as_float(ob[j]) * alpha);
                tmem_st_x16(o_taddr + 16 * hh, ob);
              }
              tmem_st_wait();
            }
            if (grow) {
              mc += bm;
              set_nb(mc);
            }
            settled = true;
          }
          // exponentials, row sum and bf16 P (two keys per 32-bit column), two key rows at a time
          uint64_t rs2 = 0ull;
#pragma unroll 1
          for (int pr = 0; pr < 4; ++pr) {
            const uint32_t need2 = (warp_rows >> (2 * pr)) & 3u;
            const uint32_t mine2 = (rowmask >> (2 * pr)) & 3u;
            uint32_t pk[2][Cfg::PCOLS_ROW];
            if (need2 == 0u) {
#pragma unroll
              for (int j = 0; j < Cfg::PCOLS_ROW; ++j) pk[0][j] = pk[1][j] = 0u;
            } else {
              uint32_t a[2][EWP];
              tmem_ld_keyrow<EWP>(s_taddr + (2 * pr) * EWP, a[0]);
              tmem_ld_keyrow<EWP>(s_taddr + (2 * pr + 1) * EWP, a[1]);
              tmem_ld_wait();
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const bool mine = (mine2 >> h) & 1u;
                const uint32_t keep = mine ? 0xffffffffu : 0u;
                uint64_t rsa = 0ull, rsb = 0ull;
#pragma unroll
                for (int k2 = 0; k2 < Cfg::PCOLS_ROW; ++k2) {
                  uint32_t packed = 0u;
                  if (k2 < EW / 2) {
                    float t0, t1;
                    unpack2(ffma2(pack2u(a[h][2 * k2], a[h][2 * k2 + 1]), c2, nb2[k2]), t0, t1);
                    const float p0 = fast_exp2(t0), p1 = fast_exp2(t1);
                    if (k2 & 1) rsb = fadd2(rsb, pack2(p0, p1)); else rsa = fadd2(rsa, pack2(p0, p1));
                    packed = pack_bf16(p0, p1) & keep;
                  }
                  pk[h][k2] = packed;
                }
                if (mine) rs2 = fadd2(rs2, fadd2(rsa, rsb));
              }
            }
            if constexpr (EWP == 16) {
              tmem_st_x16(p_taddr + 16 * pr, &pk[0][0]);
            } else {
              tmem_st_x8(p_taddr + 8 * pr, &pk[0][0]);
            }
          }
          {
            float r0, r1;
            unpack2(rs2, r0, r1);
            rs_blk = r0 + r1;
          }
          // a sum this large (or infinite, or NaN) means a score far above the reference:
          // take the maximum after all and redo the block (S is still intact)
          if (settled || !__any_sync(0xffffffffu, !(rs_blk < SUM_LIMIT))) break;
          take_max = true;
        }
        l_run += rs_blk;
        // every lane completes its P stores, then one lane arrives for the warp
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready);
        if (++st_prev == STAGES) { st_prev = 0; ph_prev ^= 1u; }
      }
      if (!ok) break;

      // item epilogue: wait for the last P V, normalise this thread's row and store it
      if (!mbar_wait(pv_done(st_prev), ph_prev, abort_flag, ST_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
      tc_fence_after();
      {
        const float inv = 1.0f / l_run;
        const long long tok = ((static_cast<long long>(it.b) * p.D + (it.d0 + zd)) * p.q_H +
                               (it.h0 + zh - p.q_h0)) * p.q_W + (it.w0 + zw - p.q_w0);
        __nv_bfloat16* op = p.out + tok * p.ldo + it.head * 64;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t ob[32];
          tmem_ld_32x32(o_taddr + 32 * hh, ob);
          tmem_ld_wait();
          if (q_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 v4;
              v4.x = pack_bf16(__uint_as_float(ob[j]) * inv, __uint_as_float(ob[j + 1]) * inv);
              v4.y = pack_bf16(__uint_as_float(ob[j + 2]) * inv, __uint_as_float(ob[j + 3]) * inv);
              v4.z = pack_bf16(__uint_as_float(ob[j + 4]) * inv, __uint_as_float(ob[j + 5]) * inv);
              v4.w = pack_bf16(__uint_as_float(ob[j + 6]) * inv, __uint_as_float(ob[j + 7]) * inv);
              *reinterpret_cast<uint4*>(op + 32 * hh + j) = v4;
            }
          }
        }
        tc_fence_before();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace strata
