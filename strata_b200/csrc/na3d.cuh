// Fused 3-D neighbourhood attention forward for sm_100a (head_dim 64, bf16, non-causal,
// dilation 1): for every query token, softmax(q.k * scale) over the kd*kh*kw keys of its
// window, times v. Windows keep their full size at the borders: along an axis of length L
// the window of query i starts at clamp(i - k/2, 0, L - k).
//
// Work decomposition (persistent kernel, one CTA per SM)
//   work item      one tile of 128 queries (QD x QH x 8 tokens) of one head of one batch entry;
//                  CTA c handles items c, c + gridDim.x, ... (neighbouring items are
//                  neighbouring tiles of the same head, so their key halos meet in L2).
//   key blocks     the union of a tile's windows is a box of ED x EH x EW keys
//                  (E* = Q* + k* - 1) starting at the window start of the tile's first query.
//                  The box is cut into units of one depth plane x 4 rows x EWP columns
//                  (EWP = EW padded) and streamed as blocks of TWO units (NKEYS = 8*EWP <= 192);
//                  TMA zero-fills whatever lies outside the tensor. Which two units share a
//                  block is a host-built table: each quarter of the tile (32 queries = one warp
//                  per softmax group = one SM sub-partition) sees only part of the box, so units
//                  are paired such that, wherever possible, every quarter finds exactly one
//                  visible unit in every block - the exponential work is then spread evenly
//                  over the sub-partitions instead of the busiest quarter setting the pace.
//   warp 0         TMA producer: Q tile (double-buffered across items) and the K / V blocks into
//                  a 2-3 stage ring (5-D tensor maps over [B, D, H, W, channels]; 128-byte
//                  swizzle, a key's 64 channels are one 128-byte row). Runs ahead across items.
//   warp 1         MMA issuer: S = Q K^T (M=128, N=NKEYS, K=64) into one of two TMEM buffers -
//                  block i+1 is issued before the softmax of block i has finished - then
//                  O_g += P_g V_g (M=128, N=64) for each key group g; O_g stays in TMEM for
//                  the whole item.
//   softmax warps  NG groups of 4 warps (NG = 4 for key blocks of up to 128 keys, else 2). A
//                  query row is shared by one thread of each group; with four groups, group g
//                  owns row g of both units of every block (the producer stores the rows
//                  group-major), with two groups, group g owns unit g. A group keeps its own
//                  reference maximum and running sum - no exchange between groups per block.
//                  Per block:
//                  pass 1 reads the thread's S row segments from TMEM and takes the masked
//                  maximum, pass 2 re-reads them, exponentiates, writes bf16 P into the
//                  swizzled A-operand layout (double-buffered) and adds to the running sum.
//                  The reference maximum moves (and the group's TMEM accumulator is rescaled
//                  through tcgen05.ld / tcgen05.st) only when a block maximum exceeds it by
//                  more than 2^8, which after the first block or two is rare. Key rows no query
//                  of the warp can see are skipped (zeros written) without touching the
//                  exponential unit. At the end of an item the groups publish (max, sum) in
//                  shared memory, and every thread combines the NG accumulators of its row
//                  straight from TMEM for its own slice of the 64 output channels.
//   mask           per (query, key): the key's box coordinates must fall in the query's window
//                  on all three axes. Columns: an additive per-thread bias vector (0 / -1e30);
//                  rows: a per-thread bit mask; planes: one comparison per block. Border
//                  clamping is therefore exact per query row.
//   barriers       all mbarrier waits are bounded. Barriers that consecutive blocks would
//                  otherwise share (S full, P ready, O full) alternate by block parity, so an
//                  arrival for block i+1 can never be counted for block i.
#pragma once
#include "common.cuh"
#include "tensormap.cuh"

// Key-row width up to which four softmax groups are used (wider key blocks need the TMEM
// columns for S and run with two).
#ifndef NA_NG4_MAX_EW
#define NA_NG4_MAX_EW 16
#endif

namespace strata {

constexpr int NA_MAX_BLOCKS = 64;   // 16 planes x 8 chunks / 2

struct Na3dParams {
  int B, D, H, W, heads;
  int kd, kh;            // kernel extents along depth and rows (columns: template KW)
  int QD, QH;            // query tile extents (QW = 8); QD*QH = 16
  int tiles_d, tiles_h, tiles_w;
  // Query region: only tokens with h in [q_h0, q_h0+q_H), w in [q_w0, q_w0+q_W) are queries
  // (the interior of a halo-padded tile; the whole plane by default). Keys come from the
  // whole [H, W] plane. Outputs are written compactly as [B, D, q_H, q_W, ldo].
  int q_h0, q_H, q_w0, q_W;
  int n_items;           // tiles_d*tiles_h*tiles_w*heads*B
  int nblk;              // key blocks per item
  // blk[i][s]: unit in slot s of block i: chunk (4 rows) in bits 0-3, plane in bits 4-7;
  // bit 15: the slot only repeats another unit to keep the block full - ignore its keys.
  unsigned short blk[NA_MAX_BLOCKS][2];
  __nv_bfloat16* out;    // [B, D, H, W, ldo] with head h at channel offset h*64
  long long ldo;
  float scale_log2e;
};

constexpr int NA_QW = 8;
constexpr int NA_TMEM_COLS = 512;

template <int KW>
struct Na3dCfg {
  static constexpr int EW = NA_QW + KW - 1;
  static constexpr int NG = (EW <= NA_NG4_MAX_EW) ? 4 : 2;      // softmax groups
  static constexpr int EWP = (NG == 4) ? (EW + 7) / 8 * 8 : (EW + 3) / 4 * 4;
  static constexpr int NKEYS = 8 * EWP;
  static constexpr int RPG = 8 / NG;                            // key rows per group
  static constexpr int GKEYS = RPG * EWP;                       // keys per group per block
  static constexpr int THREADS = 64 + 128 * NG;
  static constexpr int SCOLS = (NG == 4) ? 128 : 192;           // TMEM columns per S buffer
  static constexpr int O_COL = 2 * SCOLS;                       // O of group g at O_COL + 64 g
  static constexpr int KV_BYTES = NKEYS * 128;
  static constexpr int ROW_BYTES = EWP * 128;                   // one key row in shared memory
  static constexpr int Q_BYTES = 128 * 128;
  static constexpr int KV_OFF = 2 * Q_BYTES;
  static constexpr int ML_BYTES = 2 * NG * 128 * 8;             // [2][NG][128] (max, sum)
  // K/V ring as deep as shared memory allows: its depth hides the TMA round trip
  static constexpr int STAGES_FIT = (227 * 1024 - KV_OFF - ML_BYTES - 256) / (2 * KV_BYTES);
  static constexpr int STAGES = STAGES_FIT > 6 ? 6 : STAGES_FIT;
  static constexpr int ML_OFF = KV_OFF + STAGES * 2 * KV_BYTES;
  static constexpr int BAR_OFF = ML_OFF + ML_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256;
  static constexpr int PCOLS_ROW = EWP / 2;                     // packed-P columns per key row
  static_assert(NKEYS <= SCOLS && GKEYS % 16 == 0, "key block layout");
  static_assert(O_COL + 64 * NG <= NA_TMEM_COLS, "TMEM budget");
  static_assert(TOTAL <= 227 * 1024 && STAGES >= 2, "shared memory budget");
};

__device__ __forceinline__ int na_window_start(int i, int L, int k) {
  int s = i - (k >> 1);
  s = s < 0 ? 0 : s;
  return s > L - k ? L - k : s;
}

__device__ __forceinline__ void tmem_ld_x4(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_x8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                 "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// Loads EWP (8, 12, 16, 20 or 24) consecutive S columns of this thread's row.
template <int EWP>
__device__ __forceinline__ void tmem_ld_keyrow(uint32_t taddr, uint32_t* a) {
  if constexpr (EWP == 8) {
    tmem_ld_x8(taddr, a);
  } else if constexpr (EWP == 12) {
    tmem_ld_x8(taddr, a);
    tmem_ld_x4(taddr + 8, a + 8);
  } else if constexpr (EWP == 16) {
    tmem_ld_x16(taddr, a);
  } else if constexpr (EWP == 20) {
    tmem_ld_x16(taddr, a);
    tmem_ld_x4(taddr + 16, a + 16);
  } else {
    tmem_ld_x16(taddr, a);
    tmem_ld_x8(taddr + 16, a + 16);
  }
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_x8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]),
                 "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st_x4(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3])
               : "memory");
}
__device__ __forceinline__ void tmem_st_x2(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1])
               : "memory");
}
// Stores N (4, 6, 8, 10 or 12) consecutive 32-bit columns of this thread's row.
template <int N>
__device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const uint32_t* r) {
  static_assert(N == 4 || N == 6 || N == 8 || N == 10 || N == 12, "unsupported column count");
  if constexpr (N == 4) {
    tmem_st_x4(taddr, r);
  } else if constexpr (N == 6) {
    tmem_st_x4(taddr, r);
    tmem_st_x2(taddr + 4, r + 4);
  } else {
    tmem_st_x8(taddr, r);
    if constexpr (N == 10) tmem_st_x2(taddr + 8, r + 8);
    if constexpr (N == 12) tmem_st_x4(taddr + 8, r + 8);
  }
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

struct NaItem {
  int b, head, d0, h0, w0, bd0, bh0, bw0;
};
template <int KW>
__device__ __forceinline__ NaItem na_decode_item(int item, const Na3dParams& p) {
  NaItem it;
  int t = item;
  const int tw = t % p.tiles_w; t /= p.tiles_w;
  const int th = t % p.tiles_h; t /= p.tiles_h;
  const int td = t % p.tiles_d; t /= p.tiles_d;
  it.head = t % p.heads;
  it.b = t / p.heads;
  it.d0 = td * p.QD; it.h0 = p.q_h0 + th * p.QH; it.w0 = p.q_w0 + tw * NA_QW;
  // key box origin = window start of the tile's first query on each axis
  it.bd0 = na_window_start(it.d0, p.D, p.kd);
  it.bh0 = na_window_start(it.h0, p.H, p.kh);
  it.bw0 = na_window_start(it.w0, p.W, KW);
  return it;
}

template <int KW>
__global__ void __launch_bounds__(Na3dCfg<KW>::THREADS, 1)
na3d_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const Na3dParams p) {
  using Cfg = Na3dCfg<KW>;
  constexpr int EW = Cfg::EW;
  constexpr int EWP = Cfg::EWP;
  constexpr int NKEYS = Cfg::NKEYS;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int NG = Cfg::NG;
  constexpr int RPG = Cfg::RPG;
  constexpr int GKEYS = Cfg::GKEYS;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  if ((sbase & 1023u) != 0) {  // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(&g_status, 0, ST_BAD_TMEM);
    return;
  }
  auto q_smem = [&](int qb) { return sbase + qb * Cfg::Q_BYTES; };
  auto k_smem = [&](int st) { return sbase + Cfg::KV_OFF + st * 2 * Cfg::KV_BYTES; };
  auto v_smem = [&](int st) { return k_smem(st) + Cfg::KV_BYTES; };
  float2* ml = reinterpret_cast<float2*>(smem + Cfg::ML_OFF);
  const uint32_t bar = sbase + Cfg::BAR_OFF;
  // barriers, 8 bytes each
  auto q_full = [&](uint32_t i) { return bar + 8u * i; };             // 0,1
  auto q_empty = [&](uint32_t i) { return bar + 16u + 8u * i; };      // 2,3
  auto s_full = [&](uint32_t i) { return bar + 32u + 8u * i; };       // 4,5
  auto p_ready = [&](uint32_t i) { return bar + 48u + 8u * i; };      // 6,7   (by block parity)
  auto o_full = [&](uint32_t i) { return bar + 64u + 8u * i; };       // 8,9   (by block parity)
  auto ml_ready = [&](uint32_t i) { return bar + 80u + 8u * i; };     // 10,11 (by item parity)
  auto kv_full = [&](int st) { return bar + 96u + 8u * st; };         // 12..17
  auto kv_empty = [&](int st) { return bar + 144u + 8u * st; };       // 18..23
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::BAR_OFF + 224);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::BAR_OFF + 232);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int nblk = p.nblk;

  if (threadIdx.x == 0) {
    for (uint32_t i = 0; i < 2; ++i) {
      mbar_init(q_full(i), 1);
      mbar_init(q_empty(i), 1);
      mbar_init(s_full(i), 1);
      mbar_init(p_ready(i), 4 * NG);    // one arrival per softmax warp
      mbar_init(o_full(i), 1);
      mbar_init(ml_ready(i), 4 * NG);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), NA_TMEM_COLS);
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
      int n = 0;
      int st = 0;
      uint32_t ph = 0;
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, ++n) {
        const NaItem it = na_decode_item<KW>(item, p);
        const uint32_t qb = n & 1;
        if (!mbar_wait(q_empty(qb), ((n >> 1) & 1u) ^ 1u, abort_flag, ST_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(q_full(qb), Cfg::Q_BYTES);
        tma_load_5d(q_smem(qb), &tmQ, it.head * 64, it.w0, it.h0, it.d0, it.b, q_full(qb));
        for (int i = 0; i < nblk; ++i) {
          if (!mbar_wait(kv_empty(st), ph ^ 1u, abort_flag, ST_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          mbar_expect_tx(kv_full(st), 2 * Cfg::KV_BYTES);
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const uint32_t u = p.blk[i][s];
            const int kh0 = it.bh0 + 4 * static_cast<int>(u & 15u);
            const int kd0 = it.bd0 + static_cast<int>((u >> 4) & 15u);
            if constexpr (NG == 4) {
              // one load per key row; row r of slot s lands at position 2r + s (group-major)
#pragma unroll
              for (int r = 0; r < 4; ++r) {
                const uint32_t off = (2 * r + s) * Cfg::ROW_BYTES;
                tma_load_5d(k_smem(st) + off, &tmK, it.head * 64, it.bw0, kh0 + r, kd0, it.b,
                            kv_full(st));
                tma_load_5d(v_smem(st) + off, &tmV, it.head * 64, it.bw0, kh0 + r, kd0, it.b,
                            kv_full(st));
              }
            } else {
              const uint32_t off = s * 4 * Cfg::ROW_BYTES;
              tma_load_5d(k_smem(st) + off, &tmK, it.head * 64, it.bw0, kh0, kd0, it.b, kv_full(st));
              tma_load_5d(v_smem(st) + off, &tmV, it.head * 64, it.bw0, kh0, kd0, it.b, kv_full(st));
            }
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
    // One thread issues every MMA, so its instruction stream is kept short: descriptors are
    // two 32-bit halves (a constant high word, a low word that is a base plus compile-time
    // offsets), ring positions are carried incrementally.
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, NKEYS, false, false);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 64, false, true);
      constexpr int GROUP_STEPS = GKEYS / 16;  // 16-key MMA steps per key group
      constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t STAGE_UNITS = (2 * Cfg::KV_BYTES) >> 4;
      auto lo_of = [](uint32_t addr) { return ((addr & 0x3FFFFu) >> 4) | (1u << 16); };
      auto desc = [](uint32_t lo) { return (static_cast<uint64_t>(DESC_HI) << 32) | lo; };
      const uint32_t q_lo[2] = {lo_of(q_smem(0)), lo_of(q_smem(1))};
      const uint32_t k_lo0 = lo_of(k_smem(0));
      const uint32_t v_lo0 = lo_of(v_smem(0));
      const uint32_t o_tmem = tmem_base + Cfg::O_COL;

      // position of the next Q K^T to issue (runs one block ahead of the P V position)
      int qk_st = 0;
      uint32_t qk_ph = 0, qk_sb = 0;
      auto issue_qk = [&](uint32_t qlo) -> bool {
        if (!mbar_wait(kv_full(qk_st), qk_ph, abort_flag, ST_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint32_t klo = k_lo0 + qk_st * STAGE_UNITS;
        const uint32_t s_tmem = tmem_base + (qk_sb ? Cfg::SCOLS : 0);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_ss(s_tmem, desc(qlo + 2u * k), desc(klo + 2u * k), idesc_qk, k != 0 ? 1u : 0u);
        umma_commit(s_full(qk_sb));
        qk_sb ^= 1u;
        if (++qk_st == STAGES) { qk_st = 0; qk_ph ^= 1u; }
        return true;
      };

      bool ok = true;
      int n = 0;
      int pv_st = 0;
      uint32_t pv_par = 0;     // block parity of the next P V (p_ready / o_full barrier, P buffer)
      uint32_t pv_cnt = 0;     // number of P V blocks issued so far
      bool pre_issued = false; // S of this item's block 0 was issued at the end of the previous item
      for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, ++n) {
        const uint32_t qb = n & 1;
        if (!pre_issued) {
          if (!mbar_wait(q_full(qb), (n >> 1) & 1u, abort_flag, ST_TIMEOUT_MMA)) break;
          if (!issue_qk(q_lo[qb])) break;
        }
        pre_issued = false;
        for (int i = 0; i < nblk; ++i) {
          // run ahead: S of the next block (of this item, or block 0 of the next item)
          if (i + 1 < nblk) {
            if (!issue_qk(q_lo[qb])) { ok = false; break; }
            if (i + 2 == nblk) umma_commit(q_empty(qb));   // last Q K^T of this item issued
          } else {
            if (nblk == 1) umma_commit(q_empty(qb));
            if (item + static_cast<int>(gridDim.x) < p.n_items) {
              const uint32_t nq = (n + 1) & 1;
              if (!mbar_wait(q_full(nq), ((n + 1) >> 1) & 1u, abort_flag, ST_TIMEOUT_MMA)) {
                ok = false;
                break;
              }
              if (!issue_qk(q_lo[nq])) { ok = false; break; }
              pre_issued = true;
            }
          }
          if (!mbar_wait(p_ready(pv_par), (pv_cnt >> 1) & 1u, abort_flag, ST_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t vlo = v_lo0 + pv_st * STAGE_UNITS;
          const uint32_t p_tmem = tmem_base + (pv_par ? Cfg::SCOLS : 0);   // P aliases S
          const uint32_t acc = i != 0 ? 1u : 0u;   // O accumulates over the blocks of the item
#pragma unroll
          for (int g = 0; g < NG; ++g) {
#pragma unroll
            for (int s0 = 0; s0 < GROUP_STEPS; ++s0) {
              const int s = g * GROUP_STEPS + s0;
              // P: bf16 pairs in the group's S columns, 8 columns per 16-key step;
              // V: 16 keys = 16 rows of 128 bytes per step (2048 bytes = 128 units)
              umma_ts(o_tmem + 64 * g, p_tmem + g * GKEYS + 8 * s0, desc(vlo + 128u * s),
                      idesc_pv, s0 != 0 ? 1u : acc);
            }
          }
          umma_commit(kv_empty(pv_st));
          umma_commit(o_full(pv_par));
          pv_par ^= 1u;
          ++pv_cnt;
          if (++pv_st == STAGES) pv_st = 0;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax warps
    const int quarter = warp & 3;
    const int grp = (warp - 2) >> 2;          // key group this thread owns
    const int r = quarter * 32 + lane;        // query row
    const int zw = r & 7;
    const int zh = (r >> 3) % p.QH;
    const int zd = (r >> 3) / p.QH;
    const uint32_t lane_taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t o_taddr = lane_taddr + Cfg::O_COL + 64 * grp;
    const float c = p.scale_log2e;
    constexpr uint32_t ROWBITS = (1u << RPG) - 1u;

    bool ok = true;
    int n = 0;
    uint32_t gb = 0;
    for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, ++n) {
      const NaItem it = na_decode_item<KW>(item, p);
      const bool q_ok = (it.d0 + zd < p.D) && (it.h0 + zh < p.q_h0 + p.q_H) &&
                        (it.w0 + zw < p.q_w0 + p.q_W);
      const int id = min(it.d0 + zd, p.D - 1), ih = min(it.h0 + zh, p.H - 1),
                iw = min(it.w0 + zw, p.W - 1);
      const int wd = na_window_start(id, p.D, p.kd) - it.bd0;
      const int wh = na_window_start(ih, p.H, p.kh) - it.bh0;
      const int ww = na_window_start(iw, p.W, KW) - it.bw0;
      const uint32_t hmask_all = ((1u << p.kh) - 1u) << wh;   // bit = key row of the box

      // Scores are handled in scaled form t = s*c - mc (c = scale*log2 e), where mc is the
      // scaled reference of this thread's key group. nb2 holds, per pair of key columns, the
      // addend of that form: -mc inside the query's window, -1e30 outside (the column mask).
      // The output accumulator lives in TMEM and is touched only when the reference moves.
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
        const uint32_t sb = gb & 1u;
        if (!mbar_wait(s_full(sb), (gb >> 1) & 1u, abort_flag, ST_TIMEOUT_SOFTMAX)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t s_taddr = lane_taddr + (sb ? Cfg::SCOLS : 0) + grp * GKEYS;
        // which of this thread's RPG key rows of the block lie inside its query's window
        uint32_t rowmask;
        {
          auto plane_ok = [&](uint32_t u) {
            return (u >> 15) == 0u &&
                   static_cast<unsigned>(static_cast<int>((u >> 4) & 15u) - wd) <
                       static_cast<unsigned>(p.kd);
          };
          if constexpr (NG == 4) {
            const uint32_t u0 = p.blk[i][0], u1 = p.blk[i][1];
            const uint32_t b0 = plane_ok(u0) ? (hmask_all >> (4u * (u0 & 15u) + grp)) & 1u : 0u;
            const uint32_t b1 = plane_ok(u1) ? (hmask_all >> (4u * (u1 & 15u) + grp)) & 1u : 0u;
            rowmask = b0 | (b1 << 1);
          } else {
            const uint32_t u = p.blk[i][grp];
            rowmask = plane_ok(u) ? (hmask_all >> (4u * (u & 15u))) & ROWBITS : 0u;
          }
        }
        const uint32_t warp_rows = __reduce_or_sync(0xffffffffu, rowmask);

        // The reference of a key group moves only when a block maximum exceeds it by more than
        // 2^8 (P stays well inside bf16 / fp32 range otherwise) - or is adopted for free while
        // nothing has been accumulated yet. Moving it rescales the TMEM accumulator, which must
        // wait for the previous block's P V (o_full of that block's parity; S of the current
        // block being complete implies P V of block gb-2 is, so the parity wait cannot alias).
        auto apply_reference = [&](float bm) -> bool {
          const bool fresh = l_run == 0.f;
          const bool grow = fresh ? (bm > -1e29f) : (bm > 8.0f);
          const bool rescale = grow && !fresh;
          if (__any_sync(0xffffffffu, rescale)) {
            if (!mbar_wait(o_full((gb - 1u) & 1u), ((gb - 1u) >> 1) & 1u, abort_flag,
                           ST_TIMEOUT_SOFTMAX))
              return false;
            tc_fence_after();
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
          return true;
        };

        // While some query of the warp has no reference yet, the block maximum is taken first
        // (pass 1). Afterwards a block is handled in a single pass against the current reference;
        // its maximum is tracked on the side and, should it overshoot the 2^8 margin (rare), the
        // reference is moved and the block is redone before anything is stored.
        // (With four groups the register budget is too tight for the extra bookkeeping, and the
        // two-pass form is used for every block.)
        constexpr bool SINGLE_PASS = (NG == 2);
        bool settled = SINGLE_PASS ? __any_sync(0xffffffffu, l_run == 0.f) : true;
        if (settled) {
          float bm = -1e30f;
#pragma unroll
          for (int rr = 0; rr < RPG; ++rr) {
            if ((warp_rows >> rr) & 1u) {
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
          }
          if (!apply_reference(bm)) {
            ok = false;
            break;
          }
        }

        // exponentials, row sum and bf16 P (two keys per 32-bit column), held in registers
        // until the block is known to be final
        uint32_t pk[RPG][Cfg::PCOLS_ROW];
        uint64_t rs2;
#pragma unroll 1
        while (true) {
          rs2 = 0ull;
          float tm0 = -1e30f, tm1 = -1e30f;
#pragma unroll
          for (int rr = 0; rr < RPG; ++rr) {
            const bool need = (warp_rows >> rr) & 1u;
            const bool mine = (rowmask >> rr) & 1u;
            const uint32_t keep = mine ? 0xffffffffu : 0u;
            uint32_t a[EWP];
            uint64_t rsa = 0ull, rsb = 0ull;
            float rm0 = -1e30f, rm1 = -1e30f;
            if (need) {
              tmem_ld_keyrow<EWP>(s_taddr + rr * EWP, a);
              tmem_ld_wait();
            }
#pragma unroll
            for (int k2 = 0; k2 < Cfg::PCOLS_ROW; ++k2) {
              uint32_t packed = 0u;
              if (need && k2 < EW / 2) {
                float t0, t1;
                unpack2(ffma2(pack2u(a[2 * k2], a[2 * k2 + 1]), c2, nb2[k2]), t0, t1);
                if constexpr (SINGLE_PASS) {
                  if (k2 & 1) rm1 = fmax3(rm1, t0, t1); else rm0 = fmax3(rm0, t0, t1);
                }
                const float p0 = fast_exp2(t0), p1 = fast_exp2(t1);
                if (k2 & 1) rsb = fadd2(rsb, pack2(p0, p1)); else rsa = fadd2(rsa, pack2(p0, p1));
                packed = pack_bf16(p0, p1) & keep;
              }
              pk[rr][k2] = packed;
            }
            if constexpr (!SINGLE_PASS)   // final already: store this row's P right away
              tmem_st_cols<Cfg::PCOLS_ROW>(s_taddr + rr * Cfg::PCOLS_ROW, pk[rr]);
            if (mine) {
              rs2 = fadd2(rs2, fadd2(rsa, rsb));
              tm0 = fmaxf(tm0, rm0);
              tm1 = fmaxf(tm1, rm1);
            }
          }
          if (!SINGLE_PASS || settled) break;
          const float tmax = fmaxf(tm0, tm1);
          if (!__any_sync(0xffffffffu, tmax > 8.0f)) break;
          settled = true;
          if (!apply_reference(tmax > 8.0f ? tmax : -1e30f)) {
            ok = false;
            break;
          }
        }
        if (!ok) break;
        // P of key row rr goes to columns [rr*EWP/2, (rr+1)*EWP/2) of this thread's own S
        // segment: the S values are consumed, and no other thread reads this lane.
        if constexpr (SINGLE_PASS) {
#pragma unroll
          for (int rr = 0; rr < RPG; ++rr)
            tmem_st_cols<Cfg::PCOLS_ROW>(s_taddr + rr * Cfg::PCOLS_ROW, pk[rr]);
        }
        {
          float r0, r1;
          unpack2(rs2, r0, r1);
          l_run += r0 + r1;
        }
        // every lane completes its P stores, then one lane arrives for the warp
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready(sb));
      }
      if (!ok) break;

      // item epilogue: publish (max, sum), wait for the last P V, then every thread combines
      // the NG accumulators of its row for its own 64/NG output channels and stores them.
      const uint32_t ipar = n & 1u;
      ml[(ipar * NG + grp) * 128 + r] = make_float2(l_run > 0.f ? mc : -1e30f, l_run);
      __syncwarp();
      if (lane == 0) mbar_arrive(ml_ready(ipar));
      if (!mbar_wait(o_full((gb - 1u) & 1u), ((gb - 1u) >> 1) & 1u, abort_flag,
                     ST_TIMEOUT_SOFTMAX) ||
          !mbar_wait(ml_ready(ipar), (n >> 1) & 1u, abort_flag, ST_TIMEOUT_SOFTMAX)) {
        ok = false;
        break;
      }
      tc_fence_after();
      {
        float mj[NG], lj[NG];
        float m = -1e30f;
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          const float2 t = ml[(ipar * NG + g) * 128 + r];
          mj[g] = t.x;
          lj[g] = t.y;
          m = fmaxf(m, t.x);
        }
        float denom = 0.f;
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          mj[g] = fast_exp2(mj[g] - m);   // weight of group g (references are already scaled)
          denom += lj[g] * mj[g];
        }
        const float inv = 1.0f / denom;
        constexpr int WCOLS = 64 / NG;          // output channels this thread finishes
        float acc[WCOLS];
#pragma unroll
        for (int j = 0; j < WCOLS; ++j) acc[j] = 0.f;
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          uint32_t ob[WCOLS];
          const uint32_t ta = lane_taddr + Cfg::O_COL + 64 * g + WCOLS * grp;
          if constexpr (WCOLS == 16) tmem_ld_x16(ta, ob); else tmem_ld_32x32(ta, *reinterpret_cast<uint32_t(*)[32]>(ob));
          tmem_ld_wait();
          const float wgt = mj[g] * inv;
#pragma unroll
          for (int j = 0; j < WCOLS; ++j) acc[j] = fmaf(__uint_as_float(ob[j]), wgt, acc[j]);
        }
        tc_fence_before();
        if (q_ok) {
          const long long tok = ((static_cast<long long>(it.b) * p.D + (it.d0 + zd)) * p.q_H +
                                 (it.h0 + zh - p.q_h0)) * p.q_W + (it.w0 + zw - p.q_w0);
          __nv_bfloat16* op = p.out + tok * p.ldo + it.head * 64 + WCOLS * grp;
#pragma unroll
          for (int j = 0; j < WCOLS; j += 8) {
            uint4 v4;
            v4.x = pack_bf16(acc[j], acc[j + 1]);
            v4.y = pack_bf16(acc[j + 2], acc[j + 3]);
            v4.z = pack_bf16(acc[j + 4], acc[j + 5]);
            v4.w = pack_bf16(acc[j + 6], acc[j + 7]);
            *reinterpret_cast<uint4*>(op + j) = v4;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, NA_TMEM_COLS);
  }
}

// Cuts the key box into (plane, 4-row chunk) units and pairs them into blocks. For every unit
// the set of tile quarters (32 consecutive query rows: one warp per softmax group) that can
// see it is worked out for an interior tile; units with disjoint sets are paired first, the
// unit seen by most quarters choosing the partner that fills most of the remaining ones, so
// that the per-block work of the busiest quarter is as small as the pairing allows. Windows
// clamped at a border see fewer units than assumed here; that only affects the balance, the
// kernel's masks are exact.
inline int na_build_blocks(Na3dParams& p) {
  const int ED = p.QD + p.kd - 1;
  const int EH = p.QH + p.kh - 1;
  const int NC = (EH + 3) / 4;
  if (ED > 16 || NC > 8 || ED * NC > 2 * NA_MAX_BLOCKS) return -2;
  const int n = ED * NC;
  unsigned char seen[2 * NA_MAX_BLOCKS];
  bool used[2 * NA_MAX_BLOCKS];
  for (int pl = 0; pl < ED; ++pl)
    for (int ch = 0; ch < NC; ++ch) {
      unsigned m = 0;
      for (int q = 0; q < 4; ++q)
        for (int j = 4 * q; j < 4 * q + 4; ++j) {   // (zd, zh) pairs of the quarter
          const int zh = j % p.QH, zd = j / p.QH;
          const bool pd = pl >= zd && pl < zd + p.kd;
          const bool ph = 4 * ch + 3 >= zh && 4 * ch < zh + p.kh;
          if (pd && ph) m |= 1u << q;
        }
      seen[pl * NC + ch] = static_cast<unsigned char>(m);
      used[pl * NC + ch] = false;
    }
  auto pop = [](unsigned m) { return __builtin_popcount(m); };
  auto code = [&](int u) { return static_cast<unsigned short>((u % NC) | ((u / NC) << 4)); };
  int nb = 0;
  // pass 1: disjoint pairs, widest sets first
  for (int want = 4; want >= 1; --want)
    for (int u = 0; u < n; ++u) {
      if (used[u] || pop(seen[u]) != want) continue;
      int best = -1;
      for (int v = 0; v < n; ++v)
        if (!used[v] && v != u && (seen[u] & seen[v]) == 0 &&
            (best < 0 || pop(seen[v]) > pop(seen[best])))
          best = v;
      if (best < 0) continue;
      used[u] = used[best] = true;
      p.blk[nb][0] = code(u);
      p.blk[nb][1] = code(best);
      ++nb;
    }
  // pass 2: whatever is left, in order
  int pending = -1;
  for (int u = 0; u < n; ++u) {
    if (used[u]) continue;
    if (pending < 0) { pending = u; continue; }
    p.blk[nb][0] = code(pending);
    p.blk[nb][1] = code(u);
    ++nb;
    pending = -1;
  }
  if (pending >= 0) {
    p.blk[nb][0] = code(pending);
    p.blk[nb][1] = static_cast<unsigned short>(code(pending) | 0x8000u);
    ++nb;
  }
  p.nblk = nb;
  return 0;
}

}  // namespace strata

#include "na3d_narrow.cuh"

namespace strata {

// q/k/v: token-major bf16, element (b,d,h,w,head,c) at base + token*ld + head*64 + c where
// token = ((b*D + d)*H + h)*W + w. out likewise with ldo.
template <int KW>
inline int launch_na3d_t(const __nv_bfloat16* q, long long ldq, const __nv_bfloat16* k,
                         long long ldk, const __nv_bfloat16* v, long long ldv, Na3dParams p,
                         int sm_count, cudaStream_t stream) {
  using Cfg = Na3dCfg<KW>;
  const uint64_t chans = static_cast<uint64_t>(p.heads) * 64;
  auto make = [&](CUtensorMap* tm, const __nv_bfloat16* base, long long ld, uint32_t bw,
                  uint32_t bh, uint32_t bd) {
    uint64_t dims[5] = {chans, static_cast<uint64_t>(p.W), static_cast<uint64_t>(p.H),
                        static_cast<uint64_t>(p.D), static_cast<uint64_t>(p.B)};
    uint64_t str[4] = {static_cast<uint64_t>(ld) * 2, static_cast<uint64_t>(ld) * 2 * p.W,
                       static_cast<uint64_t>(ld) * 2 * p.W * p.H,
                       static_cast<uint64_t>(ld) * 2 * p.W * p.H * p.D};
    uint32_t box[5] = {64, bw, bh, bd, 1};
    return make_tmap_bf16(tm, base, 5, dims, str, box);
  };
  CUtensorMap tmQ, tmK, tmV;
  if (make(&tmQ, q, ldq, NA_QW, p.QH, p.QD) != 0) return -20;
  if constexpr (NA_QW + KW - 1 <= 16) {
    // narrow key rows: the two-CTAs-per-SM kernel
    using NCfg = Na3dNarrowCfg<KW>;
    if (make(&tmK, k, ldk, NCfg::EWP, 4, 1) != 0) return -20;
    if (make(&tmV, v, ldv, NCfg::EWP, 4, 1) != 0) return -20;
    auto kern = na3d_fwd_narrow_kernel<KW>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         NCfg::TOTAL);
    if (e != cudaSuccess) return -static_cast<int>(e) - 1000;
    const int grid = p.n_items < 2 * sm_count ? p.n_items : 2 * sm_count;
    kern<<<grid, NCfg::THREADS, NCfg::TOTAL, stream>>>(tmQ, tmK, tmV, p);
    e = cudaGetLastError();
    return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
  } else {
    constexpr uint32_t KV_BOX_ROWS = Cfg::NG == 4 ? 1 : 4;
    if (make(&tmK, k, ldk, Cfg::EWP, KV_BOX_ROWS, 1) != 0) return -20;
    if (make(&tmV, v, ldv, Cfg::EWP, KV_BOX_ROWS, 1) != 0) return -20;
    auto kern = na3d_fwd_kernel<KW>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::TOTAL);
    if (e != cudaSuccess) return -static_cast<int>(e) - 1000;
    const int grid = p.n_items < sm_count ? p.n_items : sm_count;
    kern<<<grid, Cfg::THREADS, Cfg::TOTAL, stream>>>(tmQ, tmK, tmV, p);
    e = cudaGetLastError();
    return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
  }
}

inline int launch_na3d(const __nv_bfloat16* q, long long ldq, const __nv_bfloat16* k, long long ldk,
                       const __nv_bfloat16* v, long long ldv, __nv_bfloat16* out, long long ldo,
                       int B, int D, int H, int W, int heads, int kd, int kh, int kw, float scale,
                       int sm_count, cudaStream_t stream, int q_h0 = 0, int q_H = -1, int q_w0 = 0,
                       int q_W = -1) {
  if (kd > D || kh > H || kw > W || kd < 1 || kh < 1 || kw < 1) return -1;
  if (kh > 15 || kd > 15) return -2;
  Na3dParams p{};
  p.B = B; p.D = D; p.H = H; p.W = W; p.heads = heads;
  p.kd = kd; p.kh = kh;
  // query tile: 2 x 8 x 8, flattened towards the rows when the tensor is shallow
  if (D >= 2) { p.QD = 2; p.QH = 8; } else { p.QD = 1; p.QH = 16; }
  if (p.QH + kh - 1 > 31) return -2;
  p.q_h0 = q_h0; p.q_w0 = q_w0;
  p.q_H = q_H < 0 ? H : q_H;
  p.q_W = q_W < 0 ? W : q_W;
  if (p.q_h0 < 0 || p.q_w0 < 0 || p.q_H < 1 || p.q_W < 1 || p.q_h0 + p.q_H > H ||
      p.q_w0 + p.q_W > W)
    return -1;
  p.tiles_d = (D + p.QD - 1) / p.QD;
  p.tiles_h = (p.q_H + p.QH - 1) / p.QH;
  p.tiles_w = (p.q_W + NA_QW - 1) / NA_QW;
  const long long items = static_cast<long long>(p.tiles_d) * p.tiles_h * p.tiles_w * heads * B;
  if (items > 0x7fffffffLL) return -2;
  p.n_items = static_cast<int>(items);
  if (na_build_blocks(p) != 0) return -2;
  p.out = out;
  p.ldo = ldo;
  p.scale_log2e = scale * 1.4426950408889634f;
  switch (kw) {
    case 1: return launch_na3d_t<1>(q, ldq, k, ldk, v, ldv, p, sm_count, stream);
    case 3: return launch_na3d_t<3>(q, ldq, k, ldk, v, ldv, p, sm_count, stream);
    case 5: return launch_na3d_t<5>(q, ldq, k, ldk, v, ldv, p, sm_count, stream);
    case 7: return launch_na3d_t<7>(q, ldq, k, ldk, v, ldv, p, sm_count, stream);
    case 9: return launch_na3d_t<9>(q, ldq, k, ldk, v, ldv, p, sm_count, stream);
    case 11: return launch_na3d_t<11>(q, ldq, k, ldk, v, ldv, p, sm_count, stream);
    case 13: return launch_na3d_t<13>(q, ldq, k, ldk, v, ldv, p, sm_count, stream);
    case 15: return launch_na3d_t<15>(q, ldq, k, ldk, v, ldv, p, sm_count, stream);
    default: return -2;
  }
}

}  // namespace strata
