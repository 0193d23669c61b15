// Fused 3-D neighbourhood attention forward for sm_100a (head_dim 64, bf16, non-causal,
// dilation 1): for every query token, softmax(q.k * scale) over the kd*kh*kw keys of its
// window, times v. Windows keep their full size at the borders: along an axis of length L
// the window of query i starts at clamp(i - k/2, 0, L - k).
//
// Work decomposition (persistent kernel, TWO CTAs per SM)
//   work item   one tile of up to 128 queries (QD x QH x QW tokens) of one head of one batch
//               entry; CTA c handles items c, c + gridDim.x, ... (neighbouring items are
//               neighbouring tiles of the same head, so their key halos meet in L2). The tile
//               is as wide as the kernel allows with key rows of at most 16 columns:
//               QW = 8 for kernel widths up to 9, 4 up to 13, 2 for 15.
//   key blocks  the union of a tile's windows is a box of ED x EH x EW keys
//               (E* = Q* + k* - 1) starting at the window start of the tile's first query.
//               The box is cut into units of one depth plane x 4 rows x EWP columns
//               (EWP = EW padded to 8 or 16) and streamed as blocks of TWO units (64 or 128
//               keys); TMA zero-fills whatever lies outside the tensor. Which two units share
//               a block is a host-built table: each quarter of the tile (32 queries = one
//               softmax warp = one SM sub-partition) sees only part of the box, so units are
//               paired such that, wherever possible, every quarter finds exactly one visible
//               unit in every block - the exponential work is then spread evenly over the
//               sub-partitions instead of the busiest quarter setting the pace.
//   TMEM        S (128 columns), P (64) and O (64) of one query tile take 256 columns - half
//               an SM's TMEM. A CTA needs only six warps, half the shared memory (one Q tile,
//               a three-stage K/V ring) and is resident twice per SM. Each CTA runs a simple,
//               strictly ordered pipeline per key block
//                   Q K^T -> S   |   softmax: S -> P   |   P V -> O
//               and the latencies of that chain (MMA issue and completion, tcgen05.ld / st
//               round trips, barrier hand-offs) are hidden by the OTHER CTA on the SM rather
//               than by deeper buffering inside one CTA.
//   warp 0      TMA producer: Q tile (single buffer, re-filled as soon as the item's last
//               Q K^T has completed) and K / V units (one box of 4 rows x EWP keys per unit;
//               5-D tensor maps over [B, D, H, W, channels], 128-byte swizzle, a key's 64
//               channels are one 128-byte row).
//   warp 1      MMA issuer. Q K^T of block i+1 is issued as soon as the softmax warps have
//               copied the scores of block i out of S (s_free), i.e. while they evaluate its
//               exponentials; P V of block i (A operand = P from TMEM) follows when P(i) is
//               ready. Barrier arrivals through tcgen05.commit are kept to two per block (P V
//               done, S full): a commit costs the issuing thread about as much as three MMAs.
//   warps 2-5   softmax, one thread per query row (TMEM lane quarter = warp & 3). Per visible
//               unit: load the 4 x EWP scores into registers, hand S back, one straight-line
//               pass of exponentials against the row's current reference, add the row sum.
//               There is no maximum pass: a row's first reference is the largest of a few
//               scores it certainly sees (any visible score serves), the running sum is the
//               detector for scores far above the reference, and at the next block's start
//               the reference then moves up by a whole number of binades e - O and the sum
//               are multiplied by 2^-e, which is exact, and nothing needs the raw scores
//               again. A row whose sum leaves the repairable range (2^100, infinite, NaN)
//               within one block is recomputed from global memory by a plain loop after the
//               CTA's last item. Everything rare - that loop, the rescale of O, the polling
//               loops of the barrier waits - and the item's output store are functions out
//               of line: rare code left inline in this loop cost 2-15 % each without running.
//               The store of an item's rows happens while the next item's first block waits
//               for the item's last P V anyway.
//   P           bf16 pairs, column j of the P region holds keys 2j, 2j+1 of the block; rows a
//               query cannot see hold zeros.
//   mask        per (query, key): the key's box coordinates must fall in the query's window
//               on all three axes. Columns: an additive per-thread bias vector (0 / -1e30);
//               rows: a per-thread bit mask; planes: one comparison per unit. Border clamping
//               is therefore exact per query row.
//   barriers    all mbarrier waits are bounded.
#pragma once
#include "common.cuh"
#include "tensormap.cuh"

namespace strata {

constexpr int NA_MAX_BLOCKS = 64;   // 16 planes x 8 chunks / 2

struct Na3dParams {
  int B, D, H, W, heads;
  int kd, kh;            // kernel extents along depth and rows (columns: template KW)
  int QD, QH, QW;        // query tile extents; QD*QH*QW <= 128
  int q_rows;            // QD*QH*QW: rows of the 128-row tile that carry a query
  int tiles_d, tiles_h, tiles_w;
  // Query region: only tokens with h in [q_h0, q_h0+q_H), w in [q_w0, q_w0+q_W) are queries
  // (the interior of a halo-padded tile; the whole plane by default). Keys come from the
  // whole [H, W] plane. Output plane: [B, D, o_H, o_W, ldo], query (h, w) lands at
  // (h - o_h0, w - o_w0) - by default the query region itself, stored compactly; a larger
  // output window lets several launches (an inner region, border strips) fill one tensor.
  int q_h0, q_H, q_w0, q_W;
  int o_h0, o_H, o_w0, o_W;
  int n_items;           // tiles_d*tiles_h*tiles_w*heads*B
  int nblk;              // key blocks per item
  // blk[i][s]: unit in slot s of block i: chunk (4 rows) in bits 0-3, plane in bits 4-7;
  // bit 15: the slot only repeats another unit to keep the block full - ignore its keys.
  unsigned short blk[NA_MAX_BLOCKS][2];
  __nv_bfloat16* out;    // [B, D, q_H, q_W, ldo] with head h at channel offset h*64
  long long ldo;
  // the operands as plain pointers (token-major, row strides in elements): only the
  // recomputation of a row whose scores left the range of the fast path reads them
  const __nv_bfloat16 *q, *k, *v;
  long long ldq, ldk, ldv;
  float scale_log2e;
};

__device__ __forceinline__ int na_window_start(int i, int L, int k) {
  int s = i - (k >> 1);
  s = s < 0 ? 0 : s;
  return s > L - k ? L - k : s;
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
// Loads EWP (8 or 16) consecutive S columns of this thread's row.
template <int EWP>
__device__ __forceinline__ void tmem_ld_keyrow(uint32_t taddr, uint32_t* a) {
  if constexpr (EWP == 8) tmem_ld_x8(taddr, a); else tmem_ld_x16(taddr, a);
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
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// One query row computed the plain way - scores, online softmax and P V in fp32 on the CUDA
// cores, operands read from global memory. Thousands of times slower than the tensor-core
// path and only used for a row whose scores rose more than 2^119 above its reference within
// one unit (or are infinite or NaN), which the fast path cannot represent.
struct NaSlowArgs {   // passed by value: a reference to the kernel's parameters would force a local copy
  const __nv_bfloat16 *q, *k, *v;
  long long ldq, ldk, ldv;
  int D, H, W, kd, kh;
  float scale_log2e;
};
template <int KW>
__device__ __noinline__ void na_slow_row(const NaSlowArgs p, int b, int head, int id, int ih,
                                         int iw, __nv_bfloat16* op) {
  auto token = [&](int d, int h, int w) {
    return ((static_cast<long long>(b) * p.D + d) * p.H + h) * p.W + w;
  };
  float qf[64], o[64];
  {
    const uint4* qp = reinterpret_cast<const uint4*>(p.q + token(id, ih, iw) * p.ldq + head * 64);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint4 x = qp[j];
      const uint32_t w4[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        qf[8 * j + 2 * t] = bf16_lo(w4[t]);
        qf[8 * j + 2 * t + 1] = bf16_hi(w4[t]);
      }
    }
  }
#pragma unroll
  for (int c = 0; c < 64; ++c) o[c] = 0.f;
  const int d0 = na_window_start(id, p.D, p.kd);
  const int h0 = na_window_start(ih, p.H, p.kh);
  const int w0 = na_window_start(iw, p.W, KW);
  float m = -3.0e38f, l = 0.f;
  const int nkeys = p.kd * p.kh * KW;
#pragma unroll 1
  for (int n = 0; n < nkeys; ++n) {
    const int ww = n % KW, hh = (n / KW) % p.kh, dd = n / (KW * p.kh);
    const long long tok = token(d0 + dd, h0 + hh, w0 + ww);
    const uint4* kp = reinterpret_cast<const uint4*>(p.k + tok * p.ldk + head * 64);
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint4 x = kp[j];
      const uint32_t w4[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        dot = fmaf(qf[8 * j + 2 * t], bf16_lo(w4[t]), dot);
        dot = fmaf(qf[8 * j + 2 * t + 1], bf16_hi(w4[t]), dot);
      }
    }
    const float t = dot * p.scale_log2e;
    if (t > m) {
      const float alpha = exp2f(m - t);
      l *= alpha;
#pragma unroll
      for (int c = 0; c < 64; ++c) o[c] *= alpha;
      m = t;
    }
    const float pw = exp2f(t - m);
    l += pw;
    const float pb = __bfloat162float(__float2bfloat16_rn(pw));   // P enters P V as bf16
    const uint4* vp = reinterpret_cast<const uint4*>(p.v + tok * p.ldv + head * 64);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint4 x = vp[j];
      const uint32_t w4[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int t2 = 0; t2 < 4; ++t2) {
        o[8 * j + 2 * t2] = fmaf(pb, bf16_lo(w4[t2]), o[8 * j + 2 * t2]);
        o[8 * j + 2 * t2 + 1] = fmaf(pb, bf16_hi(w4[t2]), o[8 * j + 2 * t2 + 1]);
      }
    }
  }
  const float inv = 1.0f / l;
#pragma unroll
  for (int j = 0; j < 64; j += 8) {
    uint4 v4;
    v4.x = pack_bf16(o[j] * inv, o[j + 1] * inv);
    v4.y = pack_bf16(o[j + 2] * inv, o[j + 3] * inv);
    v4.z = pack_bf16(o[j + 4] * inv, o[j + 5] * inv);
    v4.w = pack_bf16(o[j + 6] * inv, o[j + 7] * inv);
    *reinterpret_cast<uint4*>(op + j) = v4;
  }
}

// Multiplies this thread's row of the O accumulator (64 fp32 columns in tensor memory) by 2^-e
// and returns that factor. Called by a whole warp; out of line because it is rare.
__device__ __noinline__ float na_scale_o_row(uint32_t o_taddr, int e) {
  const float alpha = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
#pragma unroll 1
  for (int hh = 0; hh < 4; ++hh) {
    uint32_t ob[16];
    tmem_ld_x16(o_taddr + 16 * hh, ob);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 16; ++j) ob[j] = __float_as_uint(__uint_as_float(ob[j]) * alpha);
    tmem_st_x16(o_taddr + 16 * hh, ob);
  }
  tmem_st_wait();
  return alpha;
}

// Reads this thread's row of the O accumulator, scales it by inv and stores it as 64 bf16 at op
// (nullptr: the row carries no query). Called by a whole warp, once per item.
__device__ __noinline__ void na_store_o_row(uint32_t o_taddr, float inv, __nv_bfloat16* op) {
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    uint32_t ob[32];
    tmem_ld_32x32(o_taddr + 32 * hh, ob);
    tmem_ld_wait();
    if (op != nullptr) {
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

// mbar_wait with the (bounded) polling loop out of line: the common case - the phase has
// already completed - costs one test in the softmax warps' hot loop.
__device__ __noinline__ bool na_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
  return mbar_wait(bar, parity, abort_flag, code);
}
__device__ __forceinline__ bool na_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  return na_wait_slow(bar, parity, abort_flag, code);
}

struct NaItem {
  int b, head, d0, h0, w0, bd0, bh0, bw0;
};
template <int KW, int QW>
__device__ __forceinline__ NaItem na_decode_item(int item, const Na3dParams& p) {
  NaItem it;
  int t = item;
  const int tw = t % p.tiles_w; t /= p.tiles_w;
  const int th = t % p.tiles_h; t /= p.tiles_h;
  const int td = t % p.tiles_d; t /= p.tiles_d;
  it.head = t % p.heads;
  it.b = t / p.heads;
  it.d0 = td * p.QD; it.h0 = p.q_h0 + th * p.QH; it.w0 = p.q_w0 + tw * QW;
  // key box origin = window start of the tile's first query on each axis
  it.bd0 = na_window_start(it.d0, p.D, p.kd);
  it.bh0 = na_window_start(it.h0, p.H, p.kh);
  it.bw0 = na_window_start(it.w0, p.W, KW);
  return it;
}

template <int KW, int QW>
struct Na3dCfg {
  static constexpr int EW = QW + KW - 1;
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
  static_assert(EWP <= 16, "key rows of at most 16 columns");
  static_assert(TOTAL <= 115712, "two CTAs per SM: at most half of the SM's shared memory");
};

// The rows of one thread (tile position zd, zh, zw) in the CTA's items that the fast path gave
// up on: the first 64 items are remembered one by one (bad_items), later ones as a group.
template <int KW, int QW>
__device__ __noinline__ void na_slow_rows(const Na3dParams& p, uint64_t bad_items, bool bad_rest,
                                          int n_my, bool has_query, int zd, int zh, int zw) {
  const NaSlowArgs sa = {p.q, p.k, p.v, p.ldq, p.ldk, p.ldv, p.D, p.H, p.W, p.kd, p.kh, p.scale_log2e};
#pragma unroll 1
  for (int n = 0; n < n_my; ++n) {
    if (!(n < 64 ? ((bad_items >> n) & 1ull) != 0ull : bad_rest)) continue;
    const NaItem it = na_decode_item<KW, QW>(static_cast<int>(blockIdx.x) + n * static_cast<int>(gridDim.x), p);
    const bool q_ok = has_query && (it.d0 + zd < p.D) && (it.h0 + zh < p.q_h0 + p.q_H) &&
                      (it.w0 + zw < p.q_w0 + p.q_W);
    if (!q_ok) continue;
    const long long tok = ((static_cast<long long>(it.b) * p.D + (it.d0 + zd)) * p.o_H +
                           (it.h0 + zh - p.o_h0)) * p.o_W + (it.w0 + zw - p.o_w0);
    na_slow_row<KW>(sa, it.b, it.head, it.d0 + zd, it.h0 + zh, it.w0 + zw,
                    p.out + tok * p.ldo + it.head * 64);
  }
}

template <int KW, int QW>
__global__ void __launch_bounds__(Na3dCfg<KW, QW>::THREADS, 2)
na3d_fwd_kernel(const __grid_constant__ CUtensorMap tmQ,
                       const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const Na3dParams p) {
  using Cfg = Na3dCfg<KW, QW>;
  constexpr int EW = Cfg::EW;
  constexpr int EWP = Cfg::EWP;
  constexpr int NKEYS = Cfg::NKEYS;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int PC = Cfg::PCOLS_ROW;          // P columns (bf16 pairs) per key row
  constexpr int UNIT_PCOLS = 4 * PC;          // P columns of one unit (4 key rows)
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
  const uint32_t q_full = bar, q_empty = bar + 8, s_full = bar + 16, p_ready = bar + 24,
                 s_free = bar + 96;
  auto kv_full = [&](int st) { return bar + 32u + 8u * st; };
  auto pv_done = [&](int st) { return bar + 64u + 8u * st; };   // K/V stage free, O updated
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::BAR_OFF + 128);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::BAR_OFF + 136);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nblk = p.nblk;
  // items of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ... (the grid never exceeds n_items)
  const int n_my = (p.n_items - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                   static_cast<int>(gridDim.x);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_ready, 4);   // one arrival per softmax warp
    mbar_init(s_free, 4);
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
      int st = 0;
      uint32_t ph = 0;
      for (int n = 0; n < n_my && ok; ++n) {
        const NaItem it = na_decode_item<KW, QW>(static_cast<int>(blockIdx.x) + n * static_cast<int>(gridDim.x), p);
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
          if (i == 0) {
            // the item's Q tile follows its first K/V block: the wait for the previous item's last
            // Q K^T then does not hold that block back
            if (!mbar_wait(q_empty, (n & 1u) ^ 1u, abort_flag, ST_TIMEOUT_PRODUCER)) {
              ok = false;
              break;
            }
            mbar_expect_tx(q_full, static_cast<uint32_t>(p.q_rows) * 128u);
            tma_load_5d(q_smem, &tmQ, it.head * 64, it.w0, it.h0, it.d0, it.b, q_full);
          }
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
      const int G = n_my * nblk;   // key blocks of this CTA, over all its items

      // Q K^T of block g (blocks are numbered through the CTA's items): needs the item's Q tile,
      // the block's K unit pair and - from the second block on - the softmax warps' word that
      // they have copied the previous scores out of S.
      int qk_st = 0, qk_i = 0, qk_n = 0;
      uint32_t qk_ph = 0;
      auto issue_qk = [&](int g) -> bool {
        if (qk_i == 0 && !mbar_wait(q_full, qk_n & 1u, abort_flag, ST_TIMEOUT_MMA)) return false;
        if (!mbar_wait(kv_full(qk_st), qk_ph, abort_flag, ST_TIMEOUT_MMA)) return false;
        if (g > 0 && !mbar_wait(s_free, (g - 1) & 1u, abort_flag, ST_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint32_t klo = k_lo0 + qk_st * STAGE_UNITS;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_ss(s_tmem, desc(q_lo + 2u * k), desc(klo + 2u * k), idesc_qk, k != 0 ? 1u : 0u);
        umma_commit(s_full);
        if (++qk_i == nblk) {   // last Q K^T of the item: its completion frees the Q tile
          umma_commit(q_empty);
          qk_i = 0;
          ++qk_n;
        }
        if (++qk_st == STAGES) { qk_st = 0; qk_ph ^= 1u; }
        return true;
      };

      bool ok = G > 0 && issue_qk(0);
      int pv_st = 0, pv_i = 0;
      for (int g = 0; g < G && ok; ++g) {
        // scores of the next block first: they are computed while the softmax warps work on
        // this one ...
        if (g + 1 < G && !issue_qk(g + 1)) break;
        // ... then O += P V of this block, once its P is in tensor memory
        if (!mbar_wait(p_ready, g & 1u, abort_flag, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t vlo = v_lo0 + pv_st * STAGE_UNITS;
#pragma unroll
        for (int s = 0; s < PV_STEPS; ++s)
          umma_ts(o_tmem, p_tmem + 8 * s, desc(vlo + 128u * s), idesc_pv,
                  (s != 0 || pv_i != 0) ? 1u : 0u);
        umma_commit(pv_done(pv_st));
        if (++pv_st == STAGES) pv_st = 0;
        if (++pv_i == nblk) pv_i = 0;
      }
    }
  } else {
    // ------------------------------------------------------------ softmax warps
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;        // query row
    const bool has_query = r < p.q_rows;      // small tiles leave the upper rows unused
    const int zw = r % QW;
    const int zh = (r / QW) % p.QH;
    const int zd = has_query ? (r / QW) / p.QH : 0;
    const uint32_t lane_taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_taddr = lane_taddr + Cfg::S_COL;
    const uint32_t p_taddr = lane_taddr + Cfg::P_COL;
    const uint32_t o_taddr = lane_taddr + Cfg::O_COL;
    const float c = p.scale_log2e;
    constexpr float SUM_LIMIT = 65536.0f;          // 2^16
    constexpr float SUM_REPAIRABLE = 1.0e30f;      // ~2^100: P, O and 2^-e stay well inside fp32

    bool ok = true;
    uint32_t gb = 0;
    bool pend = false;            // the previous item's row is still to be stored
    float pend_inv = 0.f;
    __nv_bfloat16* pend_op = nullptr;
    uint64_t bad_items = 0ull;    // see the end of this branch
    bool bad_rest = false;
    int st_prev = STAGES - 1;     // ring stage and phase of block gb-1 (for pv_done)
    uint32_t ph_prev = 1;
    for (int n = 0; n < n_my && ok; ++n) {
      const NaItem it = na_decode_item<KW, QW>(static_cast<int>(blockIdx.x) + n * static_cast<int>(gridDim.x), p);
      const bool q_ok = has_query && (it.d0 + zd < p.D) && (it.h0 + zh < p.q_h0 + p.q_H) &&
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
          if (!has_query) rowmask = 0u;
        }
        const uint32_t warp_rows = __reduce_or_sync(0xffffffffu, rowmask);
        bool p_free = false;      // the previous block's P V has completed: P may be overwritten
        if (i != 0 && __any_sync(0xffffffffu, l_run >= SUM_LIMIT)) {
          // rare: some row's scores have risen far above its reference. Move that reference up
          // by e whole binades: what has been accumulated under the old one - O (complete once
          // the previous P V is) and the running sum - is multiplied by 2^-e, which is exact.
          // A sum beyond SUM_REPAIRABLE (or infinite, or NaN) is left alone: the row is
          // recomputed from global memory when the kernel ends.
          if (!na_wait(pv_done(st_prev), ph_prev, abort_flag, ST_TIMEOUT_SOFTMAX)) {
            ok = false;
            break;
          }
          tc_fence_after();
          p_free = true;
          const int e = (l_run >= SUM_LIMIT && l_run < SUM_REPAIRABLE)
                            ? static_cast<int>((__float_as_uint(l_run) >> 23) & 255u) - 127 : 0;
          l_run *= na_scale_o_row(o_taddr, e);
          if (e != 0) {
            mc += static_cast<float>(e);
            set_nb(mc);
          }
        }
        if (!na_wait(s_full, gb & 1u, abort_flag, ST_TIMEOUT_SOFTMAX)) {
          ok = false;
          break;
        }
        tc_fence_after();

        // The block's two units (4 key rows each) are handled one after the other with the
        // unit's scores held in registers: as soon as the last unit the warp can see has been
        // copied out of S, the warp gives S back (s_free) and the MMA warp computes the next
        // block's scores while the exponentials of this one are still being evaluated. P is
        // stored once the previous block's P V has completed (pv_done), which has normally
        // happened long before.
        //
        // The exponentials are taken against the row's current reference without looking for
        // the maximum first. A row that has no reference yet takes the maximum of its first
        // visible scores (one extra pass, once per row and item). Afterwards the running sum
        // is the detector: once it has reached 2^16 a score lies far above the reference, and
        // at the start of the next block (see above) the reference moves up. Rows of the unit
        // that this query does not see are masked (zero P, left out of the sum).
        bool s_released = false;
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint32_t need4 = (warp_rows >> (4 * u)) & 15u;   // rows some query of the warp sees
          const uint32_t mine4 = (rowmask >> (4 * u)) & 15u;     // rows this query sees
          const bool last_load = (u == 1) || ((warp_rows >> 4) == 0u);
          uint32_t pk[UNIT_PCOLS];
          if (need4 != 0u) {
            uint32_t a[4][EWP];
#pragma unroll
            for (int rr = 0; rr < 4; ++rr) tmem_ld_keyrow<EWP>(s_taddr + (4 * u + rr) * EWP, a[rr]);
            tmem_ld_wait();
            if (last_load && !s_released) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(s_free);
              s_released = true;
            }
            const bool fresh = has_query && l_run == 0.f;
            if (__any_sync(0xffffffffu, fresh)) {
              // The first reference of a row: the largest of some scores it sees in this unit
              // (scaled form). Any visible score will do - whatever lies above it by less than
              // 2^100 is absorbed by the running sum and the moves of the reference that follow
              // from it - so only the key columns that every query of the tile has in its
              // window (QW-1 .. KW-1, clamped windows included) are looked at when there are
              // any, all columns otherwise.
              constexpr int K2_LO = (KW >= QW) ? (QW - 1) / 2 : 0;
              constexpr int K2_HI = (KW >= QW) ? (QW - 1) / 2 + 1 : EW / 2;
              float bm = -1e30f;
#pragma unroll
              for (int rr = 0; rr < 4; ++rr) {
                float rm = -1e30f;
#pragma unroll
                for (int k2 = K2_LO; k2 < K2_HI; ++k2) {
                  float t0, t1;
                  unpack2(ffma2(pack2u(a[rr][2 * k2], a[rr][2 * k2 + 1]), c2, nb2[k2]), t0, t1);
                  rm = fmaxf(rm, fmaxf(t0, t1));
                }
                bm = fmaxf(bm, ((mine4 >> rr) & 1u) ? rm : -1e30f);
              }
              // nothing has been accumulated for a fresh row (its earlier P were zeros)
              if (fresh && bm > -1e29f) {
                mc += bm;
                set_nb(mc);
              }
            }
            // exponentials, row sum and bf16 P (two keys per 32-bit column)
            uint64_t rs2 = 0ull;
#pragma unroll
            for (int rr = 0; rr < 4; ++rr) {
              const bool mine = (mine4 >> rr) & 1u;
              const uint32_t keep = mine ? 0xffffffffu : 0u;
              uint64_t rsa = 0ull, rsb = 0ull;
#pragma unroll
              for (int k2 = 0; k2 < PC; ++k2) {
                uint32_t packed = 0u;
                if (k2 < EW / 2) {
                  float t0, t1;
                  unpack2(ffma2(pack2u(a[rr][2 * k2], a[rr][2 * k2 + 1]), c2, nb2[k2]), t0, t1);
                  const float p0 = fast_exp2(t0), p1 = fast_exp2(t1);
                  if (k2 & 1) rsb = fadd2(rsb, pack2(p0, p1)); else rsa = fadd2(rsa, pack2(p0, p1));
                  packed = pack_bf16(p0, p1) & keep;
                }
                pk[rr * PC + k2] = packed;
              }
              if (mine) rs2 = fadd2(rs2, fadd2(rsa, rsb));
            }
            {
              float r0, r1;
              unpack2(rs2, r0, r1);
              l_run += r0 + r1;
            }
          } else {
#pragma unroll
            for (int j = 0; j < UNIT_PCOLS; ++j) pk[j] = 0u;
            if (last_load && !s_released) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(s_free);
              s_released = true;
            }
            // The zeros of a first unit the warp does not see are stored after the second
            // unit's exponentials: the wait for the previous P V must not come before them.
            if (u == 0 && (warp_rows >> 4) != 0u) continue;
          }
          if (!p_free) {
            if (!na_wait(pv_done(st_prev), ph_prev, abort_flag, ST_TIMEOUT_SOFTMAX)) ok = false;
            tc_fence_after();
            p_free = true;
            if (i == 0 && pend && ok) {
              // O still holds the previous item (this item's first P V has not been issued):
              // its rows are normalised and stored now
              na_store_o_row(o_taddr, pend_inv, pend_op);
              pend = false;
            }
          }
          if constexpr (EWP == 16) {
            tmem_st_x16(p_taddr + u * UNIT_PCOLS, &pk[0]);
            tmem_st_x16(p_taddr + u * UNIT_PCOLS + 16, &pk[16]);
          } else {
            tmem_st_x16(p_taddr + u * UNIT_PCOLS, &pk[0]);
          }
        }
        if ((warp_rows & 15u) == 0u && (warp_rows >> 4) != 0u) {   // the postponed zeros of unit 0
          uint32_t z[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) z[j] = 0u;
          tmem_st_x16(p_taddr, z);
          if constexpr (EWP == 16) tmem_st_x16(p_taddr + 16, z);
        }
        if (!ok) break;
        // every lane completes its P stores, then one lane arrives for the warp
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready);
        if (++st_prev == STAGES) { st_prev = 0; ph_prev ^= 1u; }
      }
      if (!ok) break;

      // The item's row is normalised and stored later - while the first block of the next
      // item waits for this item's last P V anyway (or after the loop) - so that the wait is
      // spent on that block's exponentials.
      if (!(l_run < SUM_REPAIRABLE)) {   // beyond repair (or NaN): this row is computed again below
        if (n < 64) bad_items |= 1ull << n; else bad_rest = true;
      }
      {
        const long long tok = ((static_cast<long long>(it.b) * p.D + (it.d0 + zd)) * p.o_H +
                               (it.h0 + zh - p.o_h0)) * p.o_W + (it.w0 + zw - p.o_w0);
        pend_op = q_ok ? p.out + tok * p.ldo + it.head * 64 : nullptr;
        pend_inv = 1.0f / l_run;
        pend = true;
      }
    }
    if (ok && pend) {
      if (na_wait(pv_done(st_prev), ph_prev, abort_flag, ST_TIMEOUT_SOFTMAX)) {
        tc_fence_after();
        na_store_o_row(o_taddr, pend_inv, pend_op);
      } else {
        ok = false;
      }
    }
    // rows whose scores left the range of the fast path: computed again the plain way
    if (ok && (bad_items != 0ull || bad_rest)) {
      const Na3dParams pc = p;   // a callee cannot address the kernel's parameter bank
      na_slow_rows<KW, QW>(pc, bad_items, bad_rest, n_my, has_query, zd, zh, zw);
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
      const int per = 32 / p.QW;                    // (zd, zh) pairs per quarter
      for (int q = 0; q < 4; ++q)
        for (int j = per * q; j < per * (q + 1) && j < p.QD * p.QH; ++j) {
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

// q/k/v: token-major bf16, element (b,d,h,w,head,c) at base + token*ld + head*64 + c where
// token = ((b*D + d)*H + h)*W + w. out likewise with ldo.
template <int KW, int QW>
inline int launch_na3d_t(const __nv_bfloat16* q, long long ldq, const __nv_bfloat16* k,
                         long long ldk, const __nv_bfloat16* v, long long ldv, Na3dParams p,
                         int sm_count, cudaStream_t stream) {
  using Cfg = Na3dCfg<KW, QW>;
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
  if (make(&tmQ, q, ldq, QW, p.QH, p.QD) != 0) return -20;
  if (make(&tmK, k, ldk, Cfg::EWP, 4, 1) != 0) return -20;
  if (make(&tmV, v, ldv, Cfg::EWP, 4, 1) != 0) return -20;
  p.q = q; p.k = k; p.v = v;
  p.ldq = ldq; p.ldk = ldk; p.ldv = ldv;
  auto kern = na3d_fwd_kernel<KW, QW>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::TOTAL);
  if (e != cudaSuccess) return -static_cast<int>(e) - 1000;
  const int grid = p.n_items < 2 * sm_count ? p.n_items : 2 * sm_count;
  kern<<<grid, Cfg::THREADS, Cfg::TOTAL, stream>>>(tmQ, tmK, tmV, p);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

inline int launch_na3d(const __nv_bfloat16* q, long long ldq, const __nv_bfloat16* k, long long ldk,
                       const __nv_bfloat16* v, long long ldv, __nv_bfloat16* out, long long ldo,
                       int B, int D, int H, int W, int heads, int kd, int kh, int kw, float scale,
                       int sm_count, cudaStream_t stream, int q_h0 = 0, int q_H = -1, int q_w0 = 0,
                       int q_W = -1, int o_h0 = 0, int o_H = -1, int o_w0 = 0, int o_W = -1) {
  if (kd > D || kh > H || kw > W || kd < 1 || kh < 1 || kw < 1) return -1;
  if (kh > 15 || kd > 15 || kw > 15 || !(kw & 1)) return -2;
  Na3dParams p{};
  p.B = B; p.D = D; p.H = H; p.W = W; p.heads = heads;
  p.kd = kd; p.kh = kh;
  // Query tile: as wide as key rows of 16 columns allow, 16 rows when that leaves room, the
  // rest in depth - as far as the tensor is deep and the key box stays within 16 planes.
  p.QW = kw <= 9 ? 8 : (kw <= 13 ? 4 : 2);
  if (p.QW == 8) {
    // 16 query rows as 1 x 16, 2 x 8 or 4 x 4 (depth x height): the shape whose key box has the
    // fewest (plane, 4-row) units - deep windows (kd >= 7) favour 4 x 4; a tie goes to 2 x 8
    int best_units = 1 << 30;
    for (int qd = 1; qd <= 4; qd <<= 1) {
      const int qh = 16 / qd;
      if (qd > D || qd + kd - 1 > 16 || qh + kh - 1 > 31) continue;
      const int units = (qd + kd - 1) * ((qh + kh - 1 + 3) / 4);
      if (units < best_units || (units == best_units && qd == 2)) {
        best_units = units; p.QD = qd; p.QH = qh;
      }
    }
    if (best_units == (1 << 30)) return -2;
  } else {
    // narrower tiles hold 32 (QW = 4) or 64 (QW = 2) query rows: 16 or 8 rows high, the rest in
    // depth as far as the tensor is deep and the key box stays within 16 planes and 128 units;
    // among those the shape with the fewest key units (ties keep 16 rows)
    const int rows = 128 / p.QW;
    int best_units = 1 << 30;
    for (int qh = 16; qh >= 8; qh >>= 1) {
      int qd = rows / qh;
      while (qd > 1 && (qd > D || qd + kd - 1 > 16)) qd >>= 1;
      if (qh + kh - 1 > 31) continue;
      const int units = (qd + kd - 1) * ((qh + kh - 1 + 3) / 4);
      // compare per query row: a shrunk depth leaves part of the tile empty
      const long long cost = static_cast<long long>(units) * rows / (qd * qh);
      if (units <= 128 && cost < best_units) { best_units = static_cast<int>(cost); p.QD = qd; p.QH = qh; }
    }
    if (best_units == (1 << 30)) return -2;
  }
  p.q_rows = p.QD * p.QH * p.QW;
  if (p.QH + kh - 1 > 31) return -2;
  p.q_h0 = q_h0; p.q_w0 = q_w0;
  p.q_H = q_H < 0 ? H : q_H;
  p.q_W = q_W < 0 ? W : q_W;
  if (p.q_h0 < 0 || p.q_w0 < 0 || p.q_H < 1 || p.q_W < 1 || p.q_h0 + p.q_H > H ||
      p.q_w0 + p.q_W > W)
    return -1;
  if (o_H < 0 || o_W < 0) {
    p.o_h0 = p.q_h0; p.o_H = p.q_H; p.o_w0 = p.q_w0; p.o_W = p.q_W;
  } else {
    p.o_h0 = o_h0; p.o_H = o_H; p.o_w0 = o_w0; p.o_W = o_W;
    if (o_h0 > p.q_h0 || o_w0 > p.q_w0 || o_h0 + o_H < p.q_h0 + p.q_H || o_w0 + o_W < p.q_w0 + p.q_W)
      return -1;   // the output window must contain the query region
  }
  p.tiles_d = (D + p.QD - 1) / p.QD;
  p.tiles_h = (p.q_H + p.QH - 1) / p.QH;
  p.tiles_w = (p.q_W + p.QW - 1) / p.QW;
  const long long items = static_cast<long long>(p.tiles_d) * p.tiles_h * p.tiles_w * heads * B;
  if (items > 0x7fffffffLL) return -2;
  p.n_items = static_cast<int>(items);
  if (na_build_blocks(p) != 0) return -2;
  p.out = out;
  p.ldo = ldo;
  p.scale_log2e = scale * 1.4426950408889634f;
  switch (kw) {
    case 1: return launch_na3d_t<1, 8>(q, ldq, k, ldk, v, ldv, p, sm_count, stream);
    case 3: return launch_na3d_t<3, 8>(q, ldq, k, ldk, v, ldv, p, sm_count, stream);
    case 5: return launch_na3d_t<5, 8>(q, ldq, k, ldk, v, ldv, p, sm_count, stream);
    case 7: return launch_na3d_t<7, 8>(q, ldq, k, ldk, v, ldv, p, sm_count, stream);
    case 9: return launch_na3d_t<9, 8>(q, ldq, k, ldk, v, ldv, p, sm_count, stream);
    case 11: return launch_na3d_t<11, 4>(q, ldq, k, ldk, v, ldv, p, sm_count, stream);
    case 13: return launch_na3d_t<13, 4>(q, ldq, k, ldk, v, ldv, p, sm_count, stream);
    case 15: return launch_na3d_t<15, 2>(q, ldq, k, ldk, v, ldv, p, sm_count, stream);
    default: return -2;
  }
}

}  // namespace strata
