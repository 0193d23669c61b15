// Fused 3-D neighbourhood attention forward for sm_100a (head_dim 64, bf16, non-causal,
// dilation 1): for every query token, softmax(q.k * scale) over the kd*kh*kw keys of its
// window, times v. Windows keep their full size at the borders: along an axis of length L
// the window of query i starts at clamp(i - k/2, 0, L - k).
//
// Work decomposition
//   CTA            one tile of 128 queries (QD x QH x 8 tokens) of one head of one tile batch
//                  entry; two CTAs are co-resident per SM so one CTA's softmax overlaps the
//                  other's tensor work.
//   key blocks     the union of the tile's windows is a box of ED x EH x EW keys
//                  (E* = Q* + k* - 1) starting at the window start of the tile's first query.
//                  It is streamed as blocks of one depth plane x 8 rows x EW columns
//                  (NKEYS = 8*EW keys); TMA zero-fills whatever lies outside the tensor.
//   warp 0         TMA producer: Q tile once, then K and V blocks into a 2-stage ring
//                  (5-D tensor maps over [B, D, H, W, channels]; 128-byte swizzle, a key's 64
//                  channels are one 128-byte row).
//   warp 1         MMA issuer: S = Q K^T (M=128, N=NKEYS, K=64) into TMEM, then
//                  O_blk = P V (M=128, N=64, K=NKEYS) with P read from shared memory.
//   warps 2-5      softmax: each thread owns one query row. Pass 1 reads its S row from
//                  TMEM and takes the masked maximum, pass 2 re-reads it, exponentiates,
//                  writes bf16 P into the swizzled A-operand layout and keeps the running
//                  sum; the per-block P V result is read back from TMEM and accumulated
//                  in registers with the usual online-softmax rescaling. Key rows that no
//                  query of the warp can see are skipped (zeros written) without touching
//                  the exponential unit.
//   mask           per (query, key): the key's box coordinates must fall in the query's
//                  window on all three axes; evaluated from a per-thread column bit mask,
//                  a row bit mask and a plane test, so border clamping is exact per row.
#pragma once
#include "common.cuh"
#include "tensormap.cuh"

namespace strata {

struct Na3dParams {
  int B, D, H, W, heads;
  int kd, kh;            // kernel extents along depth and rows (columns: template KW)
  int QD, QH;            // query tile extents (QW = 8); QD*QH = 16
  int tiles_d, tiles_h, tiles_w;
  __nv_bfloat16* out;    // [B, D, H, W, ldo] with head h at channel offset h*64
  long long ldo;
  float scale_log2e;
};

constexpr int NA_THREADS = 192;
constexpr int NA_QW = 8;
constexpr int NA_TMEM_COLS = 256;
constexpr int NA_O_COL = 192;

template <int KW>
struct Na3dCfg {
  static constexpr int EW = NA_QW + KW - 1;
  static constexpr int NKEYS = 8 * EW;
  static constexpr int KV_BYTES = NKEYS * 128;
  static constexpr int P_ATOMS = (NKEYS + 63) / 64;
  static constexpr int Q_BYTES = 128 * 128;
  static constexpr int STAGES = 2;
  static constexpr int P_OFF = Q_BYTES + STAGES * 2 * KV_BYTES;
  static constexpr int BAR_OFF = P_OFF + P_ATOMS * 16384;
  static constexpr int TOTAL = BAR_OFF + 128;
  static_assert(NKEYS % 16 == 0 && NKEYS <= NA_O_COL, "key block must fit the S columns");
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
// Loads at least EW consecutive S columns of this thread's row (extra columns are ignored).
template <int EW>
__device__ __forceinline__ void tmem_ld_keyrow(uint32_t taddr, uint32_t (&a)[32]) {
  if constexpr (EW <= 16) {
    tmem_ld_x16(taddr, a);
  } else if constexpr (EW <= 24) {
    tmem_ld_x16(taddr, a);
    tmem_ld_x8(taddr + 16, a + 16);
  } else {
    tmem_ld_32x32(taddr, a);
  }
}

template <int KW>
__global__ void __launch_bounds__(NA_THREADS, 2)
na3d_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const Na3dParams p) {
  using Cfg = Na3dCfg<KW>;
  constexpr int EW = Cfg::EW;
  constexpr int NKEYS = Cfg::NKEYS;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  if ((sbase & 1023u) != 0) {  // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(&g_status, 0, ST_BAD_TMEM);
    return;
  }
  const uint32_t q_smem = sbase;
  auto k_smem = [&](int st) { return sbase + Cfg::Q_BYTES + st * 2 * Cfg::KV_BYTES; };
  auto v_smem = [&](int st) { return k_smem(st) + Cfg::KV_BYTES; };
  const uint32_t p_smem = sbase + Cfg::P_OFF;
  const uint32_t bar = sbase + Cfg::BAR_OFF;
  const uint32_t q_full = bar, s_full = bar + 8, p_ready = bar + 16, o_full = bar + 24;
  auto kv_full = [&](int st) { return bar + 32 + 8 * st; };
  auto kv_empty = [&](int st) { return bar + 48 + 8 * st; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::BAR_OFF + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::BAR_OFF + 72);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // tile coordinates
  int t = blockIdx.x;
  const int tw = t % p.tiles_w; t /= p.tiles_w;
  const int th = t % p.tiles_h; t /= p.tiles_h;
  const int td = t;
  const int head = blockIdx.y;
  const int b = blockIdx.z;
  const int d0 = td * p.QD, h0 = th * p.QH, w0 = tw * NA_QW;
  // key box origin = window start of the tile's first query on each axis
  const int bd0 = na_window_start(d0, p.D, p.kd);
  const int bh0 = na_window_start(h0, p.H, p.kh);
  const int bw0 = na_window_start(w0, p.W, KW);
  const int ED = p.QD + p.kd - 1;
  const int EH = p.QH + p.kh - 1;
  const int n_hb = (EH + 7) >> 3;
  const int nblk = ED * n_hb;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(s_full, 1);
    mbar_init(p_ready, 128);
    mbar_init(o_full, 1);
    for (int s = 0; s < Cfg::STAGES; ++s) {
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
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, Cfg::Q_BYTES);
      tma_load_5d(q_smem, &tmQ, head * 64, w0, h0, d0, b, q_full);
      bool ok = true;
      for (int i = 0; i < nblk; ++i) {
        const int st = i & 1;
        const uint32_t ph = (i >> 1) & 1u;
        if (!mbar_wait(kv_empty(st), ph ^ 1u, abort_flag, ST_TIMEOUT_PRODUCER)) {
          ok = false;
          break;
        }
        const int ip = i / n_hb, hb = i - ip * n_hb;
        mbar_expect_tx(kv_full(st), 2 * Cfg::KV_BYTES);
        tma_load_5d(k_smem(st), &tmK, head * 64, bw0, bh0 + 8 * hb, bd0 + ip, b, kv_full(st));
        tma_load_5d(v_smem(st), &tmV, head * 64, bw0, bh0 + 8 * hb, bd0 + ip, b, kv_full(st));
      }
      if (!ok)
        for (int i = 0; i < 2000; ++i) __nanosleep(100);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, NKEYS, false, false);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 64, false, true);
      const uint32_t s_tmem = tmem_base;
      const uint32_t o_tmem = tmem_base + NA_O_COL;
      if (mbar_wait(q_full, 0, abort_flag, ST_TIMEOUT_MMA)) {
        const uint64_t qdesc = umma_smem_desc_sw128(q_smem);
        for (int i = 0; i < nblk; ++i) {
          const int st = i & 1;
          const uint32_t ph = (i >> 1) & 1u;
          if (!mbar_wait(kv_full(st), ph, abort_flag, ST_TIMEOUT_MMA)) break;
          tc_fence_after();
          const uint64_t kdesc = umma_smem_desc_sw128(k_smem(st));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_ss(s_tmem, qdesc + 2u * k, kdesc + 2u * k, idesc_qk, k != 0 ? 1u : 0u);
          umma_commit(s_full);
          if (!mbar_wait(p_ready, i & 1u, abort_flag, ST_TIMEOUT_MMA)) break;
          tc_fence_after();
          const uint64_t vdesc = umma_smem_desc_sw128(v_smem(st));
#pragma unroll
          for (int s = 0; s < NKEYS / 16; ++s) {
            const uint64_t pdesc =
                umma_smem_desc_sw128(p_smem + (s >> 2) * 16384 + (s & 3) * 32);
            // V advances 16 keys = 16 rows of 128 bytes per step (2048 bytes, 128 units)
            umma_ss(o_tmem, pdesc, vdesc + 128u * s, idesc_pv, s != 0 ? 1u : 0u);
          }
          umma_commit(kv_empty(st));
          umma_commit(o_full);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax warps
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int zw = r & 7;
    const int zh = (r >> 3) % p.QH;
    const int zd = (r >> 3) / p.QH;
    const bool q_ok = (d0 + zd < p.D) && (h0 + zh < p.H) && (w0 + zw < p.W);
    const int id = min(d0 + zd, p.D - 1), ih = min(h0 + zh, p.H - 1), iw = min(w0 + zw, p.W - 1);
    const int wd = na_window_start(id, p.D, p.kd) - bd0;
    const int wh = na_window_start(ih, p.H, p.kh) - bh0;
    const int ww = na_window_start(iw, p.W, KW) - bw0;
    const uint32_t colmask = ((1u << KW) - 1u) << ww;
    const uint32_t hmask_all = ((1u << p.kh) - 1u) << wh;   // bit = key row of the box
    const uint32_t lane_taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t p_row = p_smem + r * 128;
    const uint32_t sw = static_cast<uint32_t>(r & 7);
    const float c = p.scale_log2e;

    float m_run = -1e30f, l_run = 0.f, alpha_prev = 1.f;
    float o[64];
#pragma unroll
    for (int j = 0; j < 64; ++j) o[j] = 0.f;

    bool ok = true;
    for (int i = 0; i < nblk && ok; ++i) {
      const int ip = i / n_hb, hb = i - ip * n_hb;
      if (!mbar_wait(s_full, i & 1u, abort_flag, ST_TIMEOUT_SOFTMAX)) { ok = false; break; }
      tc_fence_after();
      const bool dvalid = static_cast<unsigned>(ip - wd) < static_cast<unsigned>(p.kd);
      const uint32_t rowmask = dvalid ? ((hmask_all >> (8 * hb)) & 0xffu) : 0u;
      const uint32_t warp_rows = __reduce_or_sync(0xffffffffu, rowmask);

      // pass 1: masked row maximum
      float bm = -1e30f;
#pragma unroll
      for (int rr = 0; rr < 8; ++rr) {
        if ((warp_rows >> rr) & 1u) {
          uint32_t a[32];
          tmem_ld_keyrow<EW>(lane_taddr + rr * EW, a);
          tmem_ld_wait();
          const uint32_t mk = ((rowmask >> rr) & 1u) ? colmask : 0u;
#pragma unroll
          for (int cc = 0; cc < EW; ++cc)
            if ((mk >> cc) & 1u) bm = fmaxf(bm, __uint_as_float(a[cc]));
        }
      }
      const float m_new = fmaxf(m_run, bm);
      const float alpha = fast_exp2((m_run - m_new) * c);
      const float mc = m_new * c;

      // fold in the previous block's P V result
      if (i > 0) {
        if (!mbar_wait(o_full, (i - 1) & 1u, abort_flag, ST_TIMEOUT_SOFTMAX)) { ok = false; break; }
        tc_fence_after();
        uint32_t ob[32];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          tmem_ld_32x32(lane_taddr + NA_O_COL + 32 * hh, ob);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            o[32 * hh + j] = o[32 * hh + j] * alpha_prev + __uint_as_float(ob[j]);
        }
      }

      // pass 2: exponentials, row sum, bf16 P into the swizzled A-operand layout
      float rs = 0.f;
      uint32_t pk[4] = {0u, 0u, 0u, 0u};
#pragma unroll
      for (int rr = 0; rr < 8; ++rr) {
        const bool need = (warp_rows >> rr) & 1u;
        uint32_t a[32];
        uint32_t mk = 0u;
        if (need) {
          tmem_ld_keyrow<EW>(lane_taddr + rr * EW, a);
          tmem_ld_wait();
          mk = ((rowmask >> rr) & 1u) ? colmask : 0u;
        }
#pragma unroll
        for (int cc = 0; cc < EW; cc += 2) {
          const int j = rr * EW + cc;  // even
          float p0 = 0.f, p1 = 0.f;
          if (need) {
            if ((mk >> cc) & 1u) p0 = fast_exp2(__uint_as_float(a[cc]) * c - mc);
            if ((mk >> (cc + 1)) & 1u) p1 = fast_exp2(__uint_as_float(a[cc + 1]) * c - mc);
            rs += p0 + p1;
          }
          pk[(j >> 1) & 3] = pack_bf16(p0, p1);
          if ((j & 7) == 6) {
            const uint32_t chunk = static_cast<uint32_t>((j & 63) >> 3);
            const uint32_t addr = p_row + (j >> 6) * 16384 + ((chunk ^ sw) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[0]),
                         "r"(pk[1]), "r"(pk[2]), "r"(pk[3])
                         : "memory");
          }
        }
      }
      l_run = l_run * alpha + rs;
      m_run = m_new;
      alpha_prev = alpha;
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
    }

    if (ok && mbar_wait(o_full, (nblk - 1) & 1u, abort_flag, ST_TIMEOUT_SOFTMAX)) {
      tc_fence_after();
      uint32_t ob[32];
      const float inv = 1.0f / l_run;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        tmem_ld_32x32(lane_taddr + NA_O_COL + 32 * hh, ob);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j)
          o[32 * hh + j] = (o[32 * hh + j] * alpha_prev + __uint_as_float(ob[j])) * inv;
      }
      if (q_ok) {
        const long long tok =
            ((static_cast<long long>(b) * p.D + (d0 + zd)) * p.H + (h0 + zh)) * p.W + (w0 + zw);
        __nv_bfloat16* op = p.out + tok * p.ldo + head * 64;
#pragma unroll
        for (int j = 0; j < 64; j += 8) {
          uint4 v4;
          v4.x = pack_bf16(o[j], o[j + 1]);
          v4.y = pack_bf16(o[j + 2], o[j + 3]);
          v4.z = pack_bf16(o[j + 4], o[j + 5]);
          v4.w = pack_bf16(o[j + 6], o[j + 7]);
          *reinterpret_cast<uint4*>(op + j) = v4;
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

// q/k/v: token-major bf16, element (b,d,h,w,head,c) at base + token*ld + head*64 + c where
// token = ((b*D + d)*H + h)*W + w. out likewise with ldo.
template <int KW>
inline int launch_na3d_t(const __nv_bfloat16* q, long long ldq, const __nv_bfloat16* k,
                         long long ldk, const __nv_bfloat16* v, long long ldv, Na3dParams p,
                         cudaStream_t stream) {
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
  if (make(&tmK, k, ldk, Cfg::EW, 8, 1) != 0) return -20;
  if (make(&tmV, v, ldv, Cfg::EW, 8, 1) != 0) return -20;
  auto kern = na3d_fwd_kernel<KW>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::TOTAL);
  if (e != cudaSuccess) return -static_cast<int>(e) - 1000;
  dim3 grid(p.tiles_d * p.tiles_h * p.tiles_w, p.heads, p.B);
  kern<<<grid, NA_THREADS, Cfg::TOTAL, stream>>>(tmQ, tmK, tmV, p);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

inline int launch_na3d(const __nv_bfloat16* q, long long ldq, const __nv_bfloat16* k, long long ldk,
                       const __nv_bfloat16* v, long long ldv, __nv_bfloat16* out, long long ldo,
                       int B, int D, int H, int W, int heads, int kd, int kh, int kw, float scale,
                       cudaStream_t stream) {
  if (kd > D || kh > H || kw > W || kd < 1 || kh < 1 || kw < 1) return -1;
  if (kh > 15 || kd > 15) return -2;
  Na3dParams p{};
  p.B = B; p.D = D; p.H = H; p.W = W; p.heads = heads;
  p.kd = kd; p.kh = kh;
  // query tile: 2 x 8 x 8, flattened towards the rows when the tensor is shallow
  if (D >= 2) { p.QD = 2; p.QH = 8; } else { p.QD = 1; p.QH = 16; }
  if (p.QH + kh - 1 > 31) return -2;
  p.tiles_d = (D + p.QD - 1) / p.QD;
  p.tiles_h = (H + p.QH - 1) / p.QH;
  p.tiles_w = (W + NA_QW - 1) / NA_QW;
  p.out = out;
  p.ldo = ldo;
  p.scale_log2e = scale * 1.4426950408889634f;
  if (heads > 65535 || B > 65535) return -2;
  switch (kw) {
    case 1: return launch_na3d_t<1>(q, ldq, k, ldk, v, ldv, p, stream);
    case 3: return launch_na3d_t<3>(q, ldq, k, ldk, v, ldv, p, stream);
    case 5: return launch_na3d_t<5>(q, ldq, k, ldk, v, ldv, p, stream);
    case 7: return launch_na3d_t<7>(q, ldq, k, ldk, v, ldv, p, stream);
    case 9: return launch_na3d_t<9>(q, ldq, k, ldk, v, ldv, p, stream);
    case 11: return launch_na3d_t<11>(q, ldq, k, ldk, v, ldv, p, stream);
    case 13: return launch_na3d_t<13>(q, ldq, k, ldk, v, ldv, p, stream);
    case 15: return launch_na3d_t<15>(q, ldq, k, ldk, v, ldv, p, stream);
    default: return -2;
  }
}

}  // namespace strata
