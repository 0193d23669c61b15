// Cubed-sphere tile halo exchange: gather kernels and the cross-GPU flag barrier.
//
// A padded tile is assembled by GATHER: for every cell of every padded local tile a
// precomputed map names the interior cell it copies (src_a) and, on a corner diagonal, a
// second cell it is averaged with (src_b >= 0). A cell id is  g*T*T + i*T + j  with g the
// tile's position in the global tile order; id / cells_per_rank is the owning rank and the
// remainder the cell's offset inside that rank's tile buffer, so the source may sit in this
// GPU's memory or in a peer's (plain loads over NVLink through a peer-mapped pointer; no TMA,
// no multicast). Face-edge rotation and the corner rule are entirely in the map, so the
// kernel's result is bit-identical to applying the same index logic on the host (copies
// always; the two-cell mean and the weighted sums of the other kernels of this file for
// normal-range values - the library is built with flush-to-zero).
//
// Mean of two cells: (a + b) / 2 evaluated in the storage type's own arithmetic (fp32: one
// add, one halving; bf16: the sum is rounded to bf16, then halved - what a bf16 tensor
// expression produces).
//
// HBM-bound (remote part: NVLink-bound): payload bytes read once and written once.
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"

namespace strata {

constexpr int HALO_MAX_RANKS = 16;
struct PeerPtrs {
  const void* p[HALO_MAX_RANKS];
};
struct FlagPtrs {
  int* p[HALO_MAX_RANKS];
};

// 1 while the last cross-GPU flag barrier on this device completed (or none has run), 0 after
// one whose bounded wait ran out. The gather kernels that follow a barrier on the stream read
// it: after a failed barrier the peers' slots may be unpublished or stale, so they fill their
// output with NaN instead of plausible-looking numbers. Set back to 1 by the next barrier that
// completes, or when the host clears the device status word.
__device__ int g_halo_ok = 1;
__device__ __forceinline__ bool halo_exchange_failed() {
  return *reinterpret_cast<volatile int*>(&g_halo_ok) == 0;
}
constexpr uint32_t BF16_NAN2 = 0x7fc07fc0u;

// Token layout: source buffers [tiles_per_rank, D, T*T, C] bf16, output [tiles_per_rank, D, P*P, C].
// grid: x over groups of 256 padded cells (a warp takes 32 consecutive ones: lane l works out
// cell l's source rows - the integer divisions happen once per cell, 32 cells side by side -
// then the warp moves the cells one after the other, a 16-byte vector per lane at a time),
// y over (tile, depth).
__global__ void __launch_bounds__(256)
halo_gather_tokens_kernel(__nv_bfloat16* __restrict__ out, const PeerPtrs src,
                          const int* __restrict__ src_a, const int* __restrict__ src_b, int PP,
                          int TT, int D, int C, int cells_per_rank, int only_halo,
                          int halo_lo, int halo_hi, int P) {
  const int vpc = C >> 3;  // 16-byte vectors per cell
  const int tile = blockIdx.y / D;
  const int d = blockIdx.y - tile * D;
  const bool failed = halo_exchange_failed();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  for (int base = (blockIdx.x * warps + warp) * 32; base < PP; base += gridDim.x * warps * 32) {
    const int pc_l = base + lane;
    const __nv_bfloat16* my_a = nullptr;   // nullptr: nothing to do for this cell
    const __nv_bfloat16* my_b = nullptr;
    if (pc_l < PP) {
      bool skip = false;
      if (only_halo) {
        const int pi = pc_l / P, pj = pc_l - pi * P;
        skip = pi >= halo_lo && pi < halo_hi && pj >= halo_lo && pj < halo_hi;
      }
      if (!skip) {
        auto source_row = [&](int id) -> const __nv_bfloat16* {
          const int rank = id / cells_per_rank;
          const int local = id - rank * cells_per_rank;
          const int st = local / TT;
          const int sc = local - st * TT;
          return static_cast<const __nv_bfloat16*>(src.p[rank]) +
                 ((static_cast<long long>(st) * D + d) * TT + sc) * C;
        };
        my_a = source_row(__ldg(src_a + tile * PP + pc_l));
        const int b = __ldg(src_b + tile * PP + pc_l);
        if (b >= 0) my_b = source_row(b);
      }
    }
    const int n_here = min(32, PP - base);
    for (int c = 0; c < n_here; ++c) {
      const __nv_bfloat16* row_a = reinterpret_cast<const __nv_bfloat16*>(
          __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_a), c));
      const __nv_bfloat16* row_b = reinterpret_cast<const __nv_bfloat16*>(
          __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_b), c));
      if (row_a == nullptr) continue;
      __nv_bfloat16* out_row = out + ((static_cast<long long>(tile) * D + d) * PP + base + c) * C;
      constexpr int UNROLL = 4;
      for (int v0 = lane; v0 < vpc; v0 += 32 * UNROLL) {
        uint4 x[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const int v = v0 + 32 * u;
          if (v < vpc) x[u] = *reinterpret_cast<const uint4*>(row_a + (v << 3));
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const int v = v0 + 32 * u;
          if (v >= vpc) continue;
          uint4 r = x[u];
          if (row_b != nullptr) {
            const uint4 s2 = *reinterpret_cast<const uint4*>(row_b + (v << 3));
            uint32_t* rw = reinterpret_cast<uint32_t*>(&r);
            const uint32_t* sw = reinterpret_cast<const uint32_t*>(&s2);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              // sum rounded to bf16 first, then halved (exact)
              const float lo = __bfloat162float(__float2bfloat16(bf16_lo(rw[t]) + bf16_lo(sw[t]))) * 0.5f;
              const float hi = __bfloat162float(__float2bfloat16(bf16_hi(rw[t]) + bf16_hi(sw[t]))) * 0.5f;
              rw[t] = pack_bf16(lo, hi);
            }
          }
          if (failed) r = make_uint4(BF16_NAN2, BF16_NAN2, BF16_NAN2, BF16_NAN2);
          *reinterpret_cast<uint4*>(out_row + (v << 3)) = r;
        }
      }
    }
  }
}

// Field layout: source buffers [L, tiles_per_rank*T*T] fp32 (L = product of leading dims),
// output [L, tiles_per_rank*P*P]. grid: x over padded cells, y over leading index.
__global__ void __launch_bounds__(256)
halo_gather_fields_kernel(float* __restrict__ out, const PeerPtrs src,
                          const int* __restrict__ src_a, const int* __restrict__ src_b,
                          int n_out_cells, int cells_per_rank, int L) {
  const bool failed = halo_exchange_failed();
  for (int oc = blockIdx.x * blockDim.x + threadIdx.x; oc < n_out_cells;
       oc += gridDim.x * blockDim.x) {
    const int a = __ldg(src_a + oc);
    const int b = __ldg(src_b + oc);
    const int ra = a / cells_per_rank, la = a - ra * cells_per_rank;
    const float* pa = static_cast<const float*>(src.p[ra]) + la;
    const float* pb = nullptr;
    if (b >= 0) {
      const int rb = b / cells_per_rank, lb = b - rb * cells_per_rank;
      pb = static_cast<const float*>(src.p[rb]) + lb;
    }
    constexpr int UL = 4;   // leading indices in flight per thread (independent loads)
    int l = blockIdx.y;
    for (; l + (UL - 1) * static_cast<int>(gridDim.y) < L; l += UL * gridDim.y) {
      float v[UL];
#pragma unroll
      for (int u = 0; u < UL; ++u) {
        const long long so = static_cast<long long>(l + u * gridDim.y) * cells_per_rank;
        v[u] = pa[so];
        if (pb) v[u] = (v[u] + pb[so]) / 2.0f;
      }
#pragma unroll
      for (int u = 0; u < UL; ++u)
        out[static_cast<long long>(l + u * gridDim.y) * n_out_cells + oc] =
            failed ? __int_as_float(0x7fc00000) : v[u];
    }
    for (; l < L; l += gridDim.y) {
      const long long so = static_cast<long long>(l) * cells_per_rank;
      float v = pa[so];
      if (pb) v = (v + pb[so]) / 2.0f;
      out[static_cast<long long>(l) * n_out_cells + oc] = failed ? __int_as_float(0x7fc00000) : v;
    }
  }
}

// Weighted gather (k-nearest-neighbour halo): out[l, oc] = sum_j w[oc, j] * x[l, idx[oc, j]]
// with idx a global interior cell id (owner rank = id / cells_per_rank) - the sparse operator
// the reference applies to an all-gathered copy of the whole globe, evaluated here by reading
// the k source cells from the tiles of their owners (local or peer memory). Products and sums
// are rounded one by one in source order (no fused multiply-add): reproducible on the host.
// Source buffers [L, cells_per_rank] fp32 per rank; out [L, n_out_cells].
template <int K>
__global__ void __launch_bounds__(256)
halo_gather_knn_fields_kernel(float* __restrict__ out, const PeerPtrs src,
                              const int* __restrict__ idx, const float* __restrict__ w,
                              int n_out_cells, int cells_per_rank, int L) {
  const bool failed = halo_exchange_failed();
  for (int oc = blockIdx.x * blockDim.x + threadIdx.x; oc < n_out_cells;
       oc += gridDim.x * blockDim.x) {
    const float* sp[K];
    float wk[K];
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const int id = __ldg(idx + static_cast<long long>(oc) * K + j);
      const int rank = id / cells_per_rank;
      sp[j] = static_cast<const float*>(src.p[rank]) + (id - rank * cells_per_rank);
      wk[j] = __ldg(w + static_cast<long long>(oc) * K + j);
    }
    for (int l = blockIdx.y; l < L; l += gridDim.y) {
      const long long so = static_cast<long long>(l) * cells_per_rank;
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) acc = __fadd_rn(acc, __fmul_rn(wk[j], sp[j][so]));
      out[static_cast<long long>(l) * n_out_cells + oc] = failed ? __int_as_float(0x7fc00000) : acc;
    }
  }
}

// Windowed overlap-add un-pad (the normalised transpose of the field gather): every interior
// cell c of this rank collects the padded cells that were copied from it - its own image and
// its copies in neighbouring tiles' halos, in local or peer memory - as
//     out[l, c] = ( sum_j coef_j * (window[p_j] * y[l, p_j]) ) / weights[c]
// with entries offsets[c]..offsets[c+1] sorted by padded cell id. Pull form: no atomics, a
// fixed summation order, every product and sum rounded separately (no fused multiply-add), so
// the result is bit-identical to the same loop on the host for normal-range values (the library
// is built with flush-to-zero, so a denormal operand or result is zero here and not there).
// Padded sources: [L, tiles_per_rank*P*P] fp32 per rank; out [L, tiles_per_rank*T*T].
__global__ void __launch_bounds__(256)
halo_adjoint_fields_kernel(float* __restrict__ out, const PeerPtrs src,
                           const int* __restrict__ offsets, const int* __restrict__ cell,
                           const float* __restrict__ coef, const float* __restrict__ window,
                           const float* __restrict__ weights, int n_cells,
                           int padded_cells_per_rank, int PP, int L) {
  const bool failed = halo_exchange_failed();
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < n_cells; c += gridDim.x * blockDim.x) {
    const int e0 = __ldg(offsets + c), e1 = __ldg(offsets + c + 1);
    // (after a failed barrier the divisor is NaN, and with it every output)
    const float wsum = failed ? __int_as_float(0x7fc00000) : __ldg(weights + c);
    // with the copy halo's coefficients (1 or 1/2) coef * (window * y) == (coef * window) * y bit
    // for bit, so the per-entry factor and source pointer are set up once, outside the loop over
    // the leading index (general coefficients - the k-nearest-neighbour lists - agree with the
    // long-list branch below to rounding only)
    constexpr int FAST = 4;
    const int ne = e1 - e0;
    if (ne <= FAST) {
      const float* sp[FAST];
      float wc[FAST];
#pragma unroll
      for (int j = 0; j < FAST; ++j) {
        const int e = e0 + (j < ne ? j : 0);
        const int p = __ldg(cell + e);
        const int rank = p / padded_cells_per_rank;
        const int local = p - rank * padded_cells_per_rank;
        sp[j] = static_cast<const float*>(src.p[rank]) + local;
        wc[j] = j < ne ? __fmul_rn(__ldg(coef + e), __ldg(window + local % PP)) : 0.f;
      }
      constexpr int UL = 4;   // leading indices in flight per thread (independent loads)
      int l = blockIdx.y;
      for (; l + (UL - 1) * static_cast<int>(gridDim.y) < L; l += UL * gridDim.y) {
        float y[UL][FAST];
#pragma unroll
        for (int u = 0; u < UL; ++u) {
          const long long so = static_cast<long long>(l + u * gridDim.y) * padded_cells_per_rank;
#pragma unroll
          for (int j = 0; j < FAST; ++j) y[u][j] = j < ne ? sp[j][so] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < UL; ++u) {
          float acc = 0.f;
#pragma unroll
          for (int j = 0; j < FAST; ++j)
            if (j < ne) acc = __fadd_rn(acc, __fmul_rn(wc[j], y[u][j]));
          out[static_cast<long long>(l + u * gridDim.y) * n_cells + c] = __fdiv_rn(acc, wsum);
        }
      }
      for (; l < L; l += gridDim.y) {
        const long long so = static_cast<long long>(l) * padded_cells_per_rank;
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < FAST; ++j)
          if (j < ne) acc = __fadd_rn(acc, __fmul_rn(wc[j], sp[j][so]));
        out[static_cast<long long>(l) * n_cells + c] = __fdiv_rn(acc, wsum);
      }
    } else {
      for (int l = blockIdx.y; l < L; l += gridDim.y) {
        const long long so = static_cast<long long>(l) * padded_cells_per_rank;
        float acc = 0.f;
        for (int e = e0; e < e1; ++e) {
          const int p = __ldg(cell + e);
          const int rank = p / padded_cells_per_rank;
          const int local = p - rank * padded_cells_per_rank;
          const float y = static_cast<const float*>(src.p[rank])[so + local];
          const float wy = __fmul_rn(__ldg(window + local % PP), y);
          acc = __fadd_rn(acc, __fmul_rn(__ldg(coef + e), wy));
        }
        out[static_cast<long long>(l) * n_cells + c] = __fdiv_rn(acc, wsum);
      }
    }
  }
}

// Per-block K/V halo for tiles whose packed qkv rows live in halo-padded layout
// [tiles_per_rank, D, P*P, ld] (q | k | v channel blocks of C each): the interiors were written
// by this rank's QKV GEMM, this kernel fills the K and V channels of the halo cells from the
// owning tiles' interiors (local or peer memory). K arrives rotated in the SENDER tile's RoPE
// frame; it is turned into the receiver's frame on the way by the per-cell delta rotation
// dcs[tile, cell, pair] = (cos, sin)(theta_receiver - theta_sender) (IEEE half pairs), V is
// copied. Corner-diagonal cells average their two (individually rotated) sources.
// grid: x over groups of 256 halo cells (a warp takes 32 consecutive ones), y over (tile, depth).
__global__ void __launch_bounds__(256, 3)
halo_gather_kv_kernel(__nv_bfloat16* __restrict__ qkv, const PeerPtrs src,
                      const int* __restrict__ src_a, const int* __restrict__ src_b,
                      const uint32_t* __restrict__ dcs_a, const uint32_t* __restrict__ dcs_b,
                      int P, int T, int halo, int D, int C, int head_dim, long long ld,
                      int cells_per_rank) {
  const int PP = P * P, TT = T * T;
  const int vpc = (2 * C) >> 3;     // 16-byte vectors of k|v per cell
  const int kvec = C >> 3;          // the first kvec of them are K
  const int half = head_dim >> 1;
  const int tile = blockIdx.y / D;
  const int d = blockIdx.y - tile * D;
  // only the halo cells are visited: first the two full-width strips above and below the
  // interior (2*halo rows of P cells), then the 2*halo side columns of the T interior rows
  const int n_strip = 2 * halo * P;
  const int n_halo = n_strip + 2 * halo * T;
  // A warp takes 32 consecutive halo cells. Lane l works out cell l's position and source rows
  // (a dozen integer divisions: done once per cell by one lane, all 32 cells side by side), then
  // the whole warp moves the cells one after the other, every lane a 16-byte vector at a time,
  // with the cell's addresses handed round by shuffles.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const bool failed = halo_exchange_failed();   // (read once: a volatile load per store halves the copy rate)
  for (int base = (blockIdx.x * warps + warp) * 32; base < n_halo; base += gridDim.x * warps * 32) {
    const int hc = base + lane;
    const __nv_bfloat16* my_a = nullptr;
    const __nv_bfloat16* my_b = nullptr;
    int my_pc = 0;
    if (hc < n_halo) {
      int pi, pj;
      if (hc < n_strip) {
        const int row = hc / P;
        pj = hc - row * P;
        pi = row < halo ? row : row + T;
      } else {
        const int e = hc - n_strip;
        const int row = e / (2 * halo);
        const int col = e - row * 2 * halo;
        pi = halo + row;
        pj = col < halo ? col : col + T;
      }
      my_pc = pi * P + pj;
      const int a = __ldg(src_a + tile * PP + my_pc);
      const int b = __ldg(src_b + tile * PP + my_pc);
      auto source_row = [&](int id) -> const __nv_bfloat16* {
        const int rank = id / cells_per_rank;
        const int local = id - rank * cells_per_rank;
        const int st = local / TT;
        const int sc = local - st * TT;
        const int si = sc / T, sj = sc - si * T;
        const long long row = ((static_cast<long long>(st) * D + d) * P + si + halo) * P + sj + halo;
        return static_cast<const __nv_bfloat16*>(src.p[rank]) + row * ld + C;   // k|v start after q
      };
      my_a = source_row(a);
      if (b >= 0) my_b = source_row(b);
    }
    const int n_here = min(32, n_halo - base);
    for (int c = 0; c < n_here; ++c) {
      const __nv_bfloat16* row_a = reinterpret_cast<const __nv_bfloat16*>(
          __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_a), c));
      const __nv_bfloat16* row_b = reinterpret_cast<const __nv_bfloat16*>(
          __shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_b), c));
      const int pc = __shfl_sync(0xffffffffu, my_pc, c);
      const long long tab_row = (static_cast<long long>(tile) * PP + pc) * half;
      __nv_bfloat16* out_row = qkv + ((static_cast<long long>(tile) * D + d) * PP + pc) * ld + C;
      // x: eight bf16 of the source row; t4: the four (cos, sin) pairs of a K vector
      auto rotate = [&](const uint4& x, const uint4& t4, bool is_k, float (&o)[8]) {
        const uint32_t w[4] = {x.x, x.y, x.z, x.w};
        if (is_k) {
          const uint32_t tw[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 cs = __half22float2(*reinterpret_cast<const __half2*>(&tw[t]));
            const float x0 = bf16_lo(w[t]), x1 = bf16_hi(w[t]);
            o[2 * t] = x0 * cs.x - x1 * cs.y;
            o[2 * t + 1] = x0 * cs.y + x1 * cs.x;
          }
        } else {
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            o[2 * t] = bf16_lo(w[t]);
            o[2 * t + 1] = bf16_hi(w[t]);
          }
        }
      };
      auto table = [&](const uint32_t* tab, int v) {   // first channel pair of vector v: ((8v) % head_dim) / 2
        return __ldg(reinterpret_cast<const uint4*>(tab + tab_row + (((v << 3) % head_dim) >> 1)));
      };
      // four vectors per lane and pass, all loads issued before the first use: the copy is
      // bound by the bytes a thread keeps in flight
      constexpr int UNROLL = 4;
      for (int v0 = lane; v0 < vpc; v0 += 32 * UNROLL) {
        uint4 xa[UNROLL], ta[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const int v = v0 + 32 * u;
          if (v < vpc) {
            xa[u] = *reinterpret_cast<const uint4*>(row_a + (v << 3));
            if (v < kvec) ta[u] = table(dcs_a, v);
          }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const int v = v0 + 32 * u;
          if (v >= vpc) continue;
          uint4 o4 = xa[u];   // V of a cell with one source is copied as it is
          if (v < kvec || row_b != nullptr) {
            float ra[8];
            rotate(xa[u], ta[u], v < kvec, ra);
            if (row_b != nullptr) {   // corner diagonal: the mean of two individually rotated sources
              float rb[8];
              const uint4 xb = *reinterpret_cast<const uint4*>(row_b + (v << 3));
              uint4 tb = make_uint4(0u, 0u, 0u, 0u);
              if (v < kvec) tb = table(dcs_b, v);
              rotate(xb, tb, v < kvec, rb);
#pragma unroll
              for (int t = 0; t < 8; ++t) ra[t] = (ra[t] + rb[t]) * 0.5f;
            }
            o4.x = pack_bf16(ra[0], ra[1]);
            o4.y = pack_bf16(ra[2], ra[3]);
            o4.z = pack_bf16(ra[4], ra[5]);
            o4.w = pack_bf16(ra[6], ra[7]);
          }
          if (failed) o4 = make_uint4(BF16_NAN2, BF16_NAN2, BF16_NAN2, BF16_NAN2);
          *reinterpret_cast<uint4*>(out_row + (v << 3)) = o4;
        }
      }
    }
  }
}

// Cross-GPU barrier on flag words: rank `me` publishes `epoch` into slot [me] of every
// rank's flag array (release, system scope), then waits until every slot of its own array has
// reached `epoch` (acquire). One thread per peer. The wait is bounded; on expiry the status
// word records ST_TIMEOUT_PEER_FLAG and the kernel returns.
__global__ void halo_barrier_kernel(const FlagPtrs flags, int me, int world, int epoch,
                                    long long limit_cycles) {
  const int r = threadIdx.x;
  if (r >= world) return;
  if (r == 0) *reinterpret_cast<volatile int*>(&g_halo_ok) = 1;   // long before any wait can run out
  __threadfence_system();
  int* remote = flags.p[r] + me;
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  const int* mine = flags.p[me] + r;
  const long long t0 = clock64();
  while (true) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (v >= epoch) break;
    if (clock64() - t0 > limit_cycles) {
      atomicCAS(&g_status, 0, ST_TIMEOUT_PEER_FLAG);
      *reinterpret_cast<volatile int*>(&g_halo_ok) = 0;   // the gathers behind this barrier write NaN
      break;
    }
    __nanosleep(200);
  }
}

}  // namespace strata
