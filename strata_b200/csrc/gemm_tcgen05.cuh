// Persistent, warp-specialised bf16 GEMM for sm_100a:  D[M,N] = A[M,K] * W[N,K]^T  with a
// fused epilogue. One CTA per SM; each CTA walks output tiles of 128 x BN.
//
//   warp 0      TMA producer: streams 128x64 A tiles and BNx64 W tiles (128-byte swizzle)
//               into a ring of shared-memory stages.
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) from the smem
//               stages into one of two TMEM accumulators (2 x BN fp32 columns), and commits
//               stage-free / accumulator-full mbarriers.
//   warps 2-17  epilogue (16 warps: four per SM sub-partition, because the epilogue of a
//               128 x 256 tile is bound by the latency of each warp's instruction stream
//               rather than by issue slots): read the finished accumulator with tcgen05.ld
//               (each thread owns one output row, 16 columns at a time), apply bias and the
//               selected epilogue, store bf16. The other accumulator is being filled meanwhile.
//
// PAIR variant (large problems): two CTAs of a cluster share every MMA (tcgen05 cta_group::2,
// M = 256): each CTA loads its own 128 rows of A and HALF of the W tile, the instruction reads
// both halves, and each CTA's tensor memory receives its 128 rows x BN accumulator. A CTA then
// moves 32 KB per k-block through shared memory instead of 48 KB, which matters because the
// one-CTA mainloop is bound by shared-memory bandwidth (operand reads + TMA writes), not by the
// tensor pipe. The first CTA of the pair issues the MMAs; TMA loads of both CTAs signal its
// stage barriers, its commits arrive on both CTAs' barriers, and both CTAs' epilogue warps hand
// the accumulator back on its barrier. Everything else (epilogues, staging, stores) is per CTA.
//
// Epilogues (the operator each one serves in the Strata block):
//   EPI_BIAS           y = acc + b                                   (generic Linear)
//   EPI_GELU           y = gelu_tanh(acc + b)                        (mlp.layers.0 + tanh GELU)
//   EPI_RESIDUAL       y = acc + b + R[m,n]                          (attn.proj / mlp.layers.2)
//   EPI_QKV_ROPE       y = rope(rmsnorm?(acc + b)) on q,k columns    (attn.qkv + RoPE + pack)
//   EPI_GATE           y = G[m,n] * sigmoid(acc + b)                 (attn.gate_proj)
#pragma once
#include <cuda_fp16.h>

#include <atomic>

#include "common.cuh"
#include "tensormap.cuh"

namespace strata {

enum GemmEpilogue : int {
  EPI_BIAS = 0,
  EPI_GELU = 1,
  EPI_RESIDUAL = 2,
  EPI_QKV_ROPE = 3,
  EPI_GATE = 4,
};

struct GemmParams {
  int M, N, K;
  __nv_bfloat16* out;
  long long ldo;
  const float* bias;          // [N] or nullptr
  const __nv_bfloat16* aux;   // residual (EPI_RESIDUAL) or gated operand (EPI_GATE)
  long long ldaux;
  // EPI_QKV_ROPE: table [n_tiles, hw, head_dim/2] of (cos, sin) pairs in IEEE half (4 bytes per
  // rotated channel pair); token row m belongs to tile m / tokens_per_tile and to horizontal
  // position m % hw (depth levels share a table row).
  const uint32_t* rope_cs;
  int tokens_per_tile;
  int hw;
  int head_dim;
  int rope_cols;   // columns [0, rope_cols) are q and k
  int qk_norm;     // 1: RMS-normalise each head of q and k before the rotation
  float qk_eps;
  // Output row remap (pad_T > 0): the M input rows are the interior tokens of tiles
  // [tile, d, i, j] with i, j < pad_T (pad_T a multiple of 32), and row m is stored at row
  // ((tile*pad_D + d)*P + i + pad_h)*P + j + pad_h of the output, P = pad_T + 2*pad_h: the
  // interior of halo-padded tiles. A 32-row store box never leaves one interior row.
  int pad_T, pad_h, pad_D;
};

// Output row of input row m under the padded-tile remap (identity when it is off).
__device__ __forceinline__ int gemm_out_row(int m, const GemmParams& p) {
  if (p.pad_T == 0) return m;
  const int T = p.pad_T, P = T + 2 * p.pad_h;
  const int j = m % T;
  int t = m / T;
  const int i = t % T;
  t /= T;   // tile*pad_D + d
  return (t * P + i + p.pad_h) * P + j + p.pad_h;
}

#ifndef GEMM_USE_PAIRS
#define GEMM_USE_PAIRS 1
#endif

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_EPI_WARPS = 16;
constexpr int GEMM_THREADS = 64 + 32 * GEMM_EPI_WARPS;

template <int BN, bool PAIR = false>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * GEMM_BK * 2;   // a pair splits the W tile
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256 && !PAIR) ? 4 : 6;
  static constexpr int STAGING_BYTES = 32 * 32 * 2;             // one 32-row x 32-col bf16 box
  static constexpr int STAGING_OFF = STAGES * STAGE_BYTES;      // per epilogue warp
  static constexpr int BAR_OFF = STAGING_OFF + GEMM_EPI_WARPS * STAGING_BYTES;
  static constexpr int BAR_BYTES = 512;
  static constexpr int TOTAL = BAR_OFF + BAR_BYTES + 1024;      // + alignment slack
};

// TMA store of a shared-memory box to global memory (bulk async group of the issuing thread).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tm, uint32_t src, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
      ::"l"(tm), "r"(src), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_read0() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// Epilogue math on 16 consecutive columns of output row m, in place. Lane `src_lane0 + j` of
// the warp holds the bias of column j of the group; `aux` holds the residual / gated operand of
// the same columns (bf16 pairs) for the epilogues that use one; `qk_scale` is the RMS-norm
// factor of the head these columns belong to; cs: this row's (cos, sin) half pairs for the 8
// channel pairs of these 16 columns.
template <int EPI>
__device__ __forceinline__ void gemm_epilogue_16(float (&v)[16], bool rotate, float b_lane,
                                                 int src_lane0, const uint32_t (&aux)[8],
                                                 float qk_scale, const uint32_t (&cs)[8],
                                                 const GemmParams& p, const float* bias16) {
  if (p.bias != nullptr) {
    if (bias16 != nullptr) {
      // the 16 biases of this column group, the same for every row: four 16-byte loads at an
      // address that is uniform over the warp (one L1 line, broadcast) instead of one shuffle
      // per output element
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 b4 = __ldg(reinterpret_cast<const float4*>(bias16) + q);
        v[4 * q] += b4.x; v[4 * q + 1] += b4.y; v[4 * q + 2] += b4.z; v[4 * q + 3] += b4.w;
      }
    } else {   // ragged right edge of the matrix: lane j of the group holds column j's bias
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] += __shfl_sync(0xffffffffu, b_lane, src_lane0 + j);
    }
  }
  if constexpr (EPI == EPI_GELU) {
    // tanh GELU on pairs: the polynomial part runs on packed fp32x2 instructions
    const float k0 = 0.7978845608028654f, k01 = 0.7978845608028654f * 0.044715f;
    const uint64_t K0 = pack2(k0, k0), K01 = pack2(k01, k01), HALF = pack2(0.5f, 0.5f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint64_t x = pack2(v[2 * j], v[2 * j + 1]);
      const uint64_t u = fmul2(x, ffma2(fmul2(x, x), K01, K0));
      float u0, u1;
      unpack2(u, u0, u1);
      const uint64_t t = pack2(fast_tanh(u0), fast_tanh(u1));
      const uint64_t hx = fmul2(x, HALF);
      unpack2(ffma2(hx, t, hx), v[2 * j], v[2 * j + 1]);
    }
  } else if constexpr (EPI == EPI_RESIDUAL) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[2 * j] += bf16_lo(aux[j]);
      v[2 * j + 1] += bf16_hi(aux[j]);
    }
  } else if constexpr (EPI == EPI_GATE) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[2 * j] = bf16_lo(aux[j]) / (1.0f + __expf(-v[2 * j]));
      v[2 * j + 1] = bf16_hi(aux[j]) / (1.0f + __expf(-v[2 * j + 1]));
    }
  } else if constexpr (EPI == EPI_QKV_ROPE) {
    if (rotate) {
      if (p.qk_norm) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] *= qk_scale;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 t =
            __half22float2(*reinterpret_cast<const __half2*>(&cs[j]));  // (cos, sin)
        const float a = v[2 * j], b = v[2 * j + 1];
        v[2 * j] = a * t.x - b * t.y;
        v[2 * j + 1] = a * t.y + b * t.x;
      }
    }
  }
}

// Per-head RMS factors of the q/k norm for one output row: one extra pass over the warp's
// WARP_COLS accumulator columns (+ bias). head_dim 64: the warp's 64 columns are one head, both
// components carry its factor; head_dim 32: one factor per 32-column sub-chunk. Called by a
// whole warp (tensor-memory loads).
template <int NSUB>
__device__ __noinline__ float2 gemm_qk_norm_scales(uint32_t taddr, const float* bias, int n_warp0,
                                                   int N, int lane, int head_dim, float eps) {
  static_assert(NSUB == 1 || NSUB == 2, "one or two 32-column sub-chunks per warp");
  float ss[NSUB];
#pragma unroll
  for (int cc = 0; cc < NSUB; ++cc) {
    float acc = 0.f;
    float bl = 0.f;
    if (bias != nullptr && n_warp0 + 32 * cc + lane < N) bl = __ldg(bias + n_warp0 + 32 * cc + lane);
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      uint32_t r[16];
      tmem_ld_32x16(taddr + 32 * cc + 16 * g, r);
      tmem_ld_wait();
      const int nb0 = n_warp0 + 32 * cc + 16 * g;
      if (bias != nullptr && nb0 + 16 <= N) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const float4 b4 = __ldg(reinterpret_cast<const float4*>(bias + nb0) + q4);
          const float x0 = __uint_as_float(r[4 * q4]) + b4.x;
          const float x1 = __uint_as_float(r[4 * q4 + 1]) + b4.y;
          const float x2 = __uint_as_float(r[4 * q4 + 2]) + b4.z;
          const float x3 = __uint_as_float(r[4 * q4 + 3]) + b4.w;
          acc += x0 * x0 + x1 * x1 + x2 * x2 + x3 * x3;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float x = __uint_as_float(r[j]) + __shfl_sync(0xffffffffu, bl, 16 * g + j);
          acc += x * x;
        }
      }
    }
    ss[cc] = acc;
  }
  if (head_dim == 64 && NSUB == 2) {
    const float f = rsqrtf((ss[0] + ss[NSUB - 1]) * (1.0f / 64.0f) + eps);
    return make_float2(f, f);
  }
  return make_float2(rsqrtf(ss[0] * (1.0f / 32.0f) + eps), rsqrtf(ss[NSUB - 1] * (1.0f / 32.0f) + eps));
}

// mbar_wait with the (bounded) polling loop out of line, for the epilogue warps: the phase has
// usually completed, and rare code left inline in their loop costs registers and schedule.
__device__ __noinline__ bool gemm_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                            int code) {
  return mbar_wait(bar, parity, abort_flag, code);
}
__device__ __forceinline__ bool gemm_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int code) {
  if (mbar_try_wait(bar, parity)) return true;
  return gemm_wait_slow(bar, parity, abort_flag, code);
}

template <int BN, int EPI, bool PAIR = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmOut,
                    const __grid_constant__ CUtensorMap tmAux, const GemmParams p) {
  using S = GemmSmem<BN, PAIR>;
  // PAIR: this CTA is rank 0 or 1 of a cluster of two that computes 256 x BN tiles together
  const uint32_t pair_rank = PAIR ? cluster_ctarank() : 0u;
  const int unit = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int n_units = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  constexpr int TILE_M = PAIR ? 2 * GEMM_BM : GEMM_BM;
  constexpr bool HAS_AUX = (EPI == EPI_RESIDUAL || EPI == EPI_GATE);
  // Epilogues without an operand to prefetch wait for the staging box as late as possible.
  constexpr bool LATE_WAIT = (EPI == EPI_BIAS || EPI == EPI_GELU || EPI == EPI_QKV_ROPE);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t bar_base = smem_base + S::BAR_OFF;
  // barriers (8 bytes each): full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], aux[8]
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (S::STAGES + s); };
  auto accf_bar = [&](int b) { return bar_base + 8u * (2 * S::STAGES + b); };
  auto acce_bar = [&](int b) { return bar_base + 8u * (2 * S::STAGES + 2 + b); };
  auto aux_bar = [&](int w) { return bar_base + 8u * (2 * S::STAGES + 4 + w); };
  uint8_t* tail = smem_gen + S::BAR_OFF + 8 * (2 * S::STAGES + 4 + GEMM_EPI_WARPS);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_m = (p.M + TILE_M - 1) / TILE_M;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + GEMM_BK - 1) / GEMM_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(accf_bar(b), 1);
      mbar_init(acce_bar(b), PAIR ? 2 * GEMM_EPI_WARPS : GEMM_EPI_WARPS);
    }
    for (int w = 0; w < GEMM_EPI_WARPS; ++w) mbar_init(aux_bar(w), 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();   // the partner's barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = unit; t < num_tiles && ok; t += n_units) {
        const int m0 = (t / tiles_n) * TILE_M + static_cast<int>(pair_rank) * GEMM_BM;
        const int n0 = (t % tiles_n) * BN + (PAIR ? static_cast<int>(pair_rank) * (BN / 2) : 0);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, ST_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * S::STAGE_BYTES;
          const uint32_t b_dst = a_dst + S::A_BYTES;
          if constexpr (PAIR) {
            // both CTAs' loads complete on the FIRST CTA's stage barrier (it issues the MMAs);
            // that CTA's producer announces the bytes of both (a transaction count may run
            // ahead of its announcement within a phase)
            const uint32_t fb = map_to_cta(full_bar(stage), 0);
            if (pair_rank == 0) mbar_expect_tx(full_bar(stage), 2 * S::STAGE_BYTES);
            tma_load_2d_pair(a_dst, &tmA, kb * GEMM_BK, m0, fb);
            tma_load_2d_pair(b_dst, &tmB, kb * GEMM_BK, n0, fb);
          } else {
            mbar_expect_tx(full_bar(stage), S::STAGE_BYTES);
            tma_load_2d(a_dst, &tmA, kb * GEMM_BK, m0, full_bar(stage));
            tma_load_2d(b_dst, &tmB, kb * GEMM_BK, n0, full_bar(stage));
          }
          if (++stage == S::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Give loads already in flight time to land before the CTA retires.
#pragma unroll 1
        for (int i = 0; i < 2000; ++i) __nanosleep(100);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && pair_rank == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(TILE_M, BN, false, false);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = unit; t < num_tiles && ok; t += n_units, ++it) {
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(acce_bar(buf), acc_phase ^ 1u, abort_flag, ST_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, ST_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_src = smem_base + stage * S::STAGE_BYTES;
          const uint32_t b_src = a_src + S::A_BYTES;
          const uint64_t adesc = umma_smem_desc_sw128(a_src);
          const uint64_t bdesc = umma_smem_desc_sw128(b_src);
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            // advance 16 bf16 = 32 bytes along K inside the 128-byte swizzle span
            if constexpr (PAIR)
              umma_ss_pair(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
            else
              umma_ss(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          if constexpr (PAIR) umma_commit_pair(empty_bar(stage)); else umma_commit(empty_bar(stage));
          if (++stage == S::STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) {
          if constexpr (PAIR) umma_commit_pair(accf_bar(buf)); else umma_commit(accf_bar(buf));
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    // Each warp owns 32 output rows (its TMEM lane quarter) x BN/4 columns of the tile and
    // walks them in 32-column sub-chunks of two 16-column groups: TMEM -> registers -> math ->
    // 64-byte-swizzled staging box (32 rows x 32 columns) in shared memory -> TMA store
    // (clipped at the matrix edge by the tensor map). The residual / gated operand of a
    // sub-chunk is TMA-loaded into the same staging box beforehand.
    const int e = warp - 2;
    const int quarter = warp & 3;            // TMEM lane quarter this warp may read
    const int cg = e >> 2;                   // which quarter of the BN columns
    constexpr int WARP_COLS = BN / 4;
    constexpr int NSUB = WARP_COLS / 32;
    const uint32_t stage_s = smem_base + S::STAGING_OFF + e * S::STAGING_BYTES;
    const uint32_t my_row_s = stage_s + lane * 64;
    const uint32_t sw = static_cast<uint32_t>((lane >> 1) & 3);   // 64-byte swizzle of this row
    const uint32_t acce_remote0 = PAIR ? map_to_cta(acce_bar(0), 0) : 0u;
    const uint32_t acce_remote1 = PAIR ? map_to_cta(acce_bar(1), 0) : 0u;
    uint32_t aux_phase = 0;
    int it = 0;
    bool ok = true;
    for (int t = unit; t < num_tiles && ok; t += n_units, ++it) {
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      const int m0 = (t / tiles_n) * TILE_M + static_cast<int>(pair_rank) * GEMM_BM;
      const int n_tile0 = (t % tiles_n) * BN;
      const int m_warp = m0 + quarter * 32;
      const int m = m_warp + lane;
      const bool row_ok = m < p.M;
      const int n_warp0 = n_tile0 + cg * WARP_COLS;
      // EPI_QKV_ROPE: this row's rotation table (one 4-byte (cos, sin) pair per channel pair of
      // a head: a single 128-byte line for head_dim 64) is the same for every q / k head. It is
      // pulled into L1 here, before the accumulator is waited for, and read 32 bytes at a time
      // where a 16-column group needs it.
      const uint4* cs_src = nullptr;
      bool rope_tile = false;
      if constexpr (EPI == EPI_QKV_ROPE) {
        rope_tile = (p.rope_cs != nullptr) && (n_warp0 < p.rope_cols) && row_ok;
        if (rope_tile) {
          const int half = p.head_dim >> 1;
          const long long trow =
              static_cast<long long>(m / p.tokens_per_tile) * p.hw + (m % p.hw);
          cs_src = reinterpret_cast<const uint4*>(p.rope_cs + trow * half);
          asm volatile("prefetch.global.L1 [%0];" ::"l"(cs_src));
        }
      }
      bool acc_ready = false;
      // per-head RMS factor (qk norm): one extra pass over the head's 64 (or 32) accumulator
      // columns; with 64-wide heads the warp's 64 columns are exactly one head
      float qk_scale[NSUB];
#pragma unroll
      for (int c = 0; c < NSUB; ++c) qk_scale[c] = 1.f;
#pragma unroll 1
      for (int c = 0; c < NSUB; ++c) {
        const int n0 = n_warp0 + c * 32;
        const bool chunk_live = (n0 < p.N) && (m_warp < p.M);   // warp-uniform
        float b_lane = 0.f;
        if (p.bias != nullptr && n0 + lane < p.N) b_lane = __ldg(p.bias + n0 + lane);
        if constexpr (!LATE_WAIT) {
          if (chunk_live) {
            // staging box free again? (previous TMA store has finished reading it) - a
            // residual / gated operand is fetched into it right away
            if (lane == 0) tma_store_wait_read0();
            __syncwarp();
            if constexpr (HAS_AUX) {
              if (lane == 0) {
                mbar_expect_tx(aux_bar(e), S::STAGING_BYTES);
                tma_load_2d(stage_s, &tmAux, n0, m_warp, aux_bar(e));
              }
            }
          }
        }
        if (!acc_ready) {
          if (!gemm_wait(accf_bar(buf), acc_phase, abort_flag, ST_TIMEOUT_EPILOGUE)) {
            ok = false;
            break;
          }
          tc_fence_after();
          acc_ready = true;
        }
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                               static_cast<uint32_t>(buf * BN + cg * WARP_COLS + c * 32);
        if constexpr (EPI == EPI_QKV_ROPE) {
          if (c == 0 && p.qk_norm && m_warp < p.M && n_warp0 < p.rope_cols && n_warp0 < p.N) {
            // (out of line: most models run without the q/k norm)
            const float2 sc = gemm_qk_norm_scales<NSUB>(taddr, p.bias, n_warp0, p.N, lane, p.head_dim,
                                                        p.qk_eps);
            qk_scale[0] = sc.x;
            qk_scale[NSUB - 1] = sc.y;
          }
        }
        if constexpr (HAS_AUX) {
          if (chunk_live) {
            if (!gemm_wait(aux_bar(e), aux_phase, abort_flag, ST_TIMEOUT_EPILOGUE)) {
              ok = false;
              break;
            }
            aux_phase ^= 1u;
          }
        }
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          // head_dim 64: the 32-column sub-chunks of a head use table pairs [0,16) and
          // [16,32); head_dim 32: each sub-chunk is a whole head and uses pairs [0,16).
          // The table words are requested before the TMEM load so that the two latencies overlap.
          const bool rotate = rope_tile && (n0 < p.rope_cols);
          uint32_t cs[8];
          if constexpr (EPI == EPI_QKV_ROPE) {
            if (rotate && chunk_live) {
              const int pair0 = ((p.head_dim == 64) ? (n0 & 63) >> 1 : 0) + 8 * g;
              const uint4* src = cs_src + (pair0 >> 2);
#pragma unroll
              for (int q = 0; q < 2; ++q) {
                const uint4 t4 = __ldg(src + q);
                cs[4 * q] = t4.x; cs[4 * q + 1] = t4.y; cs[4 * q + 2] = t4.z; cs[4 * q + 3] = t4.w;
              }
            }
          }
          uint32_t r[16];
          if (chunk_live) {
            tmem_ld_32x16(taddr + 16 * g, r);
            tmem_ld_wait();
          }
          if (g == 1 && c == NSUB - 1) {
            // the accumulator is in registers (or not needed): hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if constexpr (PAIR) mbar_arrive_cluster(buf ? acce_remote1 : acce_remote0);
              else mbar_arrive(acce_bar(buf));
            }
          }
          if (chunk_live) {
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
            uint32_t aux[8];
            if constexpr (HAS_AUX) {
#pragma unroll
              for (int q = 0; q < 2; ++q) {
                const uint32_t addr = my_row_s + ((static_cast<uint32_t>(2 * g + q) ^ sw) << 4);
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(aux[4 * q]), "=r"(aux[4 * q + 1]), "=r"(aux[4 * q + 2]),
                               "=r"(aux[4 * q + 3])
                             : "r"(addr)
                             : "memory");
              }
            }
            // (the bias group is read directly when all its 16 columns exist; p.bias is
            // 16-byte aligned and n0 a multiple of 32)
            const float* bias16 = (p.bias != nullptr && n0 + 16 * g + 16 <= p.N)
                                      ? p.bias + n0 + 16 * g : nullptr;
            gemm_epilogue_16<EPI>(v, rotate, b_lane, 16 * g, aux, qk_scale[c], cs, p, bias16);
            if constexpr (LATE_WAIT) {
              if (g == 0) {
                // the previous sub-chunk's TMA store must have finished reading the staging
                // box before it is overwritten; waiting only now lets that drain overlap with
                // the TMEM load and the arithmetic above
                if (lane == 0) tma_store_wait_read0();
                __syncwarp();
              }
            }
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const uint32_t addr = my_row_s + ((static_cast<uint32_t>(2 * g + q) ^ sw) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                           "r"(pack_bf16(v[8 * q], v[8 * q + 1])),
                           "r"(pack_bf16(v[8 * q + 2], v[8 * q + 3])),
                           "r"(pack_bf16(v[8 * q + 4], v[8 * q + 5])),
                           "r"(pack_bf16(v[8 * q + 6], v[8 * q + 7]))
                           : "memory");
            }
          }
        }
        if (!chunk_live) continue;
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&tmOut, stage_s, n0, gemm_out_row(m_warp, p));
          tma_store_commit();
        }
      }
    }
    if (lane == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();   // no signal may reach a CTA that has already left
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// Host launcher. A: [M,K] bf16 row-major with row stride lda (elements); W: [N,K] bf16
// row-major with row stride ldw. Returns 0, or a negative argument error / CUDA error code.
template <int BN, int EPI, bool PAIR = false>
inline int launch_gemm_t(const __nv_bfloat16* A, long long lda, const __nv_bfloat16* W,
                         long long ldw, const GemmParams& p, int sm_count, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(p.K), static_cast<uint64_t>(p.M)};
    uint64_t str[1] = {static_cast<uint64_t>(lda) * 2};
    uint32_t box[2] = {GEMM_BK, GEMM_BM};
    if (make_tmap_bf16(&tmA, A, 2, dims, str, box) != 0) return -20;
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(p.K), static_cast<uint64_t>(p.N)};
    uint64_t str[1] = {static_cast<uint64_t>(ldw) * 2};
    uint32_t box[2] = {GEMM_BK, static_cast<uint32_t>(PAIR ? BN / 2 : BN)};
    if (make_tmap_bf16(&tmB, W, 2, dims, str, box) != 0) return -21;
  }
  CUtensorMap tmOut, tmAux;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(p.N), static_cast<uint64_t>(p.M)};
    uint64_t str[1] = {static_cast<uint64_t>(p.ldo) * 2};
    uint32_t box[2] = {32, 32};
    uint64_t odims[2] = {dims[0], dims[1]};
    if (p.pad_T > 0) {
      const uint64_t P = static_cast<uint64_t>(p.pad_T + 2 * p.pad_h);
      odims[1] = dims[1] / (static_cast<uint64_t>(p.pad_T) * p.pad_T) * P * P;
    }
    if (make_tmap_bf16(&tmOut, p.out, 2, odims, str, box, TMAP_SWIZZLE_64B) != 0) return -22;
    tmAux = tmOut;
    if (EPI == EPI_RESIDUAL || EPI == EPI_GATE) {
      uint64_t astr[1] = {static_cast<uint64_t>(p.ldaux) * 2};
      if (make_tmap_bf16(&tmAux, p.aux, 2, dims, astr, box, TMAP_SWIZZLE_64B) != 0) return -23;
    }
  }
  using S = GemmSmem<BN, PAIR>;
  auto kern = gemm_tcgen05_kernel<BN, EPI, PAIR>;
  {
    // Per-device attribute; setting it on every launch keeps the launcher stateless.
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return -static_cast<int>(e) - 1000;
  }
  if constexpr (PAIR) {
    const int tiles = ((p.M + 2 * GEMM_BM - 1) / (2 * GEMM_BM)) * ((p.N + BN - 1) / BN);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(sm_count & ~1));
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = S::TOTAL;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // A persistent grid must be resident at once: not every SM has a partner for a pair, so the
    // number of clusters that fit is asked for (once per kernel and device), not assumed.
    static std::atomic<int> max_clusters[64];   // per device; concurrent first calls store the same value
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return -24;
    int fit = max_clusters[dev].load(std::memory_order_relaxed);
    if (fit == 0) {
      if (cudaOccupancyMaxActiveClusters(&fit, kern, &cfg) != cudaSuccess || fit <= 0) return -24;
      max_clusters[dev].store(fit, std::memory_order_relaxed);
    }
    const int clusters = tiles < fit ? tiles : fit;
    cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters));
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmOut, tmAux, p);
    return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
  }
  const int tiles = ((p.M + GEMM_BM - 1) / GEMM_BM) * ((p.N + BN - 1) / BN);
  const int grid = tiles < sm_count ? tiles : sm_count;
  kern<<<grid, GEMM_THREADS, S::TOTAL, stream>>>(tmA, tmB, tmOut, tmAux, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

template <int EPI>
inline int launch_gemm(const __nv_bfloat16* A, long long lda, const __nv_bfloat16* W, long long ldw,
                       const GemmParams& p, int sm_count, cudaStream_t stream) {
  // 128x256 tiles when the output is wide enough to fill the machine with them.
  // (the QKV epilogue always takes 256-wide tiles: a warp's 64 columns are then one whole
  // 64-channel head, which the qk norm needs)
  if ((p.N >= 256 && (p.N % 256 == 0 || p.N > 512)) || EPI == EPI_QKV_ROPE) {
    // large problems: CTA pairs share each MMA (less shared-memory traffic per SM)
    if (GEMM_USE_PAIRS && p.M >= 1024)
      return launch_gemm_t<256, EPI, true>(A, lda, W, ldw, p, sm_count, stream);
    return launch_gemm_t<256, EPI>(A, lda, W, ldw, p, sm_count, stream);
  }
  return launch_gemm_t<128, EPI>(A, lda, W, ldw, p, sm_count, stream);
}

}  // namespace strata
