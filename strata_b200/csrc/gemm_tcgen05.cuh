// Persistent, warp-specialised bf16 GEMM for sm_100a:  D[M,N] = A[M,K] * W[N,K]^T  with a
// fused epilogue. One CTA per SM; each CTA walks output tiles of 128 x BN.
//
//   warp 0      TMA producer: streams 128x64 A tiles and BNx64 W tiles (128-byte swizzle)
//               into a ring of shared-memory stages.
//   warp 1      MMA issuer: one thread issues tcgen05.mma (M=128, N=BN, K=16) from the smem
//               stages into one of two TMEM accumulators (2 x BN fp32 columns), and commits
//               stage-free / accumulator-full mbarriers.
//   warps 2-9   epilogue: read the finished accumulator with tcgen05.ld (each thread owns
//               one output row), apply bias and the selected epilogue, store bf16. The
//               other accumulator is being filled meanwhile.
//
// Epilogues (the operator each one serves in the Strata block):
//   EPI_BIAS           y = acc + b                                   (generic Linear)
//   EPI_GELU           y = gelu_tanh(acc + b)                        (mlp.layers.0 + tanh GELU)
//   EPI_RESIDUAL       y = acc + b + R[m,n]                          (attn.proj / mlp.layers.2)
//   EPI_QKV_ROPE       y = rope(rmsnorm?(acc + b)) on q,k columns    (attn.qkv + RoPE + pack)
//   EPI_GATE           y = G[m,n] * sigmoid(acc + b)                 (attn.gate_proj)
#pragma once
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
  // EPI_QKV_ROPE: tables [n_tiles, hw, head_dim/2] fp32; token row m belongs to tile
  // m / tokens_per_tile and to horizontal position m % hw (depth levels share a table row).
  const float* rope_cos;
  const float* rope_sin;
  int tokens_per_tile;
  int hw;
  int head_dim;
  int rope_cols;   // columns [0, rope_cols) are q and k
  int qk_norm;     // 1: RMS-normalise each head of q and k before the rotation
  float qk_eps;
};

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 320;
constexpr int GEMM_EPI_WARPS = 8;

template <int BN>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int BAR_BYTES = 256;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // + alignment slack
};

template <int EPI>
__device__ __forceinline__ void gemm_epilogue_64(float (&v)[64], int m, int n0, bool row_ok,
                                                 const GemmParams& p) {
  // v holds acc for columns [n0, n0+64) of row m. Apply bias + epilogue in place.
  if (p.bias != nullptr) {
#pragma unroll
    for (int j = 0; j < 64; j += 4) {
      if (n0 + j + 3 < p.N) {
        float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + n0 + j));
        v[j] += b.x; v[j + 1] += b.y; v[j + 2] += b.z; v[j + 3] += b.w;
      } else {
#pragma unroll
        for (int t = 0; t < 4; ++t)
          if (n0 + j + t < p.N) v[j + t] += __ldg(p.bias + n0 + j + t);
      }
    }
  }
  if constexpr (EPI == EPI_GELU) {
#pragma unroll
    for (int j = 0; j < 64; ++j) v[j] = gelu_tanh(v[j]);
  } else if constexpr (EPI == EPI_RESIDUAL || EPI == EPI_GATE) {
    if (row_ok) {
      const __nv_bfloat16* rp = p.aux + static_cast<long long>(m) * p.ldaux + n0;
      if (n0 + 64 <= p.N && (p.ldaux % 8) == 0) {
#pragma unroll
        for (int j = 0; j < 64; j += 8) {
          uint4 r = __ldg(reinterpret_cast<const uint4*>(rp + j));
          const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            float lo = bf16_lo(w[t]), hi = bf16_hi(w[t]);
            if constexpr (EPI == EPI_RESIDUAL) {
              v[j + 2 * t] += lo;
              v[j + 2 * t + 1] += hi;
            } else {
              v[j + 2 * t] = lo / (1.0f + __expf(-v[j + 2 * t]));
              v[j + 2 * t + 1] = hi / (1.0f + __expf(-v[j + 2 * t + 1]));
            }
          }
        }
      } else {
        for (int j = 0; j < 64; ++j) {
          if (n0 + j < p.N) {
            float r = __bfloat162float(rp[j]);
            if constexpr (EPI == EPI_RESIDUAL) v[j] += r;
            else v[j] = r / (1.0f + __expf(-v[j]));
          }
        }
      }
    }
  } else if constexpr (EPI == EPI_QKV_ROPE) {
    if (n0 < p.rope_cols && row_ok) {
      const int hd = p.head_dim;  // 32 or 64; 64-column chunks never straddle a head
      if (p.qk_norm) {
        if (hd == 64) {
          float ss = 0.f;
#pragma unroll
          for (int j = 0; j < 64; ++j) ss += v[j] * v[j];
          const float r = rsqrtf(ss * (1.0f / 64.0f) + p.qk_eps);
#pragma unroll
          for (int j = 0; j < 64; ++j) v[j] *= r;
        } else {
          float s0 = 0.f, s1 = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) { s0 += v[j] * v[j]; s1 += v[32 + j] * v[32 + j]; }
          const float r0 = rsqrtf(s0 * (1.0f / 32.0f) + p.qk_eps);
          const float r1 = rsqrtf(s1 * (1.0f / 32.0f) + p.qk_eps);
#pragma unroll
          for (int j = 0; j < 32; ++j) { v[j] *= r0; v[32 + j] *= r1; }
        }
      }
      const int half = hd >> 1;
      const long long trow =
          static_cast<long long>(m / p.tokens_per_tile) * p.hw + (m % p.hw);
      const float* cp = p.rope_cos + trow * half;
      const float* sp = p.rope_sin + trow * half;
#pragma unroll
      for (int j = 0; j < 64; j += 8) {
        const int pj = ((n0 + j) % hd) >> 1;  // pair index within the head
        float4 c = __ldg(reinterpret_cast<const float4*>(cp + pj));
        float4 s = __ldg(reinterpret_cast<const float4*>(sp + pj));
        const float cc[4] = {c.x, c.y, c.z, c.w};
        const float sn[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          float a = v[j + 2 * t], b = v[j + 2 * t + 1];
          v[j + 2 * t] = a * cc[t] - b * sn[t];
          v[j + 2 * t + 1] = a * sn[t] + b * cc[t];
        }
      }
    }
  }
}

template <int BN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmParams p) {
  using S = GemmSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t bar_base = smem_base + S::STAGES * S::STAGE_BYTES;
  // barrier layout (8 bytes each): full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (S::STAGES + s); };
  auto accf_bar = [&](int b) { return bar_base + 8u * (2 * S::STAGES + b); };
  auto acce_bar = [&](int b) { return bar_base + 8u * (2 * S::STAGES + 2 + b); };
  uint8_t* tail = smem_gen + S::STAGES * S::STAGE_BYTES + 8 * (2 * S::STAGES + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_m = (p.M + GEMM_BM - 1) / GEMM_BM;
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
      mbar_init(acce_bar(b), GEMM_EPI_WARPS);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
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
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m0 = (t / tiles_n) * GEMM_BM;
        const int n0 = (t % tiles_n) * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, ST_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * S::STAGE_BYTES;
          const uint32_t b_dst = a_dst + S::A_BYTES;
          mbar_expect_tx(full_bar(stage), S::STAGE_BYTES);
          tma_load_2d(a_dst, &tmA, kb * GEMM_BK, m0, full_bar(stage));
          tma_load_2d(b_dst, &tmB, kb * GEMM_BK, n0, full_bar(stage));
          if (++stage == S::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Give loads already in flight time to land before the CTA retires.
        for (int i = 0; i < 2000; ++i) __nanosleep(100);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(GEMM_BM, BN, false, false);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
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
            umma_ss(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == S::STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(accf_bar(buf));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    const int e = warp - 2;
    const int quarter = warp & 3;            // TMEM lane quarter this warp may read
    const int col_half = e >> 2;             // which half of the BN columns
    constexpr int HALF_COLS = BN / 2;
    int it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      const int m0 = (t / tiles_n) * GEMM_BM;
      const int n_tile0 = (t % tiles_n) * BN;
      if (!mbar_wait(accf_bar(buf), acc_phase, abort_flag, ST_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      const int m = m0 + quarter * 32 + lane;
      const bool row_ok = m < p.M;
#pragma unroll 1
      for (int c = 0; c < HALF_COLS; c += 64) {
        const int n0 = n_tile0 + col_half * HALF_COLS + c;
        if (n0 >= p.N) break;  // warp-uniform
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                               static_cast<uint32_t>(buf * BN + col_half * HALF_COLS + c);
        uint32_t r0[32], r1[32];
        tmem_ld_32x32(taddr, r0);
        tmem_ld_32x32(taddr + 32, r1);
        tmem_ld_wait();
        float v[64];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          v[j] = __uint_as_float(r0[j]);
          v[32 + j] = __uint_as_float(r1[j]);
        }
        gemm_epilogue_64<EPI>(v, m, n0, row_ok, p);
        if (row_ok) {
          __nv_bfloat16* op = p.out + static_cast<long long>(m) * p.ldo + n0;
          if (n0 + 64 <= p.N && (p.ldo % 8) == 0) {
#pragma unroll
            for (int j = 0; j < 64; j += 8) {
              uint4 o;
              o.x = pack_bf16(v[j], v[j + 1]);
              o.y = pack_bf16(v[j + 2], v[j + 3]);
              o.z = pack_bf16(v[j + 4], v[j + 5]);
              o.w = pack_bf16(v[j + 6], v[j + 7]);
              *reinterpret_cast<uint4*>(op + j) = o;
            }
          } else {
            for (int j = 0; j < 64; ++j)
              if (n0 + j < p.N) op[j] = __float2bfloat16(v[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acce_bar(buf));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// Host launcher. A: [M,K] bf16 row-major with row stride lda (elements); W: [N,K] bf16
// row-major with row stride ldw. Returns 0, or a negative argument error / CUDA error code.
template <int BN, int EPI>
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
    uint32_t box[2] = {GEMM_BK, static_cast<uint32_t>(BN)};
    if (make_tmap_bf16(&tmB, W, 2, dims, str, box) != 0) return -21;
  }
  using S = GemmSmem<BN>;
  auto kern = gemm_tcgen05_kernel<BN, EPI>;
  {
    // Per-device attribute; setting it on every launch keeps the launcher stateless.
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    if (e != cudaSuccess) return -static_cast<int>(e) - 1000;
  }
  const int tiles = ((p.M + GEMM_BM - 1) / GEMM_BM) * ((p.N + BN - 1) / BN);
  const int grid = tiles < sm_count ? tiles : sm_count;
  kern<<<grid, GEMM_THREADS, S::TOTAL, stream>>>(tmA, tmB, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

template <int EPI>
inline int launch_gemm(const __nv_bfloat16* A, long long lda, const __nv_bfloat16* W, long long ldw,
                       const GemmParams& p, int sm_count, cudaStream_t stream) {
  // 128x256 tiles when the output is wide enough to fill the machine with them.
  if (p.N >= 256 && (p.N % 256 == 0 || p.N > 512))
    return launch_gemm_t<256, EPI>(A, lda, W, ldw, p, sm_count, stream);
  return launch_gemm_t<128, EPI>(A, lda, W, ldw, p, sm_count, stream);
}

}  // namespace strata
