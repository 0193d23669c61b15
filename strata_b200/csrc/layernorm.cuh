// Non-affine LayerNorm over the channel dimension of a token matrix, bf16 in / bf16 out,
// statistics in fp32. The Strata backbone blocks carry no norm parameters, so the
// normalisation is (x - mean) * rsqrt(var + eps) and nothing else.
//
// One warp per token row; a row of C channels is read once with 16-byte loads, kept in
// registers, reduced with warp shuffles and written once. HBM-bound: 2*C bytes read +
// 2*C bytes written per token.
#pragma once
#include "common.cuh"

namespace strata {

template <int VEC_PER_LANE>  // number of 8-element (16-byte) vectors each lane holds
__global__ void __launch_bounds__(256)
layernorm_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                      __nv_bfloat16* __restrict__ y, long long ldy, int M, int C, float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nvec = C >> 3;
  for (long long row = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
       row < M; row += static_cast<long long>(gridDim.x) * warps_per_block) {
    const uint4* xp = reinterpret_cast<const uint4*>(x + row * ldx);
    float v[VEC_PER_LANE][8];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < VEC_PER_LANE; ++i) {
      const int vi = lane + 32 * i;
      if (vi < nvec) {
        uint4 r = __ldg(xp + vi);
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          v[i][2 * t] = bf16_lo(w[t]);
          v[i][2 * t + 1] = bf16_hi(w[t]);
          sum += v[i][2 * t] + v[i][2 * t + 1];
        }
      } else {
#pragma unroll
        for (int t = 0; t < 8; ++t) v[i][t] = 0.f;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / static_cast<float>(C);
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < VEC_PER_LANE; ++i) {
      if (lane + 32 * i < nvec) {
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const float d = v[i][t] - mean;
          sq += d * d;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rstd = rsqrtf(sq / static_cast<float>(C) + eps);
    uint4* yp = reinterpret_cast<uint4*>(y + row * ldy);
#pragma unroll
    for (int i = 0; i < VEC_PER_LANE; ++i) {
      const int vi = lane + 32 * i;
      if (vi < nvec) {
        uint4 o;
        o.x = pack_bf16((v[i][0] - mean) * rstd, (v[i][1] - mean) * rstd);
        o.y = pack_bf16((v[i][2] - mean) * rstd, (v[i][3] - mean) * rstd);
        o.z = pack_bf16((v[i][4] - mean) * rstd, (v[i][5] - mean) * rstd);
        o.w = pack_bf16((v[i][6] - mean) * rstd, (v[i][7] - mean) * rstd);
        yp[vi] = o;
      }
    }
  }
}

// C must be a multiple of 8 and at most 2048; ldx/ldy multiples of 8.
inline int launch_layernorm(const __nv_bfloat16* x, long long ldx, __nv_bfloat16* y, long long ldy,
                            int M, int C, float eps, int sm_count, cudaStream_t stream) {
  if (C % 8 != 0 || C > 2048 || C <= 0 || ldx % 8 != 0 || ldy % 8 != 0) return -2;
  if (M <= 0) return 0;
  const int threads = 256;
  const int rows_per_block = threads / 32;
  long long blocks = (static_cast<long long>(M) + rows_per_block - 1) / rows_per_block;
  const long long cap = static_cast<long long>(sm_count) * 16;  // 8 resident CTAs/SM, 2 waves
  if (blocks > cap) blocks = cap;
  const int nvec = C / 8;
  const int vpl = (nvec + 31) / 32;
  const int g = static_cast<int>(blocks);
  if (vpl <= 1) layernorm_rows_kernel<1><<<g, threads, 0, stream>>>(x, ldx, y, ldy, M, C, eps);
  else if (vpl <= 2) layernorm_rows_kernel<2><<<g, threads, 0, stream>>>(x, ldx, y, ldy, M, C, eps);
  else if (vpl <= 4) layernorm_rows_kernel<4><<<g, threads, 0, stream>>>(x, ldx, y, ldy, M, C, eps);
  else layernorm_rows_kernel<8><<<g, threads, 0, stream>>>(x, ldx, y, ldy, M, C, eps);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

}  // namespace strata
