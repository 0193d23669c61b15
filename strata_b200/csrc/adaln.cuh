// Kernels of the AdaLN-conditioned pixel blocks (stage 2 of the two-stage model: 128-channel
// tokens at full pixel resolution, modulated per pixel by the backbone's tokens).
//
//   adaln_rows_kernel     x' = x + gate * y ;  out = LN(x') * (1 + scale) + shift
//                         (either half optional) - one pass over the token rows, HBM-bound:
//                         up to 5 row reads + 2 row writes of 2*C bytes per token
//   qk_norm_rows_kernel   RMS norm of every 64-channel q and k head of a packed qkv row, in place
//   adaln_cond_kernel     GELU(depthwise KSxKS conv(bilinear upsample(backbone tokens)) + b)
//                         as bf16 rows [pixels, Cb] - the A operand of the modulation projection
#pragma once
#include "common.cuh"

namespace strata {

struct AdalnRowsParams {
  const __nv_bfloat16* x;      long long ldx;
  const __nv_bfloat16* y;      long long ldy;     // nullable: no residual update
  const __nv_bfloat16* gate;   long long ldg;     // nullable with y: x' = x + y
  __nv_bfloat16* xo;           long long ldxo;    // x' (may alias x); required when y != null
  const __nv_bfloat16* shift;  const __nv_bfloat16* scale;  long long ldm;  // nullable: plain LN
  __nv_bfloat16* out;          long long ldo;     // nullable: residual update only
  int M, C;
  float eps;
};

__device__ __forceinline__ void unpack8(const uint4& r, float (&v)[8]) {
  v[0] = bf16_lo(r.x); v[1] = bf16_hi(r.x); v[2] = bf16_lo(r.y); v[3] = bf16_hi(r.y);
  v[4] = bf16_lo(r.z); v[5] = bf16_hi(r.z); v[6] = bf16_lo(r.w); v[7] = bf16_hi(r.w);
}
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 o;
  o.x = pack_bf16(v[0], v[1]); o.y = pack_bf16(v[2], v[3]);
  o.z = pack_bf16(v[4], v[5]); o.w = pack_bf16(v[6], v[7]);
  return o;
}

// LPR lanes (16 or 32) share one row; each holds VPL 16-byte vectors of it.
template <int LPR, int VPL>
__global__ void __launch_bounds__(256) adaln_rows_kernel(const AdalnRowsParams p) {
  constexpr int ROWS_PER_WARP = 32 / LPR;
  const int lane = threadIdx.x & 31;
  const int sub = lane % LPR;
  const int nvec = p.C >> 3;
  const long long rows_per_block = static_cast<long long>(blockDim.x >> 5) * ROWS_PER_WARP;
  const long long first = static_cast<long long>(blockIdx.x) * rows_per_block +
                          (threadIdx.x >> 5) * ROWS_PER_WARP + lane / LPR;
  // every lane of a warp runs the same number of iterations (the shuffles below need the
  // whole warp): rows past M are computed on row M-1 and not stored
  const long long row_iters =
      (p.M + rows_per_block * gridDim.x - 1) / (rows_per_block * gridDim.x);
  for (long long it = 0; it < row_iters; ++it) {
    const long long row_raw = first + it * rows_per_block * gridDim.x;
    const bool live = row_raw < p.M;
    const long long row = live ? row_raw : p.M - 1;
    float v[VPL][8];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = sub + LPR * i;
      if (vi < nvec) {
        unpack8(__ldg(reinterpret_cast<const uint4*>(p.x + row * p.ldx) + vi), v[i]);
        if (p.y != nullptr) {
          float yv[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(p.y + row * p.ldy) + vi), yv);
          if (p.gate != nullptr) {
            float g[8];
            unpack8(__ldg(reinterpret_cast<const uint4*>(p.gate + row * p.ldg) + vi), g);
#pragma unroll
            for (int t = 0; t < 8; ++t) v[i][t] = fmaf(g[t], yv[t], v[i][t]);
          } else {
#pragma unroll
            for (int t = 0; t < 8; ++t) v[i][t] += yv[t];
          }
          const uint4 o = pack8(v[i]);
          if (live) reinterpret_cast<uint4*>(p.xo + row * p.ldxo)[vi] = o;
          unpack8(o, v[i]);   // the norm sees the stored (bf16) residual stream
        }
#pragma unroll
        for (int t = 0; t < 8; ++t) sum += v[i][t];
      } else {
#pragma unroll
        for (int t = 0; t < 8; ++t) v[i][t] = 0.f;
      }
    }
    if (p.out == nullptr) continue;
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float mean = sum / static_cast<float>(p.C);
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      if (sub + LPR * i < nvec) {
#pragma unroll
        for (int t = 0; t < 8; ++t) {
          const float d = v[i][t] - mean;
          sq += d * d;
        }
      }
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float rstd = rsqrtf(sq / static_cast<float>(p.C) + p.eps);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int vi = sub + LPR * i;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) o[t] = (v[i][t] - mean) * rstd;
        if (p.scale != nullptr) {
          float sc[8], sh[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(p.scale + row * p.ldm) + vi), sc);
          unpack8(__ldg(reinterpret_cast<const uint4*>(p.shift + row * p.ldm) + vi), sh);
#pragma unroll
          for (int t = 0; t < 8; ++t) o[t] = fmaf(o[t], 1.0f + sc[t], sh[t]);
        }
        if (live) reinterpret_cast<uint4*>(p.out + row * p.ldo)[vi] = pack8(o);
      }
    }
  }
}

inline int launch_adaln_rows(const AdalnRowsParams& p, int sm_count, cudaStream_t stream) {
  if (p.C % 8 != 0 || p.C <= 0 || p.C > 2048) return -2;
  if (p.M <= 0) return 0;
  const int nvec = p.C / 8;
  const int lpr = nvec <= 16 ? 16 : 32;
  const int threads = 256;
  const long long rows_per_block = (threads / 32) * (32 / lpr);
  long long blocks = (p.M + rows_per_block - 1) / rows_per_block;
  const long long cap = static_cast<long long>(sm_count) * 16;
  if (blocks > cap) blocks = cap;
  const int g = static_cast<int>(blocks);
  const int vpl = (nvec + lpr - 1) / lpr;
  if (lpr == 16) adaln_rows_kernel<16, 1><<<g, threads, 0, stream>>>(p);
  else if (vpl <= 1) adaln_rows_kernel<32, 1><<<g, threads, 0, stream>>>(p);
  else if (vpl <= 2) adaln_rows_kernel<32, 2><<<g, threads, 0, stream>>>(p);
  else if (vpl <= 4) adaln_rows_kernel<32, 4><<<g, threads, 0, stream>>>(p);
  else adaln_rows_kernel<32, 8><<<g, threads, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

// RMS norm of the q and k heads (64 channels each) of packed qkv rows [M, 3C], in place:
// t <- t * rsqrt(mean(t^2) + eps). Eight lanes share a head (one 16-byte vector each).
__global__ void __launch_bounds__(256)
qk_norm_rows_kernel(__nv_bfloat16* __restrict__ qkv, long long ld, long long M, int C, float eps) {
  const int heads2 = 2 * (C >> 6);                      // q heads then k heads: columns [0, 2C)
  const long long groups = M * heads2;                  // one 8-lane group per (row, head)
  const long long n_thr = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long iters = (groups * 8 + n_thr - 1) / n_thr;
  long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (long long it = 0; it < iters; ++it, t += n_thr) {
    const long long g_raw = t >> 3;
    const bool live = g_raw < groups;
    const long long g = live ? g_raw : groups - 1;
    const long long row = g / heads2;
    const int head = static_cast<int>(g - row * heads2);
    uint4* ptr = reinterpret_cast<uint4*>(qkv + row * ld + head * 64) + (t & 7);
    float v[8];
    unpack8(*ptr, v);
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) sq = fmaf(v[i], v[i], sq);
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    const float r = rsqrtf(sq * (1.0f / 64.0f) + eps);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] *= r;
    if (live) *ptr = pack8(v);
  }
}

inline int launch_qk_norm_rows(__nv_bfloat16* qkv, long long ld, long long M, int C, float eps,
                               int sm_count, cudaStream_t stream) {
  if (C % 64 != 0 || C <= 0 || ld % 8 != 0 || ld < 3LL * C) return -2;
  if (M <= 0) return 0;
  const long long thr = M * 2 * (C / 64) * 8;
  long long blocks = (thr + 255) / 256;
  const long long cap = static_cast<long long>(sm_count) * 16;
  if (blocks > cap) blocks = cap;
  qk_norm_rows_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(qkv, ld, M, C, eps);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

// Source index and weights of a 1-D bilinear upsample by an integer factor (half-pixel
// centres, negative source coordinates clamped to 0, upper neighbour clamped to n-1).
__device__ __forceinline__ void bilinear_tap(int p, int factor, int n, int& i0, int& i1, float& l0,
                                             float& l1) {
  float s = (static_cast<float>(p) + 0.5f) / static_cast<float>(factor) - 0.5f;
  s = s < 0.f ? 0.f : s;
  i0 = static_cast<int>(s);
  if (i0 > n - 1) i0 = n - 1;
  i1 = i0 + 1 < n ? i0 + 1 : n - 1;
  l1 = s - static_cast<float>(i0);
  l0 = 1.0f - l1;
}

struct AdalnCondParams {
  const __nv_bfloat16* tok;   // backbone tokens [B, D, h, w, Cb], token-major
  const float* wdw;           // depthwise weights [Cb, KS*KS]
  const float* bdw;           // [Cb] or null
  __nv_bfloat16* out;         // rows [n_rows, Cb] for pixels row0 .. row0+n_rows of (b, d, y, x)
  long long row0, n_rows;
  int D, h, w, Cb, factor, ks;
};

// One thread: one pixel x 8 channels. Every conv tap is an upsampled value, i.e. four token
// reads; taps outside the H x W image are the convolution's zero padding.
__global__ void __launch_bounds__(256) adaln_cond_kernel(const AdalnCondParams p) {
  const int nvec = p.Cb >> 3;
  const int H = p.h * p.factor, W = p.w * p.factor;
  const int r = p.ks >> 1;
  const long long total = p.n_rows * nvec;
  for (long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long pix = p.row0 + t / nvec;
    const int cv = static_cast<int>(t % nvec);
    const int x = static_cast<int>(pix % W);
    const int y = static_cast<int>((pix / W) % H);
    const long long plane = pix / (static_cast<long long>(W) * H);   // b * D + d
    const uint4* base = reinterpret_cast<const uint4*>(p.tok + plane * p.h * p.w * p.Cb) + cv;
    float acc[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = p.bdw ? __ldg(p.bdw + cv * 8 + c) : 0.f;
    for (int dy = -r; dy <= r; ++dy) {
      const int py = y + dy;
      if (py < 0 || py >= H) continue;
      int r0, r1;
      float ly0, ly1;
      bilinear_tap(py, p.factor, p.h, r0, r1, ly0, ly1);
      for (int dx = -r; dx <= r; ++dx) {
        const int px = x + dx;
        if (px < 0 || px >= W) continue;
        int c0, c1;
        float lx0, lx1;
        bilinear_tap(px, p.factor, p.w, c0, c1, lx0, lx1);
        float a[8], b[8], c[8], d[8];
        unpack8(__ldg(base + (static_cast<long long>(r0) * p.w + c0) * nvec), a);
        unpack8(__ldg(base + (static_cast<long long>(r0) * p.w + c1) * nvec), b);
        unpack8(__ldg(base + (static_cast<long long>(r1) * p.w + c0) * nvec), c);
        unpack8(__ldg(base + (static_cast<long long>(r1) * p.w + c1) * nvec), d);
        const int tap = (dy + r) * p.ks + (dx + r);
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const float u = ly0 * (lx0 * a[ch] + lx1 * b[ch]) + ly1 * (lx0 * c[ch] + lx1 * d[ch]);
          acc[ch] = fmaf(__ldg(p.wdw + (cv * 8 + ch) * p.ks * p.ks + tap), u, acc[ch]);
        }
      }
    }
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
      const float v = acc[ch];
      const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
      acc[ch] = 0.5f * v * (1.0f + tanhf(u));
    }
    reinterpret_cast<uint4*>(p.out + (pix - p.row0) * p.Cb)[cv] = pack8(acc);
  }
}

inline int launch_adaln_cond(const AdalnCondParams& p, int sm_count, cudaStream_t stream) {
  if (p.Cb % 8 != 0 || p.Cb <= 0 || p.factor <= 0 || p.ks <= 0 || (p.ks & 1) == 0 || p.ks > 9 ||
      p.D <= 0 || p.h <= 0 || p.w <= 0 || p.row0 < 0)
    return -2;
  if (p.n_rows <= 0) return 0;
  const long long total = p.n_rows * (p.Cb / 8);
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(sm_count) * 32;
  if (blocks > cap) blocks = cap;
  adaln_cond_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

}  // namespace strata
