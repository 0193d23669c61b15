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

// Direct evaluation of one pixel x 8 channels: every conv tap is an upsampled value, i.e. four
// token reads; taps outside the H x W image are the convolution's zero padding.
__device__ __forceinline__ void cond_direct_pixel(const AdalnCondParams& p, const uint4* base,
                                                  int nvec, int H, int W, int y, int x, int cv,
                                                  float (&acc)[8]) {
  const int r = p.ks >> 1;
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
}

__device__ __forceinline__ void gelu8(float (&acc)[8]) {
#pragma unroll
  for (int ch = 0; ch < 8; ++ch) {
    const float v = acc[ch];
    const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
    acc[ch] = 0.5f * v * (1.0f + fast_tanh(u));
  }
}

// One thread: one pixel x 8 channels, direct evaluation (any factor and kernel size).
__global__ void __launch_bounds__(256) adaln_cond_kernel(const AdalnCondParams p) {
  const int nvec = p.Cb >> 3;
  const int H = p.h * p.factor, W = p.w * p.factor;
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
    cond_direct_pixel(p, base, nvec, H, W, y, x, cv, acc);
    gelu8(acc);
    reinterpret_cast<uint4*>(p.out + (pix - p.row0) * p.Cb)[cv] = pack8(acc);
  }
}

// Upsample followed by the depthwise conv is linear in the tokens: away from the image border
// a pixel of the factor x factor cell of token (R, Cc) reads the 3 x 3 tokens around (R, Cc)
// with weights that depend only on its position inside the cell (the phase) and the channel.
// This kernel folds the ks x ks taps into that table, [factor^2][9][Cb] fp32. Valid for
// factor >= 4 and ks <= 5 (then every tap of every phase falls on rows R-1 .. R+1).
__global__ void adaln_cond_table_kernel(const float* __restrict__ wdw, int Cb, int factor, int ks,
                                        float* __restrict__ table) {
  const int n = factor * factor * Cb;
  const int r = ks >> 1;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < n; t += gridDim.x * blockDim.x) {
    const int ch = t % Cb;
    const int phase = t / Cb;
    const int phy = phase / factor, phx = phase % factor;
    float acc[9];
#pragma unroll
    for (int k = 0; k < 9; ++k) acc[k] = 0.f;
    for (int dy = -r; dy <= r; ++dy) {
      int r0, r1;
      float ly0, ly1;
      bilinear_tap(factor + phy + dy, factor, 4, r0, r1, ly0, ly1);   // cell R = 1 of a 4-row grid
      for (int dx = -r; dx <= r; ++dx) {
        int c0, c1;
        float lx0, lx1;
        bilinear_tap(factor + phx + dx, factor, 4, c0, c1, lx0, lx1);
        const float wt = wdw[ch * ks * ks + (dy + r) * ks + (dx + r)];
#pragma unroll
        for (int k = 0; k < 9; ++k) {
          const int j = k / 3, i = k % 3;
          const float wy = (j == r0 ? ly0 : 0.f) + (j == r1 ? ly1 : 0.f);
          const float wx = (i == c0 ? lx0 : 0.f) + (i == c1 ? lx1 : 0.f);
          acc[k] = fmaf(wt, wy * wx, acc[k]);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 9; ++k) table[(phase * 9 + k) * Cb + ch] = acc[k];
  }
}

// One thread: one cell (factor x factor pixels of one backbone token) x 8 channels. A warp
// holds 8 consecutive cells x 4 consecutive channel vectors, so a table read is one 128-byte
// line shared by the 8 cells and a token read / row write is 64 contiguous bytes per cell.
// Interior cells only; the frame of border cells is adaln_cond_frame_kernel's.
__global__ void __launch_bounds__(256)
adaln_cond_cells_kernel(const AdalnCondParams p, const float* __restrict__ table) {
  const int nvec = p.Cb >> 3;
  const int ncvg = nvec >> 2;
  const int f = p.factor;
  const int H = p.h * f, W = p.w * f;
  const long long gR0 = p.row0 / W / f;
  const long long gR1 = (p.row0 + p.n_rows - 1) / W / f;
  const long long n_cells = (gR1 - gR0 + 1) * p.w;
  const long long n_cell_groups = (n_cells + 7) >> 3;
  const long long total_warps = n_cell_groups * ncvg;
  const int lane = threadIdx.x & 31;
  const long long warps_in_grid = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long wg = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
       wg < total_warps; wg += warps_in_grid) {
    const int cvg = static_cast<int>(wg / n_cell_groups);
    const long long cell = (wg % n_cell_groups) * 8 + (lane >> 2);
    if (cell >= n_cells) continue;
    const int cv = cvg * 4 + (lane & 3);
    const long long gR = gR0 + cell / p.w;
    const int Cc = static_cast<int>(cell % p.w);
    const long long plane = gR / p.h;
    const int R = static_cast<int>(gR % p.h);
    const uint4* base = reinterpret_cast<const uint4*>(p.tok + plane * p.h * p.w * p.Cb) + cv;
    // cells on the image border belong to adaln_cond_frame_kernel
    if (R < 1 || R > p.h - 2 || Cc < 1 || Cc > p.w - 2) continue;
    float t[9][8];
    float bias[8];
#pragma unroll
    for (int k = 0; k < 9; ++k)
      unpack8(__ldg(base + (static_cast<long long>(R - 1 + k / 3) * p.w + (Cc - 1 + k % 3)) * nvec),
              t[k]);
#pragma unroll
    for (int c = 0; c < 8; ++c) bias[c] = p.bdw ? __ldg(p.bdw + cv * 8 + c) : 0.f;
    for (int phy = 0; phy < f; ++phy) {
      const int y = R * f + phy;
      for (int phx = 0; phx < f; ++phx) {
        const int x = Cc * f + phx;
        const long long pix = (plane * H + y) * W + x;
        if (pix < p.row0 || pix >= p.row0 + p.n_rows) continue;
        float acc[8];
        const float4* tb =
            reinterpret_cast<const float4*>(table + static_cast<long long>(phy * f + phx) * 9 * p.Cb) +
            cv * 2;
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] = bias[c];
#pragma unroll
        for (int k = 0; k < 9; ++k) {
          const float4 w0 = __ldg(tb + k * (p.Cb >> 2));
          const float4 w1 = __ldg(tb + k * (p.Cb >> 2) + 1);
          acc[0] = fmaf(w0.x, t[k][0], acc[0]); acc[1] = fmaf(w0.y, t[k][1], acc[1]);
          acc[2] = fmaf(w0.z, t[k][2], acc[2]); acc[3] = fmaf(w0.w, t[k][3], acc[3]);
          acc[4] = fmaf(w1.x, t[k][4], acc[4]); acc[5] = fmaf(w1.y, t[k][5], acc[5]);
          acc[6] = fmaf(w1.z, t[k][6], acc[6]); acc[7] = fmaf(w1.w, t[k][7], acc[7]);
        }
        gelu8(acc);
        reinterpret_cast<uint4*>(p.out + (pix - p.row0) * p.Cb)[cv] = pack8(acc);
      }
    }
  }
}

// The frame of border cells (the outermost `factor` pixels on every side of each H x W plane),
// tap by tap: one thread per (frame pixel, 8 channels), frame pixels enumerated densely - top
// band, bottom band, then the left and right strips of the rows in between.
__global__ void __launch_bounds__(256) adaln_cond_frame_kernel(const AdalnCondParams p) {
  const int nvec = p.Cb >> 3;
  const int f = p.factor;
  const int H = p.h * f, W = p.w * f;
  const long long HW = static_cast<long long>(H) * W;
  const long long plane0 = p.row0 / HW;
  const long long plane1 = (p.row0 + p.n_rows - 1) / HW;
  const int band = f * W;                                   // pixels of the top (or bottom) band
  const int mid_rows = H > 2 * f ? H - 2 * f : 0;
  const int strip_w = W >= 2 * f ? 2 * f : W;               // left + right strip of a middle row
  const long long per_plane =
      (H >= 2 * f ? 2LL * band : HW) + static_cast<long long>(mid_rows) * strip_w;
  const long long total = (plane1 - plane0 + 1) * per_plane * nvec;
  for (long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int cv = static_cast<int>(t % nvec);
    const long long fp = t / nvec;
    const long long plane = plane0 + fp / per_plane;
    long long k = fp % per_plane;
    int y, x;
    if (H < 2 * f) {
      y = static_cast<int>(k / W); x = static_cast<int>(k % W);
    } else if (k < band) {
      y = static_cast<int>(k / W); x = static_cast<int>(k % W);
    } else if (k < 2LL * band) {
      k -= band;
      y = H - f + static_cast<int>(k / W); x = static_cast<int>(k % W);
    } else {
      k -= 2LL * band;
      y = f + static_cast<int>(k / strip_w);
      const int sx = static_cast<int>(k % strip_w);
      x = (W >= 2 * f && sx >= f) ? W - 2 * f + sx : sx;
    }
    const long long pix = plane * HW + static_cast<long long>(y) * W + x;
    if (pix < p.row0 || pix >= p.row0 + p.n_rows) continue;
    const uint4* base = reinterpret_cast<const uint4*>(p.tok + plane * p.h * p.w * p.Cb) + cv;
    float acc[8];
    cond_direct_pixel(p, base, nvec, H, W, y, x, cv, acc);
    gelu8(acc);
    reinterpret_cast<uint4*>(p.out + (pix - p.row0) * p.Cb)[cv] = pack8(acc);
  }
}

// Number of floats of the table the cell kernel needs, or 0 when the geometry takes the
// direct kernel (small factor, wide conv kernel, channel count not a multiple of 32).
inline long long adaln_cond_table_floats(int Cb, int factor, int ks) {
  if (factor < 4 || ks > 5 || Cb % 32 != 0) return 0;
  return static_cast<long long>(factor) * factor * 9 * Cb;
}

// table: device scratch of adaln_cond_table_floats() floats, or null for the direct kernel.
inline int launch_adaln_cond(const AdalnCondParams& p, float* table, int sm_count,
                             cudaStream_t stream) {
  if (p.Cb % 8 != 0 || p.Cb <= 0 || p.factor <= 0 || p.ks <= 0 || (p.ks & 1) == 0 || p.ks > 9 ||
      p.D <= 0 || p.h <= 0 || p.w <= 0 || p.row0 < 0)
    return -2;
  if (p.n_rows <= 0) return 0;
  if (table != nullptr && adaln_cond_table_floats(p.Cb, p.factor, p.ks) > 0) {
    const int n = p.factor * p.factor * p.Cb;
    adaln_cond_table_kernel<<<(n + 255) / 256, 256, 0, stream>>>(p.wdw, p.Cb, p.factor, p.ks, table);
    const long long W = static_cast<long long>(p.w) * p.factor;
    const long long cell_rows = (p.row0 + p.n_rows - 1) / W / p.factor - p.row0 / W / p.factor + 1;
    const long long warps = (cell_rows * p.w + 7) / 8 * (p.Cb / 32);
    long long blocks = (warps + 7) / 8;
    const long long cap = static_cast<long long>(sm_count) * 16;
    if (blocks > cap) blocks = cap;
    if (p.h > 2 && p.w > 2)
      adaln_cond_cells_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(p, table);
    {
      const long long H = static_cast<long long>(p.h) * p.factor;
      const long long planes = (p.row0 + p.n_rows - 1) / (H * W) - p.row0 / (H * W) + 1;
      const long long frame = H * W - (p.h > 2 && p.w > 2 ? (H - 2 * p.factor) * (W - 2 * p.factor) : 0);
      long long fb = (planes * frame * (p.Cb / 8) + 255) / 256;
      const long long fcap = static_cast<long long>(sm_count) * 32;
      if (fb > fcap) fb = fcap;
      adaln_cond_frame_kernel<<<static_cast<int>(fb), 256, 0, stream>>>(p);
    }
  } else {
    const long long total = p.n_rows * (p.Cb / 8);
    long long blocks = (total + 255) / 256;
    const long long cap = static_cast<long long>(sm_count) * 32;
    if (blocks > cap) blocks = cap;
    adaln_cond_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(p);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

}  // namespace strata
