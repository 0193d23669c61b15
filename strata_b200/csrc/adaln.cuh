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

// Upsample followed by the depthwise conv is linear in the tokens: a pixel of the
// factor x factor cell of token (R, Cc) reads a 3 x 3 block of tokens with weights that depend
// only on the channel and on the pixel's position class along each axis - 3 * factor classes:
// the `factor` pixels of the first cell (clamped upsample source, conv taps cut by the zero
// padding), the `factor` phases of an interior cell, the `factor` pixels of the last cell.
// The token block starts at row R-1 (0 for the first cell, h-3 for the last), same for columns.
// This kernel folds the ks x ks taps into that table, [3f][3f][9][Cb] fp32. Valid for
// factor >= 4, ks <= 5 and at least 3 cells per axis (then every tap falls inside the block).
__device__ __forceinline__ void cond_class_ref(int cls, int f, int& pos, int& base) {
  // representative pixel position and token-block base on a reference axis of 4 cells
  if (cls < f) { pos = cls; base = 0; }
  else if (cls < 2 * f) { pos = cls; base = 0; }             // cell 1, phase cls - f
  else { pos = 3 * f + (cls - 2 * f); base = 1; }            // cell 3 (last)
}

__global__ void adaln_cond_table_kernel(const float* __restrict__ wdw, int Cb, int factor, int ks,
                                        float* __restrict__ table) {
  const int ncls = 3 * factor;
  const int n = ncls * ncls * Cb;
  const int r = ks >> 1;
  const int n_ref = 4 * factor;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < n; t += gridDim.x * blockDim.x) {
    const int ch = t % Cb;
    const int cls = t / Cb;
    int y, rb, x, cb;
    cond_class_ref(cls / ncls, factor, y, rb);
    cond_class_ref(cls % ncls, factor, x, cb);
    float acc[9];
#pragma unroll
    for (int k = 0; k < 9; ++k) acc[k] = 0.f;
    for (int dy = -r; dy <= r; ++dy) {
      if (y + dy < 0 || y + dy >= n_ref) continue;
      int r0, r1;
      float ly0, ly1;
      bilinear_tap(y + dy, factor, 4, r0, r1, ly0, ly1);
      r0 -= rb; r1 -= rb;
      for (int dx = -r; dx <= r; ++dx) {
        if (x + dx < 0 || x + dx >= n_ref) continue;
        int c0, c1;
        float lx0, lx1;
        bilinear_tap(x + dx, factor, 4, c0, c1, lx0, lx1);
        c0 -= cb; c1 -= cb;
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
    for (int k = 0; k < 9; ++k) table[(static_cast<long long>(cls) * 9 + k) * Cb + ch] = acc[k];
  }
}

// acc = bias + sum_k w[k] * t[k] over the 3 x 3 token block; tb points at this thread's 8
// channels of table entry k = 0, entries `stride` float4 apart.
__device__ __forceinline__ void cond_stencil(const float4* tb, int stride, const uint4 (&tk)[9],
                                             const float* bdw, int cv, float (&acc)[8]) {
  if (bdw != nullptr) {
    const float4 b0 = __ldg(reinterpret_cast<const float4*>(bdw) + cv * 2);
    const float4 b1 = __ldg(reinterpret_cast<const float4*>(bdw) + cv * 2 + 1);
    acc[0] = b0.x; acc[1] = b0.y; acc[2] = b0.z; acc[3] = b0.w;
    acc[4] = b1.x; acc[5] = b1.y; acc[6] = b1.z; acc[7] = b1.w;
  } else {
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = 0.f;
  }
#pragma unroll
  for (int k = 0; k < 9; ++k) {
    const float4 w0 = tb[k * stride];
    const float4 w1 = tb[k * stride + 1];
    float t[8];
    unpack8(tk[k], t);
    acc[0] = fmaf(w0.x, t[0], acc[0]); acc[1] = fmaf(w0.y, t[1], acc[1]);
    acc[2] = fmaf(w0.z, t[2], acc[2]); acc[3] = fmaf(w0.w, t[3], acc[3]);
    acc[4] = fmaf(w1.x, t[4], acc[4]); acc[5] = fmaf(w1.y, t[5], acc[5]);
    acc[6] = fmaf(w1.z, t[6], acc[6]); acc[7] = fmaf(w1.w, t[7], acc[7]);
  }
}

// The four corner cells of every plane (each has its own f x f block of table classes). One
// thread: one cell (factor x factor pixels of one backbone token) x 8 channels, table entries
// read from global memory (L2).
constexpr int COND_CELLS_PER_ITEM = 256;   // interior kernel: cells a block walks per slab load
constexpr int COND_BORDER_CELLS_PER_ITEM = 64;

__global__ void __launch_bounds__(256, 2)
adaln_cond_border_kernel(const AdalnCondParams p, const float* __restrict__ table) {
  const int nvec = p.Cb >> 3;
  const int ncvg = nvec >> 2;
  const int f = p.factor;
  const int ncls = 3 * f;
  const int H = p.h * f, W = p.w * f;
  const long long gR0 = p.row0 / W / f;
  const long long gR1 = (p.row0 + p.n_rows - 1) / W / f;
  const long long ring = 4;                                  // the corner cells of one plane
  const long long plane0 = gR0 / p.h;
  const long long n_cells = (gR1 / p.h - plane0 + 1) * ring;
  const long long n_chunks = (n_cells + COND_BORDER_CELLS_PER_ITEM - 1) / COND_BORDER_CELLS_PER_ITEM;
  const long long n_items = n_chunks * ncvg;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  for (long long item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int cvg = static_cast<int>(item / n_chunks);
    const long long cell = (item % n_chunks) * COND_BORDER_CELLS_PER_ITEM + warp * 8 + (lane >> 2);
    if (cell >= n_cells) continue;
    const int cv = cvg * 4 + (lane & 3);
    const long long plane = plane0 + cell / ring;
    const int k = static_cast<int>(cell % ring);
    const int R = (k & 2) ? p.h - 1 : 0, Cc = (k & 1) ? p.w - 1 : 0;
    const int rb = R == 0 ? 0 : (R == p.h - 1 ? p.h - 3 : R - 1);
    const int cb = Cc == 0 ? 0 : (Cc == p.w - 1 ? p.w - 3 : Cc - 1);
    const int ycls0 = R == 0 ? 0 : (R == p.h - 1 ? 2 * f : f);
    const int xcls0 = Cc == 0 ? 0 : (Cc == p.w - 1 ? 2 * f : f);
    const uint4* base = reinterpret_cast<const uint4*>(p.tok + plane * p.h * p.w * p.Cb) + cv;
    uint4 tk[9];
#pragma unroll
    for (int t = 0; t < 9; ++t)
      tk[t] = __ldg(base + (static_cast<long long>(rb + t / 3) * p.w + (cb + t % 3)) * nvec);
    for (int phy = 0; phy < f; ++phy) {
      const int y = R * f + phy;
      for (int phx = 0; phx < f; ++phx) {
        const int x = Cc * f + phx;
        const long long pix = (plane * H + y) * W + x;
        if (pix < p.row0 || pix >= p.row0 + p.n_rows) continue;
        float acc[8];
        const long long cls = static_cast<long long>(ycls0 + phy) * ncls + (xcls0 + phx);
        cond_stencil(reinterpret_cast<const float4*>(table + cls * 9 * p.Cb) + cv * 2, p.Cb >> 2,
                     tk, p.bdw, cv, acc);
        gelu8(acc);
        reinterpret_cast<uint4*>(p.out + (pix - p.row0) * p.Cb)[cv] = pack8(acc);
      }
    }
  }
}

// Interior cells, second layout: one thread = TWO neighbouring cells x 4 channels. The table
// entries of a phase (read from the shared-memory slab) serve both cells, which halves the
// shared-memory reads per output - the interior kernel is paced by those reads and by
// instruction issue in about equal parts. A warp holds 4 cell pairs x 8 channel quads (32
// channels): a token read and a row write are still 64 contiguous bytes per cell.
__global__ void __launch_bounds__(256, 2)
adaln_cond_interior_kernel(const AdalnCondParams p, const float* __restrict__ table, int group0) {
  extern __shared__ __align__(16) float slab[];
  const int ncvg = p.Cb >> 5;
  const int f = p.factor;
  const int ncls = 3 * f;
  const int H = p.h * f, W = p.w * f;
  const long long gR0 = p.row0 / W / f;
  const long long gR1 = (p.row0 + p.n_rows - 1) / W / f;
  // blockIdx.y: which set of cells sharing one f x f block of table classes - 0: the interior,
  // 1 / 2: first / last cell row without its corners, 3 / 4: first / last cell column without
  // its corners (the four corner cells of a plane are left to the border kernel)
  const int group = group0 + static_cast<int>(blockIdx.y);
  const long long plane0 = gR0 / p.h;
  const long long planes = gR1 / p.h - plane0 + 1;
  const int per_plane = group == 0 ? 0 : (group <= 2 ? p.w - 2 : p.h - 2);
  const long long n_cells = group == 0 ? (gR1 - gR0 + 1) * p.w : planes * per_plane;
  const int ycls0 = group == 1 ? 0 : (group == 2 ? 2 * f : f);
  const int xcls0 = group == 3 ? 0 : (group == 4 ? 2 * f : f);
  const long long n_chunks = (n_cells + COND_CELLS_PER_ITEM - 1) / COND_CELLS_PER_ITEM;
  const long long n_items = n_chunks * ncvg;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int cq = lane & 7;
  const int slab_vec = f * f * 9 * 8;                      // float4 count of a slab
  for (long long item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int cvg = static_cast<int>(item / n_chunks);
    const long long cell0 = (item % n_chunks) * COND_CELLS_PER_ITEM;
    __syncthreads();                                       // previous item's readers are done
    for (int v = threadIdx.x; v < slab_vec; v += blockDim.x) {
      const int e = v >> 3;                                // (phase, k)
      const int phase = e / 9, k = e - phase * 9;
      const int cls = (ycls0 + phase / f) * ncls + (xcls0 + phase % f);
      reinterpret_cast<float4*>(slab)[v] = __ldg(
          reinterpret_cast<const float4*>(table + (static_cast<long long>(cls) * 9 + k) * p.Cb +
                                          cvg * 32) + (v & 7));
    }
    __syncthreads();
    const int ch0 = cvg * 32 + 4 * cq;
    float4 bias = make_float4(0.f, 0.f, 0.f, 0.f);
    if (p.bdw != nullptr) bias = __ldg(reinterpret_cast<const float4*>(p.bdw + ch0));
    for (int pass = 0; pass < COND_CELLS_PER_ITEM / 64; ++pass) {
      uint64_t ta[9][2], tb[9][2];   // fp32 pairs (channels 0-1, 2-3): the stencil runs on packed fp32x2
      long long pix_a = -1, pix_b = -1;     // first pixel of each cell; -1: the cell is skipped
#pragma unroll
      for (int s2 = 0; s2 < 2; ++s2) {
        const long long cell = cell0 + pass * 64 + warp * 8 + 2 * (lane >> 3) + s2;
        if (cell >= n_cells) continue;
        long long plane;
        int R, Cc;
        if (group == 0) {
          const long long gR = gR0 + cell / p.w;
          Cc = static_cast<int>(cell % p.w);
          plane = gR / p.h;
          R = static_cast<int>(gR % p.h);
          if (R < 1 || R > p.h - 2 || Cc < 1 || Cc > p.w - 2) continue;
        } else {
          plane = plane0 + cell / per_plane;
          const int j = 1 + static_cast<int>(cell % per_plane);
          R = group == 1 ? 0 : (group == 2 ? p.h - 1 : j);
          Cc = group == 3 ? 0 : (group == 4 ? p.w - 1 : j);
        }
        // the 3 x 3 token block starts one cell before the cell, clamped into the plane
        const int rb = R == 0 ? 0 : (R == p.h - 1 ? p.h - 3 : R - 1);
        const int cb = Cc == 0 ? 0 : (Cc == p.w - 1 ? p.w - 3 : Cc - 1);
        const __nv_bfloat16* base = p.tok + plane * p.h * p.w * p.Cb + ch0;
#pragma unroll
        for (int k = 0; k < 9; ++k) {
          const uint2 t2 = __ldg(reinterpret_cast<const uint2*>(
              base + (static_cast<long long>(rb + k / 3) * p.w + (cb + k % 3)) * p.Cb));
          if (s2 == 0) {
            ta[k][0] = pack2(bf16_lo(t2.x), bf16_hi(t2.x)); ta[k][1] = pack2(bf16_lo(t2.y), bf16_hi(t2.y));
          } else {
            tb[k][0] = pack2(bf16_lo(t2.x), bf16_hi(t2.x)); tb[k][1] = pack2(bf16_lo(t2.y), bf16_hi(t2.y));
          }
        }
        const long long pix0 = (plane * H + static_cast<long long>(R) * f) * W + static_cast<long long>(Cc) * f;
        if (s2 == 0) pix_a = pix0; else pix_b = pix0;
      }
      if (pix_a < 0 && pix_b < 0) continue;
      if (pix_a < 0) {
#pragma unroll
        for (int k = 0; k < 9; ++k) ta[k][0] = ta[k][1] = 0ull;
      }
      if (pix_b < 0) {
#pragma unroll
        for (int k = 0; k < 9; ++k) tb[k][0] = tb[k][1] = 0ull;
      }
      for (int phy = 0; phy < f; ++phy) {
        for (int phx = 0; phx < f; ++phx) {
          const float4* wv = reinterpret_cast<const float4*>(slab) + (phy * f + phx) * 72 + cq;
          uint64_t a[2] = {pack2(bias.x, bias.y), pack2(bias.z, bias.w)};
          uint64_t b[2] = {a[0], a[1]};
#pragma unroll
          for (int k = 0; k < 9; ++k) {
            const float4 w4 = wv[k * 8];
            const uint64_t w01 = pack2(w4.x, w4.y), w23 = pack2(w4.z, w4.w);
            a[0] = ffma2(w01, ta[k][0], a[0]); a[1] = ffma2(w23, ta[k][1], a[1]);
            b[0] = ffma2(w01, tb[k][0], b[0]); b[1] = ffma2(w23, tb[k][1], b[1]);
          }
          const long long off = static_cast<long long>(phy) * W + phx;
          auto finish = [&](const uint64_t (&v2)[2], long long pix0) {
            const long long pix = pix0 + off;
            if (pix0 < 0 || pix < p.row0 || pix >= p.row0 + p.n_rows) return;
            // tanh GELU, the polynomial part on packed fp32x2
            const float k0 = 0.7978845608028654f, k01 = 0.7978845608028654f * 0.044715f;
            const uint64_t K0 = pack2(k0, k0), K01 = pack2(k01, k01), HALF = pack2(0.5f, 0.5f);
            float v[4];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const uint64_t x = v2[j];
              const uint64_t u = fmul2(x, ffma2(fmul2(x, x), K01, K0));
              float u0, u1;
              unpack2(u, u0, u1);
              const uint64_t hx = fmul2(x, HALF);
              unpack2(ffma2(hx, pack2(fast_tanh(u0), fast_tanh(u1)), hx), v[2 * j], v[2 * j + 1]);
            }
            uint2 o;
            o.x = pack_bf16(v[0], v[1]);
            o.y = pack_bf16(v[2], v[3]);
            *reinterpret_cast<uint2*>(p.out + (pix - p.row0) * p.Cb + ch0) = o;
          };
          finish(a, pix_a);
          finish(b, pix_b);
        }
      }
    }
  }
}

// Number of floats of the table the cell kernel needs, or 0 when the geometry takes the
// direct kernel (small factor, wide conv kernel, channel count not a multiple of 32).
inline long long adaln_cond_table_floats(int Cb, int factor, int ks) {
  if (factor < 4 || factor > 8 || ks > 5 || Cb % 32 != 0) return 0;   // slab <= 72 KB of smem
  return 9LL * factor * factor * 9 * Cb;
}

// table: device scratch of adaln_cond_table_floats() floats, or null for the direct kernel.
inline int launch_adaln_cond(const AdalnCondParams& p, float* table, int sm_count,
                             cudaStream_t stream) {
  if (p.Cb % 8 != 0 || p.Cb <= 0 || p.factor <= 0 || p.ks <= 0 || (p.ks & 1) == 0 || p.ks > 9 ||
      p.D <= 0 || p.h <= 0 || p.w <= 0 || p.row0 < 0)
    return -2;
  if (p.n_rows <= 0) return 0;
  if (table != nullptr && p.h >= 3 && p.w >= 3 &&
      adaln_cond_table_floats(p.Cb, p.factor, p.ks) > 0) {
    const int n = 9 * p.factor * p.factor * p.Cb;
    adaln_cond_table_kernel<<<(n + 255) / 256, 256, 0, stream>>>(p.wdw, p.Cb, p.factor, p.ks, table);
    const long long W = static_cast<long long>(p.w) * p.factor;
    const long long cell_rows = (p.row0 + p.n_rows - 1) / W / p.factor - p.row0 / W / p.factor + 1;
    const long long items =
        (cell_rows * p.w + COND_CELLS_PER_ITEM - 1) / COND_CELLS_PER_ITEM * (p.Cb / 32);
    long long blocks = items;
    const long long cap = static_cast<long long>(sm_count) * 24;
    if (blocks > cap) blocks = cap;
    const int slab_bytes = p.factor * p.factor * 9 * 32 * 4;
    if (slab_bytes > 48 * 1024) {
      cudaError_t ea = cudaFuncSetAttribute(adaln_cond_interior_kernel,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, slab_bytes);
      if (ea != cudaSuccess) return -static_cast<int>(ea) - 1000;
    }
    adaln_cond_interior_kernel<<<static_cast<int>(blocks), 256, slab_bytes, stream>>>(p, table, 0);
    {
      const long long H = static_cast<long long>(p.h) * p.factor;
      const long long planes = (p.row0 + p.n_rows - 1) / (H * W) - p.row0 / (H * W) + 1;
      // the first / last cell rows and columns (groups 1-4), then the four corners per plane
      const long long edge = planes * ((p.w > p.h ? p.w : p.h) - 2);
      long long be = (edge + COND_CELLS_PER_ITEM - 1) / COND_CELLS_PER_ITEM * (p.Cb / 32);
      if (be > cap) be = cap;
      adaln_cond_interior_kernel<<<dim3(static_cast<unsigned>(be), 4), 256, slab_bytes, stream>>>(p, table, 1);
      long long bb = (planes * 4 + COND_BORDER_CELLS_PER_ITEM - 1) / COND_BORDER_CELLS_PER_ITEM * (p.Cb / 32);
      if (bb > cap) bb = cap;
      adaln_cond_border_kernel<<<static_cast<int>(bb), 256, 0, stream>>>(p, table);
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
