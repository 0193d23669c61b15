// Fused pre- and post-processing of the Strata wrapper around the token path.
//
// Pre (one pass over the input fields instead of ~40 elementwise kernels, three concatenations
// and a transposing copy): for every pixel
//   * rotate the horizontal wind (U, V) from the pixel's east / north basis into the tangent
//     basis of the tile centre,
//   * append cos(lat), sin(lat) as two more channels,
//   * write the pixel's channel values, cast to bf16, into its slot of the patch-embedding
//     GEMM operand A[token, (c, dv, dh, dw)] (non-overlapping patches: a pure permutation).
// Post: the final linear layer's output Y[token, (dv, dh, dw, c)] is un-patchified to
// [B, C_out, D, H, W] fp32 and the wind channels are rotated back to east / north.
//
// One thread per horizontal pixel (b, y, x); it walks the D levels, so the trigonometry of its
// bases is evaluated once (in double precision: the values are then rounded to fp32, which keeps
// them independent of the fast-math setting the library is built with). HBM-bound, and small:
// the fields have C_in channels where the token stream has hundreds.
#pragma once
#include "common.cuh"

namespace strata {

struct Basis {
  float e[3], n[3], r[3];
};
__device__ __forceinline__ Basis local_basis_enr(float lat, float lon) {
  double sl, cl, so, co;
  sincos(static_cast<double>(lat), &sl, &cl);
  sincos(static_cast<double>(lon), &so, &co);
  Basis b;
  const float fsl = static_cast<float>(sl), fcl = static_cast<float>(cl);
  const float fso = static_cast<float>(so), fco = static_cast<float>(co);
  b.e[0] = -fso; b.e[1] = fco; b.e[2] = 0.f;
  b.n[0] = -fsl * fco; b.n[1] = -fsl * fso; b.n[2] = fcl;
  b.r[0] = fcl * fco; b.r[1] = fcl * fso; b.r[2] = fsl;
  return b;
}

struct PrePostParams {
  int B, C, D, H, W;      // field tensor [B, C, D, H, W] (C = channels of x resp. of the output)
  int pv, ph, pw;         // patch extents
  int u_idx, v_idx;       // wind channels, -1: no rotation
  int concat_lat;         // pre only: append cos(lat), sin(lat)
  const float* lat;       // [B, H, W] radians
  const float* lon;
  const float* lat0;      // [B] tile-centre latitude / longitude (rotation only)
  const float* lon0;
  long long ld;           // row stride of the token matrix (elements)
};

// x [B, C, D, H, W] fp32 -> A [B*d*h*w, ld] bf16, columns (c, dv, dh, dw), zero beyond K.
__global__ void __launch_bounds__(256)
preprocess_patches_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ a,
                          const PrePostParams p) {
  const long long npix = static_cast<long long>(p.B) * p.H * p.W;
  const int d_tok = p.D / p.pv, h_tok = p.H / p.ph, w_tok = p.W / p.pw;
  const int pvol = p.pv * p.ph * p.pw;
  const int c_all = p.C + (p.concat_lat ? 2 : 0);
  const int K = c_all * pvol;
  for (long long pix = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; pix < npix;
       pix += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int xw = static_cast<int>(pix % p.W);
    const int yh = static_cast<int>((pix / p.W) % p.H);
    const int b = static_cast<int>(pix / (static_cast<long long>(p.W) * p.H));
    const float lat = __ldg(p.lat + pix), lon = __ldg(p.lon + pix);
    const bool rot = p.u_idx >= 0;
    Basis q{}, q0{};
    if (rot) {
      q = local_basis_enr(lat, lon);
      q0 = local_basis_enr(__ldg(p.lat0 + b), __ldg(p.lon0 + b));
    }
    float cl = 0.f, sl = 0.f;
    if (p.concat_lat) {
      double s, c;
      sincos(static_cast<double>(lat), &s, &c);
      cl = static_cast<float>(c);
      sl = static_cast<float>(s);
    }
    const int dh = yh % p.ph, dw = xw % p.pw;
    const int th = yh / p.ph, tw = xw / p.pw;
    const long long plane = static_cast<long long>(p.H) * p.W;
    const float* xb = x + (static_cast<long long>(b) * p.C * p.D) * plane +
                      static_cast<long long>(yh) * p.W + xw;
    for (int d = 0; d < p.D; ++d) {
      const int dv = d % p.pv, td = d / p.pv;
      const long long row = ((static_cast<long long>(b) * d_tok + td) * h_tok + th) * w_tok + tw;
      __nv_bfloat16* ar = a + row * p.ld + (dv * p.ph + dh) * p.pw + dw;
      float ur = 0.f, vr = 0.f;
      if (rot) {
        const float U = __ldg(xb + (static_cast<long long>(p.u_idx) * p.D + d) * plane);
        const float V = __ldg(xb + (static_cast<long long>(p.v_idx) * p.D + d) * plane);
        float v3[3], dot = 0.f;
#pragma unroll
        for (int i = 0; i < 3; ++i) {
          v3[i] = U * q.e[i] + V * q.n[i];
          dot += v3[i] * q0.r[i];
        }
#pragma unroll
        for (int i = 0; i < 3; ++i) {
          const float vt = v3[i] - dot * q0.r[i];
          ur += vt * q0.e[i];
          vr += vt * q0.n[i];
        }
      }
      auto channel = [&](int c) -> float {
        if (c >= c_all) return 0.f;                      // padding column
        if (c >= p.C) return c == p.C ? cl : sl;         // latitude channels
        if (rot && c == p.u_idx) return ur;
        if (rot && c == p.v_idx) return vr;
        return __ldg(xb + (static_cast<long long>(c) * p.D + d) * plane);
      };
      if (pvol == 1 && (p.ld & 7) == 0) {
        // one pixel = one token: the whole row (padding included) goes out in 16-byte stores
        uint4* ar4 = reinterpret_cast<uint4*>(a + row * p.ld);
        for (int c8 = 0; c8 < p.ld; c8 += 8) {
          uint4 o;
          o.x = pack_bf16(channel(c8), channel(c8 + 1));
          o.y = pack_bf16(channel(c8 + 2), channel(c8 + 3));
          o.z = pack_bf16(channel(c8 + 4), channel(c8 + 5));
          o.w = pack_bf16(channel(c8 + 6), channel(c8 + 7));
          ar4[c8 >> 3] = o;
        }
        continue;
      }
      for (int c = 0; c < p.C; ++c) ar[c * pvol] = __float2bfloat16(channel(c));
      if (p.concat_lat) {
        ar[p.C * pvol] = __float2bfloat16(cl);
        ar[(p.C + 1) * pvol] = __float2bfloat16(sl);
      }
      if (dv == 0 && dh == 0 && dw == 0)   // padding columns of the row: written once per token
        for (int k = K; k < p.ld; ++k) a[row * p.ld + k] = __float2bfloat16(0.f);
    }
  }
}

// Y [B*d*h*w, ld] bf16, columns (dv, dh, dw, c) -> out [B, C, D, H, W] fp32, wind rotated back.
__global__ void __launch_bounds__(256)
postprocess_fields_kernel(const __nv_bfloat16* __restrict__ y, float* __restrict__ out,
                          const PrePostParams p) {
  const long long npix = static_cast<long long>(p.B) * p.H * p.W;
  const int d_tok = p.D / p.pv, h_tok = p.H / p.ph, w_tok = p.W / p.pw;
  for (long long pix = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; pix < npix;
       pix += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int xw = static_cast<int>(pix % p.W);
    const int yh = static_cast<int>((pix / p.W) % p.H);
    const int b = static_cast<int>(pix / (static_cast<long long>(p.W) * p.H));
    const bool rot = p.u_idx >= 0;
    Basis q{}, q0{};
    float inv_rr = 0.f;
    if (rot) {
      q = local_basis_enr(__ldg(p.lat + pix), __ldg(p.lon + pix));
      q0 = local_basis_enr(__ldg(p.lat0 + b), __ldg(p.lon0 + b));
      inv_rr = q0.r[0] * q.r[0] + q0.r[1] * q.r[1] + q0.r[2] * q.r[2];
    }
    const int dh = yh % p.ph, dw = xw % p.pw;
    const int th = yh / p.ph, tw = xw / p.pw;
    const long long plane = static_cast<long long>(p.H) * p.W;
    float* ob = out + (static_cast<long long>(b) * p.C * p.D) * plane +
                static_cast<long long>(yh) * p.W + xw;
    for (int d = 0; d < p.D; ++d) {
      const int dv = d % p.pv, td = d / p.pv;
      const long long row = ((static_cast<long long>(b) * d_tok + td) * h_tok + th) * w_tok + tw;
      const __nv_bfloat16* yr = y + row * p.ld + ((dv * p.ph + dh) * p.pw + dw) * p.C;
      float ug = 0.f, vg = 0.f;
      if (rot) {
        const float Ul = __bfloat162float(yr[p.u_idx]), Vl = __bfloat162float(yr[p.v_idx]);
        float vt[3], num = 0.f;
#pragma unroll
        for (int i = 0; i < 3; ++i) {
          vt[i] = Ul * q0.e[i] + Vl * q0.n[i];
          num += vt[i] * q.r[i];
        }
        const float beta = -num / inv_rr;
#pragma unroll
        for (int i = 0; i < 3; ++i) {
          const float v3 = vt[i] + beta * q0.r[i];
          ug += v3 * q.e[i];
          vg += v3 * q.n[i];
        }
      }
      for (int c = 0; c < p.C; ++c) {
        float val;
        if (rot && c == p.u_idx) val = ug;
        else if (rot && c == p.v_idx) val = vg;
        else val = __bfloat162float(yr[c]);
        ob[(static_cast<long long>(c) * p.D + d) * plane] = val;
      }
    }
  }
}

// De-aliased patch gathering (reference: screamcast/dealias.py:28-143). The reference runs the
// patch convolution at stride 1 without padding, pads its output by replication, low-pass
// filters it per decimated axis and decimates by the patch size. Filtering commutes with the
// convolution, so the same tokens come from ONE strided GEMM whose operand rows are filtered
// patches:  A[token, (c, v, y, x)] = sum_k f[k] * X[c, s_d(k) + v, s_h(k) + y, s_w(k) + x]  with
// s_axis(k) = clamp(token_axis * patch + k_axis - (K_axis - 1) / 2, 0, size - patch) - the clamp
// is the replicate padding of the stride-1 output. X: pixel rows [B, D, H, W, ldx] bf16
// (channels last, the output of preprocess_patches at patch 1); A: [tokens, lda] bf16, zero
// beyond the C * pv * ph * pw valid columns.
struct DealiasParams {
  int B, C, D, H, W, pv, ph, pw;
  int kd, kh, kw;
  float fd[8], fh[8], fw[8];     // per-axis taps, each already divided by its sum
  long long ldx, lda;
};

__global__ void __launch_bounds__(256)
dealias_patches_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ a,
                       const DealiasParams p) {
  const int d_tok = p.D / p.pv, h_tok = p.H / p.ph, w_tok = p.W / p.pw;
  const int pvol = p.pv * p.ph * p.pw;
  const int K = p.C * pvol;
  const long long total = static_cast<long long>(p.B) * d_tok * h_tok * w_tok * p.lda;
  for (long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int col = static_cast<int>(t % p.lda);
    const long long tok = t / p.lda;
    if (col >= K) {
      a[t] = __float2bfloat16(0.f);
      continue;
    }
    const int c = col / pvol;
    int rem = col - c * pvol;
    const int v = rem / (p.ph * p.pw);
    rem -= v * p.ph * p.pw;
    const int yy = rem / p.pw, xx = rem - yy * p.pw;
    const int tw = static_cast<int>(tok % w_tok);
    const int th = static_cast<int>((tok / w_tok) % h_tok);
    const int td = static_cast<int>((tok / (static_cast<long long>(w_tok) * h_tok)) % d_tok);
    const long long b = tok / (static_cast<long long>(w_tok) * h_tok * d_tok);
    float acc = 0.f;
    for (int id = 0; id < p.kd; ++id) {
      int sd = td * p.pv + id - (p.kd - 1) / 2;
      sd = sd < 0 ? 0 : (sd > p.D - p.pv ? p.D - p.pv : sd);
      for (int ih = 0; ih < p.kh; ++ih) {
        int sh = th * p.ph + ih - (p.kh - 1) / 2;
        sh = sh < 0 ? 0 : (sh > p.H - p.ph ? p.H - p.ph : sh);
        const float fdh = p.fd[id] * p.fh[ih];
        const long long row = ((b * p.D + sd + v) * p.H + sh + yy) * p.W;
        for (int iw = 0; iw < p.kw; ++iw) {
          int sw = tw * p.pw + iw - (p.kw - 1) / 2;
          sw = sw < 0 ? 0 : (sw > p.W - p.pw ? p.W - p.pw : sw);
          acc = fmaf(fdh * p.fw[iw], __bfloat162float(x[(row + sw + xx) * p.ldx + c]), acc);
        }
      }
    }
    a[t] = __float2bfloat16(acc);
  }
}

}  // namespace strata
