// extern "C" entry points of libstrata_b200.so (declared in include/strata_b200.h).
// Single translation unit: the kernels live in the .cuh files included below.
#include "../../include/strata_b200.h"

#include <string.h>

#include <atomic>

#include "common.cuh"
#include "gemm_tcgen05.cuh"
#include "layernorm.cuh"
#include "na3d.cuh"
#include "halo.cuh"
#include "prepost.cuh"
#include "adaln.cuh"

using namespace strata;

namespace {

// SM count of the current device (-1: no sm_100 device). The per-device cache is written with
// relaxed atomics: concurrent first calls from several host threads store the same values.
int current_sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  constexpr int kMaxDev = 64;
  static std::atomic<int> cached_sms[kMaxDev];     // 0 = not looked up yet, -1 = not sm_100
  if (dev < 0 || dev >= kMaxDev) return -1;
  int v = cached_sms[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    int sms = 0, major = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
      return -1;
    v = (major == 10 && sms > 0) ? sms : -1;
    cached_sms[dev].store(v, std::memory_order_relaxed);
  }
  return v;
}

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" {

int strata_abi_version(void) { return 1; }

const char* strata_error_string(int code) {
  switch (code) {
    case STRATA_OK: return "ok";
    case STRATA_ERR_ARG: return "invalid argument (shape, pointer or alignment)";
    case STRATA_ERR_UNSUPPORTED: return "unsupported configuration";
    case STRATA_ERR_NO_DEVICE: return "no sm_100 CUDA device is current";
    case STRATA_ERR_SCRATCH_LIMIT:
      return "problem too large for the library's built-in 64 MiB scratch array; use the entry "
             "point that takes a caller-provided workspace";
    case STRATA_ERR_TENSORMAP:
    case -21:
    case -22:
    case -23: return "TMA tensor map could not be encoded for this operand layout";
    default: break;
  }
  if (code <= -1000) return cudaGetErrorString(static_cast<cudaError_t>(-(code + 1000)));
  return "unknown error";
}

int strata_device_status(int* h_status, int reset) {
  if (!h_status) return STRATA_ERR_ARG;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return -static_cast<int>(e) - 1000;
  e = cudaMemcpyFromSymbol(h_status, g_status, sizeof(int));
  if (e != cudaSuccess) return -static_cast<int>(e) - 1000;
  if (reset && *h_status != 0) {
    int zero = 0, one = 1;
    e = cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    if (e != cudaSuccess) return -static_cast<int>(e) - 1000;
    // a failed halo barrier also left the "exchange ok" word at 0 (gathers write NaN meanwhile)
    e = cudaMemcpyToSymbol(g_halo_ok, &one, sizeof(int));
    if (e != cudaSuccess) return -static_cast<int>(e) - 1000;
  }
  return STRATA_OK;
}

int strata_layernorm_bf16(const void* x, int64_t ldx, void* y, int64_t ldy, int M, int C,
                          float eps, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
  if (M == 0) return STRATA_OK;
  if (!x || !y || M < 0 || !aligned16(x) || !aligned16(y)) return STRATA_ERR_ARG;
  int r = launch_layernorm(static_cast<const __nv_bfloat16*>(x), ldx,
                           static_cast<__nv_bfloat16*>(y), ldy, M, C, eps, sms, as_stream(stream));
  return r == -2 ? STRATA_ERR_ARG : r;
}

int strata_linear_bf16(const void* x, int64_t ldx, const void* w, int64_t ldw, const float* bias,
                       void* y, int64_t ldy, int M, int N, int K, int epilogue, const void* aux,
                       int64_t ldaux, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
  if (M == 0 && N > 0 && K > 0) return STRATA_OK;
  if (!x || !w || !y || M < 0 || N <= 0 || K <= 0) return STRATA_ERR_ARG;
  if (K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ldx < K || ldw < K || ldy < N ||
      ldy % 8 != 0 || (aux && ldaux % 8 != 0))
    return STRATA_ERR_ARG;
  if (!aligned16(x) || !aligned16(w) || !aligned16(y) || (bias && !aligned16(bias)))
    return STRATA_ERR_ARG;
  if ((epilogue == STRATA_EPI_RESIDUAL || epilogue == STRATA_EPI_GATE) &&
      (!aux || ldaux < N || !aligned16(aux)))
    return STRATA_ERR_ARG;
  if (M == 0) return STRATA_OK;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.out = static_cast<__nv_bfloat16*>(y);
  p.ldo = ldy;
  p.bias = bias;
  p.aux = static_cast<const __nv_bfloat16*>(aux);
  p.ldaux = ldaux;
  const auto* A = static_cast<const __nv_bfloat16*>(x);
  const auto* W = static_cast<const __nv_bfloat16*>(w);
  cudaStream_t st = as_stream(stream);
  switch (epilogue) {
    case STRATA_EPI_BIAS: return launch_gemm<EPI_BIAS>(A, ldx, W, ldw, p, sms, st);
    case STRATA_EPI_GELU: return launch_gemm<EPI_GELU>(A, ldx, W, ldw, p, sms, st);
    case STRATA_EPI_RESIDUAL: return launch_gemm<EPI_RESIDUAL>(A, ldx, W, ldw, p, sms, st);
    case STRATA_EPI_GATE: return launch_gemm<EPI_GATE>(A, ldx, W, ldw, p, sms, st);
    default: return STRATA_ERR_UNSUPPORTED;
  }
}

// One row of the packed (cos, sin) half table that rotates by nothing: 32 pairs of (1.0, 0.0).
// With tokens_per_tile = M and hw = 1 every token reads this row, which lets a model with the
// q/k norm but without rotation run the same fused epilogue as one with both.
static __device__ __align__(128) uint32_t g_identity_rope_row[32] = {
    0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u,
    0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u,
    0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u,
    0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u, 0x3C00u};
namespace {
std::atomic<void*> g_identity_rope_addr[64];   // per device, written once with the same value
const void* identity_rope_row() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  void* a = g_identity_rope_addr[dev].load(std::memory_order_acquire);
  if (a == nullptr) {
    if (cudaGetSymbolAddress(&a, g_identity_rope_row) != cudaSuccess) return nullptr;
    g_identity_rope_addr[dev].store(a, std::memory_order_release);
  }
  return a;
}
}  // namespace

static int qkv_rope_impl(const void* x, int64_t ldx, const void* w, int64_t ldw, const float* bias,
                         void* qkv, int64_t ldqkv, int M, int C, int head_dim,
                         const void* rope_cs, int tokens_per_tile, int hw, int qk_norm,
                         float qk_eps, int pad_T, int pad_halo, int pad_D, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
  if (M == 0 && C > 0) return STRATA_OK;
  if (!x || !w || !qkv || M < 0 || C <= 0) return STRATA_ERR_ARG;
  if (head_dim != 32 && head_dim != 64) return STRATA_ERR_UNSUPPORTED;
  if (C % 64 != 0 || C % head_dim != 0) return STRATA_ERR_UNSUPPORTED;
  if (ldx % 8 != 0 || ldw % 8 != 0 || ldx < C || ldw < C || ldqkv < 3 * C || ldqkv % 8 != 0)
    return STRATA_ERR_ARG;
  if (!aligned16(x) || !aligned16(w) || !aligned16(qkv) || (bias && !aligned16(bias)))
    return STRATA_ERR_ARG;
  if (rope_cs) {
    if (!aligned16(rope_cs)) return STRATA_ERR_ARG;
    if (hw <= 0 || tokens_per_tile <= 0 || tokens_per_tile % hw != 0 || M % tokens_per_tile != 0)
      return STRATA_ERR_ARG;
  }
  if (M == 0) return STRATA_OK;
  GemmParams p{};
  p.M = M; p.N = 3 * C; p.K = C;
  p.out = static_cast<__nv_bfloat16*>(qkv);
  p.ldo = ldqkv;
  p.bias = bias;
  p.rope_cs = static_cast<const uint32_t*>(rope_cs);
  p.tokens_per_tile = tokens_per_tile > 0 ? tokens_per_tile : 1;
  p.hw = hw > 0 ? hw : 1;
  p.head_dim = head_dim;
  p.rope_cols = 2 * C;
  p.qk_norm = qk_norm;
  p.qk_eps = qk_eps;
  if (pad_T > 0) {
    if (pad_T % 32 != 0 || pad_halo < 0 || pad_D < 1 ||
        M % (pad_D * pad_T * pad_T) != 0)
      return STRATA_ERR_ARG;
    p.pad_T = pad_T; p.pad_h = pad_halo; p.pad_D = pad_D;
  }
  const auto* A = static_cast<const __nv_bfloat16*>(x);
  const auto* W = static_cast<const __nv_bfloat16*>(w);
  if (!rope_cs && !qk_norm) return launch_gemm<EPI_BIAS>(A, ldx, W, ldw, p, sms, as_stream(stream));
  if (!rope_cs && C < 256 && head_dim == 64) {
    // qk norm without rotation at a small width (the pixel stage: C = 128): the projection is
    // bound by its output traffic and the fused epilogue's extra arithmetic costs more than a
    // second pass - plain projection, then the in-place row kernel normalises the q and k heads
    // (measured at C = 128: 0.29 + 0.27 ms against 0.72 ms fused).
    int r = launch_gemm<EPI_BIAS>(A, ldx, W, ldw, p, sms, as_stream(stream));
    if (r != 0) return r;
    long long rows = M;
    if (pad_T > 0) {
      // padded layout: the interior rows are not contiguous - normalise every row of the padded
      // buffer (halo rows are overwritten by the exchange that follows)
      const int P = pad_T + 2 * pad_halo;
      rows = static_cast<long long>(M) / (pad_T * pad_T) * P * P;
    }
    r = launch_qk_norm_rows(static_cast<__nv_bfloat16*>(qkv), ldqkv, rows, C, qk_eps, sms,
                            as_stream(stream));
    return r == -2 ? STRATA_ERR_ARG : r;
  }
  if (!rope_cs) {
    // qk norm without rotation (rope_mode 'none' with qk_norm=True): the fused epilogue with a
    // one-row table of identity rotations that every token reads - the norm is taken from the
    // fp32 accumulators and no second pass over the q and k heads is needed
    p.rope_cs = static_cast<const uint32_t*>(identity_rope_row());
    if (p.rope_cs == nullptr) return STRATA_ERR_NO_DEVICE;
    p.tokens_per_tile = M;
    p.hw = 1;
  }
  return launch_gemm<EPI_QKV_ROPE>(A, ldx, W, ldw, p, sms, as_stream(stream));
}

int strata_qkv_rope_bf16(const void* x, int64_t ldx, const void* w, int64_t ldw, const float* bias,
                         void* qkv, int64_t ldqkv, int M, int C, int head_dim,
                         const void* rope_cs, int tokens_per_tile, int hw, int qk_norm,
                         float qk_eps, void* stream) {
  return qkv_rope_impl(x, ldx, w, ldw, bias, qkv, ldqkv, M, C, head_dim, rope_cs, tokens_per_tile,
                       hw, qk_norm, qk_eps, 0, 0, 0, stream);
}

int strata_qkv_rope_padded_bf16(const void* x, int64_t ldx, const void* w, int64_t ldw,
                                const float* bias, void* qkv_padded, int64_t ldqkv, int M, int C,
                                int head_dim, const void* rope_cs, int tokens_per_tile, int hw,
                                int qk_norm, float qk_eps, int pad_T, int pad_halo, int pad_D,
                                void* stream) {
  if (pad_T <= 0) return STRATA_ERR_ARG;
  return qkv_rope_impl(x, ldx, w, ldw, bias, qkv_padded, ldqkv, M, C, head_dim, rope_cs,
                       tokens_per_tile, hw, qk_norm, qk_eps, pad_T, pad_halo, pad_D, stream);
}

static int na3d_impl(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v,
                     int64_t ldv, void* out, int64_t ldo, int B, int D, int H, int W, int heads,
                     int head_dim, int kd, int kh, int kw, float scale, int q_h0, int q_H, int q_w0,
                     int q_W, int o_h0, int o_H, int o_w0, int o_W, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
  if (!q || !k || !v || !out || B < 0 || D <= 0 || H <= 0 || W <= 0 || heads <= 0)
    return STRATA_ERR_ARG;
  if (head_dim != 64) return STRATA_ERR_UNSUPPORTED;
  const int64_t C = static_cast<int64_t>(heads) * head_dim;
  if (ldq < C || ldk < C || ldv < C || ldo < C) return STRATA_ERR_ARG;
  if (ldq % 8 || ldk % 8 || ldv % 8 || ldo % 8) return STRATA_ERR_ARG;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return STRATA_ERR_ARG;
  if (kd < 1 || kh < 1 || kw < 1 || kd > D || kh > H || kw > W) return STRATA_ERR_ARG;
  if (B == 0) return STRATA_OK;
  const float sc = scale > 0.f ? scale : 1.0f / sqrtf(static_cast<float>(head_dim));
  int r = launch_na3d(static_cast<const __nv_bfloat16*>(q), ldq,
                      static_cast<const __nv_bfloat16*>(k), ldk,
                      static_cast<const __nv_bfloat16*>(v), ldv, static_cast<__nv_bfloat16*>(out),
                      ldo, B, D, H, W, heads, kd, kh, kw, sc, sms, as_stream(stream), q_h0, q_H,
                      q_w0, q_W, o_h0, o_H, o_w0, o_W);
  if (r == -1) return STRATA_ERR_ARG;
  if (r == -2) return STRATA_ERR_UNSUPPORTED;
  return r;
}

int strata_na3d_fwd_bf16(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v,
                         int64_t ldv, void* out, int64_t ldo, int B, int D, int H, int W,
                         int heads, int head_dim, int kd, int kh, int kw, float scale,
                         void* stream) {
  return na3d_impl(q, ldq, k, ldk, v, ldv, out, ldo, B, D, H, W, heads, head_dim, kd, kh, kw,
                   scale, 0, -1, 0, -1, 0, -1, 0, -1, stream);
}

int strata_na3d_fwd_region_bf16(const void* q, int64_t ldq, const void* k, int64_t ldk,
                                const void* v, int64_t ldv, void* out, int64_t ldo, int B, int D,
                                int H, int W, int heads, int head_dim, int kd, int kh, int kw,
                                float scale, int q_h0, int q_H, int q_w0, int q_W, int o_h0,
                                int o_H, int o_w0, int o_W, void* stream) {
  if (q_h0 < 0 || q_w0 < 0 || q_H < 1 || q_W < 1) return STRATA_ERR_ARG;
  return na3d_impl(q, ldq, k, ldk, v, ldv, out, ldo, B, D, H, W, heads, head_dim, kd, kh, kw,
                   scale, q_h0, q_H, q_w0, q_W, o_h0, o_H, o_w0, o_W, stream);
}

int64_t strata_block_workspace_bytes(int64_t M, int C, int hidden) {
  if (M < 0 || C <= 0 || hidden <= 0) return -1;
  // xn [M,C] | qkv [M,3C] | attn [M,C] | x1 [M,C] | h [M,hidden], each rounded to 256 bytes
  auto r256 = [](int64_t b) { return (b + 255) / 256 * 256; };
  return r256(M * C * 2) * 3 + r256(M * 3 * C * 2) + r256(M * static_cast<int64_t>(hidden) * 2);
}

int strata_block_forward_bf16(const void* x, void* y, int n_tiles, int D, int H, int W, int C,
                              int heads, int hidden, int kd, int kh, int kw,
                              const strata_block_weights* wts, const void* rope_cs, int qk_norm,
                              float ln_eps, float qk_eps, void* workspace,
                              int64_t workspace_bytes, void* stream) {
  if (!x || !y || !wts || !workspace || n_tiles < 0 || D <= 0 || H <= 0 || W <= 0)
    return STRATA_ERR_ARG;
  if (heads <= 0 || C % heads != 0) return STRATA_ERR_ARG;
  const int hd = C / heads;
  if (hd != 64) return STRATA_ERR_UNSUPPORTED;
  const int64_t M64 = static_cast<int64_t>(n_tiles) * D * H * W;
  if (M64 > 0x7fffffffLL) return STRATA_ERR_ARG;
  const int M = static_cast<int>(M64);
  if (workspace_bytes < strata_block_workspace_bytes(M, C, hidden)) return STRATA_ERR_ARG;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return STRATA_ERR_ARG;
  if (!wts->w_qkv || !wts->w_proj || !wts->w_fc1 || !wts->w_fc2) return STRATA_ERR_ARG;
  if (M == 0) return STRATA_OK;
  auto r256 = [](int64_t b) { return (b + 255) / 256 * 256; };
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  void* xn = ws;               ws += r256(M64 * C * 2);
  void* qkv = ws;              ws += r256(M64 * 3 * C * 2);
  void* attn = ws;             ws += r256(M64 * C * 2);
  void* x1 = ws;               ws += r256(M64 * C * 2);
  void* hbuf = ws;
  const int tokens_per_tile = D * H * W;
  int r;
  if ((r = strata_layernorm_bf16(x, C, xn, C, M, C, ln_eps, stream)) != 0) return r;
  if ((r = strata_qkv_rope_bf16(xn, C, wts->w_qkv, C, wts->b_qkv, qkv, 3 * C, M, C, hd, rope_cs,
                                tokens_per_tile, H * W, qk_norm, qk_eps, stream)) != 0)
    return r;
  const __nv_bfloat16* qp = static_cast<const __nv_bfloat16*>(qkv);
  if ((r = strata_na3d_fwd_bf16(qp, 3 * C, qp + C, 3 * C, qp + 2 * C, 3 * C, attn, C, n_tiles, D, H,
                                W, heads, hd, kd, kh, kw, 0.f, stream)) != 0)
    return r;
  if (wts->w_gate) {
    if ((r = strata_linear_bf16(xn, C, wts->w_gate, C, wts->b_gate, attn, C, M, C, C,
                                STRATA_EPI_GATE, attn, C, stream)) != 0)
      return r;
  }
  if ((r = strata_linear_bf16(attn, C, wts->w_proj, C, wts->b_proj, x1, C, M, C, C,
                              STRATA_EPI_RESIDUAL, x, C, stream)) != 0)
    return r;
  if ((r = strata_layernorm_bf16(x1, C, xn, C, M, C, ln_eps, stream)) != 0) return r;
  if ((r = strata_linear_bf16(xn, C, wts->w_fc1, C, wts->b_fc1, hbuf, hidden, M, hidden, C,
                              STRATA_EPI_GELU, nullptr, 0, stream)) != 0)
    return r;
  return strata_linear_bf16(hbuf, hidden, wts->w_fc2, hidden, wts->b_fc2, y, C, M, C, hidden,
                            STRATA_EPI_RESIDUAL, x1, C, stream);
}

static int prepost_check(int B, int C, int D, int H, int W, int pv, int ph, int pw, const float* lat,
                         const float* lon, const float* lat0, const float* lon0, int u_idx,
                         int v_idx, int need_latlon) {
  if (B < 0 || C <= 0 || D <= 0 || H <= 0 || W <= 0 || pv <= 0 || ph <= 0 || pw <= 0)
    return STRATA_ERR_ARG;
  if (D % pv || H % ph || W % pw) return STRATA_ERR_ARG;
  const bool rot = u_idx >= 0 || v_idx >= 0;
  if (rot && (u_idx < 0 || v_idx < 0 || u_idx >= C || v_idx >= C || u_idx == v_idx || !lat0 || !lon0))
    return STRATA_ERR_ARG;
  if ((rot || need_latlon) && (!lat || !lon)) return STRATA_ERR_ARG;
  if (static_cast<long long>(B) * (D / pv) * (H / ph) * (W / pw) > 0x7fffffffLL) return STRATA_ERR_ARG;
  return STRATA_OK;
}

int strata_preprocess_patches_bf16(const float* x, int B, int C_in, int D, int H, int W,
                                   const float* lat, const float* lon, const float* lat0,
                                   const float* lon0, int u_idx, int v_idx, int concat_lat, int pv,
                                   int ph, int pw, void* a, int64_t lda, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
  int r = prepost_check(B, C_in, D, H, W, pv, ph, pw, lat, lon, lat0, lon0, u_idx, v_idx, concat_lat);
  if (r != STRATA_OK) return r;
  if (!x || !a) return STRATA_ERR_ARG;
  const long long K = static_cast<long long>(C_in + (concat_lat ? 2 : 0)) * pv * ph * pw;
  if (lda < K) return STRATA_ERR_ARG;
  if (B == 0) return STRATA_OK;
  PrePostParams p{B, C_in, D, H, W, pv, ph, pw, u_idx < 0 ? -1 : u_idx, u_idx < 0 ? -1 : v_idx,
                  concat_lat ? 1 : 0, lat, lon, lat0, lon0, lda};
  const long long npix = static_cast<long long>(B) * H * W;
  long long blocks = (npix + 255) / 256;
  if (blocks > static_cast<long long>(sms) * 16) blocks = static_cast<long long>(sms) * 16;
  preprocess_patches_kernel<<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
      x, static_cast<__nv_bfloat16*>(a), p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

int strata_postprocess_fields_f32(const void* y, int64_t ldy, int B, int C_out, int D, int H, int W,
                                  const float* lat, const float* lon, const float* lat0,
                                  const float* lon0, int u_idx, int v_idx, int pv, int ph, int pw,
                                  float* out, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
  int r = prepost_check(B, C_out, D, H, W, pv, ph, pw, lat, lon, lat0, lon0, u_idx, v_idx, 0);
  if (r != STRATA_OK) return r;
  if (!y || !out || ldy < static_cast<long long>(C_out) * pv * ph * pw) return STRATA_ERR_ARG;
  if (B == 0) return STRATA_OK;
  PrePostParams p{B, C_out, D, H, W, pv, ph, pw, u_idx < 0 ? -1 : u_idx, u_idx < 0 ? -1 : v_idx, 0,
                  lat, lon, lat0, lon0, ldy};
  const long long npix = static_cast<long long>(B) * H * W;
  long long blocks = (npix + 255) / 256;
  if (blocks > static_cast<long long>(sms) * 16) blocks = static_cast<long long>(sms) * 16;
  postprocess_fields_kernel<<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
      static_cast<const __nv_bfloat16*>(y), out, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

int strata_halo_gather_tokens_bf16(void* out, const void* const* h_peer_src, int world,
                                   const int32_t* src_a, const int32_t* src_b, int tiles_per_rank,
                                   int D, int T, int halo, int C, int only_halo, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
  if (!out || !h_peer_src || !src_a || !src_b) return STRATA_ERR_ARG;
  if (world < 1 || world > HALO_MAX_RANKS) return STRATA_ERR_UNSUPPORTED;
  if (tiles_per_rank <= 0 || D <= 0 || T <= 0 || halo < 0 || C <= 0 || C % 8 != 0)
    return STRATA_ERR_ARG;
  if (!aligned16(out)) return STRATA_ERR_ARG;
  PeerPtrs pp{};
  for (int r = 0; r < world; ++r) {
    if (!h_peer_src[r] || !aligned16(h_peer_src[r])) return STRATA_ERR_ARG;
    pp.p[r] = h_peer_src[r];
  }
  const int P = T + 2 * halo;
  const long long cells = static_cast<long long>(tiles_per_rank) * T * T;
  if (cells * world > 0x7fffffffLL) return STRATA_ERR_ARG;
  const long long work = static_cast<long long>(P) * P;   // padded cells of one (tile, depth) slice
  long long bx = (work + 255) / 256;                      // a block's eight warps take 32 cells each
  const long long cap = static_cast<long long>(sms) * 8;
  if (bx > cap) bx = cap;
  dim3 grid(static_cast<unsigned>(bx), static_cast<unsigned>(tiles_per_rank * D));
  if (static_cast<long long>(tiles_per_rank) * D > 65535) return STRATA_ERR_UNSUPPORTED;
  halo_gather_tokens_kernel<<<grid, 256, 0, as_stream(stream)>>>(
      static_cast<__nv_bfloat16*>(out), pp, src_a, src_b, P * P, T * T, D, C,
      static_cast<int>(cells), only_halo, halo, halo + T, P);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

int strata_halo_gather_fields_f32(float* out, const void* const* h_peer_src, int world,
                                  const int32_t* src_a, const int32_t* src_b, int tiles_per_rank,
                                  int T, int halo, int64_t L, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
  if (!out || !h_peer_src || !src_a || !src_b) return STRATA_ERR_ARG;
  if (world < 1 || world > HALO_MAX_RANKS) return STRATA_ERR_UNSUPPORTED;
  if (tiles_per_rank <= 0 || T <= 0 || halo < 0 || L < 0) return STRATA_ERR_ARG;
  if (L == 0) return STRATA_OK;
  PeerPtrs pp{};
  for (int r = 0; r < world; ++r) {
    if (!h_peer_src[r]) return STRATA_ERR_ARG;
    pp.p[r] = h_peer_src[r];
  }
  const int P = T + 2 * halo;
  const long long cells = static_cast<long long>(tiles_per_rank) * T * T;
  const long long ocells = static_cast<long long>(tiles_per_rank) * P * P;
  if (cells * world > 0x7fffffffLL || ocells > 0x7fffffffLL || L > 0x7fffffffLL)
    return STRATA_ERR_ARG;
  long long bx = (ocells + 255) / 256;
  if (bx > 4096) bx = 4096;
  long long by = L;
  const long long want = static_cast<long long>(sms) * 16;  // enough CTAs for two waves
  if (bx * by > want) by = (want + bx - 1) / bx;
  if (by < 1) by = 1;
  if (by > 65535) by = 65535;
  dim3 grid(static_cast<unsigned>(bx), static_cast<unsigned>(by));
  halo_gather_fields_kernel<<<grid, 256, 0, as_stream(stream)>>>(
      out, pp, src_a, src_b, static_cast<int>(ocells), static_cast<int>(cells),
      static_cast<int>(L));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

int strata_halo_gather_knn_fields_f32(float* out, const void* const* h_peer_src, int world,
                                      const int32_t* idx, const float* weights, int k,
                                      int tiles_per_rank, int T, int halo, int64_t L, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
  if (!out || !h_peer_src || !idx || !weights) return STRATA_ERR_ARG;
  if (world < 1 || world > HALO_MAX_RANKS) return STRATA_ERR_UNSUPPORTED;
  if (tiles_per_rank <= 0 || T <= 0 || halo < 0 || L < 0) return STRATA_ERR_ARG;
  if (k != 1 && k != 2 && k != 4 && k != 8) return STRATA_ERR_UNSUPPORTED;
  if (L == 0) return STRATA_OK;
  PeerPtrs pp{};
  for (int r = 0; r < world; ++r) {
    if (!h_peer_src[r]) return STRATA_ERR_ARG;
    pp.p[r] = h_peer_src[r];
  }
  const int P = T + 2 * halo;
  const long long cells = static_cast<long long>(tiles_per_rank) * T * T;
  const long long ocells = static_cast<long long>(tiles_per_rank) * P * P;
  if (cells * world > 0x7fffffffLL || ocells > 0x7fffffffLL || L > 0x7fffffffLL)
    return STRATA_ERR_ARG;
  long long bx = (ocells + 255) / 256;
  if (bx > 4096) bx = 4096;
  long long by = L;
  const long long want = static_cast<long long>(sms) * 16;
  if (bx * by > want) by = (want + bx - 1) / bx;
  if (by < 1) by = 1;
  if (by > 65535) by = 65535;
  dim3 grid(static_cast<unsigned>(bx), static_cast<unsigned>(by));
  cudaStream_t st = as_stream(stream);
  const int no = static_cast<int>(ocells), nc = static_cast<int>(cells), nl = static_cast<int>(L);
  switch (k) {
    case 1: halo_gather_knn_fields_kernel<1><<<grid, 256, 0, st>>>(out, pp, idx, weights, no, nc, nl); break;
    case 2: halo_gather_knn_fields_kernel<2><<<grid, 256, 0, st>>>(out, pp, idx, weights, no, nc, nl); break;
    case 4: halo_gather_knn_fields_kernel<4><<<grid, 256, 0, st>>>(out, pp, idx, weights, no, nc, nl); break;
    default: halo_gather_knn_fields_kernel<8><<<grid, 256, 0, st>>>(out, pp, idx, weights, no, nc, nl); break;
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

int strata_halo_adjoint_fields_f32(float* out, const void* const* h_peer_padded, int world,
                                   const int32_t* offsets, const int32_t* cell, const float* coef,
                                   const float* window, const float* weights, int tiles_per_rank,
                                   int T, int halo, int64_t L, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
  if (!out || !h_peer_padded || !offsets || !cell || !coef || !window || !weights)
    return STRATA_ERR_ARG;
  if (world < 1 || world > HALO_MAX_RANKS) return STRATA_ERR_UNSUPPORTED;
  if (tiles_per_rank <= 0 || T <= 0 || halo < 0 || L < 0) return STRATA_ERR_ARG;
  if (L == 0) return STRATA_OK;
  PeerPtrs pp{};
  for (int r = 0; r < world; ++r) {
    if (!h_peer_padded[r]) return STRATA_ERR_ARG;
    pp.p[r] = h_peer_padded[r];
  }
  const int P = T + 2 * halo;
  const long long cells = static_cast<long long>(tiles_per_rank) * T * T;
  const long long pcells = static_cast<long long>(tiles_per_rank) * P * P;
  if (pcells * world > 0x7fffffffLL || L > 0x7fffffffLL) return STRATA_ERR_ARG;
  long long bx = (cells + 255) / 256;
  if (bx > 4096) bx = 4096;
  long long by = L;
  const long long want = static_cast<long long>(sms) * 16;
  if (bx * by > want) by = (want + bx - 1) / bx;
  if (by < 1) by = 1;
  if (by > 65535) by = 65535;
  dim3 grid(static_cast<unsigned>(bx), static_cast<unsigned>(by));
  halo_adjoint_fields_kernel<<<grid, 256, 0, as_stream(stream)>>>(
      out, pp, offsets, cell, coef, window, weights, static_cast<int>(cells),
      static_cast<int>(pcells), P * P, static_cast<int>(L));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

int strata_halo_gather_kv_bf16(void* qkv, const void* const* h_peer_qkv, int world,
                               const int32_t* src_a, const int32_t* src_b, const void* dcs_a,
                               const void* dcs_b, int tiles_per_rank, int D, int T, int halo, int C,
                               int head_dim, int64_t ldqkv, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
  if (!qkv || !h_peer_qkv || !src_a || !src_b || !dcs_a || !dcs_b) return STRATA_ERR_ARG;
  if (world < 1 || world > HALO_MAX_RANKS) return STRATA_ERR_UNSUPPORTED;
  if (tiles_per_rank <= 0 || D <= 0 || T <= 0 || halo < 0 || C <= 0 || C % 8 != 0 ||
      head_dim < 8 || head_dim % 8 != 0 || C % head_dim != 0 || ldqkv < 3 * C || ldqkv % 8 != 0)
    return STRATA_ERR_ARG;
  if (!aligned16(qkv) || !aligned16(dcs_a) || !aligned16(dcs_b)) return STRATA_ERR_ARG;
  if (halo == 0) return STRATA_OK;
  PeerPtrs pp{};
  for (int r = 0; r < world; ++r) {
    if (!h_peer_qkv[r] || !aligned16(h_peer_qkv[r])) return STRATA_ERR_ARG;
    pp.p[r] = h_peer_qkv[r];
  }
  const int P = T + 2 * halo;
  const long long cells = static_cast<long long>(tiles_per_rank) * T * T;
  if (cells * world > 0x7fffffffLL) return STRATA_ERR_ARG;
  if (static_cast<long long>(tiles_per_rank) * D > 65535) return STRATA_ERR_UNSUPPORTED;
  const long long work = static_cast<long long>(P) * P - static_cast<long long>(T) * T;   // halo cells
  long long bx = (work + 255) / 256;   // a block's eight warps take 32 halo cells each
  const long long cap = static_cast<long long>(sms) * 8;
  if (bx > cap) bx = cap;
  if (bx < 1) return STRATA_OK;   // no halo
  dim3 grid(static_cast<unsigned>(bx), static_cast<unsigned>(tiles_per_rank * D));
  halo_gather_kv_kernel<<<grid, 256, 0, as_stream(stream)>>>(
      static_cast<__nv_bfloat16*>(qkv), pp, src_a, src_b, static_cast<const uint32_t*>(dcs_a),
      static_cast<const uint32_t*>(dcs_b), P, T, halo, D, C, head_dim, ldqkv,
      static_cast<int>(cells));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

int strata_halo_barrier(int* const* h_flags, int me, int world, int epoch, int timeout_ms,
                        void* stream) {
  if (!h_flags || world < 1 || world > HALO_MAX_RANKS || me < 0 || me >= world)
    return STRATA_ERR_ARG;
  FlagPtrs fp{};
  for (int r = 0; r < world; ++r) {
    if (!h_flags[r]) return STRATA_ERR_ARG;
    fp.p[r] = h_flags[r];
  }
  if (timeout_ms <= 0) timeout_ms = 2000;
  const long long limit = static_cast<long long>(timeout_ms) * 2000000LL;  // ~2 GHz
  halo_barrier_kernel<<<1, 32, 0, as_stream(stream)>>>(fp, me, world, epoch, limit);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

int strata_ipc_alloc(int64_t bytes, void** dptr, void* h_handle64) {
  if (bytes <= 0 || !dptr || !h_handle64) return STRATA_ERR_ARG;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, static_cast<size_t>(bytes));
  if (e != cudaSuccess) return -static_cast<int>(e) - 1000;
  e = cudaMemset(p, 0, static_cast<size_t>(bytes));
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(h_handle64), p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return -static_cast<int>(e) - 1000;
  }
  *dptr = p;
  return STRATA_OK;
}

int strata_ipc_open(const void* h_handle64, void** dptr) {
  if (!h_handle64 || !dptr) return STRATA_ERR_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, h_handle64, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(dptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

int strata_ipc_close(void* dptr) {
  if (!dptr) return STRATA_ERR_ARG;
  cudaError_t e = cudaIpcCloseMemHandle(dptr);
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

int strata_ipc_free(void* dptr) {
  if (!dptr) return STRATA_ERR_ARG;
  cudaError_t e = cudaFree(dptr);
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

int strata_adaln_rows_bf16(const void* x, int64_t ldx, const void* y, int64_t ldy, const void* gate,
                           int64_t ldg, void* x_out, int64_t ldxo, const void* shift,
                           const void* scale, int64_t ldm, void* out, int64_t ldo, int M, int C,
                           float eps, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
  if (M == 0) return STRATA_OK;
  if (!x || M < 0 || C <= 0 || C % 8 || ldx % 8 || ldx < C || !aligned16(x)) return STRATA_ERR_ARG;
  if (!y && !out) return STRATA_ERR_ARG;
  if (y && (!x_out || !aligned16(y) || !aligned16(x_out) || ldy % 8 || ldy < C || ldxo % 8 ||
            ldxo < C))
    return STRATA_ERR_ARG;
  if (!y && gate) return STRATA_ERR_ARG;
  if (gate && (!aligned16(gate) || ldg % 8 || ldg < C)) return STRATA_ERR_ARG;
  if ((shift == nullptr) != (scale == nullptr)) return STRATA_ERR_ARG;
  if (shift && (!out || !aligned16(shift) || !aligned16(scale) || ldm % 8 || ldm < C))
    return STRATA_ERR_ARG;
  if (out && (!aligned16(out) || ldo % 8 || ldo < C)) return STRATA_ERR_ARG;
  AdalnRowsParams p;
  p.x = static_cast<const __nv_bfloat16*>(x); p.ldx = ldx;
  p.y = static_cast<const __nv_bfloat16*>(y); p.ldy = ldy;
  p.gate = static_cast<const __nv_bfloat16*>(gate); p.ldg = ldg;
  p.xo = static_cast<__nv_bfloat16*>(x_out); p.ldxo = ldxo;
  p.shift = static_cast<const __nv_bfloat16*>(shift);
  p.scale = static_cast<const __nv_bfloat16*>(scale); p.ldm = ldm;
  p.out = static_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.M = M; p.C = C; p.eps = eps;
  int r = launch_adaln_rows(p, sms, as_stream(stream));
  return r == -2 ? STRATA_ERR_ARG : r;
}

int strata_qk_norm_rows_bf16(void* qkv, int64_t ld, int64_t M, int C, float eps, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
  if (M == 0) return STRATA_OK;
  if (!qkv || M < 0 || !aligned16(qkv)) return STRATA_ERR_ARG;
  int r = launch_qk_norm_rows(static_cast<__nv_bfloat16*>(qkv), ld, M, C, eps, sms,
                              as_stream(stream));
  return r == -2 ? STRATA_ERR_ARG : r;
}

int strata_dealias_patches_bf16(const void* x_rows, int64_t ldx, int B, int C, int D, int H, int W,
                                int pv, int ph, int pw, const float* taps, int n_taps, void* a,
                                int64_t lda, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
  if (B < 0 || C <= 0 || D <= 0 || H <= 0 || W <= 0 || pv <= 0 || ph <= 0 || pw <= 0)
    return STRATA_ERR_ARG;
  if (D % pv || H % ph || W % pw || !x_rows || !a || !taps || n_taps < 1 || n_taps > 8)
    return STRATA_ERR_ARG;
  if (ldx < C || lda < static_cast<int64_t>(C) * pv * ph * pw) return STRATA_ERR_ARG;
  if (B == 0) return STRATA_OK;
  DealiasParams p{};
  p.B = B; p.C = C; p.D = D; p.H = H; p.W = W; p.pv = pv; p.ph = ph; p.pw = pw;
  p.ldx = ldx; p.lda = lda;
  // host taps: the filter acts on decimated axes only (a stride-1 axis keeps a single unit tap)
  float sum = 0.f;
  for (int i = 0; i < n_taps; ++i) sum += taps[i];
  if (sum == 0.f) return STRATA_ERR_ARG;
  auto fill = [&](int patch, int& k, float* f) {
    if (patch == 1) { k = 1; f[0] = 1.f; return; }
    k = n_taps;
    for (int i = 0; i < n_taps; ++i) f[i] = taps[i] / sum;
  };
  fill(pv, p.kd, p.fd); fill(ph, p.kh, p.fh); fill(pw, p.kw, p.fw);
  const long long total = static_cast<long long>(B) * (D / pv) * (H / ph) * (W / pw) * lda;
  long long blocks = (total + 255) / 256;
  if (blocks > static_cast<long long>(sms) * 32) blocks = static_cast<long long>(sms) * 32;
  dealias_patches_kernel<<<static_cast<unsigned>(blocks), 256, 0, as_stream(stream)>>>(
      static_cast<const __nv_bfloat16*>(x_rows), static_cast<__nv_bfloat16*>(a), p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : -static_cast<int>(e) - 1000;
}

int64_t strata_adaln_cond_table_floats(int Cb, int factor, int ks) {
  return adaln_cond_table_floats(Cb, factor, ks);
}

int strata_adaln_cond_bf16(const void* tokens, int B, int D, int h, int w, int Cb, int factor,
                           const float* w_dw, const float* b_dw, int ks, int64_t row0,
                           int64_t n_rows, void* out, float* table_ws, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
  if (n_rows == 0) return STRATA_OK;
  if (!tokens || !w_dw || !out || !aligned16(tokens) || !aligned16(out) || B <= 0 || n_rows < 0)
    return STRATA_ERR_ARG;
  if (D <= 0 || h <= 0 || w <= 0 || factor <= 0) return STRATA_ERR_ARG;
  if (!aligned16(w_dw) || (b_dw && !aligned16(b_dw))) return STRATA_ERR_ARG;
  const int64_t pixels = static_cast<int64_t>(B) * D * h * factor * w * factor;
  if (row0 < 0 || row0 + n_rows > pixels) return STRATA_ERR_ARG;
  AdalnCondParams p;
  p.tok = static_cast<const __nv_bfloat16*>(tokens);
  p.wdw = w_dw; p.bdw = b_dw;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.row0 = row0; p.n_rows = n_rows;
  p.D = D; p.h = h; p.w = w; p.Cb = Cb; p.factor = factor; p.ks = ks;
  if (table_ws && !aligned16(table_ws)) return STRATA_ERR_ARG;
  int r = launch_adaln_cond(p, table_ws, sms, as_stream(stream));
  return r == -2 ? STRATA_ERR_ARG : r;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// Allocation-free variant of the block forward: its scratch is this file-scope device array.
// In host code the name below is only a handle for the runtime (not a device address); the
// address kernels can use is obtained once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[STRATA_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
// written once per device with the same value by whichever host thread calls first
std::atomic<void*> g_static_scratch_addr[kMaxDevices];
}  // namespace

extern "C" int strata_block_forward_static_scratch_bf16(
    const void* x, void* y, int n_tiles, int D, int H, int W, int C, int heads, int hidden, int kd,
    int kh, int kw, const strata_block_weights* wts, const void* rope_cs, int qk_norm, float ln_eps,
    float qk_eps, void* stream) {
  if (n_tiles < 0 || D <= 0 || H <= 0 || W <= 0 || C <= 0 || hidden <= 0) return STRATA_ERR_ARG;
  const int64_t M = static_cast<int64_t>(n_tiles) * D * H * W;
  const int64_t need = strata_block_workspace_bytes(M, C, hidden);
  if (need < 0) return STRATA_ERR_ARG;
  if (need > STRATA_STATIC_SCRATCH_BYTES) return STRATA_ERR_SCRATCH_LIMIT;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return -static_cast<int>(e) - 1000;
  if (dev < 0 || dev >= kMaxDevices) return STRATA_ERR_NO_DEVICE;
  void* scratch = g_static_scratch_addr[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    // One-time set-up for this device (which is current): resolve the array's device address.
    e = cudaGetSymbolAddress(&scratch, g_static_scratch);
    if (e != cudaSuccess) return -static_cast<int>(e) - 1000;
    if (scratch == nullptr) return STRATA_ERR_NO_DEVICE;
    g_static_scratch_addr[dev].store(scratch, std::memory_order_release);
  }
  return strata_block_forward_bf16(x, y, n_tiles, D, H, W, C, heads, hidden, kd, kh, kw, wts,
                                   rope_cs, qk_norm, ln_eps, qk_eps, scratch,
                                   STRATA_STATIC_SCRATCH_BYTES, stream);
}
