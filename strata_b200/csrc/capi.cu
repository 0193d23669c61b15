// extern "C" entry points of libstrata_b200.so (declared in include/strata_b200.h).
// Single translation unit: the kernels live in the .cuh files included below.
#include "../../include/strata_b200.h"

#include "common.cuh"
#include "gemm_tcgen05.cuh"
#include "layernorm.cuh"
#include "na3d.cuh"

using namespace strata;

namespace {

int current_sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  static int cached_dev = -1, cached_sms = 0, cached_major = 0;
  if (dev != cached_dev) {
    int sms = 0, major = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
      return -1;
    cached_dev = dev;
    cached_sms = sms;
    cached_major = major;
  }
  if (cached_major != 10) return -1;
  return cached_sms;
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
    case STRATA_ERR_TENSORMAP:
    case -21: return "TMA tensor map could not be encoded for this operand layout";
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
    int zero = 0;
    e = cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    if (e != cudaSuccess) return -static_cast<int>(e) - 1000;
  }
  return STRATA_OK;
}

int strata_layernorm_bf16(const void* x, int64_t ldx, void* y, int64_t ldy, int M, int C,
                          float eps, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
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
  if (!x || !w || !y || M < 0 || N <= 0 || K <= 0) return STRATA_ERR_ARG;
  if (K % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ldx < K || ldw < K || ldy < N)
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

int strata_qkv_rope_bf16(const void* x, int64_t ldx, const void* w, int64_t ldw, const float* bias,
                         void* qkv, int64_t ldqkv, int M, int C, int head_dim,
                         const float* rope_cos, const float* rope_sin, int tokens_per_tile, int hw,
                         int qk_norm, float qk_eps, void* stream) {
  const int sms = current_sm_count();
  if (sms <= 0) return STRATA_ERR_NO_DEVICE;
  if (!x || !w || !qkv || M < 0 || C <= 0) return STRATA_ERR_ARG;
  if (head_dim != 32 && head_dim != 64) return STRATA_ERR_UNSUPPORTED;
  if (C % 64 != 0 || C % head_dim != 0) return STRATA_ERR_UNSUPPORTED;
  if (ldx % 8 != 0 || ldw % 8 != 0 || ldx < C || ldw < C || ldqkv < 3 * C || ldqkv % 8 != 0)
    return STRATA_ERR_ARG;
  if (!aligned16(x) || !aligned16(w) || !aligned16(qkv) || (bias && !aligned16(bias)))
    return STRATA_ERR_ARG;
  if ((rope_cos == nullptr) != (rope_sin == nullptr)) return STRATA_ERR_ARG;
  if (rope_cos) {
    if (!aligned16(rope_cos) || !aligned16(rope_sin)) return STRATA_ERR_ARG;
    if (hw <= 0 || tokens_per_tile <= 0 || tokens_per_tile % hw != 0 || M % tokens_per_tile != 0)
      return STRATA_ERR_ARG;
  }
  if (M == 0) return STRATA_OK;
  GemmParams p{};
  p.M = M; p.N = 3 * C; p.K = C;
  p.out = static_cast<__nv_bfloat16*>(qkv);
  p.ldo = ldqkv;
  p.bias = bias;
  p.rope_cos = rope_cos;
  p.rope_sin = rope_sin;
  p.tokens_per_tile = tokens_per_tile > 0 ? tokens_per_tile : 1;
  p.hw = hw > 0 ? hw : 1;
  p.head_dim = head_dim;
  p.rope_cols = 2 * C;
  p.qk_norm = qk_norm;
  p.qk_eps = qk_eps;
  const auto* A = static_cast<const __nv_bfloat16*>(x);
  const auto* W = static_cast<const __nv_bfloat16*>(w);
  if (!rope_cos && !qk_norm) return launch_gemm<EPI_BIAS>(A, ldx, W, ldw, p, sms, as_stream(stream));
  if (!rope_cos) return STRATA_ERR_UNSUPPORTED;  // qk norm without rotation: not on the path
  return launch_gemm<EPI_QKV_ROPE>(A, ldx, W, ldw, p, sms, as_stream(stream));
}

int strata_na3d_fwd_bf16(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v,
                         int64_t ldv, void* out, int64_t ldo, int B, int D, int H, int W,
                         int heads, int head_dim, int kd, int kh, int kw, float scale,
                         void* stream) {
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
                      ldo, B, D, H, W, heads, kd, kh, kw, sc, as_stream(stream));
  if (r == -1) return STRATA_ERR_ARG;
  if (r == -2) return STRATA_ERR_UNSUPPORTED;
  return r;
}

}  // extern "C"
