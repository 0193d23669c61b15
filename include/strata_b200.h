/* C ABI of libstrata_b200.so — hand-written sm_100a kernels for the Strata transformer-block
 * hot path and the cubed-sphere tile halo exchange.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its name starts with "h_".
 *   - bf16 tensors are passed as void*; leading dimensions ("ld*") and strides are in
 *     ELEMENTS, not bytes.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *   - Calls are asynchronous on `stream`. The return value reports argument / launch
 *     errors only: 0 = ok, negative = error (see strata_error_string). Failures detected on
 *     the device (a bounded wait that ran out) are recorded in a device status word read
 *     back with strata_device_status().
 *   - Unless stated otherwise no entry point allocates device memory; scratch is passed in.
 *   - Entry points may be called from several host threads (one stream each); the few
 *     per-device values the library caches on first use are stored atomically.
 *
 * The reference implements this path in Python on top of third-party kernels; each entry
 * point cites the reference call it stands in for (path inside the reference project).
 */
#ifndef STRATA_B200_H
#define STRATA_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define STRATA_OK 0
#define STRATA_ERR_ARG (-1)         /* invalid shape / pointer / alignment */
#define STRATA_ERR_UNSUPPORTED (-2) /* configuration this build has no kernel for */
#define STRATA_ERR_NO_DEVICE (-3)   /* no sm_100 device current */
#define STRATA_ERR_SCRATCH_LIMIT (-4) /* problem needs more than the built-in scratch array holds */
#define STRATA_ERR_TENSORMAP (-20)  /* cuTensorMapEncodeTiled refused the operand layout */
/* <= -1000: -(cudaError_t) - 1000 from a launch or runtime call */

/* Epilogue selector of strata_linear_bf16. */
#define STRATA_EPI_BIAS 0     /* y = x W^T + b */
#define STRATA_EPI_GELU 1     /* y = gelu_tanh(x W^T + b) */
#define STRATA_EPI_RESIDUAL 2 /* y = x W^T + b + aux */
#define STRATA_EPI_GATE 4     /* y = aux * sigmoid(x W^T + b) */

int strata_abi_version(void);
const char* strata_error_string(int code);

/* Reads (and, if reset != 0, clears) the device status word of the current device.
 * Synchronises the device. *h_status: 0 = ok, 101..105 = a bounded wait timed out. */
int strata_device_status(int* h_status, int reset);

/* Non-affine LayerNorm over channels: y[m,:] = (x[m,:] - mean) * rsqrt(var + eps).
 * Replaces the block's norm1/norm2 (physicsnemo StrataTransformer3DBlock; the parameter
 * manifests tests/regression_data/ *.param_order.txt list no norm parameters). */
int strata_layernorm_bf16(const void* x, int64_t ldx, void* y, int64_t ldy, int M, int C,
                          float eps, void* stream);

/* y[M,N] = epilogue(x[M,K] W[N,K]^T + bias). W is an nn.Linear weight ([out,in]); bias is
 * fp32 [N] or NULL; aux is the bf16 residual / gated operand or NULL.
 * Replaces nn.Linear calls of the block: attn.proj, attn.gate_proj, mlp.layers.0 (+ the
 * tanh GELU of screamcast/strata_wrappers.py:76-100), mlp.layers.2. */
int strata_linear_bf16(const void* x, int64_t ldx, const void* w, int64_t ldw, const float* bias,
                       void* y, int64_t ldy, int M, int N, int K, int epilogue, const void* aux,
                       int64_t ldaux, void* stream);

/* qkv[M,3C] = x[M,C] Wqkv[3C,C]^T + b with, fused in the epilogue, optional per-head RMS
 * norm of q and k and the 2-D rotary embedding of q and k by the token's (cos,sin) row.
 * rope_cs: [n_tiles, hw, head_dim/2] pairs (cos, sin) in IEEE half, 4 bytes per pair (channel
 * pair p of a head rotates channels 2p, 2p+1); row m of x is token
 * (tile = m / tokens_per_tile, horizontal cell = m % hw). Column layout of qkv:
 * [q heads | k heads | v heads], each head head_dim wide (nn.Linear(C,3C) reshaped
 * [.., 3, heads, head_dim]). Pass rope_cs = NULL for no rotation (with qk_norm set the norm is
 * still fused - the epilogue then runs with an internal one-row table of identity rotations -
 * except below C = 256, where a plain projection followed by strata_qk_norm_rows_bf16's kernel
 * is faster).
 * Replaces attn.qkv + qk norm + stereographic/axial RoPE + head split of the block
 * (tables: screamcast/strata_wrappers.py:636-642). */
int strata_qkv_rope_bf16(const void* x, int64_t ldx, const void* w, int64_t ldw, const float* bias,
                         void* qkv, int64_t ldqkv, int M, int C, int head_dim,
                         const void* rope_cs, int tokens_per_tile, int hw, int qk_norm,
                         float qk_eps, void* stream);

/* 3-D neighbourhood attention forward (non-causal, dilation 1, head_dim 64).
 * q, k, v, out are token-major: element (b,d,h,w,head,c) lives at
 * base + token*ld + head*head_dim + c with token = ((b*D + d)*H + h)*W + w, so q/k/v may be
 * column slices of one packed [M,3C] qkv matrix (ld = 3C) and out a [M,C] matrix.
 * Window of query i along an axis of length L: [s, s+k) with s = clamp(i - k/2, 0, L-k).
 * scale <= 0 selects head_dim^-0.5. Requires kd<=D, kh<=H, kw<=W, odd kw <= 15, kh <= 15.
 * Replaces NATTEN na3d as called by the physicsnemo Strata block (backend selector
 * screamcast/config.py:99, passed at screamcast/strata_wrappers.py:331). */
int strata_na3d_fwd_bf16(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v,
                         int64_t ldv, void* out, int64_t ldo, int B, int D, int H, int W,
                         int heads, int head_dim, int kd, int kh, int kw, float scale,
                         void* stream);

/* Weights of one backbone block, all DEVICE pointers. w_*: bf16 nn.Linear weights [out,in]
 * (row-major, contiguous); b_*: fp32 biases or NULL. w_gate/b_gate NULL = ungated block.
 * Names follow the reference's parameter manifest
 * (tests/regression_data/ *.param_order.txt: attn.qkv, attn.proj, attn.gate_proj,
 * mlp.layers.0, mlp.layers.2). */
typedef struct strata_block_weights {
  const void* w_qkv;   /* [3C, C] */
  const float* b_qkv;  /* [3C] */
  const void* w_proj;  /* [C, C] */
  const float* b_proj;
  const void* w_gate;  /* [C, C] or NULL */
  const float* b_gate;
  const void* w_fc1;   /* [hidden, C] */
  const float* b_fc1;
  const void* w_fc2;   /* [C, hidden] */
  const float* b_fc2;
} strata_block_weights;

/* Scratch bytes strata_block_forward_bf16 needs for M tokens. */
int64_t strata_block_workspace_bytes(int64_t M, int C, int hidden);

/* One Strata backbone block forward over n_tiles tiles of D*H*W tokens (tokens in d,h,w order,
 * C channels innermost, bf16):
 *   xn = LN(x); qkv = rope(xn Wqkv^T + b); a = NA3D(q,k,v); [a *= sigmoid(xn Wg^T + bg)]
 *   x1 = x + a Wp^T + bp; y = x1 + fc2(gelu_tanh(fc1(LN(x1))))
 * x and y are [n_tiles*D*H*W, C]; y may alias x. rope_cs as in strata_qkv_rope_bf16
 * (NULL = no rotation). workspace: strata_block_workspace_bytes(M, C, hidden) bytes of device
 * scratch, 256-byte aligned, owned by the caller. Seven (eight if gated) kernels are launched
 * on `stream`.
 * Replaces one physicsnemo StrataTransformer3D block as driven by
 * screamcast/strata_wrappers.py:314-341,414 (self.strata(x, pos=pos)). */
int strata_block_forward_bf16(const void* x, void* y, int n_tiles, int D, int H, int W, int C,
                              int heads, int hidden, int kd, int kh, int kw,
                              const strata_block_weights* h_weights, const void* rope_cs,
                              int qk_norm, float ln_eps, float qk_eps, void* workspace,
                              int64_t workspace_bytes, void* stream);

/* ---- cubed-sphere tile halo exchange ------------------------------------------------------
 * Gather maps: int32 arrays over the cells of this rank's padded tiles
 * [tiles_per_rank, P, P] (P = tile + 2*halo). src_a[c] is the global id of the interior cell
 * that padded cell c copies; src_b[c] >= 0 marks a corner-diagonal cell that is the mean of
 * cells src_a[c] and src_b[c]. Cell id = g*T*T + i*T + j, g = index of the tile in the global
 * tile order product(face, ti, tj); owner rank = id / cells_per_rank with
 * cells_per_rank = tiles_per_rank*T*T. h_peer_src[r] is the DEVICE pointer through which this
 * GPU reads rank r's tile buffer (its own buffer for r = me, a peer-mapped pointer otherwise);
 * the array itself is in HOST memory, world <= 16.
 * Together they replace the halo padding of screamcast/distributed_halo.py:305-327 (all-gather +
 * regrid) by the copy / rot90 / diagonal-corner index logic of
 * screamcast/cubesphere_transforms.py:357-445 applied per tile
 * (screamcast/distributed_halo.py:451-473), reading only the neighbours' cells. */

/* Token-space halo: buffers [tiles_per_rank, D, T*T, C] bf16 -> out [tiles_per_rank, D, P*P, C].
 * only_halo != 0 leaves the interior cells of `out` untouched. */
int strata_halo_gather_tokens_bf16(void* out, const void* const* h_peer_src, int world,
                                   const int32_t* src_a, const int32_t* src_b, int tiles_per_rank,
                                   int D, int T, int halo, int C, int only_halo, void* stream);

/* Field-space halo (the reference module's interface): buffers [L, tiles_per_rank, T, T] fp32
 * -> out [L, tiles_per_rank, P, P]; L = product of the leading dims. */
int strata_halo_gather_fields_f32(float* out, const void* const* h_peer_src, int world,
                                  const int32_t* src_a, const int32_t* src_b, int tiles_per_rank,
                                  int T, int halo, int64_t L, void* stream);

/* k-nearest-neighbour halo: out[l, oc] = sum_j weights[oc, j] * x[l, idx[oc, j]] over this rank's
 * padded cells oc (replaces DistributedTileKNNHaloPadding_AllGather.forward,
 * screamcast/distributed_halo.py:305-327: all_gather of every rank's tiles + sparse regrid).
 * idx: [tiles_per_rank*P*P, k] global interior cell ids g*T*T + i*T + j (owner rank = id /
 * (tiles_per_rank*T*T)), weights: same shape, fp32; k in {1, 2, 4, 8}. h_peer_src[r]: rank r's
 * tiles [L, tiles_per_rank*T*T] fp32; out: [L, tiles_per_rank*P*P]. Products and sums are
 * rounded one by one in source order. */
int strata_halo_gather_knn_fields_f32(float* out, const void* const* h_peer_src, int world,
                                      const int32_t* idx, const float* weights, int k,
                                      int tiles_per_rank, int T, int halo, int64_t L, void* stream);

/* Windowed overlap-add un-pad: the normalised transpose D_w^-1 A^T (w . y) of the field gather A
 * above (replaces NormalizedHaloAdjoint.forward, screamcast/distributed_halo.py:438-448, whose
 * transpose runs as a vector-Jacobian product of the regrid plus a reduce_scatter). h_peer_padded[r]:
 * rank r's published padded tiles [L, tiles_per_rank*P*P] fp32 (P = T + 2*halo). offsets / cell /
 * coef: for each local interior cell the padded cells copied from it (global padded cell ids
 * g*P*P + pi*P + pj, coefficient 1 or 1/2), window [P*P], weights [tiles_per_rank*T*T] = the
 * per-cell sum of coef*window. out: [L, tiles_per_rank*T*T]. Sums run entry by entry in fp32
 * without fused multiply-add, so the result is reproducible bit for bit on the host. */
int strata_halo_adjoint_fields_f32(float* out, const void* const* h_peer_padded, int world,
                                   const int32_t* offsets, const int32_t* cell, const float* coef,
                                   const float* window, const float* weights, int tiles_per_rank,
                                   int T, int halo, int64_t L, void* stream);

/* Per-block K/V halo (token space, halo exchange every block). The packed qkv rows of each rank
 * live in halo-padded layout [tiles_per_rank, D, P*P, ldqkv] (channels q | k | v, C each); the
 * interiors are written by strata_qkv_rope_padded_bf16. This call fills the k and v channels of
 * the halo cells of `qkv` from the owning tiles' interiors (h_peer_qkv[r]: rank r's padded qkv
 * buffer as mapped into this process), following the same gather maps as above. K is stored by
 * its owner rotated in the owner's RoPE frame and is re-rotated into this tile's frame with
 * dcs_a / dcs_b: [tiles_per_rank, P*P, head_dim/2] (cos, sin) half pairs of the angle difference
 * receiver - sender for the cell's first / second source. New relative to the reference, which
 * exchanges halos once per model step in field space (scripts/ace/run_screamcast_nudged.py:455). */
int strata_halo_gather_kv_bf16(void* qkv, const void* const* h_peer_qkv, int world,
                               const int32_t* src_a, const int32_t* src_b, const void* dcs_a,
                               const void* dcs_b, int tiles_per_rank, int D, int T, int halo, int C,
                               int head_dim, int64_t ldqkv, void* stream);

/* strata_qkv_rope_bf16 whose M = n_tiles*pad_D*pad_T*pad_T input rows are the interior tokens of
 * tiles and whose output rows go to the interior of the halo-padded layout
 * [n_tiles, pad_D, P*P, ldqkv], P = pad_T + 2*pad_halo (pad_T a multiple of 32). */
int strata_qkv_rope_padded_bf16(const void* x, int64_t ldx, const void* w, int64_t ldw,
                                const float* bias, void* qkv_padded, int64_t ldqkv, int M, int C,
                                int head_dim, const void* rope_cs, int tokens_per_tile, int hw,
                                int qk_norm, float qk_eps, int pad_T, int pad_halo, int pad_D,
                                void* stream);

/* strata_na3d_fwd_bf16 restricted to a query region: only tokens with h in [q_h0, q_h0+q_H) and
 * w in [q_w0, q_w0+q_W) are queries (the interior of a halo-padded tile); keys come from the
 * whole [H, W] plane, windows clamp at the plane's (padded) borders. out is the plane
 * [B, D, o_H, o_W, ldo] in which query (h, w) lands at (h - o_h0, w - o_w0); the output window
 * must contain the query region. o_H < 0 or o_W < 0: the query region itself, stored compactly.
 * A larger window lets several calls (an inner region, then border strips) fill one tensor. */
int strata_na3d_fwd_region_bf16(const void* q, int64_t ldq, const void* k, int64_t ldk,
                                const void* v, int64_t ldv, void* out, int64_t ldo, int B, int D,
                                int H, int W, int heads, int head_dim, int kd, int kh, int kw,
                                float scale, int q_h0, int q_H, int q_w0, int q_W, int o_h0,
                                int o_H, int o_w0, int o_W, void* stream);

/* Fused pre-processing of the model wrapper (replaces _StrataModelBase._preprocess,
 * screamcast/strata_wrappers.py:206-238, forward_uv_to_tile, screamcast/wind_rotation.py:49-92,
 * and the patch gathering of the patch-embedding convolution): x [B, C_in, D, H, W] fp32 ->
 * a [B*(D/pv)*(H/ph)*(W/pw), lda] bf16, the operand of the patch-embedding GEMM with columns in
 * (channel, dv, dh, dw) order - the layout of a flattened Conv3d weight - and zeros beyond
 * K = (C_in + 2*concat_lat)*pv*ph*pw. u_idx, v_idx >= 0: those two channels are the east / north
 * wind and are rotated into the tangent basis of the tile centre (lat0, lon0 [B], radians);
 * concat_lat: cos(lat), sin(lat) are appended as channels C_in, C_in+1. lat, lon: [B, H, W]. */
int strata_preprocess_patches_bf16(const float* x, int B, int C_in, int D, int H, int W,
                                   const float* lat, const float* lon, const float* lat0,
                                   const float* lon0, int u_idx, int v_idx, int concat_lat, int pv,
                                   int ph, int pw, void* a, int64_t lda, void* stream);

/* Fused post-processing (replaces unpatchify + _postprocess, strata_wrappers.py:240-249, and
 * inverse_tile_to_uv, wind_rotation.py:95-144): y [tokens, ldy] bf16, the final linear layer's
 * output with columns in (dv, dh, dw, channel) order -> out [B, C_out, D, H, W] fp32, wind
 * channels rotated back to east / north. */
int strata_postprocess_fields_f32(const void* y, int64_t ldy, int B, int C_out, int D, int H, int W,
                                  const float* lat, const float* lon, const float* lat0,
                                  const float* lon0, int u_idx, int v_idx, int pv, int ph, int pw,
                                  float* out, void* stream);

/* Pixel-stage (two-stage model) row kernel: x' = x + gate * y (written to x_out; skipped when y
 * is NULL; gate NULL means x + y), then out = LN(x') * (1 + scale) + shift with a non-affine
 * LayerNorm (skipped when out is NULL; shift/scale NULL means plain LN). All operands bf16 rows
 * of C channels; shift and scale share the row stride ldm (two column blocks of the per-pixel
 * modulation matrix). Replaces the modulate / gated-residual arithmetic of physicsnemo's
 * StrataPixel3DBlock (adaln-zero: screamcast train.py:279-299 states shift=0, scale=1, gate=0
 * at initialisation). */
int strata_adaln_rows_bf16(const void* x, int64_t ldx, const void* y, int64_t ldy, const void* gate,
                           int64_t ldg, void* x_out, int64_t ldxo, const void* shift,
                           const void* scale, int64_t ldm, void* out, int64_t ldo, int M, int C,
                           float eps, void* stream);

/* In-place RMS norm of the q and k heads (64 channels each) of packed rows [M, 3C]
 * (qk_norm_pixel of screamcast/strata_wrappers.py:437, non-affine). */
int strata_qk_norm_rows_bf16(void* qkv, int64_t ld, int64_t M, int C, float eps, void* stream);

/* Conditioning rows of the "bilinear_dw" AdaLN mode (screamcast/strata_wrappers.py:491-495;
 * parameters adaln_bilinear_dw_conv.{weight,bias} of the parameter manifest
 * tests/regression_data/pixeldit_*.param_order.txt:253-254): backbone tokens [B, D, h, w, Cb]
 * bf16 are upsampled bilinearly by `factor` in h and w (half-pixel centres), convolved depthwise
 * with a ks x ks kernel (zero padding), biased and passed through the tanh GELU; rows
 * row0 .. row0 + n_rows of the flattened (b, d, y, x) pixel order are written as bf16 [n_rows, Cb]
 * (fastest when the range covers whole groups of `factor` image rows). */
int strata_adaln_cond_bf16(const void* tokens, int B, int D, int h, int w, int Cb, int factor,
                           const float* w_dw, const float* b_dw, int ks, int64_t row0,
                           int64_t n_rows, void* out, float* table_ws, void* stream);

/* Floats of device scratch (`table_ws` above) that let strata_adaln_cond_bf16 fold upsample and
 * convolution into one 3 x 3 token stencil per pixel phase (factor >= 4, ks <= 5, Cb % 32 == 0);
 * 0 when the geometry has no such form. With table_ws NULL every pixel is evaluated tap by tap. */
int64_t strata_adaln_cond_table_floats(int Cb, int factor, int ks);

/* Operand rows of the de-aliased patch embedding (screamcast/dealias.py:28-143,
 * DealiasedPatchEmbed3D): x_rows = pixel rows [B, D, H, W, ldx] bf16, channels last (what
 * strata_preprocess_patches_bf16 writes at patch 1x1x1); a[token, (c, v, y, x)] = the low-pass
 * filtered patch, so that strata_linear_bf16 with the proj weight gives the module's tokens.
 * taps: HOST array of the 1-D resample filter (n_taps <= 8, e.g. 1 4 6 4 1), applied on the
 * axes whose patch size exceeds 1, normalised by its sum; edges replicate as in the reference. */
int strata_dealias_patches_bf16(const void* x_rows, int64_t ldx, int B, int C, int D, int H, int W,
                                int pv, int ph, int pw, const float* taps, int n_taps, void* a,
                                int64_t lda, void* stream);

/* Cross-GPU barrier on the stream: publishes `epoch` (monotonically increasing per use) in slot
 * [me] of every rank's flag array h_flags[r] (int32[world], zero-initialised, peer-mapped) and
 * waits - for at most timeout_ms - until all slots of this rank's own array reached it. Work
 * enqueued before it is visible to the peers' kernels enqueued after their barrier. A timeout
 * sets device status 105 and, until the next barrier that completes or until the status is
 * cleared with strata_device_status(.., reset = 1), makes every halo gather / adjoint kernel of
 * this device fill its output with NaN (the peers' data may be missing or stale): a failed
 * exchange cannot pass for a good one even if the caller polls the status rarely. Every rank
 * must run on its own GPU. */
int strata_halo_barrier(int* const* h_flags, int me, int world, int epoch, int timeout_ms,
                        void* stream);

/* Peer-shareable device memory (CUDA IPC). These four calls DO allocate / map memory; use
 * them at set-up. handle: 64 bytes, exchanged between the processes of one node by any means. */
int strata_ipc_alloc(int64_t bytes, void** dptr, void* h_handle64);
int strata_ipc_open(const void* h_handle64, void** dptr);
int strata_ipc_close(void* dptr);
int strata_ipc_free(void* dptr);

/* Size in bytes of the scratch array built into the library for
 * strata_block_forward_static_scratch_bf16. */
#define STRATA_STATIC_SCRATCH_BYTES (64ll * 1024 * 1024)

/* Same computation and same arguments as strata_block_forward_bf16, except that the caller
 * passes no workspace: the scratch lives in a 64 MiB array that is part of the library image.
 * (This entry point has no counterpart in the reference; it is an addition of this library.)
 *
 * Who it is for: code that must run the block but is not in a position to obtain device
 * memory of its own - a plugin called from inside someone else's inference loop with a fixed
 * memory budget, a host whose allocator must not be touched while a latency-critical section
 * or another library's memory pool is active, or an embedder that is handed input and output
 * buffers and nothing else. Such callers cannot call cudaMalloc (or have torch do it), so the
 * ordinary entry point, which wants a caller-allocated workspace, is closed to them.
 *
 * Contract
 *   - Allocates nothing: no cudaMalloc/cudaFree, no allocating library call. Inputs, outputs,
 *     weights and RoPE tables are still the caller's buffers.
 *   - Limit: strata_block_workspace_bytes(M, C, hidden) must not exceed
 *     STRATA_STATIC_SCRATCH_BYTES (e.g. 26 214 tokens at C=128, hidden=512); larger problems
 *     are refused with STRATA_ERR_SCRATCH_LIMIT before anything is launched.
 *   - Cost: every GPU on which the library is loaded keeps the 64 MiB array until the
 *     process exits, whether or not this entry point is ever called.
 *   - The first call on each device looks up the array's device address (with that device
 *     current). Make that first call outside any stream capture.
 *   - All calls on a device share the one array. It keeps whatever the previous call left in
 *     it; nothing in it has to start at zero because every scratch buffer is fully written
 *     before it is read. Two calls whose kernels can overlap on the GPU (different streams
 *     without an ordering between them, or different host threads) race on the array and
 *     corrupt each other: serialise them. */
int strata_block_forward_static_scratch_bf16(const void* x, void* y, int n_tiles, int D, int H,
                                             int W, int C, int heads, int hidden, int kd, int kh,
                                             int kw, const strata_block_weights* h_weights,
                                             const void* rope_cs, int qk_norm, float ln_eps,
                                             float qk_eps, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* STRATA_B200_H */
