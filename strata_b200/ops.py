"""Tensor-level wrappers over the C ABI (device pointers + current CUDA stream).

Each function checks dtypes/devices on the Python side, passes raw pointers to
libstrata_b200.so and raises on any error code. Nothing here computes on the host and
nothing falls back to PyTorch kernels.
"""
from __future__ import annotations

import torch

from . import _lib
from .rope import pack_rope_tables

EPI_BIAS = 0
EPI_GELU = 1
EPI_RESIDUAL = 2
EPI_GATE = 4


def _stream_ptr(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _require_cuda_bf16(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise _lib.StrataLibraryError(
            f"{name} must be a CUDA tensor: strata_b200 has no CPU path")
    if t.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be bfloat16, got {t.dtype}")


def _as_rows(t: torch.Tensor, name: str) -> tuple[torch.Tensor, int, int, int]:
    """View t as [M, C] with unit inner stride; returns (tensor, M, C, ld)."""
    if t.dim() < 2:
        raise ValueError(f"{name} must have at least 2 dims")
    c = t.shape[-1]
    t2 = t.reshape(-1, c)
    if t2.stride(-1) != 1:
        t2 = t2.contiguous()
    ld = t2.stride(0) if t2.shape[0] > 1 else max(t2.stride(0), c)
    return t2, t2.shape[0], c, ld


def _f32_or_none(t, name):
    if t is None:
        return None
    if t.dtype != torch.float32:
        raise TypeError(f"{name} must be float32")
    return t.contiguous()


def _rope_cs(rope_cos, rope_sin, rope_cs, want_shape, device):
    """Packed half (cos, sin) table for the kernels, from fp32 tables unless already packed."""
    if rope_cs is None:
        if rope_cos is None:
            return None
        rope_cos = _f32_or_none(rope_cos, "rope_cos")
        rope_sin = _f32_or_none(rope_sin, "rope_sin")
        if tuple(rope_cos.shape) != want_shape or tuple(rope_sin.shape) != want_shape:
            raise ValueError(f"rope tables must be {want_shape}, got {tuple(rope_cos.shape)}")
        rope_cs = pack_rope_tables(rope_cos, rope_sin)
    if rope_cs.dtype != torch.float16 or tuple(rope_cs.shape) != (*want_shape, 2):
        raise ValueError(f"rope_cs must be float16 {(*want_shape, 2)}, got {rope_cs.dtype} "
                         f"{tuple(rope_cs.shape)}")
    if not rope_cs.is_cuda:
        rope_cs = rope_cs.to(device)
    return rope_cs.contiguous()


def layernorm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Non-affine LayerNorm over the last dim (bf16 in, bf16 out)."""
    _require_cuda_bf16(x, "x")
    x2, M, C, ld = _as_rows(x, "x")
    y = torch.empty((M, C), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().strata_layernorm_bf16(x2.data_ptr(), ld, y.data_ptr(), C, M, C,
                                                     float(eps), _stream_ptr(x)),
                   "strata_layernorm_bf16")
    return y.reshape(x.shape)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
           epilogue: int = EPI_BIAS, aux: torch.Tensor | None = None,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """y = epilogue(x @ weight.T + bias); weight is [N, K] (nn.Linear layout), bias fp32."""
    _require_cuda_bf16(x, "x")
    _require_cuda_bf16(weight, "weight")
    x2, M, K, ldx = _as_rows(x, "x")
    if weight.dim() != 2 or weight.shape[1] != K:
        raise ValueError(f"weight must be [N, {K}], got {tuple(weight.shape)}")
    w = weight if weight.stride(1) == 1 else weight.contiguous()
    N = w.shape[0]
    bias = _f32_or_none(bias, "bias")
    aux_ptr, ldaux = None, 0
    if epilogue in (EPI_RESIDUAL, EPI_GATE):
        if aux is None:
            raise ValueError("this epilogue needs `aux`")
        _require_cuda_bf16(aux, "aux")
        a2, Ma, Na, ldaux = _as_rows(aux, "aux")
        if (Ma, Na) != (M, N):
            raise ValueError(f"aux must be [{M}, {N}], got [{Ma}, {Na}]")
        aux_ptr = a2.data_ptr()
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    else:
        _require_cuda_bf16(out, "out")
        if out.shape != (M, N) or out.stride(1) != 1:
            raise ValueError("out must be [M, N] with unit inner stride")
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().strata_linear_bf16(
            x2.data_ptr(), ldx, w.data_ptr(), w.stride(0),
            None if bias is None else bias.data_ptr(), out.data_ptr(), out.stride(0), M, N, K,
            int(epilogue), aux_ptr, ldaux, _stream_ptr(x)), "strata_linear_bf16")
    return out if x.dim() == 2 else out.reshape(*x.shape[:-1], N)


def qkv_rope(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, head_dim: int,
             rope_cos: torch.Tensor | None, rope_sin: torch.Tensor | None, tokens_per_tile: int,
             hw: int, qk_norm: bool = False, qk_eps: float = 1e-6,
             rope_cs: torch.Tensor | None = None) -> torch.Tensor:
    """Fused QKV projection + optional qk RMS norm + rotary embedding; returns [M, 3C].
    Tables: fp32 rope_cos / rope_sin [n_tiles, hw, head_dim/2], or the packed half table
    rope_cs (see rope.pack_rope_tables)."""
    _require_cuda_bf16(x, "x")
    _require_cuda_bf16(weight, "weight")
    x2, M, C, ldx = _as_rows(x, "x")
    if weight.shape != (3 * C, C):
        raise ValueError(f"qkv weight must be [{3 * C}, {C}], got {tuple(weight.shape)}")
    w = weight if weight.stride(1) == 1 else weight.contiguous()
    bias = _f32_or_none(bias, "bias")
    n_tiles = M // max(tokens_per_tile, 1)
    cs = _rope_cs(rope_cos, rope_sin, rope_cs, (n_tiles, hw, head_dim // 2), x.device)
    out = torch.empty((M, 3 * C), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().strata_qkv_rope_bf16(
            x2.data_ptr(), ldx, w.data_ptr(), w.stride(0),
            None if bias is None else bias.data_ptr(), out.data_ptr(), 3 * C, M, C, head_dim,
            None if cs is None else cs.data_ptr(), int(tokens_per_tile), int(hw),
            1 if qk_norm else 0, float(qk_eps), _stream_ptr(x)), "strata_qkv_rope_bf16")
    return out


def _token_major(t: torch.Tensor, name: str) -> int:
    """Check a [B,D,H,W,heads,hd] view is token-major; return its token stride."""
    if t.dim() != 6:
        raise ValueError(f"{name} must be [B, D, H, W, heads, head_dim]")
    B, D, H, W, nh, hd = t.shape
    sb, sd, sh, sw, sn, sc = t.stride()
    ld = sw
    ok = sc == 1 and sn == hd and sh == W * ld and sd == H * W * ld and (B == 1 or sb == D * H * W * ld)
    if not ok:
        raise ValueError(f"{name} is not token-major (strides {t.stride()}); call .contiguous()")
    return ld


def na3d(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kernel, scale: float | None = None,
         out: torch.Tensor | None = None) -> torch.Tensor:
    """3-D neighbourhood attention. q, k, v: [B, D, H, W, heads, 64] bf16 (token-major views,
    e.g. slices of a packed qkv tensor). Returns [B, D, H, W, heads, 64]."""
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _require_cuda_bf16(t, n)
    if not (q.shape == k.shape == v.shape):
        raise ValueError("q, k, v must have the same shape")
    B, D, H, W, nh, hd = q.shape
    kd, kh, kw = (int(kernel),) * 3 if isinstance(kernel, int) else tuple(int(x) for x in kernel)
    ldq, ldk, ldv = _token_major(q, "q"), _token_major(k, "k"), _token_major(v, "v")
    if out is None:
        out = torch.empty((B, D, H, W, nh, hd), dtype=torch.bfloat16, device=q.device)
    ldo = _token_major(out, "out")
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().strata_na3d_fwd_bf16(
            q.data_ptr(), ldq, k.data_ptr(), ldk, v.data_ptr(), ldv, out.data_ptr(), ldo,
            B, D, H, W, nh, hd, kd, kh, kw, float(scale) if scale else 0.0, _stream_ptr(q)),
            "strata_na3d_fwd_bf16")
    return out


def block_workspace_bytes(M: int, C: int, hidden: int) -> int:
    return int(_lib.load().strata_block_workspace_bytes(int(M), int(C), int(hidden)))


def block_forward(x: torch.Tensor, weights: dict, *, grid, num_heads: int, kernel,
                  rope_cos: torch.Tensor | None, rope_sin: torch.Tensor | None,
                  qk_norm: bool = False, ln_eps: float = 1e-6, qk_eps: float = 1e-6,
                  workspace: torch.Tensor | None = None, out: torch.Tensor | None = None,
                  rope_cs: torch.Tensor | None = None):
    """One backbone block through strata_block_forward_bf16.

    x: [n_tiles, D*H*W, C] bf16 contiguous. weights: bf16 'w_*' [out,in] and fp32 'b_*'
    tensors keyed qkv/proj/gate/fc1/fc2 (gate optional). workspace: uint8 scratch of at least
    block_workspace_bytes(M, C, hidden) bytes (allocated here when None).
    """
    _require_cuda_bf16(x, "x")
    if x.dim() != 3 or not x.is_contiguous():
        raise ValueError("x must be a contiguous [n_tiles, D*H*W, C] tensor")
    D, H, W = grid
    n_tiles, T, C = x.shape
    if T != D * H * W:
        raise ValueError(f"x has {T} tokens per tile, grid {grid} has {D * H * W}")
    kd, kh, kw = (int(kernel),) * 3 if isinstance(kernel, int) else tuple(int(v) for v in kernel)
    hidden = weights["w_fc1"].shape[0]
    M = n_tiles * T
    need = block_workspace_bytes(M, C, hidden)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    if workspace.numel() * workspace.element_size() < need:
        raise ValueError(f"workspace too small: need {need} bytes")
    if out is None:
        out = torch.empty_like(x)
    wstruct = _lib.BlockWeights()
    keep = []
    for name in ("qkv", "proj", "gate", "fc1", "fc2"):
        w = weights.get(f"w_{name}")
        b = weights.get(f"b_{name}")
        if w is not None:
            _require_cuda_bf16(w, f"w_{name}")
            if not w.is_contiguous():
                raise ValueError(f"w_{name} must be contiguous")
            keep.append(w)
        if b is not None:
            if b.dtype != torch.float32 or not b.is_contiguous() or not b.is_cuda:
                raise TypeError(f"b_{name} must be a contiguous CUDA float32 tensor")
            keep.append(b)
        setattr(wstruct, f"w_{name}", None if w is None else w.data_ptr())
        setattr(wstruct, f"b_{name}", None if b is None else b.data_ptr())
    cs = _rope_cs(rope_cos, rope_sin, rope_cs, (n_tiles, H * W, (C // num_heads) // 2), x.device)
    import ctypes
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().strata_block_forward_bf16(
            x.data_ptr(), out.data_ptr(), n_tiles, D, H, W, C, num_heads, hidden, kd, kh, kw,
            ctypes.byref(wstruct), None if cs is None else cs.data_ptr(),
            1 if qk_norm else 0, float(ln_eps),
            float(qk_eps), workspace.data_ptr(), workspace.numel() * workspace.element_size(),
            _stream_ptr(x)), "strata_block_forward_bf16")
    return out


def qkv_rope_padded(x: torch.Tensor, weight: torch.Tensor, bias, head_dim: int,
                    rope_cs: torch.Tensor | None, tokens_per_tile: int, hw: int, out: torch.Tensor,
                    tile: int, halo: int, depth: int, qk_norm: bool = False,
                    qk_eps: float = 1e-6) -> torch.Tensor:
    """Fused QKV projection whose output rows land in the interior of halo-padded tiles.
    x: [n_tiles*depth*tile*tile, C] interior tokens; out: [n_tiles*depth*P*P, 3C], P = tile+2*halo."""
    _require_cuda_bf16(x, "x")
    _require_cuda_bf16(weight, "weight")
    _require_cuda_bf16(out, "out")
    x2, M, C, ldx = _as_rows(x, "x")
    P = tile + 2 * halo
    n_tiles = M // (depth * tile * tile)
    if out.dim() != 2 or out.shape != (n_tiles * depth * P * P, 3 * C) or out.stride(1) != 1:
        raise ValueError(f"out must be [{n_tiles * depth * P * P}, {3 * C}]")
    w = weight if weight.stride(1) == 1 else weight.contiguous()
    bias = _f32_or_none(bias, "bias")
    cs = _rope_cs(None, None, rope_cs, (n_tiles, hw, head_dim // 2), x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().strata_qkv_rope_padded_bf16(
            x2.data_ptr(), ldx, w.data_ptr(), w.stride(0),
            None if bias is None else bias.data_ptr(), out.data_ptr(), out.stride(0), M, C, head_dim,
            None if cs is None else cs.data_ptr(), int(tokens_per_tile), int(hw),
            1 if qk_norm else 0, float(qk_eps), int(tile), int(halo), int(depth), _stream_ptr(x)),
            "strata_qkv_rope_padded_bf16")
    return out


def na3d_region(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kernel, region,
                scale: float | None = None, out: torch.Tensor | None = None,
                out_window=None) -> torch.Tensor:
    """Neighbourhood attention where only region = (h0, Hq, w0, Wq) of each [H, W] plane holds
    queries; returns [B, D, Hq, Wq, heads, 64]. With `out` [B, D, Ho, Wo, heads, 64] and
    out_window = (oh0, Ho, ow0, Wo) the queries land at (h - oh0, w - ow0) of that tensor, so
    several calls can fill one output."""
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _require_cuda_bf16(t, n)
    B, D, H, W, nh, hd = q.shape
    kd, kh, kw = (int(kernel),) * 3 if isinstance(kernel, int) else tuple(int(x) for x in kernel)
    h0, Hq, w0, Wq = (int(t) for t in region)
    ldq, ldk, ldv = _token_major(q, "q"), _token_major(k, "k"), _token_major(v, "v")
    if out is None:
        out = torch.empty((B, D, Hq, Wq, nh, hd), dtype=torch.bfloat16, device=q.device)
        oh0, Ho, ow0, Wo = 0, -1, 0, -1
    else:
        _require_cuda_bf16(out, "out")
        oh0, Ho, ow0, Wo = (int(t) for t in out_window)
        if tuple(out.shape) != (B, D, Ho, Wo, nh, hd) or not out.is_contiguous():
            raise ValueError("out must be a contiguous [B, D, Ho, Wo, heads, 64] tensor")
    with torch.cuda.device(q.device):
        _lib.check(_lib.load().strata_na3d_fwd_region_bf16(
            q.data_ptr(), ldq, k.data_ptr(), ldk, v.data_ptr(), ldv, out.data_ptr(), nh * hd,
            B, D, H, W, nh, hd, kd, kh, kw, float(scale) if scale else 0.0, h0, Hq, w0, Wq,
            oh0, Ho, ow0, Wo, _stream_ptr(q)), "strata_na3d_fwd_region_bf16")
    return out


def _f32_dev(t, name, shape=None):
    if t is None:
        return None
    if t.dtype != torch.float32 or not t.is_cuda:
        raise TypeError(f"{name} must be a CUDA float32 tensor")
    t = t.contiguous()
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")
    return t


def preprocess_patches(x: torch.Tensor, lat, lon, lat0=None, lon0=None, wind=None,
                       concat_lat: bool = False, patch=(1, 1, 1), k_pad: int | None = None):
    """Fused wind rotation + latitude channels + patch gathering + bf16 cast.

    x [B, C_in, D, H, W] fp32 -> [B*(D/pv)*(H/ph)*(W/pw), Kp] bf16 with columns (channel, dv, dh,
    dw), K = (C_in + 2*concat_lat)*pv*ph*pw padded with zeros to Kp (default: next multiple of
    8). lat / lon [B, H, W] radians (needed for rotation or latitude channels); wind = (u, v)
    channel indices with lat0 / lon0 [B] the tile centres."""
    if x.dtype != torch.float32 or not x.is_cuda or x.dim() != 5:
        raise TypeError("x must be a CUDA float32 [B, C, D, H, W] tensor")
    x = x.contiguous()
    B, C, D, H, W = x.shape
    pv, ph, pw = (int(v) for v in patch)
    K = (C + (2 if concat_lat else 0)) * pv * ph * pw
    Kp = (K + 7) // 8 * 8 if k_pad is None else int(k_pad)
    u, v = (-1, -1) if wind is None else (int(wind[0]), int(wind[1]))
    lat = _f32_dev(lat, "lat", (B, H, W))
    lon = _f32_dev(lon, "lon", (B, H, W))
    lat0 = None if lat0 is None else _f32_dev(lat0.reshape(-1), "lat0", (B,))
    lon0 = None if lon0 is None else _f32_dev(lon0.reshape(-1), "lon0", (B,))
    if D % pv or H % ph or W % pw:
        raise ValueError(f"grid {(D, H, W)} is not divisible by the patch {(pv, ph, pw)}")
    a = torch.empty(B * (D // pv) * (H // ph) * (W // pw), Kp, dtype=torch.bfloat16, device=x.device)
    p = lambda t: None if t is None else t.data_ptr()
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().strata_preprocess_patches_bf16(
            x.data_ptr(), B, C, D, H, W, p(lat), p(lon), p(lat0), p(lon0), u, v,
            1 if concat_lat else 0, pv, ph, pw, a.data_ptr(), Kp, _stream_ptr(x)),
            "strata_preprocess_patches_bf16")
    return a


def postprocess_fields(y: torch.Tensor, shape, lat=None, lon=None, lat0=None, lon0=None, wind=None,
                       patch=(1, 1, 1)) -> torch.Tensor:
    """Fused unpatchify + inverse wind rotation: y [tokens, >= pv*ph*pw*C_out] bf16 with columns
    (dv, dh, dw, channel) -> [B, C_out, D, H, W] fp32 (shape = (B, C_out, D, H, W))."""
    _require_cuda_bf16(y, "y")
    if y.dim() != 2 or y.stride(1) != 1:
        raise ValueError("y must be a row-major [tokens, columns] matrix")
    B, C, D, H, W = (int(v) for v in shape)
    pv, ph, pw = (int(v) for v in patch)
    if D % pv or H % ph or W % pw:
        raise ValueError(f"grid {(D, H, W)} is not divisible by the patch {(pv, ph, pw)}")
    if y.shape[0] != B * (D // pv) * (H // ph) * (W // pw) or y.shape[1] < C * pv * ph * pw:
        raise ValueError("y does not match the requested field shape")
    u, v = (-1, -1) if wind is None else (int(wind[0]), int(wind[1]))
    lat = _f32_dev(lat, "lat", (B, H, W))
    lon = _f32_dev(lon, "lon", (B, H, W))
    lat0 = None if lat0 is None else _f32_dev(lat0.reshape(-1), "lat0", (B,))
    lon0 = None if lon0 is None else _f32_dev(lon0.reshape(-1), "lon0", (B,))
    out = torch.empty(B, C, D, H, W, dtype=torch.float32, device=y.device)
    p = lambda t: None if t is None else t.data_ptr()
    with torch.cuda.device(y.device):
        _lib.check(_lib.load().strata_postprocess_fields_f32(
            y.data_ptr(), y.stride(0), B, C, D, H, W, p(lat), p(lon), p(lat0), p(lon0), u, v,
            pv, ph, pw, out.data_ptr(), _stream_ptr(y)), "strata_postprocess_fields_f32")
    return out


# ------------------------------------------------------------------ pixel stage (AdaLN blocks)
def _rows_or_none(t, name, C):
    if t is None:
        return None, 0
    _require_cuda_bf16(t, name)
    if t.dim() != 2 or t.shape[1] != C or t.stride(1) != 1:
        raise ValueError(f"{name} must be [M, {C}] rows with unit inner stride")
    return t.data_ptr(), t.stride(0)


def adaln_rows(x: torch.Tensor, *, y: torch.Tensor | None = None, gate: torch.Tensor | None = None,
               shift: torch.Tensor | None = None, scale: torch.Tensor | None = None,
               norm: bool = True, eps: float = 1e-6):
    """One pass over token rows [M, C] (bf16): x <- x + gate * y in place (when y is given;
    gate None means x + y), then - when `norm` - returns LN(x) * (1 + scale) + shift (plain
    non-affine LN when shift/scale are None). y, gate, shift, scale may be column slices of wider
    matrices. Returns the normalised rows, or None when norm is False."""
    _require_cuda_bf16(x, "x")
    if x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be [M, C] rows with unit inner stride")
    M, C = x.shape
    if y is None and not norm:
        raise ValueError("nothing to do: give y and/or norm=True")
    if (shift is None) != (scale is None):
        raise ValueError("shift and scale come together")
    yp, ldy = _rows_or_none(y, "y", C)
    gp, ldg = _rows_or_none(gate, "gate", C)
    sp, lds = _rows_or_none(shift, "shift", C)
    cp, ldc = _rows_or_none(scale, "scale", C)
    if sp is not None and lds != ldc:
        raise ValueError("shift and scale must share a row stride")
    out = torch.empty((M, C), dtype=torch.bfloat16, device=x.device) if norm else None
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().strata_adaln_rows_bf16(
            x.data_ptr(), x.stride(0), yp, ldy, gp, ldg, x.data_ptr() if yp else None, x.stride(0),
            sp, cp, lds, None if out is None else out.data_ptr(), C, M, C, float(eps),
            _stream_ptr(x)), "strata_adaln_rows_bf16")
    return out


def qk_norm_rows_(qkv: torch.Tensor, C: int, eps: float = 1e-6) -> torch.Tensor:
    """In-place RMS norm of the 64-channel q and k heads of packed rows [M, 3C]."""
    _require_cuda_bf16(qkv, "qkv")
    if qkv.dim() != 2 or qkv.shape[1] != 3 * C or qkv.stride(1) != 1:
        raise ValueError(f"qkv must be [M, {3 * C}] rows")
    with torch.cuda.device(qkv.device):
        _lib.check(_lib.load().strata_qk_norm_rows_bf16(
            qkv.data_ptr(), qkv.stride(0), qkv.shape[0], int(C), float(eps), _stream_ptr(qkv)),
            "strata_qk_norm_rows_bf16")
    return qkv


def adaln_cond(tokens: torch.Tensor, w_dw: torch.Tensor, b_dw: torch.Tensor | None, factor: int,
               row0: int = 0, n_rows: int | None = None, out: torch.Tensor | None = None,
               direct: bool = False):
    """GELU(depthwise conv(bilinear upsample(tokens)) + bias) as bf16 rows. tokens: bf16
    [B, D, h, w, Cb] contiguous; w_dw fp32 [Cb, ks, ks]; rows row0 .. row0+n_rows of the
    flattened (b, d, y, x) pixels at resolution (h*factor, w*factor). direct=True evaluates
    every pixel tap by tap instead of through the folded 3x3 stencil table."""
    _require_cuda_bf16(tokens, "tokens")
    if tokens.dim() != 5 or not tokens.is_contiguous():
        raise ValueError("tokens must be contiguous [B, D, h, w, Cb]")
    B, D, h, w, Cb = tokens.shape
    w_dw = _f32_dev(w_dw, "w_dw")
    if w_dw.dim() != 3 or w_dw.shape[0] != Cb or w_dw.shape[1] != w_dw.shape[2]:
        raise ValueError(f"w_dw must be [{Cb}, ks, ks]")
    ks = w_dw.shape[1]
    b_dw = None if b_dw is None else _f32_dev(b_dw, "b_dw", (Cb,))
    pixels = B * D * h * factor * w * factor
    if n_rows is None:
        n_rows = pixels - row0
    if out is None:
        out = torch.empty((n_rows, Cb), dtype=torch.bfloat16, device=tokens.device)
    elif out.shape != (n_rows, Cb) or not out.is_contiguous() or out.dtype != torch.bfloat16:
        raise ValueError("out must be contiguous bf16 [n_rows, Cb]")
    lib = _lib.load()
    n_table = 0 if direct else int(lib.strata_adaln_cond_table_floats(Cb, int(factor), ks))
    table = torch.empty(n_table, dtype=torch.float32, device=tokens.device) if n_table else None
    with torch.cuda.device(tokens.device):
        _lib.check(lib.strata_adaln_cond_bf16(
            tokens.data_ptr(), B, D, h, w, Cb, int(factor), w_dw.data_ptr(),
            None if b_dw is None else b_dw.data_ptr(), ks, int(row0), int(n_rows), out.data_ptr(),
            None if table is None else table.data_ptr(), _stream_ptr(tokens)),
            "strata_adaln_cond_bf16")
    return out


def dealias_patches(x_rows: torch.Tensor, shape, channels: int, patch, taps, k_pad: int | None = None):
    """Filtered patch rows of the de-aliased patch embedding. x_rows: bf16 pixel rows
    [B*D*H*W, ld] (channels last, `preprocess_patches` at patch 1); shape = (B, D, H, W);
    taps: the 1-D resample filter (python floats). Returns bf16 [tokens, k_pad]."""
    import ctypes
    _require_cuda_bf16(x_rows, "x_rows")
    B, D, H, W = (int(v) for v in shape)
    pv, ph, pw = (int(v) for v in patch)
    if x_rows.dim() != 2 or x_rows.shape[0] != B * D * H * W or x_rows.stride(1) != 1:
        raise ValueError("x_rows must be [B*D*H*W, ld] pixel rows")
    K = channels * pv * ph * pw
    k_pad = K if k_pad is None else int(k_pad)
    tokens = B * (D // pv) * (H // ph) * (W // pw)
    a = torch.empty((tokens, k_pad), dtype=torch.bfloat16, device=x_rows.device)
    t = (ctypes.c_float * len(taps))(*[float(v) for v in taps])
    with torch.cuda.device(x_rows.device):
        _lib.check(_lib.load().strata_dealias_patches_bf16(
            x_rows.data_ptr(), x_rows.stride(0), B, int(channels), D, H, W, pv, ph, pw,
            ctypes.cast(t, ctypes.c_void_p), len(taps), a.data_ptr(), k_pad, _stream_ptr(x_rows)),
            "strata_dealias_patches_bf16")
    return a
