"""CPU oracle for the Strata transformer block (TEST INFRASTRUCTURE, not product code).

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may
import this module. The product path (strata_b200/) never does.

PARITY UNPINNED. The block's arithmetic lives in third-party packages that are absent from
the reference tree and from this machine: NVIDIA/physicsnemo @ 07cdcc8b65f10bee733a32a77b4b76e20c70c54c
(physicsnemo.experimental.models.strata: StrataTransformer3D, its blocks, the RoPE builders)
and NATTEN v0.21.5 (na3d). The reference ships no golden tensors for it (its
tests/regression_data/*.pt are git-ignored). This file restates the published algorithms and
anchors on what the reference tree does pin:

  * wiring and hyper-parameters      screamcast/strata_wrappers.py:261-341
  * parameter tree / Linear shapes   tests/regression_data/*.param_order.txt
                                     (attn.qkv, attn.proj, [attn.gate_proj], mlp.layers.0,
                                     mlp.layers.2; no norm parameters => non-affine norms)
  * tanh GELU                        screamcast/strata_wrappers.py:76-100
  * RoPE unit system                 screamcast/strata_wrappers.py:134-150,
                                     screamcast/tile_geometry.py:157-170
  * RoPE table length = D*H*W, shared over depth   tests/test_dit_3d.py:99-101,
                                     screamcast/strata_wrappers.py:636-642

Every choice the reference tree does not pin is listed in oracle/ASSUMPTIONS.md and made in
exactly one place below.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

LN_EPS = 1e-6
QK_EPS = 1e-6


# --------------------------------------------------------------------------- geometry
def window_starts(length: int, k: int) -> torch.Tensor:
    """First key index of each query's window along one axis.

    Neighbourhood attention (NATTEN, non-causal, dilation 1) keeps every window at full
    size k: away from the borders it is centred on the query, at a border it is shifted
    inwards: start(i) = clamp(i - k//2, 0, length - k).
    """
    if k > length:
        raise ValueError(f"kernel {k} larger than axis length {length}")
    i = torch.arange(length)
    return (i - k // 2).clamp(0, length - k)


def spherical_centroid(lat: torch.Tensor, lon: torch.Tensor):
    """Centre of a tile: the normalised mean of its unit vectors. lat/lon [B,H,W] rad."""
    x = (torch.cos(lat) * torch.cos(lon)).mean(dim=(-2, -1))
    y = (torch.cos(lat) * torch.sin(lon)).mean(dim=(-2, -1))
    z = torch.sin(lat).mean(dim=(-2, -1))
    n = torch.sqrt(x * x + y * y + z * z)
    lat0 = torch.asin((z / n).clamp(-1, 1))
    lon0 = torch.atan2(y, x)
    return lat0, lon0


def stereographic_projection(lat, lon, lat0, lon0):
    """Stereographic map about (lat0, lon0) on the unit sphere; returns (x east, y north)."""
    lat0 = lat0[..., None, None]
    dlon = lon - lon0[..., None, None]
    cosc = torch.sin(lat0) * torch.sin(lat) + torch.cos(lat0) * torch.cos(lat) * torch.cos(dlon)
    kk = 2.0 / (1.0 + cosc)
    x = kk * torch.cos(lat) * torch.sin(dlon)
    y = kk * (torch.cos(lat0) * torch.sin(lat) - torch.sin(lat0) * torch.cos(lat) * torch.cos(dlon))
    return x, y


def rope_frequencies(head_dim: int, theta: float) -> torch.Tensor:
    """Frequency ladder of one axis: head_dim/4 values theta^(-i/(head_dim/4))."""
    n = head_dim // 4
    return theta ** (-torch.arange(n, dtype=torch.float64) / n)


def rope_tables_from_coords(xc: torch.Tensor, yc: torch.Tensor, head_dim: int, theta: float):
    """2-D continuous axial RoPE tables from per-token coordinates.

    xc, yc: [..., T]. Returns cos, sin of shape [..., T, head_dim/2]: the first head_dim/4
    angles are xc * f_i, the next head_dim/4 are yc * f_i. Pair p rotates channels
    (2p, 2p+1) of a head.
    """
    if head_dim % 4 != 0:
        raise ValueError("head_dim must be a multiple of 4 for 2-D RoPE")
    f = rope_frequencies(head_dim, theta)
    ax = xc.double()[..., None] * f
    ay = yc.double()[..., None] * f
    ang = torch.cat([ax, ay], dim=-1)
    return torch.cos(ang).float(), torch.sin(ang).float()


def stereographic_rope_tables(lat, lon, head_dim: int, patch: int, length_scale: float,
                              theta: float = 100.0):
    """Tables [B, (H/patch)*(W/patch), head_dim/2] from per-pixel lat/lon [B,H,W] (radians).

    Pixels are projected about the tile's spherical centroid, averaged over each
    patch x patch token footprint and divided by length_scale
    (= default_rope_length_scale(1) * patch for the backbone, screamcast/strata_wrappers.py:333-338).
    """
    lat0, lon0 = spherical_centroid(lat.double(), lon.double())
    x, y = stereographic_projection(lat.double(), lon.double(), lat0, lon0)
    if patch > 1:
        x = F.avg_pool2d(x[:, None], patch)[:, 0]
        y = F.avg_pool2d(y[:, None], patch)[:, 0]
    x = (x / length_scale).flatten(1)
    y = (y / length_scale).flatten(1)
    return rope_tables_from_coords(x, y, head_dim, theta)


def axial_rope_tables(h: int, w: int, head_dim: int, theta: float = 100.0):
    """Tables [1, h*w, head_dim/2] for the axial mode: coordinates are token row / column."""
    ii, jj = torch.meshgrid(torch.arange(h, dtype=torch.float64),
                            torch.arange(w, dtype=torch.float64), indexing="ij")
    return rope_tables_from_coords(jj.flatten()[None], ii.flatten()[None], head_dim, theta)


def default_rope_length_scale(patch_size_horiz: int) -> float:
    """screamcast/tile_geometry.py:157-170."""
    return math.sqrt(math.pi * patch_size_horiz ** 2 / (3.0 * 1024 ** 2))


# --------------------------------------------------------------------------- pieces
def apply_rope(t: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """t [B, D, HW, heads, hd]; cos/sin [B or 1, HW, hd/2]. Interleaved pairs (2p, 2p+1)."""
    a = t[..., 0::2]
    b = t[..., 1::2]
    c = cos[:, None, :, None, :]
    s = sin[:, None, :, None, :]
    out = torch.stack([a * c - b * s, a * s + b * c], dim=-1)
    return out.flatten(-2)


def rms_norm(t: torch.Tensor, eps: float = QK_EPS) -> torch.Tensor:
    return t * torch.rsqrt(t.pow(2).mean(dim=-1, keepdim=True) + eps)


def na3d(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kernel, scale: float | None = None):
    """3-D neighbourhood attention by explicit gathering.

    q, k, v: [B, D, H, W, heads, hd]. Each query attends the kd*kh*kw keys of its clamped
    window; softmax over them with scale hd^-0.5. Returns [B, D, H, W, heads, hd].
    """
    B, D, H, W, nh, hd = q.shape
    kd, kh, kw = kernel
    scale = hd ** -0.5 if scale is None else scale
    sd, sh, sw = window_starts(D, kd), window_starts(H, kh), window_starts(W, kw)
    idx_h = sh[:, None] + torch.arange(kh)[None]      # [H, kh]
    idx_w = sw[:, None] + torch.arange(kw)[None]      # [W, kw]
    out = torch.empty_like(q)
    for d in range(D):
        d0 = int(sd[d])
        kk = k[:, d0:d0 + kd]                          # [B, kd, H, W, nh, hd]
        vv = v[:, d0:d0 + kd]
        # gather H windows then W windows -> [B, kd, H, kh, W, kw, nh, hd]
        kk = kk[:, :, idx_h][:, :, :, :, idx_w]
        vv = vv[:, :, idx_h][:, :, :, :, idx_w]
        kk = kk.permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B, H, W, nh, kd * kh * kw, hd)
        vv = vv.permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B, H, W, nh, kd * kh * kw, hd)
        s = torch.einsum("bhwnc,bhwnkc->bhwnk", q[:, d], kk) * scale
        p = torch.softmax(s, dim=-1)
        out[:, d] = torch.einsum("bhwnk,bhwnkc->bhwnc", p, vv)
    return out


def na3d_masked(q, k, v, kernel, scale: float | None = None):
    """Same operator restated as dense attention with a window mask (tiny shapes only)."""
    B, D, H, W, nh, hd = q.shape
    kd, kh, kw = kernel
    scale = hd ** -0.5 if scale is None else scale
    sd, sh, sw = window_starts(D, kd), window_starts(H, kh), window_starts(W, kw)

    def axis_mask(starts, length, kk):
        j = torch.arange(length)[None]
        return (j >= starts[:, None]) & (j < starts[:, None] + kk)   # [L(query), L(key)]

    md, mh, mw = axis_mask(sd, D, kd), axis_mask(sh, H, kh), axis_mask(sw, W, kw)
    mask = (md[:, None, None, :, None, None] & mh[None, :, None, None, :, None]
            & mw[None, None, :, None, None, :]).reshape(D * H * W, D * H * W)
    qf = q.reshape(B, D * H * W, nh, hd).permute(0, 2, 1, 3)
    kf = k.reshape(B, D * H * W, nh, hd).permute(0, 2, 1, 3)
    vf = v.reshape(B, D * H * W, nh, hd).permute(0, 2, 1, 3)
    s = (qf @ kf.transpose(-1, -2)) * scale
    s = s.masked_fill(~mask, float("-inf"))
    o = torch.softmax(s, dim=-1) @ vf
    return o.permute(0, 2, 1, 3).reshape(B, D, H, W, nh, hd)


def _round(t: torch.Tensor, emulate_bf16: bool) -> torch.Tensor:
    return t.bfloat16().float() if emulate_bf16 else t


def _weight(w: torch.Tensor, emulate_bf16: bool) -> torch.Tensor:
    return w.float().bfloat16().float() if emulate_bf16 else w.float()


# --------------------------------------------------------------------------- the block
def block_forward(x: torch.Tensor, params: dict, *, grid, num_heads: int, kernel,
                  rope_cos: torch.Tensor | None, rope_sin: torch.Tensor | None,
                  qk_norm: bool = False, gated: bool = False, emulate_bf16: bool = False,
                  return_intermediates: bool = False):
    """One backbone block.  x: [B, D*H*W, C] (tokens in d, h, w order).

    params: 'attn.qkv.weight' [3C,C], 'attn.qkv.bias' [3C], 'attn.proj.weight' [C,C],
    'attn.proj.bias', optional 'attn.gate_proj.weight/bias' [C,C], 'mlp.layers.0.weight'
    [4C,C], 'mlp.layers.0.bias', 'mlp.layers.2.weight' [C,4C], 'mlp.layers.2.bias'.

    emulate_bf16=True rounds weights and every stored activation to bf16 at the points where
    the GPU path stores bf16 (accumulation stays fp32) - the "fp32-accumulate agreement"
    comparison; False is the plain fp32 model the 2e-2 tolerance is stated against.
    """
    D, H, W = grid
    B, T, C = x.shape
    assert T == D * H * W
    hd = C // num_heads
    r = lambda t: _round(t, emulate_bf16)
    wt = lambda name: _weight(params[name], emulate_bf16)
    x = r(x.float())

    xn = r(F.layer_norm(x, (C,), eps=LN_EPS))
    qkv = F.linear(xn, wt("attn.qkv.weight"), params["attn.qkv.bias"].float())
    qkv = qkv.reshape(B, D, H * W, 3, num_heads, hd)
    q, k, v = qkv[:, :, :, 0], qkv[:, :, :, 1], qkv[:, :, :, 2]
    if qk_norm:
        q, k = rms_norm(q), rms_norm(k)
    if rope_cos is not None:
        q = apply_rope(q, rope_cos, rope_sin)
        k = apply_rope(k, rope_cos, rope_sin)
    q, k, v = r(q), r(k), r(v)
    shape6 = (B, D, H, W, num_heads, hd)
    o = na3d(q.reshape(shape6), k.reshape(shape6), v.reshape(shape6), kernel)
    o = r(o.reshape(B, T, C))
    if gated:
        g = F.linear(xn, wt("attn.gate_proj.weight"), params["attn.gate_proj.bias"].float())
        o = r(o * torch.sigmoid(g))
    x1 = r(x + F.linear(o, wt("attn.proj.weight"), params["attn.proj.bias"].float()))

    xn2 = r(F.layer_norm(x1, (C,), eps=LN_EPS))
    h = F.linear(xn2, wt("mlp.layers.0.weight"), params["mlp.layers.0.bias"].float())
    h = r(F.gelu(h, approximate="tanh"))
    y = r(x1 + F.linear(h, wt("mlp.layers.2.weight"), params["mlp.layers.2.bias"].float()))
    if return_intermediates:
        return y, {"xn": xn, "q": q.reshape(B, T, C), "k": k.reshape(B, T, C),
                   "v": v.reshape(B, T, C), "attn": o, "x1": x1, "h": h}
    return y


def init_block_params(C: int, mlp_ratio: float = 4.0, gated: bool = False, *, seed: int = 0,
                      scheme: str = "trunc_normal") -> dict:
    """Synthetic weights: trunc-normal(0.02) or Xavier-uniform Linear weights, zero biases
    replaced by small random biases so that the bias path is exercised."""
    g = torch.Generator().manual_seed(seed)
    hidden = int(C * mlp_ratio)

    def lin(n_out, n_in):
        w = torch.empty(n_out, n_in)
        if scheme == "xavier":
            bound = math.sqrt(6.0 / (n_in + n_out))
            w.uniform_(-bound, bound, generator=g)
        else:
            torch.nn.init.trunc_normal_(w, std=0.02, a=-0.04, b=0.04, generator=g)
        b = torch.empty(n_out).uniform_(-0.02, 0.02, generator=g)
        return w, b

    p = {}
    p["attn.qkv.weight"], p["attn.qkv.bias"] = lin(3 * C, C)
    p["attn.proj.weight"], p["attn.proj.bias"] = lin(C, C)
    if gated:
        p["attn.gate_proj.weight"], p["attn.gate_proj.bias"] = lin(C, C)
    p["mlp.layers.0.weight"], p["mlp.layers.0.bias"] = lin(hidden, C)
    p["mlp.layers.2.weight"], p["mlp.layers.2.bias"] = lin(C, hidden)
    return p


def block_flops_per_token(C: int, kernel, mlp_ratio: float = 4.0, gated: bool = False) -> float:
    """Algorithmic flop per token per block: 24 C^2 + 4 K C (+ 2 C^2 if gated) at ratio 4."""
    K = kernel[0] * kernel[1] * kernel[2]
    return 6 * C * C + 4 * K * C + 2 * C * C + 4 * mlp_ratio * C * C + (2 * C * C if gated else 0)


# --------------------------------------------------------------------------- whole backbone
def backbone_forward(x: torch.Tensor, state: dict, *, patch, num_heads: int, kernel, num_layers: int,
                     lat: torch.Tensor, lon: torch.Tensor, rope_mode: str = "stereographic",
                     rope_length_scale: float | None = None, rope_base: float = 100.0,
                     qk_norm: bool = False, gated: bool = False, concat_latitude: bool = True,
                     wind_channels=None, alt_depthwise: bool = False, emulate_bf16: bool = False,
                     dealias_filter=None):
    """Single-stage model: the wrapper's pre/post-processing (wind rotation, cos/sin(lat)
    concat: screamcast/strata_wrappers.py:206-249) around patch embed -> blocks -> final layer.

    x [B, C, D, H, W] fp32; lat/lon [B, H, W] radians; state: a `strata.*` state dict
    (parameter names of tests/regression_data/sweep1_*.param_order.txt).
    """
    from oracle import halo_oracle as ho
    B, _, D, H, W = x.shape
    pv, ph, pw = patch
    x = x.float()
    lat_lon = None
    if wind_channels is not None:
        u, v = wind_channels
        lat0, lon0 = ho.tile_center(lat.numpy(), lon.numpy())
        ul, vl = ho.forward_uv_to_tile(x[:, u].numpy(), x[:, v].numpy(), lat.numpy(), lon.numpy(),
                                       lat0, lon0)
        x = x.clone()
        x[:, u], x[:, v] = torch.from_numpy(ul), torch.from_numpy(vl)
        lat_lon = (lat0, lon0)
    if concat_latitude:
        le = lat[:, None, None].expand(B, 1, D, H, W)
        x = torch.cat([x, torch.cos(le), torch.sin(le)], dim=1)
    r = lambda t: _round(t, emulate_bf16)
    w = state["strata.patch_embed.proj.weight"].float()
    if dealias_filter is not None:
        t = dealiased_patch_embed(r(x), _weight(w, emulate_bf16),
                                  state["strata.patch_embed.proj.bias"], patch, dealias_filter)
    else:
        t = F.conv3d(r(x), _weight(w, emulate_bf16), state["strata.patch_embed.proj.bias"].float(),
                     stride=patch)
    C = t.shape[1]
    grid = (D // pv, H // ph, W // pw)
    t = r(t.flatten(2).transpose(1, 2))
    hd = C // num_heads
    if rope_mode == "stereographic":
        scale = rope_length_scale if rope_length_scale else default_rope_length_scale(1) * ph
        cos, sin = stereographic_rope_tables(lat, lon, hd, ph, scale, rope_base)
    elif rope_mode == "axial":
        cos, sin = axial_rope_tables(grid[1], grid[2], hd, rope_base)
    else:
        cos = sin = None
    kernel = (kernel,) * 3 if isinstance(kernel, int) else tuple(kernel)
    for i in range(num_layers):
        p = {k[len(f"strata.blocks.{i}."):]: v for k, v in state.items()
             if k.startswith(f"strata.blocks.{i}.")}
        k_i = (kernel[0], 1, 1) if (alt_depthwise and i % 2 == 1) else kernel
        t = block_forward(t, p, grid=grid, num_heads=num_heads, kernel=k_i, rope_cos=cos,
                          rope_sin=sin, qk_norm=qk_norm, gated=gated, emulate_bf16=emulate_bf16)
    y = F.layer_norm(t, (C,), eps=LN_EPS)
    y = F.linear(y, state["strata.final_layer.linear.weight"].float(),
                 state["strata.final_layer.linear.bias"].float())
    c_out = y.shape[-1] // (pv * ph * pw)
    d, h, wd = grid
    y = y.reshape(B, d, h, wd, pv, ph, pw, c_out).permute(0, 7, 1, 4, 2, 5, 3, 6)
    y = y.reshape(B, c_out, D, H, W)
    if wind_channels is not None:
        u, v = wind_channels
        ug, vg = ho.inverse_tile_to_uv(y[:, u].numpy(), y[:, v].numpy(), lat.numpy(), lon.numpy(),
                                       *lat_lon)
        y = y.clone()
        y[:, u], y[:, v] = torch.from_numpy(ug), torch.from_numpy(vg)
    return y


def dealiased_patch_embed(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, patch,
                          resample_filter) -> torch.Tensor:
    """De-aliased patch embedding (screamcast/dealias.py:116-143): the patch convolution at
    stride 1 on the unpadded input, replicate padding of ITS OUTPUT by (k-1)//2 before and the
    rest after on every decimated axis, then a normalised separable low-pass applied per channel
    at stride = patch. Axes with patch 1 are not filtered. x [B, C, D, H, W] -> [B, E, D', H', W']."""
    pd, ph, pw = patch
    s1 = F.conv3d(x.float(), weight.float(), bias.float())
    f = torch.as_tensor(resample_filter, dtype=torch.float32)
    taps = [f / f.sum() if p > 1 else torch.ones(1) for p in (pd, ph, pw)]
    kd, kh, kw = (len(t) for t in taps)
    pads = []
    for k in (kw, kh, kd):                      # F.pad lists the last axis first
        pads += [(k - 1) // 2, (k - 1) - (k - 1) // 2]
    if max(kd, kh, kw) > 1:
        s1 = F.pad(s1, pads, mode="replicate")
    f3 = taps[0][:, None, None] * taps[1][None, :, None] * taps[2][None, None, :]
    E = s1.shape[1]
    return F.conv3d(s1, f3[None, None].repeat(E, 1, 1, 1, 1), groups=E, stride=(pd, ph, pw))


# --------------------------------------------------------------------------- per-block halo
def tiled_block_forward(x_all: torch.Tensor, params: dict, *, face: int, tile: int, halo: int,
                        depth: int, num_heads: int, kernel, lat_deg, lon_deg,
                        rope_base: float = 100.0, length_scale: float | None = None,
                        qk_norm: bool = False, gated: bool = False, return_attention: bool = False):
    """One block over ALL tiles of a cubed sphere with a K/V halo exchange inside the block.

    x_all [G, depth*tile*tile, C] (global tile order); lat_deg / lon_deg [G, tile, tile].
    Only interior tokens are queries. Every tile sees its neighbours' pre-RoPE keys and values
    through the copy-halo maps (halo_oracle), and rotates ALL keys of its padded plane in its
    own stereographic frame (centre = spherical centroid of its interior). Returns [G, ...].
    """
    import numpy as np
    from oracle import halo_oracle as ho
    G, Ttok, C = x_all.shape
    T, h, P, D = tile, halo, tile + 2 * halo, depth
    hd = C // num_heads
    scale = length_scale or default_rope_length_scale(1)
    x = x_all.float()
    xn = F.layer_norm(x, (C,), eps=LN_EPS)
    qkv = F.linear(xn, params["attn.qkv.weight"].float(), params["attn.qkv.bias"].float())
    qkv = qkv.reshape(G, D, T, T, 3, num_heads, hd)
    q, k, v = qkv[..., 0, :, :], qkv[..., 1, :, :], qkv[..., 2, :, :]
    if qk_norm:
        q, k = rms_norm(q), rms_norm(k)
    topo = ho.TileTopology(1, 0, face, tile, halo)

    def pad(t):   # [G, D, T, T, nh, hd] -> [G, D, P, P, nh, hd] via the copy halo
        lead = t.permute(1, 4, 5, 0, 2, 3).numpy()                       # [D, nh, hd, G, T, T]
        return torch.from_numpy(ho.padded_local_tiles(lead, topo)).permute(3, 0, 4, 5, 1, 2)
    kp, vp = pad(k), pad(v)
    # receiver-frame coordinates of every padded cell
    la, lo = np.radians(np.asarray(lat_deg)), np.radians(np.asarray(lon_deg))
    xyz = np.stack([np.cos(la) * np.cos(lo), np.cos(la) * np.sin(lo), np.sin(la)])
    pxyz = ho.padded_local_tiles(xyz, topo)                              # [3, G, P, P]
    plat = torch.from_numpy(np.arctan2(pxyz[2], np.hypot(pxyz[0], pxyz[1])))
    plon = torch.from_numpy(np.arctan2(pxyz[1], pxyz[0]))
    lat0, lon0 = spherical_centroid(torch.from_numpy(la), torch.from_numpy(lo))
    px, py = stereographic_projection(plat, plon, lat0, lon0)
    cos, sin = rope_tables_from_coords((px / scale).flatten(1), (py / scale).flatten(1), hd, rope_base)
    kp = apply_rope(kp.reshape(G, D, P * P, num_heads, hd), cos, sin).reshape(G, D, P, P, num_heads, hd)
    qp = torch.zeros(G, D, P, P, num_heads, hd)
    qp[:, :, h:h + T, h:h + T] = q
    qp = apply_rope(qp.reshape(G, D, P * P, num_heads, hd), cos, sin).reshape(G, D, P, P, num_heads, hd)
    o = na3d(qp, kp, vp, kernel)[:, :, h:h + T, h:h + T].reshape(G, Ttok, C)
    if return_attention:
        return o
    if gated:
        g = F.linear(xn, params["attn.gate_proj.weight"].float(), params["attn.gate_proj.bias"].float())
        o = o * torch.sigmoid(g)
    x1 = x + F.linear(o, params["attn.proj.weight"].float(), params["attn.proj.bias"].float())
    hmid = F.gelu(F.linear(F.layer_norm(x1, (C,), eps=LN_EPS), params["mlp.layers.0.weight"].float(),
                           params["mlp.layers.0.bias"].float()), approximate="tanh")
    return x1 + F.linear(hmid, params["mlp.layers.2.weight"].float(), params["mlp.layers.2.bias"].float())
