"""TEST INFRASTRUCTURE ONLY - CPU restatement of the two-stage model's pixel stage.

PARITY UNPINNED. The pixel stage (`Strata.pixel_patch_embed`, `pixel_blocks[i]`,
`pixel_final_layer`) lives in physicsnemo (`physicsnemo.experimental.models.strata`,
pinned by the reference's pyproject as a git dependency), which is absent from the reference
tree, and the reference's own tests for it are shape-only (tests/test_dit_3d_pixel.py:28-205).
What the reference itself fixes, and what this file follows:

  * parameter names and order: tests/regression_data/pixeldit_*.param_order.txt:243-294
    (pixel_patch_embed.proj, pixel_blocks.{i}.attn.{qkv,proj}, .mlp.layers.{0,2},
    .adaln_bilinear_dw_conv, .adaln_bilinear_dw_proj, pixel_final_layer.linear; no backbone
    final layer in the two-stage model);
  * the conditioning is adaLN-zero - "shift=0 / scale=1 / gate=0 at the start ... blocks start
    as identity" (train.py:279-299) - i.e. x + gate * f(LN(x) * (1 + scale) + shift);
  * "bilinear_dw" mode = bilinear upsample (H and W only, patch_size_vert must be 1:
    screamcast/strata_wrappers.py:471-476) -> depthwise conv -> GELU -> projection;
  * every GELU is the tanh form (screamcast/strata_wrappers.py:76-100, 509);
  * the pixel patch is 1x1x1 (tests/test_dit_3d_pixel.py:199-200), heads = embed_dim // 64,
    RoPE off in the production pixel config (tests/test_dit_3d_pixel.py:229-279); when on, the
    backbone's table construction at patch 1 (length scale = the per-pixel base).

Assumed (listed in oracle/ASSUMPTIONS.md): the six modulation chunks are ordered
(shift, scale, gate) for attention then (shift, scale, gate) for the MLP; the depthwise kernel
is 5x5 with zero padding over (H, W); the upsample uses half-pixel centres
(align_corners=False); the projection is one Linear(C_backbone, 6 * C_pixel) applied per pixel.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from oracle.block_oracle import (LN_EPS, _round, _weight, apply_rope, axial_rope_tables, block_forward,
                                 default_rope_length_scale, na3d, rms_norm,
                                 stereographic_rope_tables)


def adaln_cond(tokens: torch.Tensor, w_dw: torch.Tensor, b_dw, factor: int) -> torch.Tensor:
    """tokens [B, D, h, w, Cb] -> GELU(dwconv(upsample)) rows [B, D*H*W, Cb] (fp32)."""
    B, D, h, w, Cb = tokens.shape
    ks = w_dw.shape[-1]
    t = tokens.float().permute(0, 1, 4, 2, 3).reshape(B * D, Cb, h, w)
    u = F.interpolate(t, scale_factor=factor, mode="bilinear", align_corners=False)
    c = F.conv2d(u, w_dw.float().reshape(Cb, 1, ks, ks), None if b_dw is None else b_dw.float(),
                 padding=ks // 2, groups=Cb)
    g = F.gelu(c, approximate="tanh")
    return g.permute(0, 2, 3, 1).reshape(B, D * h * factor * w * factor, Cb)


def modulation(cond_rows: torch.Tensor, params: dict, emulate_bf16: bool) -> torch.Tensor:
    """[B, T, Cb] conditioning rows -> [B, T, 6C] modulation (stored bf16 on the GPU path)."""
    r = lambda t: _round(t, emulate_bf16)
    return r(F.linear(r(cond_rows), _weight(params["adaln_bilinear_dw_proj.weight"], emulate_bf16),
                      params["adaln_bilinear_dw_proj.bias"].float()))


def modulation_pixel_proj(tokens: torch.Tensor, params: dict, patch, emulate_bf16: bool):
    """"pixel_proj" mode: tokens [B, d, h, w, Cb] -> Linear(SiLU(token)) = the modulation of the
    pv x ph x pw pixels under each token, laid out (v, y, x, 6C) -> [B, pixels, 6C]."""
    r = lambda t: _round(t, emulate_bf16)
    B, d, h, w, Cb = tokens.shape
    pv, ph, pw = patch
    m = r(F.linear(r(F.silu(tokens.float())), _weight(params["adaln_pixel_proj.1.weight"], emulate_bf16),
                   params["adaln_pixel_proj.1.bias"].float()))
    m = m.reshape(B, d, h, w, pv, ph, pw, -1).permute(0, 1, 4, 2, 5, 3, 6, 7)
    return m.reshape(B, d * pv * h * ph * w * pw, -1)


def pixel_block_forward(x: torch.Tensor, mod, params: dict, *, grid, num_heads: int, kernel,
                        qk_norm: bool = False, emulate_bf16: bool = False, rope_cos=None,
                        rope_sin=None) -> torch.Tensor:
    """One pixel block. x [B, T, C]; mod [B, T, 6C] or None (a block without AdaLN parameters
    runs as a plain pre-norm block); rope_cos / rope_sin [B or 1, H*W, hd/2] or None."""
    D, H, W = grid
    B, T, C = x.shape
    hd = C // num_heads
    r = lambda t: _round(t, emulate_bf16)
    wt = lambda name: _weight(params[name], emulate_bf16)
    x = r(x.float())
    if mod is None:
        zero, one = torch.zeros(()), torch.ones(())
        sh1 = sc1 = sh2 = sc2 = zero
        g1 = g2 = one
    else:
        sh1, sc1, g1, sh2, sc2, g2 = mod.float().chunk(6, dim=-1)
    xn = r(F.layer_norm(x, (C,), eps=LN_EPS) * (1 + sc1) + sh1)
    qkv = F.linear(xn, wt("attn.qkv.weight"), params["attn.qkv.bias"].float())
    if rope_cos is None:
        # GPU path: bias GEMM stores bf16, the q/k norm then runs in place on the stored rows
        qkv = r(qkv).reshape(B, T, 3, num_heads, hd)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        if qk_norm:
            q, k = r(rms_norm(q)), r(rms_norm(k))
    else:
        # GPU path: norm and rotation in the GEMM epilogue, one rounding at the store
        qkv = qkv.reshape(B, D, H * W, 3, num_heads, hd)
        q, k, v = qkv[:, :, :, 0], qkv[:, :, :, 1], qkv[:, :, :, 2]
        if qk_norm:
            q, k = rms_norm(q), rms_norm(k)
        q, k = apply_rope(q, rope_cos, rope_sin), apply_rope(k, rope_cos, rope_sin)
        q, k, v = r(q), r(k), r(v)
    shape6 = (B, D, H, W, num_heads, hd)
    o = r(na3d(q.reshape(shape6), k.reshape(shape6), v.reshape(shape6), kernel).reshape(B, T, C))
    y = r(F.linear(o, wt("attn.proj.weight"), params["attn.proj.bias"].float()))
    x1 = r(x + g1 * y)
    xn2 = r(F.layer_norm(x1, (C,), eps=LN_EPS) * (1 + sc2) + sh2)
    h = r(F.gelu(F.linear(xn2, wt("mlp.layers.0.weight"), params["mlp.layers.0.bias"].float()),
                 approximate="tanh"))
    y2 = r(F.linear(h, wt("mlp.layers.2.weight"), params["mlp.layers.2.bias"].float()))
    return r(x1 + g2 * y2)


def _sub(state: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in state.items() if k.startswith(prefix)}


def two_stage_forward(x: torch.Tensor, state: dict, *, patch, num_heads: int, kernel,
                      num_layers: int, num_heads_pixel: int, kernel_pixel, num_layers_pixel: int,
                      lat: torch.Tensor, lon: torch.Tensor, rope_length_scale: float | None = None,
                      rope_base: float = 100.0, qk_norm: bool = False, gated: bool = False,
                      qk_norm_pixel: bool = False, concat_latitude: bool = True, wind_channels=None,
                      alt_depthwise: bool = False, emulate_bf16: bool = False,
                      rope_mode_pixel: str = "none"):
    """Two-stage model (screamcast/strata_wrappers.py:418-533): the wrapper's pre-processing,
    backbone patch embed + blocks (stereographic RoPE), then the pixel stage on the same
    pre-processed fields conditioned on the backbone tokens, and the inverse wind rotation."""
    from oracle import halo_oracle as ho
    B, _, D, H, W = x.shape
    pv, ph, pw = patch
    assert ph == pw
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
    xr = r(x)
    # ---- stage 1: backbone tokens
    t = F.conv3d(xr, _weight(state["strata.backbone.patch_embed.proj.weight"], emulate_bf16),
                 state["strata.backbone.patch_embed.proj.bias"].float(), stride=patch)
    Cb = t.shape[1]
    grid = (D // pv, H // ph, W // pw)
    t = r(t.flatten(2).transpose(1, 2))
    scale = rope_length_scale if rope_length_scale else default_rope_length_scale(1) * ph
    cos, sin = stereographic_rope_tables(lat, lon, Cb // num_heads, ph, scale, rope_base)
    kernel = (kernel,) * 3 if isinstance(kernel, int) else tuple(kernel)
    for i in range(num_layers):
        k_i = (kernel[0], 1, 1) if (alt_depthwise and i % 2 == 1) else kernel
        t = block_forward(t, _sub(state, f"strata.backbone.blocks.{i}."), grid=grid,
                          num_heads=num_heads, kernel=k_i, rope_cos=cos, rope_sin=sin,
                          qk_norm=qk_norm, gated=gated, emulate_bf16=emulate_bf16)
    s = t.reshape(B, *grid, Cb)
    # ---- stage 2: pixel tokens
    p = F.conv3d(xr, _weight(state["strata.pixel_patch_embed.proj.weight"], emulate_bf16),
                 state["strata.pixel_patch_embed.proj.bias"].float())
    C = p.shape[1]
    p = r(p.flatten(2).transpose(1, 2))
    kernel_pixel = (kernel_pixel,) * 3 if isinstance(kernel_pixel, int) else tuple(kernel_pixel)
    # pixel-stage RoPE: same tables as the backbone's at patch 1 and the per-pixel length scale
    # (screamcast/strata_wrappers.py:499-504: rope_base_pixel=100, scale = the resolved base)
    pcos = psin = None
    if rope_mode_pixel == "stereographic":
        base = rope_length_scale / ph if rope_length_scale else default_rope_length_scale(1)
        pcos, psin = stereographic_rope_tables(lat, lon, C // num_heads_pixel, 1, base, rope_base)
    elif rope_mode_pixel == "axial":
        pcos, psin = axial_rope_tables(H, W, C // num_heads_pixel, rope_base)
    for i in range(num_layers_pixel):
        bp = _sub(state, f"strata.pixel_blocks.{i}.")
        mod = None
        if "adaln_pixel_proj.1.weight" in bp:
            mod = modulation_pixel_proj(s, bp, patch, emulate_bf16)
        elif "adaln_bilinear_dw_proj.weight" in bp:
            cond = adaln_cond(s, bp["adaln_bilinear_dw_conv.weight"].float().squeeze(1).squeeze(1),
                              bp["adaln_bilinear_dw_conv.bias"], ph)
            mod = modulation(cond, bp, emulate_bf16)
        p = pixel_block_forward(p, mod, bp, grid=(D, H, W), num_heads=num_heads_pixel,
                                kernel=kernel_pixel, qk_norm=qk_norm_pixel,
                                emulate_bf16=emulate_bf16, rope_cos=pcos, rope_sin=psin)
    y = r(F.layer_norm(p, (C,), eps=LN_EPS))
    y = F.linear(y, _weight(state["strata.pixel_final_layer.linear.weight"], emulate_bf16),
                 state["strata.pixel_final_layer.linear.bias"].float())
    c_out = y.shape[-1]
    y = r(y).reshape(B, D, H, W, c_out).permute(0, 4, 1, 2, 3).contiguous()
    if wind_channels is not None:
        u, v = wind_channels
        ug, vg = ho.inverse_tile_to_uv(y[:, u].numpy(), y[:, v].numpy(), lat.numpy(), lon.numpy(),
                                       *lat_lon)
        y = y.clone()
        y[:, u], y[:, v] = torch.from_numpy(ug), torch.from_numpy(vg)
    return y
