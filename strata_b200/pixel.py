"""Two-stage Strata: the backbone's tokens condition a stack of AdaLN pixel blocks that run
at full pixel resolution (patch 1x1x1, 128 channels in production).

Module tree and parameter order follow the reference's two-stage manifest
(tests/regression_data/pixeldit_*.param_order.txt): `backbone.*` (no final layer),
`pixel_patch_embed.proj`, `pixel_blocks.{i}.attn.{qkv,proj[,gate_proj]}`,
`pixel_blocks.{i}.mlp.layers.{0,2}`, `pixel_blocks.{i}.adaln_bilinear_dw_{conv,proj}`,
`pixel_final_layer.linear`; constructor arguments are the ones the reference wrapper passes
(screamcast/strata_wrappers.py:480-508). The projections zero-initialise (adaLN-zero,
train.py:279-299), so a fresh block is the identity.

Everything on the token path runs through libstrata_b200.so: the tcgen05 GEMM, the 3-D
neighbourhood attention kernel, the fused LayerNorm / modulate / gated-residual row kernel and
the bilinear + depthwise-conv + GELU conditioning kernel. There is no PyTorch fallback.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops, rope
from .ops import EPI_BIAS, EPI_GATE, EPI_GELU
from .strata import FinalLayer, Mlp, NeighborhoodAttention3D, PatchEmbed3D, StrataTransformer3D, _triple

# pixel rows whose conditioning matrix [rows, C_backbone] is materialised at a time
_COND_CHUNK_ROWS = 1 << 18


class StrataPixel3DBlock(nn.Module):
    """x += g1 * proj(NA3D(qkv(LN(x) * (1 + s1) + b1)));  x += g2 * fc2(gelu(fc1(LN(x) * (1 + s2) + b2)))
    with (b1, s1, g1, b2, s2, g2) = chunks of proj6(GELU(dwconv(bilinear_up(backbone tokens)))).
    In the "pixel_proj" mode the chunks come from Linear(SiLU(backbone token)) instead, one set per
    pixel of the token's patch. A block built without AdaLN parameters (first_block_only_adaln)
    runs unmodulated."""

    def __init__(self, dim: int, num_heads: int, mlp_ratio: float, qk_norm: bool, gated: bool,
                 kernel, cond_dim: int, adaln: bool, dw_kernel: int = 5,
                 adaln_mode: str = "bilinear_dw", patch=(1, 1, 1)):
        super().__init__()
        self.dim, self.num_heads, self.qk_norm = dim, num_heads, qk_norm
        self.kernel = _triple(kernel)
        self.patch = _triple(patch)
        self.attn = NeighborhoodAttention3D(dim, num_heads, True, gated)
        self.mlp = Mlp(dim, int(dim * mlp_ratio))
        if adaln and adaln_mode == "pixel_proj":
            # every backbone token emits the modulation of the pv x ph x pw pixels it covers
            pv, ph, pw = self.patch
            self.adaln_pixel_proj = nn.Sequential(nn.SiLU(),
                                                  nn.Linear(cond_dim, pv * ph * pw * 6 * dim))
            nn.init.zeros_(self.adaln_pixel_proj[-1].weight)
            nn.init.zeros_(self.adaln_pixel_proj[-1].bias)
        elif adaln:
            self.adaln_bilinear_dw_conv = nn.Conv3d(cond_dim, cond_dim, (1, dw_kernel, dw_kernel),
                                                    padding=(0, dw_kernel // 2, dw_kernel // 2),
                                                    groups=cond_dim)
            self.adaln_bilinear_dw_proj = nn.Linear(cond_dim, 6 * dim)
            nn.init.zeros_(self.adaln_bilinear_dw_proj.weight)
            nn.init.zeros_(self.adaln_bilinear_dw_proj.bias)
        self._cache = None
        self._key = None

    @property
    def has_adaln(self) -> bool:
        return hasattr(self, "adaln_bilinear_dw_proj") or hasattr(self, "adaln_pixel_proj")

    def device_weights(self) -> dict:
        key = tuple((p.data_ptr(), p._version, p.device) for p in self.parameters())
        if self._cache is not None and key == self._key:
            return self._cache
        w = lambda lin: lin.weight.detach().to(torch.bfloat16).contiguous()
        b = lambda lin: None if lin.bias is None else lin.bias.detach().float().contiguous()
        c = {"w_qkv": w(self.attn.qkv), "b_qkv": b(self.attn.qkv),
             "w_proj": w(self.attn.proj), "b_proj": b(self.attn.proj),
             "w_fc1": w(self.mlp.layers[0]), "b_fc1": b(self.mlp.layers[0]),
             "w_fc2": w(self.mlp.layers[2]), "b_fc2": b(self.mlp.layers[2])}
        if hasattr(self.attn, "gate_proj"):
            c["w_gate"], c["b_gate"] = w(self.attn.gate_proj), b(self.attn.gate_proj)
        if hasattr(self, "adaln_pixel_proj"):
            c["w_pp"], c["b_pp"] = w(self.adaln_pixel_proj[-1]), b(self.adaln_pixel_proj[-1])
        elif self.has_adaln:
            conv = self.adaln_bilinear_dw_conv
            ks = conv.kernel_size[-1]
            c["w_dw"] = conv.weight.detach().float().reshape(conv.out_channels, ks, ks).contiguous()
            c["b_dw"] = b(conv)
            c["w_mod"], c["b_mod"] = w(self.adaln_bilinear_dw_proj), b(self.adaln_bilinear_dw_proj)
        self._cache, self._key = c, key
        return c

    def modulation(self, backbone_tokens: torch.Tensor, factor: int) -> torch.Tensor | None:
        """backbone tokens bf16 [B, D, h, w, Cb] -> bf16 [pixels, 6 * dim]."""
        if not self.has_adaln:
            return None
        c = self.device_weights()
        B, D, h, w, Cb = backbone_tokens.shape
        if "w_pp" in c:
            pv, ph, pw = self.patch
            a = torch.nn.functional.silu(backbone_tokens).view(-1, Cb)
            m = ops.linear(a, c["w_pp"], c["b_pp"], EPI_BIAS)
            m = m.view(B, D, h, w, pv, ph, pw, 6 * self.dim).permute(0, 1, 4, 2, 5, 3, 6, 7)
            return m.reshape(B * D * pv * h * ph * w * pw, 6 * self.dim)   # one strided copy
        pixels = B * D * h * factor * w * factor
        mod = torch.empty((pixels, 6 * self.dim), dtype=torch.bfloat16, device=backbone_tokens.device)
        # whole groups of `factor` image rows per chunk, so that no cell straddles two chunks
        band = factor * w * factor
        chunk = min(pixels, max(band, _COND_CHUNK_ROWS // band * band))
        buf = torch.empty((chunk, Cb), dtype=torch.bfloat16, device=backbone_tokens.device)
        for r0 in range(0, pixels, chunk):
            n = min(chunk, pixels - r0)
            ops.adaln_cond(backbone_tokens, c["w_dw"], c["b_dw"], factor, r0, n, out=buf[:n])
            ops.linear(buf[:n], c["w_mod"], c["b_mod"], EPI_BIAS, out=mod[r0:r0 + n])
        return mod

    def forward(self, x: torch.Tensor, grid, mod: torch.Tensor | None, n_tiles: int,
                rope_cs: torch.Tensor | None = None) -> torch.Tensor:
        """x: bf16 rows [n_tiles * D*H*W, dim], updated in place and returned. rope_cs: packed
        half (cos, sin) table [n_tiles, H*W, 32, 2] or None."""
        if not (isinstance(self.mlp.layers[1], nn.GELU) and self.mlp.layers[1].approximate == "tanh"):
            raise RuntimeError("the fused MLP kernel implements the tanh GELU; this block's Mlp "
                               "still holds an exact GELU (the wrapper's tanh swap did not run)")
        C = self.dim
        c = self.device_weights()
        D, H, W = grid
        sl = (lambda i: mod[:, i * C:(i + 1) * C]) if mod is not None else (lambda i: None)
        xn = ops.adaln_rows(x, shift=sl(0), scale=sl(1))
        if rope_cs is not None or self.qk_norm:
            # rotation and / or the q/k norm in the GEMM epilogue, as in the backbone blocks
            qkv = ops.qkv_rope(xn, c["w_qkv"], c["b_qkv"], C // self.num_heads, None, None,
                               D * H * W, H * W, qk_norm=self.qk_norm, rope_cs=rope_cs)
        else:
            qkv = ops.linear(xn, c["w_qkv"], c["b_qkv"])
        q6 = qkv.view(n_tiles, D, H, W, 3, self.num_heads, C // self.num_heads)
        attn = ops.na3d(q6[:, :, :, :, 0], q6[:, :, :, :, 1], q6[:, :, :, :, 2], self.kernel)
        attn = attn.view(-1, C)
        if "w_gate" in c:
            attn = ops.linear(xn, c["w_gate"], c["b_gate"], EPI_GATE, aux=attn, out=attn)
        y = ops.linear(attn, c["w_proj"], c["b_proj"])
        xn2 = ops.adaln_rows(x, y=y, gate=sl(2), shift=sl(3), scale=sl(4))
        h = ops.linear(xn2, c["w_fc1"], c["b_fc1"], EPI_GELU)
        y2 = ops.linear(h, c["w_fc2"], c["b_fc2"])
        ops.adaln_rows(x, y=y2, gate=sl(5), norm=False)
        return x


class Strata(nn.Module):
    """Backbone + pixel stage (the module the reference composes under `self.strata`,
    screamcast/strata_wrappers.py:480-509)."""

    def __init__(self, *, backbone_config: dict, embed_dim_pixel: int = 128,
                 num_layers_pixel: int = 4, num_heads_pixel: int | None = None,
                 mlp_ratio_pixel: float = 4.0, attn_kernel_pixel=3,
                 gated_attention_pixel: bool = False, qk_norm_pixel: bool = False,
                 qk_norm_affine_pixel: bool = False, na3d_backend_pixel: str | None = None,
                 adaln_mode: str = "pixel_proj", first_block_only_adaln: bool = False,
                 use_chunked_depthwise_conv: bool = True, rope_mode_pixel: str = "none",
                 rope_base_pixel: float = 100.0, rope_length_scale_pixel: float = 1.0,
                 bf16_mixed_pixel: bool = False, activation_checkpointing_pixel: bool | float = False,
                 adaln_dw_kernel: int = 5):
        super().__init__()
        if adaln_mode not in ("bilinear_dw", "pixel_proj"):
            raise ValueError(f"unknown adaln_mode {adaln_mode!r}")
        if rope_mode_pixel not in ("none", "axial", "stereographic"):
            raise ValueError(f"unknown rope_mode_pixel {rope_mode_pixel!r}")
        if qk_norm_affine_pixel:
            raise ValueError("qk_norm_affine_pixel=True is not supported")
        self.backbone = StrataTransformer3D(**backbone_config)
        self.backbone.final_layer = None     # the two-stage model has no backbone output head
        pv, ph, pw = self.backbone.patch_size
        if adaln_mode == "bilinear_dw" and (pv != 1 or ph != pw):
            raise ValueError("the bilinear_dw AdaLN needs patch_size_vert == 1 and square patches")
        heads = num_heads_pixel if num_heads_pixel is not None else max(embed_dim_pixel // 64, 1)
        if embed_dim_pixel % heads or embed_dim_pixel // heads != 64:
            raise ValueError("head_dim must be 64 for the sm_100a attention kernel")
        self.in_channels, self.out_channels = self.backbone.in_channels, self.backbone.out_channels
        self.depth, self.height, self.width = self.backbone.depth, self.backbone.height, self.backbone.width
        self.embed_dim_pixel, self.num_heads_pixel = embed_dim_pixel, heads
        self.head_dim_pixel = embed_dim_pixel // heads
        self.adaln_mode, self.rope_mode_pixel = adaln_mode, rope_mode_pixel
        self.rope_base_pixel, self.rope_length_scale_pixel = rope_base_pixel, rope_length_scale_pixel
        self.use_chunked_depthwise_conv = use_chunked_depthwise_conv   # one chunked kernel here
        self.na3d_backend_pixel = na3d_backend_pixel
        self.bf16_mixed_pixel = bf16_mixed_pixel
        self._activation_checkpointing_ratio_pixel = float(activation_checkpointing_pixel)
        self.pixel_patch_embed = PatchEmbed3D(self.in_channels, embed_dim_pixel, (1, 1, 1))
        self.pixel_blocks = nn.ModuleList([
            StrataPixel3DBlock(embed_dim_pixel, heads, mlp_ratio_pixel, qk_norm_pixel,
                               gated_attention_pixel, attn_kernel_pixel, self.backbone.embed_dim,
                               adaln=(i == 0 or not first_block_only_adaln), dw_kernel=adaln_dw_kernel,
                               adaln_mode=adaln_mode, patch=self.backbone.patch_size)
            for i in range(num_layers_pixel)])
        self.pixel_final_layer = FinalLayer(embed_dim_pixel, self.out_channels)
        if rope_mode_pixel == "axial":
            self._build_axial_rope_pixel()

    def _build_axial_rope_pixel(self, device=None) -> None:
        """Non-persistent buffers `_rope_cos_pixel` / `_rope_sin_pixel` [D*H*W, head_dim/2] for the
        axial mode (one row per pixel token; the reference's wrapper rebuilds them in
        set_tile_size, screamcast/strata_wrappers.py:634-645)."""
        cos, sin = rope.axial_rope_tables(self.height, self.width, self.head_dim_pixel,
                                          self.rope_base_pixel, device=device)
        self.register_buffer("_rope_cos_pixel", cos[0].repeat(self.depth, 1), persistent=False)
        self.register_buffer("_rope_sin_pixel", sin[0].repeat(self.depth, 1), persistent=False)

    def rope_tables_pixel(self, pos: torch.Tensor | None, n_tiles: int, grid_px):
        """Packed half (cos, sin) table [n_tiles, H*W, head_dim/2, 2] of the pixel tokens, or None."""
        D, H, W = grid_px
        if self.rope_mode_pixel == "none":
            return None
        if self.rope_mode_pixel == "axial":
            hw = H * W
            if self._rope_cos_pixel.shape[0] != D * hw:
                raise ValueError(f"axial pixel RoPE tables were built for {self._rope_cos_pixel.shape[0]} "
                                 f"tokens, the input has {D * hw}; call set_tile_size first")
            cos = self._rope_cos_pixel[:hw].expand(n_tiles, -1, -1).contiguous()
            sin = self._rope_sin_pixel[:hw].expand(n_tiles, -1, -1).contiguous()
        else:
            if pos is None:
                raise ValueError("stereographic RoPE needs pos=[B, 2, H, W] (lat, lon)")
            cos, sin = rope.stereographic_rope_tables(pos, self.head_dim_pixel, 1,
                                                      self.rope_length_scale_pixel,
                                                      self.rope_base_pixel)
        return rope.pack_rope_tables(cos, sin)

    def pixel_stage(self, pixel_tokens: torch.Tensor, backbone_tokens: torch.Tensor, grid_px,
                    rope_cs: torch.Tensor | None = None):
        """pixel_tokens bf16 [B, D*H*W, C] (modified in place), backbone_tokens bf16
        [B, D, h, w, Cb] -> pixel tokens after the blocks."""
        B = pixel_tokens.shape[0]
        factor = self.backbone.patch_size[1]
        x = pixel_tokens.view(-1, self.embed_dim_pixel)
        for blk in self.pixel_blocks:
            mod = blk.modulation(backbone_tokens, factor)
            blk(x, grid_px, mod, B, rope_cs)
            del mod
        return pixel_tokens

    def forward_fused(self, x: torch.Tensor, pos: torch.Tensor | None, *, lat=None, lon=None,
                      lat0=None, lon0=None, wind=None, concat_lat: bool = False) -> torch.Tensor:
        """Raw fields [B, C_raw, D, H, W] fp32 in, fields [B, C_out, D, H, W] fp32 out; the wind
        rotation, latitude channels and patch gathering are one kernel per stage on the way in,
        the un-patchify and inverse rotation one kernel on the way out."""
        bb = self.backbone
        B, _, D, H, W = x.shape
        grid = bb.token_grid(D, H, W)
        tokens = bb.embed_fused(x, lat, lon, lat0, lon0, wind, concat_lat)
        cos, sin = bb.rope_tables(pos, B, grid)
        tokens = bb.forward_tokens(tokens, grid, cos, sin)
        _, _, _, Kpp = self.pixel_patch_embed._gemm_weights()
        ap = ops.preprocess_patches(x, lat, lon, lat0, lon0, wind=wind, concat_lat=concat_lat,
                                    patch=(1, 1, 1), k_pad=Kpp)
        px = self.pixel_patch_embed.tokens_from_patches(ap, B)
        del ap
        px = self.pixel_stage(px, tokens.view(B, *grid, bb.embed_dim), (D, H, W),
                              self.rope_tables_pixel(pos, B, (D, H, W)))
        y, _ = self.pixel_final_layer.matrix_bf16(px)
        return ops.postprocess_fields(y, (B, self.out_channels, D, H, W), lat, lon, lat0, lon0,
                                      wind=wind, patch=(1, 1, 1))
