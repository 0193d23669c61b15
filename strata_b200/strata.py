"""StrataTransformer3D — the backbone the reference composes under `self.strata`
(screamcast/strata_wrappers.py:314-341), rebuilt on the sm_100a kernels of this package.

The module tree, parameter names, shapes and order follow the reference's parameter
manifest (tests/regression_data/sweep1_*.param_order.txt):

    patch_embed.proj.{weight,bias}                 Conv3d, kernel = stride = patch_size
    blocks.{i}.attn.qkv.{weight,bias}              Linear(C, 3C)
    blocks.{i}.attn.proj.{weight,bias}             Linear(C, C)
    blocks.{i}.attn.gate_proj.{weight,bias}        Linear(C, C), only if gated_attention
    blocks.{i}.mlp.layers.0.{weight,bias}          Linear(C, ratio*C)
    blocks.{i}.mlp.layers.2.{weight,bias}          Linear(ratio*C, C)
    final_layer.linear.{weight,bias}               Linear(C, pv*ph*ph*out_channels)

so checkpoints keyed `strata.*` load unchanged. The blocks run in bf16 through
libstrata_b200.so (fused QKV+RoPE GEMM, 3-D neighbourhood attention, GELU / residual GEMM
epilogues); there is no PyTorch fallback for them. The patch embedding (one strided bf16 copy
of the patches, or the fused pre-processing kernel) and the final projection (LayerNorm kernel)
feed the same tcgen05 GEMM. The one place foreign code runs is a `patch_embed` module that a
caller has assigned in place of the two this package provides (the reference leaves that
attribute assignable): it is the caller's module and is executed as given.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops, rope


def _triple(v):
    return (int(v),) * 3 if isinstance(v, int) else tuple(int(t) for t in v)


class PatchEmbed3D(nn.Module):
    """[B, C_in, D, H, W] -> tokens [B, D'*H'*W', embed_dim] (d, h, w order)."""

    def __init__(self, in_chans: int, embed_dim: int, patch_size):
        super().__init__()
        self.patch_size = _triple(patch_size)
        self.proj = nn.Conv3d(in_chans, embed_dim, kernel_size=self.patch_size,
                              stride=self.patch_size)

        self._gemm_cache = None
        self._gemm_key = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.proj(x)
        return y.flatten(2).transpose(1, 2)

    def _gemm_weights(self):
        """The convolution as a GEMM: weight [embed_dim, K] with K = C_in*pv*ph*pw in
        (c, v, h, w) order, K padded with zero columns to a multiple of 8; bf16, re-cast when
        a parameter changes."""
        key = tuple((p.data_ptr(), p._version, p.device) for p in self.proj.parameters())
        if self._gemm_cache is not None and key == self._gemm_key:
            return self._gemm_cache
        w = self.proj.weight.detach()
        K = w[0].numel()
        Kp = (K + 7) // 8 * 8
        wm = torch.zeros(w.shape[0], Kp, dtype=torch.bfloat16, device=w.device)
        wm[:, :K] = w.reshape(w.shape[0], K)
        b = None if self.proj.bias is None else self.proj.bias.detach().float().contiguous()
        self._gemm_cache, self._gemm_key = (wm, b, K, Kp), key
        return self._gemm_cache

    def tokens_bf16(self, x: torch.Tensor) -> torch.Tensor:
        """[B, C_in, D, H, W] -> bf16 tokens [B, D'*H'*W', embed_dim] on the tensor cores: the
        non-overlapping patches are laid out as rows of a [tokens, K] matrix (one strided copy,
        which also casts to bf16) and multiplied by the convolution weight with the bias epilogue.
        Same arithmetic as the Conv3d under bf16 autocast, without its channels-first output and
        the transposing copy that would follow."""
        B, cin, D, H, W = x.shape
        pv, ph, pw = self.patch_size
        d, h, w = D // pv, H // ph, W // pw
        wm, bias, K, Kp = self._gemm_weights()
        a = torch.empty(B * d * h * w, Kp, dtype=torch.bfloat16, device=x.device)
        if Kp != K:
            a[:, K:].zero_()
        a.view(B, d, h, w, Kp)[..., :K].view(B, d, h, w, cin, pv, ph, pw).copy_(
            x.view(B, cin, d, pv, h, ph, w, pw).permute(0, 2, 4, 6, 1, 3, 5, 7))
        return ops.linear(a, wm, bias).view(B, d * h * w, wm.shape[0])

    def tokens_from_patches(self, a: torch.Tensor, n_tiles: int) -> torch.Tensor:
        """Rows already gathered and cast (ops.preprocess_patches with k_pad = the padded K of
        `_gemm_weights`) -> bf16 tokens [n_tiles, tokens, embed_dim]."""
        wm, bias, _, Kp = self._gemm_weights()
        if a.shape[1] != Kp:
            raise ValueError(f"patch matrix has {a.shape[1]} columns, the embedding expects {Kp}")
        return ops.linear(a, wm, bias).view(n_tiles, -1, wm.shape[0])


class DealiasedPatchEmbed3D(nn.Module):
    """Patch embedding with a fixed low-pass before the decimation (reference:
    screamcast/dealias.py:28-143; same constructor, same `proj` shape and state-dict keys as the
    plain embedding, the filter a non-persistent buffer). The reference convolves at stride 1,
    replicate-pads, filters and decimates; here the filter is applied to the patches while they
    are gathered (`ops.dealias_patches`) and one tcgen05 GEMM with the `proj` weight follows -
    the same linear map, 1/patch-volume of the multiply-adds."""

    def __init__(self, depth, height, width, patch_size=16, in_chans=3, embed_dim=768,
                 resample_filter=(1, 1)):
        super().__init__()
        self.patch_size = _triple(patch_size)
        pd, ph, pw = self.patch_size
        for size, p_, what in ((depth, pd, "Depth"), (height, ph, "Height"), (width, pw, "Width")):
            if size % p_ != 0:
                kind = "vertical" if what == "Depth" else "horizontal"
                raise ValueError(f"{what} ({size}) must be divisible by {kind} patch size ({p_})")
        self.depth, self.height, self.width = depth, height, width
        self.num_patches = (depth // pd) * (height // ph) * (width // pw)
        self.proj = nn.Conv3d(in_chans, embed_dim, kernel_size=self.patch_size, stride=1, padding=0,
                              bias=True)
        self.resample_filter = tuple(float(v) for v in resample_filter)
        f = torch.tensor(self.resample_filter, dtype=torch.float32)
        one = torch.ones(1)
        fd, fh, fw = (one if pd == 1 else f), (one if ph == 1 else f), (one if pw == 1 else f)
        f3d = fd[:, None, None] * fh[None, :, None] * fw[None, None, :]
        self.register_buffer("dealias_filter", (f3d / f3d.sum())[None, None], persistent=False)
        self._embed_dim = embed_dim
        self._gemm_cache = None
        self._gemm_key = None

    _gemm_weights = PatchEmbed3D._gemm_weights

    def tokens_from_pixel_rows(self, rows: torch.Tensor, shape) -> torch.Tensor:
        """rows: bf16 pixel rows [B*D*H*W, ld] of the pre-processed fields (channels last);
        shape = (B, D, H, W). Returns bf16 tokens [B, tokens, embed_dim]."""
        wm, bias, _, Kp = self._gemm_weights()
        a = ops.dealias_patches(rows, shape, self.proj.in_channels, self.patch_size,
                                self.resample_filter, k_pad=Kp)
        return ops.linear(a, wm, bias).view(shape[0], -1, wm.shape[0])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """[B, C, D, H, W] -> [B, embed_dim, D', H', W'] (the reference module's output layout)."""
        if not x.is_cuda:
            raise RuntimeError("DealiasedPatchEmbed3D runs on CUDA only (its kernels have no CPU "
                               "fallback)")
        B, C, D, H, W = x.shape
        rows = x.permute(0, 2, 3, 4, 1).to(torch.bfloat16).reshape(B * D * H * W, C)
        Cp = (C + 7) // 8 * 8
        if Cp != C:
            rows = torch.nn.functional.pad(rows, (0, Cp - C))
        t = self.tokens_from_pixel_rows(rows.contiguous(), (B, D, H, W))
        pd, ph, pw = self.patch_size
        return t.view(B, D // pd, H // ph, W // pw, -1).permute(0, 4, 1, 2, 3)


class Mlp(nn.Module):
    """layers = Sequential(fc1, GELU, fc2); the reference's wrapper swaps the GELU to the tanh
    approximation (screamcast/strata_wrappers.py:76-100)."""

    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.layers = nn.Sequential(nn.Linear(dim, hidden), nn.GELU(approximate="none"),
                                    nn.Linear(hidden, dim))


class NeighborhoodAttention3D(nn.Module):
    def __init__(self, dim: int, num_heads: int, qkv_bias: bool, gated: bool):
        super().__init__()
        self.num_heads = num_heads
        self.qkv = nn.Linear(dim, 3 * dim, bias=qkv_bias)
        self.proj = nn.Linear(dim, dim)
        if gated:
            self.gate_proj = nn.Linear(dim, dim)


class StrataTransformer3DBlock(nn.Module):
    """Pre-norm block without norm parameters: x += proj(gate * NA3D(rope(qkv(LN(x)))));
    x += fc2(gelu(fc1(LN(x))))."""

    def __init__(self, dim: int, num_heads: int, mlp_ratio: float, qkv_bias: bool, qk_norm: bool,
                 gated: bool, kernel):
        super().__init__()
        self.dim, self.num_heads = dim, num_heads
        self.qk_norm = qk_norm
        self.kernel = _triple(kernel)
        self.attn = NeighborhoodAttention3D(dim, num_heads, qkv_bias, gated)
        self.mlp = Mlp(dim, int(dim * mlp_ratio))
        self._bf16_cache = None
        self._bf16_key = None

    def _gelu_is_tanh(self) -> bool:
        act = self.mlp.layers[1]
        return isinstance(act, nn.GELU) and act.approximate == "tanh"

    def device_weights(self) -> dict:
        """bf16 weights / fp32 biases for the C ABI, re-cast whenever a parameter changes."""
        key = tuple((p.data_ptr(), p._version, p.device) for p in self.parameters())
        if self._bf16_cache is not None and key == self._bf16_key:
            return self._bf16_cache

        def w(lin):
            return lin.weight.detach().to(torch.bfloat16).contiguous()

        def b(lin):
            return None if lin.bias is None else lin.bias.detach().float().contiguous()

        cache = {"w_qkv": w(self.attn.qkv), "b_qkv": b(self.attn.qkv),
                 "w_proj": w(self.attn.proj), "b_proj": b(self.attn.proj),
                 "w_fc1": w(self.mlp.layers[0]), "b_fc1": b(self.mlp.layers[0]),
                 "w_fc2": w(self.mlp.layers[2]), "b_fc2": b(self.mlp.layers[2])}
        if hasattr(self.attn, "gate_proj"):
            cache["w_gate"], cache["b_gate"] = w(self.attn.gate_proj), b(self.attn.gate_proj)
        self._bf16_cache, self._bf16_key = cache, key
        return cache

    def forward(self, x: torch.Tensor, grid, rope_cs, workspace=None) -> torch.Tensor:
        """x: [n_tiles, D*H*W, C] bf16 contiguous; rope_cs: packed half (cos, sin) table or
        None; returns the same shape as x."""
        if not self._gelu_is_tanh():
            raise RuntimeError(
                "the fused MLP kernel implements the tanh GELU the Strata checkpoints were "
                "trained with; this block's Mlp still holds an exact GELU (the wrapper's "
                "tanh swap did not run)")
        return ops.block_forward(x, self.device_weights(), grid=grid, num_heads=self.num_heads,
                                 kernel=self.kernel, rope_cos=None, rope_sin=None,
                                 rope_cs=rope_cs, qk_norm=self.qk_norm, workspace=workspace)


class FinalLayer(nn.Module):
    """Non-affine LayerNorm + Linear to patch pixels."""

    def __init__(self, dim: int, out_features: int):
        super().__init__()
        self.linear = nn.Linear(dim, out_features)
        self._gemm_cache = None
        self._gemm_key = None

    def forward_bf16(self, tokens: torch.Tensor) -> torch.Tensor:
        """bf16 tokens [..., dim] -> fp32 [..., out_features] through the library's LayerNorm
        and GEMM kernels (output rows padded to a multiple of 8 columns for the store)."""
        lead = tokens.shape[:-1]
        y, N = self.matrix_bf16(tokens)
        return y[:, :N].float().view(*lead, N)

    def _refresh(self) -> None:
        key = tuple((p.data_ptr(), p._version, p.device) for p in self.linear.parameters())
        if self._gemm_cache is None or key != self._gemm_key:
            w = self.linear.weight.detach()
            N = w.shape[0]
            Np = (N + 7) // 8 * 8
            wm = torch.zeros(Np, w.shape[1], dtype=torch.bfloat16, device=w.device)
            wm[:N] = w
            b = None
            if self.linear.bias is not None:
                b = torch.zeros(Np, dtype=torch.float32, device=w.device)
                b[:N] = self.linear.bias.detach().float()
            self._gemm_cache, self._gemm_key = (wm, b, N), key

    def matrix_bf16(self, tokens: torch.Tensor):
        """bf16 tokens [..., dim] -> (bf16 [rows, Np], N): the layer's output rows, N valid
        columns of a row stride padded to a multiple of 8."""
        self._refresh()
        wm, b, N = self._gemm_cache
        return ops.linear(ops.layernorm(tokens.reshape(-1, tokens.shape[-1])), wm, b), N


class StrataTransformer3D(nn.Module):
    """Backbone: patch embed -> N blocks -> final projection -> unpatchify.

    forward(x[B, C_in, D, H, W], pos[B, 2, H, W] lat/lon radians) -> [B, C_out, D, H, W].
    """

    def __init__(self, *, in_channels: int, out_channels: int, input_shape, patch_size=(1, 1, 1),
                 embed_dim: int = 768, num_heads: int = 16, num_layers: int = 12,
                 mlp_ratio: float = 4.0, qkv_bias: bool = True, qk_norm: bool = False,
                 qk_norm_affine: bool = False, attn_kernel=3, na_dilation: int = 3,
                 do_interleaved_dilation: bool = False, do_alt_depthwise_attn: bool = False,
                 gated_attention: bool = False, na3d_backend: str | None = None,
                 rope_mode: str = "none", rope_base: float = 100.0, rope_length_scale: float = 1.0,
                 activation_checkpointing: bool | float = False, bf16_mixed: bool = False):
        super().__init__()
        if rope_mode not in ("none", "axial", "stereographic"):
            raise ValueError(f"unknown rope_mode {rope_mode!r}")
        if qk_norm_affine:
            raise ValueError("qk_norm_affine=True is not supported (production configs use "
                             "non-affine qk norm)")
        if do_interleaved_dilation:
            raise ValueError("dilated neighbourhood attention is not supported "
                             "(production configs use dilation 1)")
        if embed_dim % num_heads or embed_dim // num_heads != 64:
            raise ValueError("head_dim must be 64 for the sm_100a attention kernel")
        self.in_channels, self.out_channels = in_channels, out_channels
        self.depth, self.height, self.width = (int(v) for v in input_shape)
        self.patch_size = _triple(patch_size)
        self.embed_dim, self.num_heads = embed_dim, num_heads
        self.head_dim = embed_dim // num_heads
        self.rope_mode, self.rope_base = rope_mode, float(rope_base)
        self.rope_length_scale = float(rope_length_scale)
        self.na3d_backend = na3d_backend  # accepted for config compatibility; one backend here
        self.bf16_mixed = bf16_mixed
        self._activation_checkpointing_ratio = float(activation_checkpointing)
        kernel = _triple(attn_kernel)
        self.attn_kernel = kernel
        self.patch_embed = PatchEmbed3D(in_channels, embed_dim, self.patch_size)
        blocks = []
        for i in range(num_layers):
            k = kernel
            if do_alt_depthwise_attn and i % 2 == 1:
                # every other block attends along depth only (kd x 1 x 1 window)
                k = (kernel[0], 1, 1)
            blocks.append(StrataTransformer3DBlock(embed_dim, num_heads, mlp_ratio, qkv_bias,
                                                   qk_norm, gated_attention, k))
        self.blocks = nn.ModuleList(blocks)
        pv, ph, pw = self.patch_size
        self.final_layer = FinalLayer(embed_dim, pv * ph * pw * out_channels)
        self._workspace = None

    # ---------------------------------------------------------------- geometry
    def set_tile_size(self, height: int, width: int) -> None:
        self.height, self.width = int(height), int(width)

    def token_grid(self, D: int, H: int, W: int):
        pv, ph, pw = self.patch_size
        return D // pv, H // ph, W // pw

    def rope_tables(self, pos: torch.Tensor | None, n_tiles: int, grid):
        _, h, w = grid
        if self.rope_mode == "none":
            return None, None
        if self.rope_mode == "axial":
            cos, sin = rope.axial_rope_tables(h, w, self.head_dim, self.rope_base,
                                              device=self.patch_embed.proj.weight.device)
            return cos.expand(n_tiles, -1, -1).contiguous(), sin.expand(n_tiles, -1, -1).contiguous()
        if pos is None:
            raise ValueError("stereographic RoPE needs pos=[B, 2, H, W] (lat, lon)")
        return rope.stereographic_rope_tables(pos, self.head_dim, self.patch_size[1],
                                              self.rope_length_scale, self.rope_base)

    def _get_workspace(self, M: int, device) -> torch.Tensor:
        hidden = self.blocks[0].mlp.layers[0].out_features
        need = ops.block_workspace_bytes(M, self.embed_dim, hidden)
        ws = self._workspace
        if ws is None or ws.numel() < need or ws.device != device:
            ws = torch.empty(need, dtype=torch.uint8, device=device)
            self._workspace = ws
        return ws

    # ---------------------------------------------------------------- forward
    def forward_tokens(self, tokens: torch.Tensor, grid, rope_cos, rope_sin) -> torch.Tensor:
        """Runs the block stack on bf16 tokens [n_tiles, D*H*W, C]."""
        ws = self._get_workspace(tokens.shape[0] * tokens.shape[1], tokens.device)
        cs = None if rope_cos is None else rope.pack_rope_tables(rope_cos, rope_sin)
        x = tokens
        for blk in self.blocks:
            x = blk(x, grid, cs, workspace=ws)
        return x

    def forward(self, x: torch.Tensor, pos: torch.Tensor | None = None) -> torch.Tensor:
        B, _, D, H, W = x.shape
        grid = self.token_grid(D, H, W)
        if isinstance(self.patch_embed, PatchEmbed3D):
            tokens = self.patch_embed.tokens_bf16(x.contiguous())
        elif isinstance(self.patch_embed, DealiasedPatchEmbed3D):
            tokens = self.patch_embed(x).flatten(2).transpose(1, 2).contiguous()
        else:   # a caller-assigned embed module (not one of this package's): the caller's own
            # code, run as it is - the only step of the forward that is not a kernel of this library
            with torch.autocast("cuda", dtype=torch.bfloat16, enabled=x.is_cuda):
                tokens = self.patch_embed(x)
            tokens = tokens.to(torch.bfloat16).contiguous()
        cos, sin = self.rope_tables(pos, B, grid)
        tokens = self.forward_tokens(tokens, grid, cos, sin)
        return self.unpatchify(self.final_layer.forward_bf16(tokens), grid)

    def fused_path_available(self, x: torch.Tensor) -> bool:
        """The fused pre/post-processing kernels serve the plain patch embedding on CUDA fp32
        inputs; anything else (a caller-assigned embed module) goes through `forward`."""
        return (isinstance(self.patch_embed, (PatchEmbed3D, DealiasedPatchEmbed3D)) and x.is_cuda
                and x.dtype == torch.float32)

    def embed_fused(self, x, lat, lon, lat0, lon0, wind, concat_lat):
        """Raw fields -> bf16 backbone tokens [B, tokens, C]: pre-processing kernel (wind rotation,
        latitude channels, patch gathering) + the patch-embedding GEMM; the de-aliased embedding
        gathers pixel rows first and filters them while forming the patches."""
        B, _, D, H, W = x.shape
        _, _, _, Kp = self.patch_embed._gemm_weights()
        if isinstance(self.patch_embed, DealiasedPatchEmbed3D):
            cin = self.patch_embed.proj.in_channels
            rows = ops.preprocess_patches(x, lat, lon, lat0, lon0, wind=wind, concat_lat=concat_lat,
                                          patch=(1, 1, 1), k_pad=(cin + 7) // 8 * 8)
            return self.patch_embed.tokens_from_pixel_rows(rows, (B, D, H, W))
        a = ops.preprocess_patches(x, lat, lon, lat0, lon0, wind=wind, concat_lat=concat_lat,
                                   patch=self.patch_size, k_pad=Kp)
        return self.patch_embed.tokens_from_patches(a, B)

    def forward_fused(self, x: torch.Tensor, pos: torch.Tensor | None, *, lat=None, lon=None,
                      lat0=None, lon0=None, wind=None, concat_lat: bool = False) -> torch.Tensor:
        """Raw fields in, fields out, with the wrapper's pre- and post-processing inside:
        x [B, C_raw, D, H, W] fp32 (before wind rotation and latitude channels) ->
        [B, C_out, D, H, W] fp32 (wind channels rotated back). One kernel gathers, rotates,
        appends and casts the patch rows, one un-patchifies and rotates back."""
        B, _, D, H, W = x.shape
        grid = self.token_grid(D, H, W)
        tokens = self.embed_fused(x, lat, lon, lat0, lon0, wind, concat_lat)
        cos, sin = self.rope_tables(pos, B, grid)
        tokens = self.forward_tokens(tokens, grid, cos, sin)
        y, _ = self.final_layer.matrix_bf16(tokens)
        return ops.postprocess_fields(y, (B, self.out_channels, D, H, W), lat, lon, lat0, lon0,
                                      wind=wind, patch=self.patch_size)

    def unpatchify(self, y: torch.Tensor, grid) -> torch.Tensor:
        B = y.shape[0]
        d, h, w = grid
        pv, ph, pw = self.patch_size
        c = self.out_channels
        y = y.reshape(B, d, h, w, pv, ph, pw, c)
        y = y.permute(0, 7, 1, 4, 2, 5, 3, 6)
        return y.reshape(B, c, d * pv, h * ph, w * pw)
