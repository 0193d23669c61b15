"""Drop-in counterparts of the reference's model wrappers (screamcast/strata_wrappers.py):
same class names, constructor arguments, methods, properties, error behaviour and
state-dict keys (`strata.*`), with `self.strata` built from this package's sm_100a backbone
instead of physicsnemo + NATTEN.

    network = StrataBackboneModel(depth=..., height=..., width=..., embed_dim=..., ...)
    y = network(x, index)      # x [B, C, D, H, W]; index: column ids or {"lat","lon"} radians
"""
from __future__ import annotations

import math
from typing import Mapping, Optional, Tuple

import torch
import torch.nn as nn

from . import rope, torch_ops
from .checkpoint_compat import remap_legacy_pre_hook
from .strata import Mlp, StrataTransformer3D


# --------------------------------------------------------------------------- helpers
def _replace_channels(x: torch.Tensor, replacements: dict) -> torch.Tensor:
    """Channel-dim rebuild by slice + cat (reference: strata_wrappers.py:61-73)."""
    pieces = [replacements[c].unsqueeze(1) if c in replacements else x[:, c:c + 1]
              for c in range(x.shape[1])]
    return torch.cat(pieces, dim=1)


def _use_tanh_gelu(model: nn.Module) -> None:
    """Swap every Mlp's exact GELU for the tanh approximation (strata_wrappers.py:76-100)."""
    n = 0
    for module in model.modules():
        if isinstance(module, Mlp):
            for i, layer in enumerate(module.layers):
                if isinstance(layer, nn.GELU) and layer.approximate == "none":
                    module.layers[i] = nn.GELU(approximate="tanh")
                    n += 1
    if n == 0:
        raise RuntimeError("_use_tanh_gelu found no exact-GELU Mlp layers to swap")


def _resolve_rope_base(rope_length_scale: Optional[float]) -> float:
    """None / 0 -> the historical default; negative raises (strata_wrappers.py:134-150)."""
    if rope_length_scale is not None and rope_length_scale < 0:
        raise ValueError("rope_length_scale must be positive (or 0/None for the default); "
                         f"got {rope_length_scale}")
    return rope_length_scale or TileGeometry.default_rope_length_scale(1)


def _rope_mode(do_rope_2d: bool, do_rope_2d_stereographic: bool) -> str:
    if do_rope_2d and do_rope_2d_stereographic:
        raise ValueError("Cannot use both row/column RoPE and stereographic RoPE simultaneously")
    if do_rope_2d_stereographic:
        return "stereographic"
    return "axial" if do_rope_2d else "none"


def mean_longitude(lon: torch.Tensor, reduce_dims=(-2, -1), return_0_2pi: bool = True):
    """Circular mean of longitude (reference: screamcast/tile_geometry.py:33-61)."""
    s = lon.sin().mean(dim=reduce_dims, keepdim=True)
    c = lon.cos().mean(dim=reduce_dims, keepdim=True)
    m = torch.atan2(s, c)
    return m % (2 * torch.pi) if return_0_2pi else m


class TileGeometry(nn.Module):
    """index -> per-pixel lat/lon (radians). Explicit {"lat","lon"} indices pass through;
    integer column ids need lookup tables, which the reference reads from earth2grid or a
    grid file (screamcast/tile_geometry.py:64-112) and which are supplied here with
    set_lookup_tables() because neither source is part of this package."""

    def __init__(self, grid_type: str = "healpix", nside: int = 1024,
                 cubesphere_latlon_path: str | None = None, index_is_latlon: bool = False):
        super().__init__()
        self.grid_type = (grid_type or "healpix").lower()
        if self.grid_type not in {"healpix", "cubesphere"}:
            raise ValueError(f"Unsupported grid_type='{grid_type}'. Expected 'healpix' or "
                             "'cubesphere'.")
        self.nside = nside
        self.index_is_latlon = index_is_latlon
        self.register_buffer("_lat_radians", torch.zeros(0), persistent=False)
        self.register_buffer("_lon_radians", torch.zeros(0), persistent=False)

    def set_lookup_tables(self, lat_radians: torch.Tensor, lon_radians: torch.Tensor) -> None:
        self.register_buffer("_lat_radians", lat_radians.float(), persistent=False)
        self.register_buffer("_lon_radians", lon_radians.float(), persistent=False)

    def lat_lon_from_index(self, index):
        if self.index_is_latlon:
            try:
                lat, lon = index["lat"], index["lon"]
            except Exception as exc:
                raise ValueError("index must provide 'lat' and 'lon' tensors when "
                                 "index_is_latlon is True") from exc
            if lat.ndim == 2:
                lat = lat.unsqueeze(0)
            if lon.ndim == 2:
                lon = lon.unsqueeze(0)
            if lat.ndim != 3 or lon.ndim != 3:
                raise ValueError("lat/lon tensors must be 2D or 3D with shape [B, H, W]")
            if lat.shape != lon.shape:
                raise ValueError("lat/lon tensors must have matching shapes")
            return lat, lon
        if self._lat_radians.numel() == 0:
            raise ValueError("integer tile indices need lat/lon lookup tables: call "
                             "geometry.set_lookup_tables(lat, lon) or use index_is_latlon=True")
        return self._lat_radians[index.long()], self._lon_radians[index.long()]

    @staticmethod
    def tile_center(lat: torch.Tensor, lon: torch.Tensor):
        """Arithmetic-mean latitude, circular-mean longitude, each [B, 1, 1]."""
        return lat.mean(dim=(1, 2), keepdim=True), mean_longitude(lon)

    @staticmethod
    def default_rope_length_scale(patch_size_horiz: int) -> float:
        return rope.default_rope_length_scale(patch_size_horiz)


# --------------------------------------------------------------------------- wind rotation
def local_basis_ENR(lat, lon):
    """East, north, radial unit vectors (reference: screamcast/wind_rotation.py:26-46)."""
    cl, sl, co, so = torch.cos(lat), torch.sin(lat), torch.cos(lon), torch.sin(lon)
    return (-so, co, torch.zeros_like(lat)), (-sl * co, -sl * so, cl), (cl * co, cl * so, sl)


def forward_uv_to_tile(U, V, lat, lon, lat0, lon0):
    """(U,V) east/north at each pixel -> components in the tile centre's tangent basis
    (reference: screamcast/wind_rotation.py:49-92)."""
    lat, lon, lat0, lon0 = lat.unsqueeze(1), lon.unsqueeze(1), lat0.unsqueeze(1), lon0.unsqueeze(1)
    E, N, _ = local_basis_ENR(lat, lon)
    v = [U * E[i] + V * N[i] for i in range(3)]
    E0, N0, R0 = local_basis_ENR(lat0, lon0)
    d = v[0] * R0[0] + v[1] * R0[1] + v[2] * R0[2]
    vt = [v[i] - d * R0[i] for i in range(3)]
    return (vt[0] * E0[0] + vt[1] * E0[1] + vt[2] * E0[2],
            vt[0] * N0[0] + vt[1] * N0[1] + vt[2] * N0[2])


def inverse_tile_to_uv(U_loc, V_loc, lat, lon, lat0, lon0):
    """Inverse of forward_uv_to_tile (reference: screamcast/wind_rotation.py:95-144)."""
    lat, lon, lat0, lon0 = lat.unsqueeze(1), lon.unsqueeze(1), lat0.unsqueeze(1), lon0.unsqueeze(1)
    E0, N0, R0 = local_basis_ENR(lat0, lon0)
    vt = [U_loc * E0[i] + V_loc * N0[i] for i in range(3)]
    E, N, R = local_basis_ENR(lat, lon)
    beta = -(vt[0] * R[0] + vt[1] * R[1] + vt[2] * R[2]) / (R0[0] * R[0] + R0[1] * R[1] + R0[2] * R[2])
    v = [vt[i] + beta * R0[i] for i in range(3)]
    return (v[0] * E[0] + v[1] * E[1] + v[2] * E[2], v[0] * N[0] + v[1] * N[1] + v[2] * N[2])


# --------------------------------------------------------------------------- wrappers
class _StrataModelBase(nn.Module):
    """Geometry / wind / latitude-concat plumbing (reference: strata_wrappers.py:165-249)."""

    def __init__(self, *, do_concat_latitude: bool, do_rotate_wind: bool,
                 wind_channel_indices: Optional[Tuple[int, int]], grid_type: str, nside: int,
                 cubesphere_latlon_path: str, index_is_latlon: bool):
        super().__init__()
        if do_rotate_wind and wind_channel_indices is None:
            raise ValueError("Must specify wind_channel_indices when do_rotate_wind is True")
        self._do_concat_latitude = do_concat_latitude
        self._do_rotate_wind = do_rotate_wind
        self._wind_channel_indices = wind_channel_indices
        self.geometry = TileGeometry(grid_type=grid_type, nside=nside,
                                     cubesphere_latlon_path=cubesphere_latlon_path,
                                     index_is_latlon=index_is_latlon)
        # legacy checkpoint keys are translated inside the load machinery itself, so the
        # translation also happens when this wrapper is a submodule of the module being loaded
        # (reference: strata_wrappers.py:193-199)
        self.register_load_state_dict_pre_hook(remap_legacy_pre_hook)
        self._op_handle = torch_ops.register_module(self)

    def __setstate__(self, state):
        # a copy (copy.deepcopy, pickle) is a module of its own for the operator registry
        super().__setstate__(state)
        self._op_handle = torch_ops.register_module(self)

    @property
    def _index_is_latlon(self) -> bool:
        return self.geometry.index_is_latlon

    def forward(self, x: torch.Tensor, index) -> torch.Tensor:
        """network(x[B, C, D, H, W], index) -> [B, C_out, D, H, W] (reference:
        strata_wrappers.py:408-415, 673-680). The index lookup is plain tensor code; everything
        behind it is one registered operator, so the module can be compiled whole
        (`torch.compile(network)`, also with fullgraph=True) and called under inference mode."""
        lat, lon = self.geometry.lat_lon_from_index(index)
        return torch.ops.strata_b200.network_forward(x, lat, lon, self._op_handle)

    def _latlon_for(self, x: torch.Tensor, lat: torch.Tensor, lon: torch.Tensor):
        B = x.shape[0]
        if lat.shape[0] != B:
            lat = lat.expand(B, -1, -1)
            lon = lon.expand(B, -1, -1)
        return lat, lon

    def _preprocess(self, x, index):
        lat, lon = self.geometry.lat_lon_from_index(index)
        return self._preprocess_latlon(x, lat, lon)

    def _preprocess_latlon(self, x, lat, lon):
        B, _, dd, _, _ = x.shape
        lat, lon = self._latlon_for(x, lat, lon)
        lat_lon_data = None
        if self._do_rotate_wind:
            lat0, lon0 = TileGeometry.tile_center(lat, lon)
            lat_lon_data = (lat, lon, lat0, lon0)
            u_idx, v_idx = self._wind_channel_indices
            u_rot, v_rot = forward_uv_to_tile(x[:, u_idx], x[:, v_idx], lat, lon, lat0, lon0)
            x = _replace_channels(x, {u_idx: u_rot, v_idx: v_rot})
        if self._do_concat_latitude:
            lat_e = lat.unsqueeze(1).unsqueeze(2).expand(-1, 1, dd, -1, -1)
            x = torch.cat([x, torch.cos(lat_e), torch.sin(lat_e)], dim=1)
        pos = torch.cat([lat.unsqueeze(1), lon.unsqueeze(1)], dim=1)
        return x, pos, lat_lon_data

    def _postprocess(self, x, lat_lon_data):
        if self._do_rotate_wind and lat_lon_data is not None:
            lat, lon, lat0, lon0 = lat_lon_data
            u_idx, v_idx = self._wind_channel_indices
            u_geo, v_geo = inverse_tile_to_uv(x[:, u_idx], x[:, v_idx], lat, lon, lat0, lon0)
            x = _replace_channels(x, {u_idx: u_geo, v_idx: v_geo})
        return x


def _dealiased_embed(depth, height, width, patch, in_chans, embed_dim, resample_filter):
    """The swapped-in de-aliased patch embedding with the reference's initialisation of it
    (xavier-uniform on the flattened conv weight, zero bias: strata_wrappers.py:103-107)."""
    from .strata import DealiasedPatchEmbed3D
    pe = DealiasedPatchEmbed3D(depth=depth, height=height, width=width, patch_size=patch,
                               in_chans=in_chans, embed_dim=embed_dim,
                               resample_filter=resample_filter)
    w = pe.proj.weight.data
    nn.init.xavier_uniform_(w.view([w.shape[0], -1]))
    nn.init.constant_(pe.proj.bias, 0.0)
    return pe


class StrataBackboneModel(_StrataModelBase):
    """Single-stage model (reference: strata_wrappers.py:252-415). Constructor argument
    names and defaults are the reference's."""

    def __init__(self, *, depth: int = 256, height: int = 256, width: int = 256,
                 n_layers: int = 12, nside: int = 1024, patch_size: int = 1,
                 patch_size_vert: int | None = None, patch_size_horiz: int | None = None,
                 in_chans: int = 3, base_out_chans: int = 3, embed_dim: int = 768,
                 num_heads: int = 16, mlp_ratio: float = 4.0, qkv_bias: bool = True,
                 qk_norm: bool = False, qk_norm_elementwise_affine: bool = False,
                 attn_kernel: int | tuple[int, int, int] = 3, do_alt_depthwise_attn: bool = False,
                 do_interleaved_dilation: bool = False, na_dilations: int = 3,
                 do_rope_2d: bool = False, do_rope_2d_stereographic: bool = False,
                 do_concat_latitude: bool = True, do_rotate_wind: bool = False,
                 wind_channel_indices: Optional[Tuple[int, int]] = None,
                 do_bf16_mixed: bool = False, do_activation_checkpointing: bool | float = False,
                 gated_attention: bool = False, na3d_backend: Optional[str] = None,
                 grid_type: str = "healpix", cubesphere_latlon_path: str = "data/latlon_ne1024pg2.nc",
                 rope_length_scale: Optional[float] = None, index_is_latlon: bool = False,
                 use_dealiased_patch_embed: bool = False,
                 dealias_resample_filter: tuple = (1, 4, 6, 4, 1)):
        super().__init__(do_concat_latitude=do_concat_latitude, do_rotate_wind=do_rotate_wind,
                         wind_channel_indices=wind_channel_indices, grid_type=grid_type,
                         nside=nside, cubesphere_latlon_path=cubesphere_latlon_path,
                         index_is_latlon=index_is_latlon)
        pv = patch_size_vert if patch_size_vert is not None else patch_size
        ph = patch_size_horiz if patch_size_horiz is not None else patch_size
        rope_mode = _rope_mode(do_rope_2d, do_rope_2d_stereographic)
        self._rope_length_scale_base = _resolve_rope_base(rope_length_scale)
        self.strata = StrataTransformer3D(
            in_channels=in_chans + (2 if do_concat_latitude else 0),
            out_channels=base_out_chans, input_shape=(depth, height, width),
            patch_size=(pv, ph, ph), embed_dim=embed_dim, num_heads=num_heads,
            num_layers=n_layers, mlp_ratio=mlp_ratio, qkv_bias=qkv_bias, qk_norm=qk_norm,
            qk_norm_affine=qk_norm_elementwise_affine, attn_kernel=attn_kernel,
            na_dilation=na_dilations, do_interleaved_dilation=do_interleaved_dilation,
            do_alt_depthwise_attn=do_alt_depthwise_attn, gated_attention=gated_attention,
            na3d_backend=na3d_backend, rope_mode=rope_mode, rope_base=100.0,
            rope_length_scale=(self._rope_length_scale_base * ph
                               if rope_mode == "stereographic" else 1.0),
            activation_checkpointing=do_activation_checkpointing, bf16_mixed=do_bf16_mixed)
        _use_tanh_gelu(self.strata)
        if use_dealiased_patch_embed:
            self.strata.patch_embed = _dealiased_embed(depth, height, width, (pv, ph, ph),
                                                       self.strata.in_channels, embed_dim,
                                                       dealias_resample_filter)

    @property
    def _out_chans(self) -> int:
        return self.strata.out_channels

    @property
    def _depth(self) -> int:
        return self.strata.depth

    @property
    def _height(self) -> int:
        return self.strata.height

    @property
    def _width(self) -> int:
        return self.strata.width

    @property
    def _activation_checkpointing_ratio(self) -> float:
        return self.strata._activation_checkpointing_ratio

    @_activation_checkpointing_ratio.setter
    def _activation_checkpointing_ratio(self, value: float) -> None:
        _ = self.strata._activation_checkpointing_ratio
        self.strata._activation_checkpointing_ratio = value

    def disable_activation_checkpointing(self) -> None:
        self._activation_checkpointing_ratio = 0.0

    def set_tile_size(self, height: int, width: int) -> None:
        self.strata.set_tile_size(height, width)

    def set_rope_length_scale(self, base: float) -> None:
        if base <= 0:
            raise ValueError(f"rope length scale base must be positive, got {base}")
        if self.strata.rope_mode != "stereographic":
            raise ValueError("set_rope_length_scale is only meaningful for stereographic RoPE")
        self._rope_length_scale_base = base
        self.strata.rope_length_scale = base * self.strata.patch_size[1]

    def _forward_eager(self, x: torch.Tensor, lat: torch.Tensor, lon: torch.Tensor) -> torch.Tensor:
        """What `strata_b200::network_forward` runs for this module."""
        if self.strata.fused_path_available(x):
            return self._forward_fused(x, lat, lon).to(x.dtype)
        xin, pos, lat_lon_data = self._preprocess_latlon(x, lat, lon)
        y = self.strata(xin, pos=pos)
        return self._postprocess(y, lat_lon_data).to(x.dtype)

    def _forward_fused(self, x: torch.Tensor, lat: torch.Tensor, lon: torch.Tensor) -> torch.Tensor:
        """Same result as _preprocess -> strata -> _postprocess, with the wind rotation, the
        latitude channels and the patch gathering done by one kernel on the way in and the
        un-patchify and inverse rotation by one kernel on the way out."""
        lat, lon = self._latlon_for(x, lat, lon)
        lat = lat.to(device=x.device, dtype=torch.float32).contiguous()
        lon = lon.to(device=x.device, dtype=torch.float32).contiguous()
        lat0 = lon0 = wind = None
        if self._do_rotate_wind:
            lat0, lon0 = TileGeometry.tile_center(lat, lon)
            wind = self._wind_channel_indices
        pos = torch.stack([lat, lon], dim=1)
        return self.strata.forward_fused(x, pos, lat=lat, lon=lon, lat0=lat0, lon0=lon0, wind=wind,
                                         concat_lat=self._do_concat_latitude)


class StrataModel(_StrataModelBase):
    """Two-stage model (reference: screamcast/strata_wrappers.py:418-687): a backbone and an
    AdaLN pixel stage under `self.strata`. Pixel-stage arguments carry the `_pixel` suffix;
    every other keyword is a backbone argument of `StrataBackboneModel`."""

    _WRAPPER_KEYS = ("do_concat_latitude", "do_rotate_wind", "wind_channel_indices", "grid_type",
                     "nside", "cubesphere_latlon_path", "index_is_latlon",
                     "use_dealiased_patch_embed", "dealias_resample_filter")

    def __init__(self, *, embed_dim_pixel: int = 128, n_layers_pixel: int = 4,
                 num_heads_pixel: int | None = None, mlp_ratio_pixel: float = 4.0,
                 attn_kernel_pixel: int = 3, gated_attention_pixel: bool = False,
                 qk_norm_pixel: bool = False, qk_norm_elementwise_affine_pixel: bool = False,
                 na3d_backend_pixel: Optional[str] = None, do_bf16_mixed_pixel: bool = False,
                 freeze_semantic: bool = False, freeze_pixel_blocks: bool = False,
                 use_bilinear_dw_gelu_project_adaln_pixel: bool = False,
                 use_chunked_depthwise_conv_pixel: bool = True,
                 first_block_only_adaln_pixel: bool = False, do_rope_2d_pixel: bool = False,
                 do_rope_2d_stereographic_pixel: bool = False,
                 do_activation_checkpointing_pixel: bool | float = False, **semantic_kwargs):
        from .pixel import Strata
        sk = dict(semantic_kwargs)
        super().__init__(do_concat_latitude=sk.get("do_concat_latitude", True),
                         do_rotate_wind=sk.get("do_rotate_wind", False),
                         wind_channel_indices=sk.get("wind_channel_indices", None),
                         grid_type=sk.get("grid_type", "healpix"), nside=sk.get("nside", 1024),
                         cubesphere_latlon_path=sk.get("cubesphere_latlon_path",
                                                       "data/latlon_ne1024pg2.nc"),
                         index_is_latlon=sk.get("index_is_latlon", False))
        self._rope_length_scale_base = _resolve_rope_base(sk.get("rope_length_scale"))
        backbone_config = self._backbone_config(sk)
        if use_bilinear_dw_gelu_project_adaln_pixel and backbone_config["patch_size"][0] != 1:
            raise ValueError("use_bilinear_dw_gelu_project_adaln requires patch_size_vert=1 "
                             "(the bilinear upsample covers H and W only); got patch_size_vert="
                             f"{backbone_config['patch_size'][0]}")
        rope_mode_pixel = _rope_mode(do_rope_2d_pixel, do_rope_2d_stereographic_pixel)
        self.strata = Strata(
            backbone_config=backbone_config, embed_dim_pixel=embed_dim_pixel,
            num_layers_pixel=n_layers_pixel, num_heads_pixel=num_heads_pixel,
            mlp_ratio_pixel=mlp_ratio_pixel, attn_kernel_pixel=attn_kernel_pixel,
            gated_attention_pixel=gated_attention_pixel, qk_norm_pixel=qk_norm_pixel,
            qk_norm_affine_pixel=qk_norm_elementwise_affine_pixel,
            na3d_backend_pixel=na3d_backend_pixel,
            adaln_mode="bilinear_dw" if use_bilinear_dw_gelu_project_adaln_pixel else "pixel_proj",
            first_block_only_adaln=first_block_only_adaln_pixel,
            use_chunked_depthwise_conv=use_chunked_depthwise_conv_pixel,
            rope_mode_pixel=rope_mode_pixel, rope_base_pixel=100.0,
            rope_length_scale_pixel=(self._rope_length_scale_base
                                     if rope_mode_pixel == "stereographic" else 1.0),
            bf16_mixed_pixel=do_bf16_mixed_pixel,
            activation_checkpointing_pixel=do_activation_checkpointing_pixel)
        _use_tanh_gelu(self.strata)
        if sk.get("use_dealiased_patch_embed", False):
            self.strata.backbone.patch_embed = _dealiased_embed(
                *backbone_config["input_shape"], backbone_config["patch_size"],
                backbone_config["in_channels"], backbone_config["embed_dim"],
                sk.get("dealias_resample_filter", (1, 4, 6, 4, 1)))
        if freeze_semantic:
            for p in self.strata.backbone.parameters():
                p.requires_grad_(False)
        if freeze_pixel_blocks:
            for p in self.strata.pixel_blocks.parameters():
                p.requires_grad_(False)
            for p in self.strata.pixel_final_layer.parameters():
                p.requires_grad_(False)

    def _backbone_config(self, semantic_kwargs: dict) -> dict:
        """Backbone keywords of the single-stage wrapper -> StrataTransformer3D arguments;
        unknown keywords raise TypeError as in the reference (strata_wrappers.py:593-596)."""
        sk = {k: v for k, v in semantic_kwargs.items() if k not in self._WRAPPER_KEYS}
        sk.pop("rope_length_scale", None)
        shape = (sk.pop("depth"), sk.pop("height"), sk.pop("width"))
        patch = sk.pop("patch_size", 1)
        pv, ph = sk.pop("patch_size_vert", None), sk.pop("patch_size_horiz", None)
        pv = patch if pv is None else pv
        ph = patch if ph is None else ph
        rope_mode = _rope_mode(sk.pop("do_rope_2d", False), sk.pop("do_rope_2d_stereographic", False))
        config = dict(
            in_channels=sk.pop("in_chans") + (2 if self._do_concat_latitude else 0),
            out_channels=sk.pop("base_out_chans"), input_shape=shape, patch_size=(pv, ph, ph),
            embed_dim=sk.pop("embed_dim", 768), num_heads=sk.pop("num_heads", 16),
            num_layers=sk.pop("n_layers", 12), mlp_ratio=sk.pop("mlp_ratio", 4.0),
            qkv_bias=sk.pop("qkv_bias", True), qk_norm=sk.pop("qk_norm", False),
            qk_norm_affine=sk.pop("qk_norm_elementwise_affine", False),
            attn_kernel=sk.pop("attn_kernel", 3), na_dilation=sk.pop("na_dilations", 3),
            do_interleaved_dilation=sk.pop("do_interleaved_dilation", False),
            do_alt_depthwise_attn=sk.pop("do_alt_depthwise_attn", False),
            gated_attention=sk.pop("gated_attention", False),
            na3d_backend=sk.pop("na3d_backend", None), rope_mode=rope_mode, rope_base=100.0,
            rope_length_scale=(self._rope_length_scale_base * ph
                               if rope_mode == "stereographic" else 1.0),
            activation_checkpointing=sk.pop("do_activation_checkpointing", False),
            bf16_mixed=sk.pop("do_bf16_mixed", False))
        if sk:
            raise TypeError(f"Unsupported legacy DiT kwargs for the Strata backbone: {sorted(sk)}")
        return config

    @property
    def _out_chans(self) -> int:
        return self.strata.out_channels

    @property
    def _depth(self) -> int:
        return self.strata.depth

    @property
    def _height(self) -> int:
        return self.strata.height

    @property
    def _width(self) -> int:
        return self.strata.width

    def disable_activation_checkpointing(self) -> None:
        _ = self.strata.backbone._activation_checkpointing_ratio
        _ = self.strata._activation_checkpointing_ratio_pixel
        self.strata.backbone._activation_checkpointing_ratio = 0.0
        self.strata._activation_checkpointing_ratio_pixel = 0.0

    def set_tile_size(self, height: int, width: int) -> None:
        self.strata.backbone.set_tile_size(height, width)
        self.strata.height, self.strata.width = int(height), int(width)
        if self.strata.rope_mode_pixel == "axial":
            self.strata._build_axial_rope_pixel(device=self.strata._rope_cos_pixel.device)

    def set_rope_length_scale(self, base: float) -> None:
        if base <= 0:
            raise ValueError(f"rope length scale base must be positive, got {base}")
        backbone_stereo = self.strata.backbone.rope_mode == "stereographic"
        pixel_stereo = self.strata.rope_mode_pixel == "stereographic"
        if not (backbone_stereo or pixel_stereo):
            raise ValueError("set_rope_length_scale is only meaningful for stereographic RoPE")
        self._rope_length_scale_base = base
        if backbone_stereo:
            self.strata.backbone.rope_length_scale = base * self.strata.backbone.patch_size[1]
        if pixel_stereo:
            self.strata.rope_length_scale_pixel = base

    def _forward_eager(self, x: torch.Tensor, lat: torch.Tensor, lon: torch.Tensor) -> torch.Tensor:
        """What `strata_b200::network_forward` runs for this module."""
        if not (x.is_cuda and x.dtype == torch.float32):
            raise RuntimeError("the two-stage model runs on CUDA fp32 fields only (its kernels "
                               "have no CPU fallback)")
        lat, lon = self._latlon_for(x, lat, lon)
        lat = lat.to(device=x.device, dtype=torch.float32).contiguous()
        lon = lon.to(device=x.device, dtype=torch.float32).contiguous()
        lat0 = lon0 = wind = None
        if self._do_rotate_wind:
            lat0, lon0 = TileGeometry.tile_center(lat, lon)
            wind = self._wind_channel_indices
        pos = torch.stack([lat, lon], dim=1)
        return self.strata.forward_fused(x, pos, lat=lat, lon=lon, lat0=lat0, lon0=lon0, wind=wind,
                                         concat_lat=self._do_concat_latitude)
