"""Rotary-embedding tables for the Strata block (host-side geometry, runs on any device).

Mirrors the helpers the reference imports from physicsnemo
(screamcast/strata_wrappers.py:50-52: build_axial_token_coords,
build_axial_rope_cos_sin_2d_continuous; spherical_centroid / stereographic_projection are
named in its module docstring, lines 38-43). The tables are 2-D (horizontal): one row per
(h, w) token position, shared by every depth level and every head.

Table layout consumed by the fused QKV kernel: cos, sin of shape [n_tiles, H*W, head_dim/2]
fp32; pair p of a head rotates channels (2p, 2p+1); pairs [0, head_dim/4) turn with the
x coordinate, pairs [head_dim/4, head_dim/2) with the y coordinate.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def default_rope_length_scale(patch_size_horiz: int) -> float:
    """sqrt of the area of a token on the unit sphere at HEALPix nside=1024 density
    (reference: screamcast/tile_geometry.py:157-170)."""
    return math.sqrt(math.pi * patch_size_horiz ** 2 / (3.0 * 1024 ** 2))


def build_axial_token_coords(depth: int, h: int, w: int, device=None) -> torch.Tensor:
    """[depth*h*w, 2] (x = column, y = row) coordinates of every token, depth-major."""
    ii, jj = torch.meshgrid(torch.arange(h, dtype=torch.float32, device=device),
                            torch.arange(w, dtype=torch.float32, device=device), indexing="ij")
    xy = torch.stack([jj.flatten(), ii.flatten()], dim=-1)
    return xy.repeat(depth, 1)


def build_axial_rope_cos_sin_2d_continuous(x: torch.Tensor, y: torch.Tensor, head_dim: int,
                                           theta: float = 100.0):
    """cos, sin of shape [..., head_dim/2] for continuous coordinates x, y of shape [...]."""
    if head_dim % 4:
        raise ValueError(f"head_dim must be a multiple of 4 for 2-D RoPE, got {head_dim}")
    n = head_dim // 4
    f = theta ** (-torch.arange(n, dtype=torch.float64, device=x.device) / n)
    ang = torch.cat([x.double()[..., None] * f, y.double()[..., None] * f], dim=-1)
    return torch.cos(ang).float(), torch.sin(ang).float()


def spherical_centroid(lat: torch.Tensor, lon: torch.Tensor):
    """Normalised mean unit vector of a tile, as (lat0, lon0); lat/lon [B, H, W] radians."""
    cl = torch.cos(lat)
    x = (cl * torch.cos(lon)).mean(dim=(-2, -1))
    y = (cl * torch.sin(lon)).mean(dim=(-2, -1))
    z = torch.sin(lat).mean(dim=(-2, -1))
    n = torch.sqrt(x * x + y * y + z * z)
    return torch.asin((z / n).clamp(-1, 1)), torch.atan2(y, x)


def stereographic_projection(lat, lon, lat0, lon0):
    """Stereographic coordinates (x east, y north) about (lat0, lon0) on the unit sphere."""
    lat0 = lat0[..., None, None]
    dlon = lon - lon0[..., None, None]
    cosc = torch.sin(lat0) * torch.sin(lat) + torch.cos(lat0) * torch.cos(lat) * torch.cos(dlon)
    k = 2.0 / (1.0 + cosc)
    return (k * torch.cos(lat) * torch.sin(dlon),
            k * (torch.cos(lat0) * torch.sin(lat) - torch.sin(lat0) * torch.cos(lat) * torch.cos(dlon)))


def stereographic_token_coords(pos: torch.Tensor, patch: int, length_scale: float):
    """pos [B, 2, H, W] (lat, lon radians) -> token coordinates x, y [B, (H/patch)*(W/patch)]
    in units of length_scale, averaged over each token's patch x patch pixels."""
    lat, lon = pos[:, 0].double(), pos[:, 1].double()
    lat0, lon0 = spherical_centroid(lat, lon)
    x, y = stereographic_projection(lat, lon, lat0, lon0)
    if patch > 1:
        x = F.avg_pool2d(x[:, None], patch)[:, 0]
        y = F.avg_pool2d(y[:, None], patch)[:, 0]
    return (x / length_scale).flatten(1), (y / length_scale).flatten(1)


def stereographic_rope_tables(pos: torch.Tensor, head_dim: int, patch: int, length_scale: float,
                              theta: float = 100.0):
    """Tables [B, tokens_hw, head_dim/2] from per-pixel lat/lon."""
    x, y = stereographic_token_coords(pos, patch, length_scale)
    return build_axial_rope_cos_sin_2d_continuous(x, y, head_dim, theta)


def axial_rope_tables(h: int, w: int, head_dim: int, theta: float = 100.0, device=None):
    """Tables [1, h*w, head_dim/2] for row/column RoPE."""
    c = build_axial_token_coords(1, h, w, device=device)
    cos, sin = build_axial_rope_cos_sin_2d_continuous(c[:, 0], c[:, 1], head_dim, theta)
    return cos[None], sin[None]


def pack_rope_tables(cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """[n_tiles, hw, head_dim/2] fp32 cos / sin -> [n_tiles, hw, head_dim/2, 2] IEEE half
    (cos, sin) pairs: the 4-bytes-per-pair table the fused QKV kernel reads."""
    return torch.stack([cos, sin], dim=-1).to(torch.float16).contiguous()
