"""One model step over a tiled cubed sphere: halo exchange -> network on padded tiles -> crop.

This is the body of the reference's distributed rollout loop
(scripts/ace/run_screamcast_nudged.py:452-477: `x_with_halo = pad(x)`, `model(x_with_halo)`,
`unpad(out)`) with this package's pieces: the peer-memory copy halo
(strata_b200/halo.py) in place of the all-gather + regrid, the sm_100a backbone in place of
physicsnemo + NATTEN, and `TileTopology.crop` as the un-pad. Tiles are the batch dimension of the
network, exactly as the reference feeds faces/tiles as batch entries.

Also here: a synthetic equiangular cubed-sphere lat/lon generator, standing in for the grid
files (`ne1024pg2_scrip.nc`, ...) that are not distributed with the reference.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .halo import DistributedTileCopyHaloPadding, NormalizedCopyHaloAdjoint, kbd_window
from .topology import TileTopology, apply_maps_numpy, halo_source_maps


def equiangular_cubed_sphere_latlon(n: int):
    """(lat, lon) in degrees, each [6, n, n], of cell centres of an equiangular gnomonic cubed
    sphere. Faces 0-3 run around the equator (centre longitudes 0, 90, 180, 270), face 4 is the
    south cap, face 5 the north cap; rows grow northwards on the equatorial faces."""
    ang = (np.arange(n) + 0.5) / n * (math.pi / 2) - math.pi / 4
    a, b = np.meshgrid(np.tan(ang), np.tan(ang), indexing="xy")   # a: column (east), b: row (north)
    lat = np.empty((6, n, n))
    lon = np.empty((6, n, n))
    for f in range(4):
        x, y, z = np.ones_like(a), a, b
        lon[f] = np.degrees(np.arctan2(y, x)) + 90.0 * f
        lat[f] = np.degrees(np.arctan2(z, np.hypot(x, y)))
    # caps: local axes chosen so that the bottom edge of the north cap meets face 0's top edge
    x, y, z = -b, a, np.ones_like(a)
    lon[5] = np.degrees(np.arctan2(y, x))
    lat[5] = np.degrees(np.arctan2(z, np.hypot(x, y)))
    x, y, z = b, a, -np.ones_like(a)
    lon[4] = np.degrees(np.arctan2(y, x))
    lat[4] = np.degrees(np.arctan2(z, np.hypot(x, y)))
    return lat, np.mod(lon, 360.0)


def padded_face_latlon(n: int, pad: int):
    """(lat, lon) in degrees, each [6, n + 2*pad, n + 2*pad]: the faces of
    `equiangular_cubed_sphere_latlon` continued beyond their edges along the same gnomonic
    lines, so that every halo cell carries its own true position (what the reference reads from
    its halo grid files for DistributedTileKNNHaloPadding_AllGather.from_padded_face_grid)."""
    ang = (np.arange(-pad, n + pad) + 0.5) / n * (math.pi / 2) - math.pi / 4
    ang = np.clip(ang, -math.pi / 2 + 1e-3, math.pi / 2 - 1e-3)
    a, b = np.meshgrid(np.tan(ang), np.tan(ang), indexing="xy")
    m = n + 2 * pad
    lat = np.empty((6, m, m))
    lon = np.empty((6, m, m))
    for f in range(4):
        x, y, z = np.ones_like(a), a, b
        lon[f] = np.degrees(np.arctan2(y, x)) + 90.0 * f
        lat[f] = np.degrees(np.arctan2(z, np.hypot(x, y)))
    x, y, z = -b, a, np.ones_like(a)
    lon[5] = np.degrees(np.arctan2(y, x))
    lat[5] = np.degrees(np.arctan2(z, np.hypot(x, y)))
    x, y, z = b, a, -np.ones_like(a)
    lon[4] = np.degrees(np.arctan2(y, x))
    lat[4] = np.degrees(np.arctan2(z, np.hypot(x, y)))
    return lat, np.mod(lon, 360.0)


def padded_tile_latlon(topology: TileTopology):
    """lat/lon (degrees) of this rank's padded tiles [tiles_per_rank, P, P]: interior cells
    from the synthetic grid, halo cells copied from the neighbouring tile / face like any other
    field (so a halo cell carries the coordinates of the cell whose data it receives)."""
    lat, lon = equiangular_cubed_sphere_latlon(topology.face_size)
    full = TileTopology(1, 0, topology.face_size, topology.tile_size, topology.halo_width)
    T = topology.tile_size

    def tiles(g):
        return np.stack([g[f, ti * T:(ti + 1) * T, tj * T:(tj + 1) * T]
                         for f, ti, tj in full.global_tiles])
    a, b = halo_source_maps(topology)
    # corner diagonals average two cells; do it on unit vectors to stay clear of the lon seam
    la, lo = np.radians(tiles(lat)), np.radians(tiles(lon))
    xyz = np.stack([np.cos(la) * np.cos(lo), np.cos(la) * np.sin(lo), np.sin(la)])
    pad = apply_maps_numpy(xyz, a, b)
    plat = np.degrees(np.arctan2(pad[2], np.hypot(pad[0], pad[1])))
    plon = np.mod(np.degrees(np.arctan2(pad[1], pad[0])), 360.0)
    return plat, plon


class TiledSphereStepper(torch.nn.Module):
    """halo exchange -> network -> crop for this rank's tiles.

    forward(x[C, D, tiles_per_rank, T, T] fp32) -> [C_out, D, tiles_per_rank, T, T].
    `network` follows the wrapper contract `network(x[B, C, D, H, W], index)` with
    `index = {"lat", "lon"}` in radians (index_is_latlon=True) and tile size T + 2*halo.
    """

    def __init__(self, network: torch.nn.Module, topology: TileTopology, device=None, group=None,
                 unpad: str = "crop", window: str | None = None, check_every: int = 0,
                 out_channels: int | None = None, in_channels: int | None = None, depth: int | None = None):
        """unpad: "crop" (drop the halo, `topology.crop`) or "adjoint" (windowed overlap-add of
        the padded outputs, `--halo-adjoint` of the reference's launcher); window: None
        (uniform) or "kbd" (`--halo-window`).

        A halo barrier whose wait runs out does not stop the stream: the padded tiles (and
        everything computed from them) come back as NaN and the device status word is set.
        check_every = n > 0 additionally synchronises and raises on every n-th step (callers
        that must not synchronise poll `halo.check_status()` themselves, e.g. where they write
        output anyway). in_channels / out_channels / depth, when given, size the peer-shared
        buffer for the larger of the two payloads (input fields, padded outputs of the adjoint)
        at construction; otherwise the first step that needs more room re-allocates it, which is
        a collective over the group."""
        super().__init__()
        self.check_every = int(check_every)
        self._steps = 0
        if unpad not in ("crop", "adjoint"):
            raise ValueError(f"unpad must be 'crop' or 'adjoint', got {unpad!r}")
        self.network = network
        self.topology = topology
        plat, plon = padded_tile_latlon(topology)
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        max_bytes = 0
        if depth is not None and (in_channels is not None or out_channels is not None):
            T, P, tpr = topology.tile_size, topology.padded_tile_size, topology.tiles_per_rank
            max_bytes = 4 * depth * tpr * max((in_channels or 0) * T * T,
                                              (out_channels or 0) * P * P if unpad == "adjoint" else 0)
        self.halo = DistributedTileCopyHaloPadding(
            topology=topology, lat_deg=torch.from_numpy(plat).float().to(dev),
            lon_deg=torch.from_numpy(plon).float().to(dev), device=dev, group=group,
            **({"max_bytes_per_call": max_bytes} if max_bytes else {}))
        self.unpad = None
        if unpad == "adjoint":
            win = kbd_window(topology.padded_tile_size) if window == "kbd" else None
            self.unpad = NormalizedCopyHaloAdjoint(self.halo, window=win)
        self.register_buffer("lat_rad", torch.deg2rad(self.halo.lat_deg), persistent=False)
        self.register_buffer("lon_rad", torch.deg2rad(self.halo.lon_deg), persistent=False)

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        padded = self.halo(x)                                   # [C, D, tpr, P, P]
        xin = padded.permute(2, 0, 1, 3, 4).contiguous()        # tiles become the batch
        y = self.network(xin, {"lat": self.lat_rad, "lon": self.lon_rad})
        if self.unpad is None:
            y = self.topology.crop(y)                           # [tpr, C_out, D, T, T]
            out = y.permute(1, 2, 0, 3, 4).contiguous()
        else:
            out = self.unpad(y.permute(1, 2, 0, 3, 4).float().contiguous())
        self._steps += 1
        if self.check_every > 0 and self._steps % self.check_every == 0:
            self.halo.check_status()
        return out

    def close(self):
        self.halo.close()
