"""Backbone blocks over tiled cubed-sphere tokens with a K/V halo exchange in EVERY block.

Only a tile's own (interior) tokens are queries; their neighbourhoods reach into the
neighbouring tiles, whose keys and values arrive through peer memory each block:

    xn = LN(x)                                   interior tokens, compact
    qkv -> interior rows of this rank's halo-padded qkv buffer   (fused GEMM + RoPE, row remap)
    flag barrier                                 every rank has published its interiors
    K, V of the halo cells <- owners' interiors  (gather maps: copy / rot90 / corner rule;
                                                  K re-rotated from the owner's RoPE frame into
                                                  this tile's frame)
    attention of the interior queries over the padded K/V planes
    projection, residual, LN, MLP               interior tokens, compact

The exchange runs in line on the compute stream: it moves about 3 % of a block's time, and
hiding it behind the attention of the queries whose windows stay inside the tile was built and
measured slower (the four border strips that have to follow fill their 128-query tiles badly
and cost four more launches per block), so that variant was taken out again. Everything that
is token-wise (LN, the GEMMs) runs in chunks of tiles, so that only x, y, the attention output
and the padded qkv buffer are ever held for all tiles at once.

Stereographic RoPE coordinates are relative to each tile's centre, so a key rotated in its
owner's frame is wrong for the receiver; the owner stores K in its own frame (it needs that
for its own queries) and the receiver applies the rotation by the angle difference, a table
that is fixed for a given grid. The reference itself exchanges halos once per model step in
field space (scripts/ace/run_screamcast_nudged.py:455) - that mode is strata_b200.rollout; this
module is the per-block mode. Tokens are pixels here (patch size 1), tile size a multiple of 32,
halo at least half the horizontal kernel.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _lib, ops, rope
from .halo import PeerSharedBuffer
from .topology import TileTopology, apply_maps_numpy, halo_source_maps


def _tile_frame_coords(lat_deg: np.ndarray, lon_deg: np.ndarray, centre_from=None):
    """Stereographic (x, y) of points (degrees, [n, ...]) about the spherical centroid of
    `centre_from` (default: the points themselves), per leading entry. float64 torch."""
    lat = torch.deg2rad(torch.as_tensor(lat_deg, dtype=torch.float64))
    lon = torch.deg2rad(torch.as_tensor(lon_deg, dtype=torch.float64))
    if centre_from is None:
        clat, clon = lat, lon
    else:
        clat = torch.deg2rad(torch.as_tensor(centre_from[0], dtype=torch.float64))
        clon = torch.deg2rad(torch.as_tensor(centre_from[1], dtype=torch.float64))
    lat0, lon0 = rope.spherical_centroid(clat, clon)
    return rope.stereographic_projection(lat, lon, lat0, lon0)


class TiledBlockRunner:
    """Set-up (maps, RoPE tables, delta tables, peer buffers) and per-block execution."""

    FLAG_BYTES = 256

    def __init__(self, topology: TileTopology, *, depth: int, dim: int, num_heads: int, kernel,
                 lat_deg: np.ndarray, lon_deg: np.ndarray, rope_base: float = 100.0,
                 rope_length_scale: float | None = None, device=None, group=None,
                 timeout_ms: int = 2000, chunk_tiles: int | None = None):
        """lat_deg / lon_deg: [total_tiles, T, T] cell centres of ALL tiles in global tile order."""
        T, h = topology.tile_size, topology.halo_width
        kd, kh, kw = (int(kernel),) * 3 if isinstance(kernel, int) else tuple(int(v) for v in kernel)
        if T % 32:
            raise ValueError("tile size must be a multiple of 32 for the padded QKV store")
        if h < max(kh, kw) // 2:
            raise ValueError("halo must cover half the horizontal kernel")
        if dim % num_heads or dim // num_heads != 64:
            raise ValueError("head_dim must be 64")
        self.topology, self.depth, self.dim, self.heads = topology, depth, dim, num_heads
        self.kernel = (kd, kh, kw)
        self.group, self.timeout_ms = group, int(timeout_ms)
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.device = dev
        P = topology.padded_tile_size
        hd = dim // num_heads
        scale = rope_length_scale or rope.default_rope_length_scale(1)
        a, b = halo_source_maps(topology)
        self.src_a = torch.from_numpy(a).to(dev)
        self.src_b = torch.from_numpy(b).to(dev)
        tpr = topology.tiles_per_rank
        s = topology.rank * tpr
        # every tile's interior coordinates in its OWN frame (needed for halo sources)
        xs, ys = _tile_frame_coords(lat_deg, lon_deg)                       # [G, T, T]
        xs, ys = (xs / scale).reshape(-1), (ys / scale).reshape(-1)
        cos, sin = rope.build_axial_rope_cos_sin_2d_continuous(
            xs.reshape(topology.total_tiles, T * T)[s:s + tpr],
            ys.reshape(topology.total_tiles, T * T)[s:s + tpr], hd, rope_base)
        self.rope_cs = rope.pack_rope_tables(cos, sin).to(dev)              # interior, own frame
        # padded cells of the local tiles in the RECEIVER's frame: coordinates of the halo cells
        # travel like any other field (unit vectors, so the corner mean stays off the lon seam)
        la, lo = np.radians(lat_deg), np.radians(lon_deg)
        xyz = np.stack([np.cos(la) * np.cos(lo), np.cos(la) * np.sin(lo), np.sin(la)])
        pad = apply_maps_numpy(xyz, a, b)                                   # [3, tpr, P, P]
        plat = np.degrees(np.arctan2(pad[2], np.hypot(pad[0], pad[1])))
        plon = np.degrees(np.arctan2(pad[1], pad[0]))
        xr, yr = _tile_frame_coords(plat, plon, centre_from=(lat_deg[s:s + tpr], lon_deg[s:s + tpr]))
        xr, yr = xr / scale, yr / scale                                     # [tpr, P, P]
        n = hd // 4
        f = rope_base ** (-torch.arange(n, dtype=torch.float64) / n)

        def delta(src):
            idx = torch.from_numpy(np.where(src < 0, 0, src).astype(np.int64))
            dx = xr - xs[idx]
            dy = yr - ys[idx]
            ang = torch.cat([dx[..., None] * f, dy[..., None] * f], dim=-1)  # [tpr, P, P, hd/2]
            return rope.pack_rope_tables(torch.cos(ang).float(), torch.sin(ang).float()
                                         ).reshape(tpr, P * P, hd // 2, 2).to(dev)
        self.dcs_a, self.dcs_b = delta(a), delta(b)
        # peer-visible padded qkv: [flags | slot 0 | slot 1]. Two alternating slots keep a rank
        # that is already one block ahead from overwriting what a slower peer still reads; a
        # single GPU is ordered by its stream and needs one.
        self._slot_bytes = tpr * depth * P * P * 3 * dim * 2
        self._n_slots = 2 if topology.world_size > 1 else 1
        self._epoch = 0
        total = self.FLAG_BYTES + self._n_slots * self._slot_bytes
        if topology.world_size > 1:
            self._shared = PeerSharedBuffer(total, group=group)
            self._local = self._shared.local
        else:
            self._shared = None
            self._local = torch.zeros(total, dtype=torch.uint8, device=dev)
        if chunk_tiles is None:   # hidden activations of a chunk stay below ~4 GB
            chunk_tiles = max(1, int(4e9 // (depth * T * T * 4 * dim * 2)))
        self.chunk_tiles = min(int(chunk_tiles), tpr)

    def _slot(self, parity: int):
        off = self.FLAG_BYTES + (parity % self._n_slots) * self._slot_bytes
        topo = self.topology
        P = topo.padded_tile_size
        rows = topo.tiles_per_rank * self.depth * P * P
        view = self._local[off:off + self._slot_bytes].view(torch.bfloat16).view(rows, 3 * self.dim)
        if self._shared is not None:
            ptrs = self._shared.ptr_array(off)
        else:
            ptrs = (ctypes.c_void_p * 1)(view.data_ptr())
        return view, ptrs

    def _chunks(self):
        tpr = self.topology.tiles_per_rank
        return [(t0, min(t0 + self.chunk_tiles, tpr)) for t0 in range(0, tpr, self.chunk_tiles)]

    def _exchange(self, qkv, ptrs):
        """Flag barrier (every rank's interiors are published) + K/V halo gather, on the
        current stream."""
        topo, D, C = self.topology, self.depth, self.dim
        lib = _lib.load()
        stream = torch.cuda.current_stream().cuda_stream
        if topo.world_size > 1:
            _lib.check(lib.strata_halo_barrier(self._shared.ptr_array(0), topo.rank, topo.world_size,
                                               self._epoch, self.timeout_ms, stream),
                       "strata_halo_barrier")
        _lib.check(lib.strata_halo_gather_kv_bf16(
            qkv.data_ptr(), ptrs, topo.world_size, self.src_a.data_ptr(), self.src_b.data_ptr(),
            self.dcs_a.data_ptr(), self.dcs_b.data_ptr(), topo.tiles_per_rank, D, topo.tile_size,
            topo.halo_width, C, C // self.heads, 3 * C, stream), "strata_halo_gather_kv_bf16")

    def attention(self, xn, w_qkv, b_qkv, qk_norm: bool = False) -> torch.Tensor:
        """LN'ed interior tokens [tiles_per_rank*D*T*T, C] (a tensor, or a callable
        chunk(t0, t1) -> rows of tiles [t0, t1)) -> attention output, same shape."""
        topo, D, C = self.topology, self.depth, self.dim
        T, h, P = topo.tile_size, topo.halo_width, topo.padded_tile_size
        tpr = topo.tiles_per_rank
        self._epoch += 1
        qkv, ptrs = self._slot(self._epoch)
        rows_t, prow_t = D * T * T, D * P * P
        for t0, t1 in self._chunks():
            xc = xn(t0, t1) if callable(xn) else xn[t0 * rows_t:t1 * rows_t]
            ops.qkv_rope_padded(xc, w_qkv, b_qkv, C // self.heads, self.rope_cs[t0:t1], rows_t, T * T,
                                qkv[t0 * prow_t:t1 * prow_t], tile=T, halo=h, depth=D,
                                qk_norm=qk_norm)
        q6 = qkv.view(tpr, D, P, P, 3, self.heads, C // self.heads)
        q, k, v = q6[..., 0, :, :], q6[..., 1, :, :], q6[..., 2, :, :]
        self._exchange(qkv, ptrs)
        o = ops.na3d_region(q, k, v, self.kernel, (h, T, h, T))
        return o.view(tpr * D * T * T, C)

    def block_forward(self, x: torch.Tensor, weights: dict, qk_norm: bool = False) -> torch.Tensor:
        """x: [tiles_per_rank, D*T*T, C] bf16 interior tokens; weights as ops.block_forward."""
        tpr, tokens, C = x.shape
        x2 = x.reshape(tpr * tokens, C)
        attn = self.attention(lambda t0, t1: ops.layernorm(x2[t0 * tokens:t1 * tokens]),
                              weights["w_qkv"], weights.get("b_qkv"), qk_norm)
        y = torch.empty_like(x2)
        for t0, t1 in self._chunks():
            sl = slice(t0 * tokens, t1 * tokens)
            xc, ac = x2[sl], attn[sl]
            if weights.get("w_gate") is not None:
                ac = ops.linear(ops.layernorm(xc), weights["w_gate"], weights.get("b_gate"),
                                ops.EPI_GATE, ac)
            x1 = ops.linear(ac, weights["w_proj"], weights.get("b_proj"), ops.EPI_RESIDUAL, xc)
            hmid = ops.linear(ops.layernorm(x1), weights["w_fc1"], weights.get("b_fc1"), ops.EPI_GELU)
            ops.linear(hmid, weights["w_fc2"], weights.get("b_fc2"), ops.EPI_RESIDUAL, x1, out=y[sl])
        return y.view(tpr, tokens, C)

    def check_status(self) -> None:
        st = _lib.device_status()
        if st != 0:
            raise RuntimeError(f"tiled block run failed on the device (status {st})")

    def close(self):
        if self._shared is not None:
            self._shared.close()
            self._shared = None
