"""CPU oracle for the cubed-sphere tile / halo index logic (TEST INFRASTRUCTURE only).

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may
import this module; strata_b200/ never does.

numpy restatement of the reference's pure index code, pinned bit-exactly by the fixtures in
tests/golden/ (generated from the reference itself by tests/golden/make_golden.py):

  get_cubesphere_neighbors          screamcast/cubesphere_transforms.py:149-196
  extract_edge_raw_batched          screamcast/cubesphere_transforms.py:199-227
  rotate_edge_to_canonical_batched  screamcast/cubesphere_transforms.py:230-251
  rotate_canonical_to_halo_batched  screamcast/cubesphere_transforms.py:254-273
  fill_corners_batched              screamcast/cubesphere_transforms.py:276-354
  create_padded_faces_batched       screamcast/cubesphere_transforms.py:357-445
  halo_dst_flat_indices             screamcast/cubesphere_transforms.py:448-473
  TileTopology                      screamcast/distributed_halo.py:57-205
  _select_padded_tile               screamcast/distributed_halo.py:451-473
  forward_uv_to_tile / inverse      screamcast/wind_rotation.py:49-144
  tile_center / mean_longitude      screamcast/tile_geometry.py:33-61,141-155
"""
from __future__ import annotations

import itertools

import numpy as np

# neighbors[face][to_dir] = (neighbour face, neighbour edge); layout
#   | 5 |
#   | 0 | 1 | 2 | 3 |
#   | 4 |
NEIGHBORS = {
    0: {"top": (5, "bottom"), "right": (1, "left"), "bottom": (4, "top"), "left": (3, "right")},
    1: {"top": (5, "right"), "right": (2, "left"), "bottom": (4, "right"), "left": (0, "right")},
    2: {"top": (5, "top"), "right": (3, "left"), "bottom": (4, "bottom"), "left": (1, "right")},
    3: {"top": (5, "left"), "right": (0, "left"), "bottom": (4, "left"), "left": (2, "right")},
    4: {"top": (0, "bottom"), "right": (1, "bottom"), "bottom": (2, "bottom"), "left": (3, "bottom")},
    5: {"top": (2, "top"), "right": (1, "top"), "bottom": (0, "top"), "left": (3, "top")},
}
_TO_CANON = {"bottom": 0, "left": -1, "right": 1, "top": 2}
_TO_HALO = {"top": 0, "right": 1, "left": -1, "bottom": 2}


def extract_edge(face: np.ndarray, edge: str, p: int) -> np.ndarray:
    """Axis -2 grows 'upwards': bottom = first p rows, top = last p rows."""
    if edge == "top":
        return face[..., -p:, :]
    if edge == "bottom":
        return face[..., :p, :]
    if edge == "left":
        return face[..., :, :p]
    if edge == "right":
        return face[..., :, -p:]
    raise ValueError(edge)


def _rot(a: np.ndarray, k: int) -> np.ndarray:
    return np.rot90(a, k=k, axes=(-2, -1)) if k else a


def fill_corners(padded: np.ndarray, p: int, fs: int) -> None:
    """Diagonal rule: one side of the (main/anti) diagonal copies the adjacent column of the
    vertical halo, the other the adjacent row of the horizontal halo, the diagonal their mean."""
    S = fs + 2 * p
    i = np.arange(p)[:, None]
    j = np.arange(p)[None, :]
    main_below, main_above = i > j, i < j
    anti_below, anti_above = (i + j) > (p - 1), (i + j) < (p - 1)
    corners = [
        (slice(0, p), slice(0, p), p, p, "main", "above"),
        (slice(0, p), slice(p + fs, S), p + fs - 1, p, "anti", "above"),
        (slice(p + fs, S), slice(0, p), p, p + fs - 1, "anti", "below"),
        (slice(p + fs, S), slice(p + fs, S), p + fs - 1, p + fs - 1, "main", "below"),
    ]
    for rs, cs, v_col, h_row, diag, v_side in corners:
        v = np.broadcast_to(padded[..., rs, v_col:v_col + 1], padded.shape[:-2] + (p, p))
        h = np.broadcast_to(padded[..., h_row:h_row + 1, cs], padded.shape[:-2] + (p, p))
        above, below = (main_above, main_below) if diag == "main" else (anti_above, anti_below)
        v_mask, h_mask = (above, below) if v_side == "above" else (below, above)
        padded[..., rs, cs] = np.where(v_mask, v, np.where(h_mask, h, (v + h) / 2))


def create_padded_faces(data: np.ndarray, p: int) -> np.ndarray:
    """(..., 6, N, N) -> (..., 6, N+2p, N+2p): copy + rot90 edge halos, diagonal-rule corners."""
    if p == 0:
        return data
    *lead, nf, N, N2 = data.shape
    if nf != 6 or N != N2:
        raise ValueError("expected (..., 6, N, N)")
    S = N + 2 * p
    fill = np.nan if np.issubdtype(data.dtype, np.floating) else 0
    out = np.full(tuple(lead) + (6, S, S), fill, dtype=data.dtype)
    for f in range(6):
        out[..., f, p:p + N, p:p + N] = data[..., f, :, :]
        for to_dir, (nb, nb_edge) in NEIGHBORS[f].items():
            strip = _rot(_rot(extract_edge(data[..., nb, :, :], nb_edge, p), _TO_CANON[nb_edge]),
                         _TO_HALO[to_dir])
            if to_dir == "top":
                out[..., f, S - p:, p:p + N] = strip
            elif to_dir == "bottom":
                out[..., f, :p, p:p + N] = strip
            elif to_dir == "left":
                out[..., f, p:p + N, :p] = strip
            else:
                out[..., f, p:p + N, S - p:] = strip
    fill_corners(out, p, N)
    return out


def halo_dst_flat_indices(N: int, p: int) -> np.ndarray:
    S = N + 2 * p
    ii, jj = np.meshgrid(np.arange(S), np.arange(S), indexing="ij")
    halo = (ii < p) | (ii >= p + N) | (jj < p) | (jj >= p + N)
    ih, jh = ii[halo].astype(np.int64), jj[halo].astype(np.int64)
    return np.concatenate([f * S * S + ih * S + jh for f in range(6)]).astype(np.int64)


def unstructured_to_6faces(x: np.ndarray, ne: int, npg: int) -> np.ndarray:
    """(..., 6*ne*ne*npg*npg) element-major columns -> (..., 6, ne*npg, ne*npg) rasters."""
    *lead, n = x.shape
    x = x.reshape(*lead, 6, ne, ne, npg, npg)
    nd = len(lead)
    x = np.moveaxis(x, nd + 3, nd + 2)  # (..., 6, ne, npg, ne, npg)
    return x.reshape(*lead, 6, ne * npg, ne * npg)


def faces_to_unstructured(x: np.ndarray, ne: int, npg: int) -> np.ndarray:
    *lead, nf, n1, n2 = x.shape
    x = x.reshape(*lead, 6, ne, npg, ne, npg)
    nd = len(lead)
    x = np.moveaxis(x, nd + 3, nd + 2)
    return x.reshape(*lead, 6 * ne * ne * npg * npg)


# --------------------------------------------------------------------------- tiles
class TileTopology:
    """Tile <-> rank decomposition: tiles enumerate product(face, ti, tj); rank r owns the
    contiguous slice [r*tpr, (r+1)*tpr)."""

    def __init__(self, world_size, rank, face_size, tile_size, halo_width, n_faces=6):
        if face_size % tile_size:
            raise ValueError("face_size must be divisible by tile_size")
        self.world_size, self.rank = world_size, rank
        self.face_size, self.tile_size, self.halo_width = face_size, tile_size, halo_width
        self.n_faces = n_faces
        if self.total_tiles % world_size:
            raise ValueError("number of tiles must be divisible by world_size")

    @property
    def tiles_per_dim(self):
        return self.face_size // self.tile_size

    @property
    def total_tiles(self):
        return self.n_faces * self.tiles_per_dim ** 2

    @property
    def tiles_per_rank(self):
        return self.total_tiles // self.world_size

    @property
    def padded_tile_size(self):
        return self.tile_size + 2 * self.halo_width

    @property
    def global_tiles(self):
        return list(itertools.product(range(self.n_faces), range(self.tiles_per_dim),
                                      range(self.tiles_per_dim)))

    @property
    def local_tiles(self):
        s = self.rank * self.tiles_per_rank
        return self.global_tiles[s:s + self.tiles_per_rank]

    def crop(self, x):
        h = self.halo_width
        return x if h == 0 else x[..., h:-h, h:-h]

    def faces_to_local_tiles(self, x):
        ts = self.tile_size
        return np.stack([x[..., f, ti * ts:(ti + 1) * ts, tj * ts:(tj + 1) * ts]
                         for f, ti, tj in self.local_tiles], axis=-3)

    def tiles_to_faces(self, all_tiles):
        """all_tiles (..., total_tiles, T, T) in global_tiles order -> (..., 6, N, N)."""
        ts = self.tile_size
        out = np.zeros(all_tiles.shape[:-3] + (self.n_faces, self.face_size, self.face_size),
                       dtype=all_tiles.dtype)
        for g, (f, ti, tj) in enumerate(self.global_tiles):
            out[..., f, ti * ts:(ti + 1) * ts, tj * ts:(tj + 1) * ts] = all_tiles[..., g, :, :]
        return out


def select_padded_tile(x, tile, tile_size, halo_width, pad_width_data):
    f, ti, tj = tile
    a = pad_width_data + ti * tile_size - halo_width
    b = pad_width_data + (ti + 1) * tile_size + halo_width
    c = pad_width_data + tj * tile_size - halo_width
    d = pad_width_data + (tj + 1) * tile_size + halo_width
    return x[..., f, a:b, c:d]


def padded_local_tiles(all_tiles: np.ndarray, topo: TileTopology) -> np.ndarray:
    """Copy-halo exchange for tiles: every tile of the globe (global_tiles order, any leading
    dims) -> this rank's tiles padded by halo_width, via faces -> create_padded_faces ->
    window slicing (the composition the reference's in-tree functions define)."""
    faces = topo.tiles_to_faces(all_tiles)
    padded = create_padded_faces(faces, topo.halo_width)
    return np.stack([select_padded_tile(padded, t, topo.tile_size, topo.halo_width, topo.halo_width)
                     for t in topo.local_tiles], axis=-3)


def halo_adjoint(padded_all: np.ndarray, topo: TileTopology, window: np.ndarray | None = None):
    """Windowed overlap-add un-pad D_w^-1 A^T (w . y) of the copy-halo exchange A
    (`padded_local_tiles`), after the reference's NormalizedHaloAdjoint
    (screamcast/distributed_halo.py:330-448; there A is the KNN regrid, here the copy halo).

    padded_all: (..., total_tiles, P, P) float32, the padded tiles of EVERY rank in global tile
    order. Returns this rank's (..., tiles_per_rank, T, T).

    A is recovered from `padded_local_tiles` itself, applied to an array of cell labels: the
    index logic under test is not re-used. Every padded cell is either a copy of one interior
    cell or the mean of two; the transpose hands its (windowed) value back with coefficient 1 or
    1/2. Contributions are summed per interior cell in the order of the padded cell ids, every
    product and sum rounded to float32 (the CUDA kernel keeps the same order: bit-exact).
    """
    T, P, G = topo.tile_size, topo.padded_tile_size, topo.total_tiles
    full = TileTopology(1, 0, topo.face_size, T, topo.halo_width)
    # labels: two probes with different cell values identify a(p), b(p) of every padded cell
    ids = np.arange(G * T * T, dtype=np.float64).reshape(G, T, T)
    pa = padded_local_tiles(ids, full)                    # a, or (a+b)/2
    pb = padded_local_tiles(ids * ids, full)              # a^2, or (a^2+b^2)/2
    s, q = pa.reshape(-1), pb.reshape(-1)
    # single source: q == s^2; two sources: a, b = s +- sqrt(q - s^2)
    d = np.sqrt(np.maximum(q - s * s, 0.0))
    a = np.rint(s - d).astype(np.int64)
    b = np.where(d > 0.25, np.rint(s + d).astype(np.int64), -1)
    w = np.ones((P, P), np.float32) if window is None else np.asarray(window, np.float32)
    wflat = np.tile(w.reshape(-1), G)
    lead = padded_all.shape[:-3]
    y = padded_all.reshape(*lead, -1).astype(np.float32)
    wy = (wflat * y).astype(np.float32)
    n_local = topo.tiles_per_rank * T * T
    lo = topo.rank * n_local
    acc = np.zeros((*lead, n_local), np.float32)
    wsum = np.zeros(n_local, np.float32)
    for p in range(a.size):                               # padded cells in id order
        for src, coef in ((a[p], 1.0 if b[p] < 0 else 0.5), (b[p], 0.5)):
            if src < lo or src >= lo + n_local:
                continue
            c = src - lo
            acc[..., c] = (acc[..., c] + (np.float32(coef) * wy[..., p]).astype(np.float32)
                           ).astype(np.float32)
            wsum[c] = np.float32(wsum[c] + np.float32(coef) * wflat[p])
    return (acc / wsum).astype(np.float32).reshape(*lead, topo.tiles_per_rank, T, T)


def knn_halo_adjoint(padded_all: np.ndarray, topo: TileTopology, idx_all: np.ndarray,
                     w_all: np.ndarray, window: np.ndarray | None = None):
    """D_w^-1 A^T (w . y) for the k-nearest-neighbour halo A (out[p] = sum_j w[p,j] x[idx[p,j]]),
    the operator of the reference's NormalizedHaloAdjoint (screamcast/distributed_halo.py:330-448),
    evaluated densely in float64: scatter-add of every padded cell's windowed value to its k
    sources, divided by the scatter-add of the window itself.

    padded_all: (..., total_tiles, P, P), idx_all / w_all: [total_tiles*P*P, k] for the padded
    cells of every tile in global tile order. Returns this rank's (..., tiles_per_rank, T, T).
    """
    T, P, G = topo.tile_size, topo.padded_tile_size, topo.total_tiles
    w = np.ones((P, P)) if window is None else np.asarray(window, np.float64)
    wflat = np.tile(w.reshape(-1), G)
    lead = padded_all.shape[:-3]
    y = padded_all.reshape(*lead, -1).astype(np.float64) * wflat
    n_src = G * T * T
    acc = np.zeros((*lead, n_src))
    wsum = np.zeros(n_src)
    for j in range(idx_all.shape[1]):
        np.add.at(wsum, idx_all[:, j], w_all[:, j].astype(np.float64) * wflat)
        flat_acc = acc.reshape(-1, n_src)
        flat_y = y.reshape(-1, y.shape[-1])
        for r in range(flat_acc.shape[0]):
            np.add.at(flat_acc[r], idx_all[:, j], w_all[:, j].astype(np.float64) * flat_y[r])
    n_local = topo.tiles_per_rank * T * T
    lo = topo.rank * n_local
    with np.errstate(invalid="ignore", divide="ignore"):
        out = acc[..., lo:lo + n_local] / wsum[lo:lo + n_local]
    return out.reshape(*lead, topo.tiles_per_rank, T, T)


def knn_halo(all_tiles: np.ndarray, topo: TileTopology, lon_deg: np.ndarray, lat_deg: np.ndarray,
             pad_width_data: int, k: int = 4, eps: float = 1e-7):
    """k-nearest-neighbour halo of this rank's tiles, after
    DistributedTileKNNHaloPadding_AllGather (screamcast/distributed_halo.py:225-327): sources =
    interiors of all tiles in global order (`_select_tile_interior`), destinations = the padded
    windows of the local tiles (`_select_padded_tile`), weights 1 / (chord distance + eps)
    normalised over the k nearest sources (earth2grid's KNNS2Interpolator is absent: this
    weight formula is an assumption). Brute-force neighbour search (small grids only).

    all_tiles: (..., total_tiles, T, T) float32. Returns ((..., tiles_per_rank, P, P), idx, w);
    sums run in neighbour order (nearest first), every product and sum rounded to float32.
    """
    T, P = topo.tile_size, topo.padded_tile_size
    full = TileTopology(1, 0, topo.face_size, T, topo.halo_width)

    def unit(lon, lat):
        lo, la = np.radians(lon.astype(np.float64)), np.radians(lat.astype(np.float64))
        return np.stack([np.cos(la) * np.cos(lo), np.cos(la) * np.sin(lo), np.sin(la)], axis=-1)

    def interior(g, tile):
        f, ti, tj = tile
        pw = pad_width_data
        return g[f, pw + ti * T:pw + (ti + 1) * T, pw + tj * T:pw + (tj + 1) * T]
    src = np.concatenate([unit(interior(lon_deg, t), interior(lat_deg, t)).reshape(-1, 3)
                          for t in full.global_tiles])
    dst = np.concatenate([unit(select_padded_tile(lon_deg, t, T, topo.halo_width, pad_width_data),
                               select_padded_tile(lat_deg, t, T, topo.halo_width, pad_width_data)
                               ).reshape(-1, 3) for t in topo.local_tiles])
    d = np.sqrt(np.maximum(((dst[:, None, :] - src[None, :, :]) ** 2).sum(-1), 0.0))
    idx = np.argsort(d, axis=1, kind="stable")[:, :k]
    dist = np.take_along_axis(d, idx, axis=1)
    lam = 1.0 / (dist + eps)
    w = (lam / lam.sum(axis=1, keepdims=True)).astype(np.float32)
    lead = all_tiles.shape[:-3]
    flat = all_tiles.reshape(*lead, -1).astype(np.float32)
    acc = np.zeros((*lead, dst.shape[0]), np.float32)
    for j in range(k):
        acc = (acc + (w[:, j] * flat[..., idx[:, j]]).astype(np.float32)).astype(np.float32)
    return acc.reshape(*lead, topo.tiles_per_rank, P, P), idx.astype(np.int32), w


def plan_halo_forward(all_tiles: np.ndarray, entries, tile_size: int, halo_width: int,
                      local_tile_ids) -> np.ndarray:
    """Forward of the plan-based tile halo after DistributedTileKNNHaloPadding.forward
    (screamcast/distributed_cubesphere_transforms.py:697-781), without the transport: padded
    tiles start as NaN, interiors are copied, and every plan entry (source tile id, destination
    tile id, positions [n] in the padded tile, index [n, k] into the source tile, weight [n, k])
    scatters its interpolated values into its destination tile.

    all_tiles: (..., total_tiles, T, T) float32 in global tile order; entries: iterable of
    (src_tile_id, dst_tile_id, positions, index, weight). Returns (..., len(local_tile_ids), S, S).
    Sums run in neighbour order, every product and sum rounded to float32 (no fused multiply-add).
    """
    T, h = tile_size, halo_width
    S = T + 2 * h
    lead = all_tiles.shape[:-3]
    local = list(local_tile_ids)
    out = np.full((*lead, len(local), S, S), np.nan, np.float32)
    for n, g in enumerate(local):
        out[..., n, h:h + T, h:h + T] = all_tiles[..., g, :, :]
    flat_out = out.reshape(*lead, len(local), S * S)
    where = {g: n for n, g in enumerate(local)}
    for src, dst, pos, index, weight in entries:
        if dst not in where:
            continue
        tile = all_tiles[..., src, :, :].reshape(*lead, T * T).astype(np.float32)
        acc = np.zeros((*lead, len(pos)), np.float32)
        for j in range(index.shape[1]):
            acc = (acc + (weight[:, j].astype(np.float32) * tile[..., index[:, j]]).astype(np.float32)
                   ).astype(np.float32)
        flat_out[..., where[dst], np.asarray(pos)] = acc
    return flat_out.reshape(*lead, len(local), S, S)


# --------------------------------------------------------------------------- wind rotation
def _basis(lat, lon):
    R = (np.cos(lat) * np.cos(lon), np.cos(lat) * np.sin(lon), np.sin(lat))
    E = (-np.sin(lon), np.cos(lon), np.zeros_like(lat))
    Nn = (-np.sin(lat) * np.cos(lon), -np.sin(lat) * np.sin(lon), np.cos(lat))
    return E, Nn, R


def mean_longitude(lon, return_0_2pi=True):
    m = np.arctan2(np.sin(lon).mean(axis=(-2, -1), keepdims=True),
                   np.cos(lon).mean(axis=(-2, -1), keepdims=True))
    return m % (2 * np.pi) if return_0_2pi else m


def tile_center(lat, lon):
    return lat.mean(axis=(1, 2), keepdims=True), mean_longitude(lon)


def forward_uv_to_tile(U, V, lat, lon, lat0, lon0):
    lat, lon, lat0, lon0 = lat[:, None], lon[:, None], lat0[:, None], lon0[:, None]
    E, Nn, _ = _basis(lat, lon)
    v = [U * E[i] + V * Nn[i] for i in range(3)]
    E0, N0, R0 = _basis(lat0, lon0)
    dot = v[0] * R0[0] + v[1] * R0[1] + v[2] * R0[2]
    vt = [v[i] - dot * R0[i] for i in range(3)]
    return (vt[0] * E0[0] + vt[1] * E0[1] + vt[2] * E0[2],
            vt[0] * N0[0] + vt[1] * N0[1] + vt[2] * N0[2])


def inverse_tile_to_uv(Ul, Vl, lat, lon, lat0, lon0):
    lat, lon, lat0, lon0 = lat[:, None], lon[:, None], lat0[:, None], lon0[:, None]
    E0, N0, R0 = _basis(lat0, lon0)
    vt = [Ul * E0[i] + Vl * N0[i] for i in range(3)]
    E, Nn, R = _basis(lat, lon)
    beta = -(vt[0] * R[0] + vt[1] * R[1] + vt[2] * R[2]) / (R0[0] * R[0] + R0[1] * R[1] + R0[2] * R[2])
    v = [vt[i] + beta * R0[i] for i in range(3)]
    return (v[0] * E[0] + v[1] * E[1] + v[2] * E[2], v[0] * Nn[0] + v[1] * Nn[1] + v[2] * Nn[2])
