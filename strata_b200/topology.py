"""Cubed-sphere tile decomposition and halo index maps (host side, numpy / torch).

`TileTopology` keeps the reference's interface (screamcast/distributed_halo.py:57-205):
tiles enumerate product(face, ti, tj) and rank r owns the contiguous slice
[r * tiles_per_rank, (r + 1) * tiles_per_rank).

The halo of a tile is built by COPY from the neighbouring tile or face — the index logic of the
reference's face padding (screamcast/cubesphere_transforms.py:149-445): edge strips of the
neighbouring face re-oriented into this face's frame, and corner blocks filled by the diagonal
rule. Here that logic is compiled once into gather maps (`halo_source_maps`): for every cell of
every padded local tile, the id of the interior cell it copies (and, on a corner diagonal, the
second cell it averages with). The GPU gather kernel then applies face-edge rotation and
corner rule by following the map, reading the source cell from local or peer memory.

Conventions (as in the reference): arrays are [row i, col j]; "bottom" = first rows, "top" =
last rows, "left" = first columns, "right" = last columns; face layout
    | 5 |
    | 0 | 1 | 2 | 3 |
    | 4 |
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass

import numpy as np
import torch

Tile = tuple  # (face, tile_i, tile_j)

# FACE_LINKS[face][side] = (neighbour face, neighbour's edge that touches this side)
FACE_LINKS = (
    {"top": (5, "bottom"), "right": (1, "left"), "bottom": (4, "top"), "left": (3, "right")},
    {"top": (5, "right"), "right": (2, "left"), "bottom": (4, "right"), "left": (0, "right")},
    {"top": (5, "top"), "right": (3, "left"), "bottom": (4, "bottom"), "left": (1, "right")},
    {"top": (5, "left"), "right": (0, "left"), "bottom": (4, "left"), "left": (2, "right")},
    {"top": (0, "bottom"), "right": (1, "bottom"), "bottom": (2, "bottom"), "left": (3, "bottom")},
    {"top": (2, "top"), "right": (1, "top"), "bottom": (0, "top"), "left": (3, "top")},
)


# ---------------------------------------------------------------- element order <-> face rasters
# The model's native column order lists, face by face, the ne x ne spectral elements and inside
# each element its npg x npg physics points; a face raster is the (ne*npg) x (ne*npg) image of
# the same values. Pure index permutations (bit-exact), interface of
# screamcast/cubesphere_transforms.py:20-146.

def _swap_element_axes(x: torch.Tensor, lead: tuple, a: int, b: int, c: int, d: int) -> torch.Tensor:
    """View the trailing block as [a, b, c, d] and exchange the two middle axes."""
    n = len(lead)
    return x.reshape(*lead, a, b, c, d).transpose(n + 1, n + 2)


def reorder_cubesphere_to_2d_tensor(array: torch.Tensor, *, ne: int, npg: int) -> torch.Tensor:
    """(..., ne*ne*npg*npg) element-major values of one face -> (..., ne*npg, ne*npg) raster."""
    if ne <= 0 or npg <= 0:
        raise ValueError(f"ne and npg must be positive, got ne={ne}, npg={npg}")
    expected = ne * ne * npg * npg
    if array.size(-1) != expected:
        raise ValueError(f"Expected last dim = {expected} (=ne^2*npg^2), got {array.size(-1)}")
    lead = tuple(array.shape[:-1])
    return _swap_element_axes(array, lead, ne, ne, npg, npg).reshape(*lead, ne * npg, ne * npg)


def reorder_2d_tensor_to_cubesphere(array: torch.Tensor, *, ne: int, npg: int) -> torch.Tensor:
    """Inverse of reorder_cubesphere_to_2d_tensor: (..., ne*npg, ne*npg) -> (..., ne*ne*npg*npg)."""
    if ne <= 0 or npg <= 0:
        raise ValueError(f"ne and npg must be positive, got ne={ne}, npg={npg}")
    side = ne * npg
    if array.shape[-1] != side or array.shape[-2] != side:
        raise ValueError(f"Expected last two dims = ({side}, {side}), got {tuple(array.shape[-2:])}")
    lead = tuple(array.shape[:-2])
    return _swap_element_axes(array, lead, ne, npg, ne, npg).reshape(*lead, ne * ne * npg * npg)


def unstructured_to_6faces(data: torch.Tensor, ne: int = 1024, npg: int = 2) -> torch.Tensor:
    """(..., 6*ne^2*npg^2) global columns -> (..., 6, ne*npg, ne*npg) face rasters."""
    per_face = (ne * npg) ** 2
    if data.shape[-1] != 6 * per_face:
        raise ValueError(f"Expected last dim = {6 * per_face} (=6*ne^2*npg^2), got {data.shape[-1]}")
    faces = data.reshape(*data.shape[:-1], 6, per_face)
    return reorder_cubesphere_to_2d_tensor(faces, ne=ne, npg=npg)


def faces_to_unstructured(data: torch.Tensor, ne: int = 1024, npg: int = 2) -> torch.Tensor:
    """Inverse of unstructured_to_6faces: (..., 6, ne*npg, ne*npg) -> (..., 6*ne^2*npg^2)."""
    side = ne * npg
    if data.dim() < 3 or tuple(data.shape[-3:]) != (6, side, side):
        raise ValueError(f"Expected last 3 dims = (6, {side}, {side}), got {tuple(data.shape[-3:])}")
    flat = reorder_2d_tensor_to_cubesphere(data, ne=ne, npg=npg)
    return flat.reshape(*data.shape[:-3], 6 * side * side)


@dataclass(frozen=True)
class TileTopology:
    """Distributed cubed-sphere tile decomposition (same fields and methods as the reference)."""

    world_size: int
    rank: int
    face_size: int
    tile_size: int
    halo_width: int
    n_faces: int = 6

    def __post_init__(self) -> None:
        if self.face_size % self.tile_size != 0:
            raise ValueError(
                f"face_size={self.face_size} must be divisible by tile_size={self.tile_size}")
        if self.total_tiles % self.world_size != 0:
            raise ValueError(f"Number of tiles ({self.total_tiles}) must be divisible by "
                             f"world_size ({self.world_size})")

    @property
    def tiles_per_dim(self) -> int:
        return self.face_size // self.tile_size

    @property
    def total_tiles(self) -> int:
        return self.n_faces * self.tiles_per_dim * self.tiles_per_dim

    @property
    def tiles_per_rank(self) -> int:
        return self.total_tiles // self.world_size

    @property
    def padded_tile_size(self) -> int:
        return self.tile_size + 2 * self.halo_width

    @property
    def global_tiles(self) -> list:
        return list(itertools.product(range(self.n_faces), range(self.tiles_per_dim),
                                      range(self.tiles_per_dim)))

    @property
    def local_tiles(self) -> list:
        start = self.rank * self.tiles_per_rank
        return self.global_tiles[start:start + self.tiles_per_rank]

    def interior_origin(self, tile: Tile) -> tuple:
        _, ti, tj = tile
        return ti * self.tile_size, tj * self.tile_size

    def _tile_coords(self, coords: dict, size: int) -> dict:
        out = dict(coords)
        out["face"] = np.arange(len(self.local_tiles))
        out["x"] = np.arange(size)
        out["y"] = np.arange(size)
        return out

    def interior_coords(self, base_coords: dict, *, time=None) -> dict:
        coords = dict(base_coords)
        if time is not None:
            coords["time"] = time
        return self._tile_coords(coords, self.tile_size)

    def pad_coords(self, coords: dict) -> dict:
        return self._tile_coords(coords, self.padded_tile_size)

    def crop_coords(self, coords: dict) -> dict:
        return self._tile_coords(coords, self.tile_size)

    def crop(self, x):
        h = self.halo_width
        return x if h == 0 else x[..., h:-h, h:-h]

    def faces_to_local_tiles(self, x: torch.Tensor) -> torch.Tensor:
        """(..., n_faces, N, N) -> (..., tiles_per_rank, T, T); no communication."""
        ts = self.tile_size
        return torch.stack([x[..., f, ti * ts:(ti + 1) * ts, tj * ts:(tj + 1) * ts]
                            for f, ti, tj in self.local_tiles], dim=-3)

    def gather_tiles_to_faces(self, x: torch.Tensor) -> torch.Tensor:
        """All-gather local interior tiles (..., tiles_per_rank, T, T) into (..., 6, N, N)."""
        *lead, tpr, nx, ny = x.shape
        if tpr != self.tiles_per_rank:
            raise ValueError(f"Expected {self.tiles_per_rank} local tiles, got {tpr}")
        if nx != self.tile_size or ny != self.tile_size:
            raise ValueError(f"Expected interior tile shape ({self.tile_size}, {self.tile_size}), "
                             f"got ({nx}, {ny})")
        if self.world_size == 1:
            gathered = x
        else:
            parts = [torch.zeros_like(x) for _ in range(self.world_size)]
            torch.distributed.all_gather(parts, x.contiguous())
            gathered = torch.cat(parts, dim=-3)
        out = gathered.new_zeros(*lead, self.n_faces, self.face_size, self.face_size)
        ts = self.tile_size
        for g, (f, ti, tj) in enumerate(self.global_tiles):
            out[..., f, ti * ts:(ti + 1) * ts, tj * ts:(tj + 1) * ts] = gathered[..., g, :, :]
        return out


# --------------------------------------------------------------------------- halo maps
def _edge_source(face: int, side: str, depth: np.ndarray, along: np.ndarray, N: int):
    """Source cell (face', i', j') of the halo cells beyond `side` of `face`.

    depth: distance outwards from the edge (0 = the halo line touching the face);
    along: position along the edge in this face's own row/column direction.
    The copied cell sits at the same depth INSIDE the neighbouring face; its position along
    the neighbour's edge runs the same or the opposite way depending on the two sides.
    """
    nb, nb_edge = FACE_LINKS[face][side]
    # position along the strip once it is laid out the canonical way
    canon = along if side in ("top", "left") else N - 1 - along
    u = canon if nb_edge in ("bottom", "right") else N - 1 - canon
    if nb_edge == "bottom":
        i, j = depth, u
    elif nb_edge == "top":
        i, j = N - 1 - depth, u
    elif nb_edge == "left":
        i, j = u, depth
    else:  # right
        i, j = u, N - 1 - depth
    return np.full_like(i, nb), i, j


def face_halo_sources(N: int, p: int):
    """Sources of every cell of the 6 padded faces.

    Returns (src_a, src_b), int64 arrays [6, N+2p, N+2p] of flat ids f*N*N + i*N + j into the
    unpadded faces. src_b is -1 except on corner diagonals, where the cell is the mean of the
    two sources.
    """
    S = N + 2 * p
    I, J = np.meshgrid(np.arange(S), np.arange(S), indexing="ij")
    src_a = np.full((6, S, S), -1, dtype=np.int64)
    src_b = np.full((6, S, S), -1, dtype=np.int64)
    inside_i = (I >= p) & (I < p + N)
    inside_j = (J >= p) & (J < p + N)

    def flat(f, i, j):
        return f * N * N + i * N + j

    for face in range(6):
        a = src_a[face]
        m = inside_i & inside_j
        a[m] = flat(face, I[m] - p, J[m] - p)
        regions = {
            "bottom": ((I < p) & inside_j, lambda: (p - 1 - I, J - p)),
            "top": ((I >= p + N) & inside_j, lambda: (I - (p + N), J - p)),
            "left": (inside_i & (J < p), lambda: (p - 1 - J, I - p)),
            "right": (inside_i & (J >= p + N), lambda: (J - (p + N), I - p)),
        }
        for side, (mask, da) in regions.items():
            depth, along = da()
            f2, i2, j2 = _edge_source(face, side, depth[mask], along[mask], N)
            a[mask] = flat(f2, i2, j2)
    if p == 0:
        return src_a, src_b
    # Corner blocks: each cell looks sideways to the vertical-strip neighbour in its own row
    # (column `vcol` of the bottom/top halo) and up/down to the horizontal-strip neighbour in its
    # own column (row `hrow` of the left/right halo); which of the two it copies is decided by
    # the side of the block's diagonal it lies on, the diagonal itself takes their mean.
    lo, hi = p, p + N - 1
    li = np.arange(p)[:, None]
    lj = np.arange(p)[None, :]
    main_upper, main_lower = li < lj, li > lj
    anti_upper, anti_lower = (li + lj) < (p - 1), (li + lj) > (p - 1)
    corner_specs = (
        (0, 0, lo, lo, main_upper, main_lower),            # bottom-left
        (0, p + N, hi, lo, anti_upper, anti_lower),        # bottom-right
        (p + N, 0, lo, hi, anti_lower, anti_upper),        # top-left
        (p + N, p + N, hi, hi, main_lower, main_upper),    # top-right
    )
    for face in range(6):
        edges = src_a[face].copy()
        for r0, c0, vcol, hrow, take_v, take_h in corner_specs:
            v = np.broadcast_to(edges[r0:r0 + p, vcol:vcol + 1], (p, p))
            h = np.broadcast_to(edges[hrow:hrow + 1, c0:c0 + p], (p, p))
            diag = ~(take_v | take_h)
            src_a[face, r0:r0 + p, c0:c0 + p] = np.where(take_h, h, v)
            src_b[face, r0:r0 + p, c0:c0 + p] = np.where(diag, h, -1)
    return src_a, src_b


def halo_source_maps(topo: TileTopology):
    """Gather maps for this rank's padded tiles.

    Returns (src_a, src_b): int32 arrays [tiles_per_rank, P, P] (P = padded tile size) of
    GLOBAL cell ids  g * T*T + i*T + j  where g indexes `global_tiles` (so the owning rank is
    id // (tiles_per_rank*T*T) and the offset inside that rank's buffer is the remainder).
    src_b = -1 except where the cell is the mean of two sources.
    """
    N, T, h = topo.face_size, topo.tile_size, topo.halo_width
    tpd = topo.tiles_per_dim
    fa, fb = face_halo_sources(N, h)

    def to_tile_ids(ids):
        f, rem = np.divmod(ids, N * N)
        i, j = np.divmod(rem, N)
        g = f * tpd * tpd + (i // T) * tpd + (j // T)
        out = g * T * T + (i % T) * T + (j % T)
        return np.where(ids < 0, -1, out)

    P = T + 2 * h
    a = np.empty((topo.tiles_per_rank, P, P), dtype=np.int64)
    b = np.empty_like(a)
    for n, (f, ti, tj) in enumerate(topo.local_tiles):
        sl = (f, slice(ti * T, ti * T + P), slice(tj * T, tj * T + P))
        a[n] = to_tile_ids(fa[sl])
        b[n] = to_tile_ids(fb[sl])
    if topo.total_tiles * T * T >= 2 ** 31:
        raise ValueError("grid too large for 32-bit cell ids")
    return a.astype(np.int32), b.astype(np.int32)


def apply_maps_numpy(all_tiles: np.ndarray, src_a: np.ndarray, src_b: np.ndarray) -> np.ndarray:
    """Host evaluation of the maps (used by tests and set-up code, e.g. to pad lat/lon grids):
    all_tiles (..., total_tiles, T, T) in global order -> (..., tiles_per_rank, P, P)."""
    lead = all_tiles.shape[:-3]
    flat = all_tiles.reshape(*lead, -1)
    va = flat[..., src_a]
    vb = flat[..., np.where(src_b < 0, 0, src_b)]
    return np.where(src_b < 0, va, (va + vb) / 2).astype(all_tiles.dtype)


def halo_adjoint_lists(topo: TileTopology, window: np.ndarray | None = None):
    """Transpose of the halo gather, as pull lists for this rank's interior cells.

    The gather fills padded cell p with x[a(p)] (or the mean of x[a(p)] and x[b(p)]). Its
    transpose sends every padded cell's value back to the interior cell(s) it was copied from.
    Seen from an interior cell c that is a list of padded cells - its own image in its own
    tile, plus its copies in the halos of neighbouring tiles, on whichever rank they live -
    with a coefficient each (1, or 1/2 for a corner mean).

    Returns (offsets int32 [n_local + 1], cell int32 [n_entries], coef float32 [n_entries],
    weights float32 [n_local]): entries of local interior cell c are offsets[c]:offsets[c+1],
    sorted by padded-cell id; `cell` is the GLOBAL padded cell id  g*P*P + pi*P + pj  (g in
    global tile order, so the owning rank is id // (tiles_per_rank*P*P)); weights[c] =
    sum coef * window[pi, pj] (window of ones by default) - the normaliser of the windowed
    overlap-add (reference: NormalizedHaloAdjoint, screamcast/distributed_halo.py:330-448).
    """
    T, P = topo.tile_size, topo.padded_tile_size
    full = TileTopology(1, 0, topo.face_size, T, topo.halo_width)
    a, b = halo_source_maps(full)                       # [G, P, P], global interior cell ids
    pid = np.arange(a.size, dtype=np.int64)
    af, bf = a.reshape(-1).astype(np.int64), b.reshape(-1).astype(np.int64)
    single = bf < 0
    src = np.concatenate([af[single], af[~single], bf[~single]])
    dst = np.concatenate([pid[single], pid[~single], pid[~single]])
    coef = np.concatenate([np.ones(single.sum(), np.float32),
                           np.full(2 * (~single).sum(), 0.5, np.float32)])
    return _pull_lists(topo, src, dst, coef, window)


def _pull_lists(topo: TileTopology, src: np.ndarray, dst: np.ndarray, coef: np.ndarray, window):
    """Entries (interior cell src <- padded cell dst, coefficient) of a gather operator, grouped
    by this rank's interior cells: (offsets, cell, coef, weights) as `halo_adjoint_lists` returns."""
    T, P = topo.tile_size, topo.padded_tile_size
    n_local = topo.tiles_per_rank * T * T
    lo = topo.rank * n_local
    keep = (src >= lo) & (src < lo + n_local)
    src, dst, coef = src[keep] - lo, dst[keep], coef[keep].astype(np.float32)
    order = np.lexsort((dst, src))
    src, dst, coef = src[order], dst[order], coef[order]
    offsets = np.zeros(n_local + 1, dtype=np.int64)
    np.add.at(offsets, src + 1, 1)
    offsets = np.cumsum(offsets)
    if dst.size and dst.max() >= 2 ** 31:
        raise ValueError("grid too large for 32-bit padded cell ids")
    w = np.ones((P, P), np.float32) if window is None else np.asarray(window, np.float32)
    if w.shape != (P, P):
        raise ValueError(f"window must be [{P}, {P}]")
    wv = (coef * w.reshape(-1)[dst % (P * P)]).astype(np.float32)
    weights = np.zeros(n_local, dtype=np.float32)
    # same summation order as the kernel: entry by entry, in float32
    k = np.arange(dst.size) - offsets[src]
    for j in range(int(k.max()) + 1 if dst.size else 0):
        m = k == j
        weights[src[m]] = (weights[src[m]] + wv[m]).astype(np.float32)
    return offsets.astype(np.int32), dst.astype(np.int32), coef, weights


def knn_adjoint_lists(topo: TileTopology, idx_all: np.ndarray, weights_all: np.ndarray,
                      window: np.ndarray | None = None):
    """Transpose of the k-nearest-neighbour halo operator A (out[p] = sum_j w[p, j] x[idx[p, j]]),
    as pull lists for this rank's interior cells - the operator whose normalised transpose
    D_w^-1 A^T (w . y) the reference's NormalizedHaloAdjoint applies
    (screamcast/distributed_halo.py:330-448, there as a vector-Jacobian product of the regrid
    followed by a reduce_scatter).

    idx_all / weights_all: [total_tiles*P*P, k] for the padded cells of EVERY tile of the globe in
    global tile order (the concatenation of all ranks' `knn_halo_weights` results). Returns the
    same four arrays as `halo_adjoint_lists`; an interior cell that no padded cell draws on gets
    weight 0 (and the kernel's division then yields NaN for it, as the reference's does).
    """
    P = topo.padded_tile_size
    n_padded = topo.total_tiles * P * P
    idx_all = np.asarray(idx_all)
    weights_all = np.asarray(weights_all, np.float32)
    if idx_all.shape != weights_all.shape or idx_all.ndim != 2 or idx_all.shape[0] != n_padded:
        raise ValueError(f"idx_all / weights_all must be [{n_padded}, k]")
    k = idx_all.shape[1]
    src = idx_all.reshape(-1).astype(np.int64)
    dst = np.repeat(np.arange(n_padded, dtype=np.int64), k)
    return _pull_lists(topo, src, dst, weights_all.reshape(-1), window)


def knn_halo_weights(topo: TileTopology, lon_deg: np.ndarray, lat_deg: np.ndarray,
                     pad_width_data: int, k: int = 4, eps: float = 1e-7):
    """k-nearest-neighbour interpolation weights of this rank's padded tiles.

    lon_deg / lat_deg: padded face grids [6, N + 2*pad, N + 2*pad] (degrees) that carry the TRUE
    coordinates of the cells beyond each face edge (reference input:
    DistributedTileKNNHaloPadding_AllGather.from_padded_face_grid,
    screamcast/distributed_halo.py:225-303). Sources are the interior cells of every tile of
    the globe; every padded cell of a local tile (its window of the padded face grid) gets its
    k nearest sources on the sphere with inverse-distance weights 1 / (chord distance + eps),
    normalised. A cell that coincides with a source gets (almost) all the weight: interiors
    are preserved, halos inside a face reproduce the neighbouring tile, halos across a face
    edge are interpolated between the neighbouring face's cells.

    Returns (idx int32 [tiles_per_rank*P*P, k] of GLOBAL interior cell ids g*T*T + i*T + j,
    weights float32 of the same shape).
    """
    from scipy.spatial import cKDTree
    T, h, N = topo.tile_size, topo.halo_width, topo.face_size
    pw = int(pad_width_data)
    if lon_deg.shape != lat_deg.shape or lon_deg.shape[0] != 6 or lon_deg.shape[1] != N + 2 * pw:
        raise ValueError(f"padded face grids must be [6, {N + 2 * pw}, {N + 2 * pw}]")
    if pw < h:
        raise ValueError("pad_width_data must cover the halo width")

    def unit(lon, lat):
        lo, la = np.radians(lon.astype(np.float64)), np.radians(lat.astype(np.float64))
        return np.stack([np.cos(la) * np.cos(lo), np.cos(la) * np.sin(lo), np.sin(la)], axis=-1)
    full = TileTopology(1, 0, N, T, h)
    src = np.concatenate([unit(lon_deg[f, pw + ti * T:pw + (ti + 1) * T, pw + tj * T:pw + (tj + 1) * T],
                               lat_deg[f, pw + ti * T:pw + (ti + 1) * T, pw + tj * T:pw + (tj + 1) * T]
                               ).reshape(-1, 3) for f, ti, tj in full.global_tiles])
    dst = np.concatenate([unit(lon_deg[f, pw + ti * T - h:pw + (ti + 1) * T + h,
                                       pw + tj * T - h:pw + (tj + 1) * T + h],
                               lat_deg[f, pw + ti * T - h:pw + (ti + 1) * T + h,
                                       pw + tj * T - h:pw + (tj + 1) * T + h]).reshape(-1, 3)
                          for f, ti, tj in topo.local_tiles])
    if src.shape[0] >= 2 ** 31:
        raise ValueError("grid too large for 32-bit cell ids")
    dist, idx = cKDTree(src).query(dst, k=k)
    if k == 1:
        dist, idx = dist[:, None], idx[:, None]
    lam = 1.0 / (dist + eps)
    lam = lam / lam.sum(axis=1, keepdims=True)
    return idx.astype(np.int32), lam.astype(np.float32)


# --------------------------------------------------------------------------- plan-based KNN halo
@dataclass
class TileSendEntry:
    """One (source tile -> part of a destination tile's halo) entry of a plan, as the reference
    lays it out (screamcast/distributed_cubesphere_transforms.py:48-55). The regridder state is
    {"index": int64 [n, k] cells of the source tile (row-major T*T), "weight": float32 [n, k]}."""

    src_tile: tuple
    regridder_state_dict: dict
    dst_halo_positions: torch.Tensor


@dataclass
class TileHaloPlan:
    """Routing plan of the tile-level KNN halo: fields of the reference's TileHaloPlan
    (screamcast/distributed_cubesphere_transforms.py:57-78) plus the same information as dense
    tables, which is what the gather kernel consumes.

    Every tile has the same halo cells (`halo_positions`: flat row-major positions in the padded
    tile, ascending). Halo cell n of tile g is interpolated from the k cells `knn_index[g, n]`
    (row-major inside the source tile) of tile `src_tile_id[g, n]` with `knn_weight[g, n]`.
    """

    face_size: int
    tile_size: int
    tiles_per_dim: int
    halo_width: int
    ne: int
    npg: int
    world_size: int
    tiles_per_rank: int
    tile_to_rank: dict
    recv_counts: dict
    send_sizes: dict
    recv_sizes: dict
    halo_positions: np.ndarray      # [n_halo] int64
    src_tile_id: np.ndarray         # [total_tiles, n_halo] int32
    knn_index: np.ndarray           # [total_tiles, n_halo, k] int32
    knn_weight: np.ndarray          # [total_tiles, n_halo, k] float32

    @property
    def send_plans(self) -> dict:
        """send_plans[src_rank][(face, ti, tj) of the destination] = [TileSendEntry, ...], built
        on demand from the tables (one entry per source tile, ascending tile id)."""
        tpd = self.tiles_per_dim
        out = {r: {} for r in range(self.world_size)}
        for g in range(self.src_tile_id.shape[0]):
            dst_tile = tile_id_to_tuple(g, tpd)
            for s in np.unique(self.src_tile_id[g]):
                m = self.src_tile_id[g] == s
                src_tile = tile_id_to_tuple(int(s), tpd)
                entry = TileSendEntry(
                    src_tile=src_tile,
                    regridder_state_dict={
                        "index": torch.from_numpy(self.knn_index[g][m].astype(np.int64)),
                        "weight": torch.from_numpy(self.knn_weight[g][m])},
                    dst_halo_positions=torch.from_numpy(self.halo_positions[m]))
                out[self.tile_to_rank[src_tile]].setdefault(dst_tile, []).append(entry)
        return out


def tile_halo_plan_from_reference(plan) -> TileHaloPlan:
    """Dense tables from a plan in the reference's layout - e.g. one that the reference's own
    `build_distributed_tile_halo_plan` produced with earth2grid's interpolator and saved - so
    that its exact weights are used. `plan` needs the reference TileHaloPlan's attributes;
    every `send_plans[src_rank][dst_tile]` entry needs `src_tile`, `dst_halo_positions` [n] and
    a `regridder_state_dict` with "index" [n, k] (cells of the source tile, row-major) and
    "weight" (or "weights") [n, k]."""
    T, h, tpd = int(plan.tile_size), int(plan.halo_width), int(plan.tiles_per_dim)
    total = 6 * tpd * tpd
    pos = tile_halo_positions(T, h)
    where = {int(pp): n for n, pp in enumerate(pos)}
    src_tile_id = np.full((total, len(pos)), -1, np.int32)
    knn_index = knn_weight = None
    for by_dst in plan.send_plans.values():
        for dst_tile, entries in by_dst.items():
            g = tile_tuple_to_id(*dst_tile, tpd)
            for e in entries:
                sd = e.regridder_state_dict
                index = np.asarray(sd["index"]).reshape(len(e.dst_halo_positions), -1)
                weight = np.asarray(sd["weight"] if "weight" in sd else sd["weights"], np.float32
                                    ).reshape(index.shape)
                if knn_index is None:
                    k = index.shape[1]
                    knn_index = np.zeros((total, len(pos), k), np.int32)
                    knn_weight = np.zeros((total, len(pos), k), np.float32)
                rows = np.array([where[int(pp)] for pp in np.asarray(e.dst_halo_positions)], np.int64)
                if (src_tile_id[g, rows] >= 0).any():
                    raise ValueError(f"halo positions of tile {dst_tile} listed twice")
                src_tile_id[g, rows] = tile_tuple_to_id(*e.src_tile, tpd)
                knn_index[g, rows] = index
                knn_weight[g, rows] = weight
    if len(pos) and (knn_index is None or (src_tile_id < 0).any()):
        raise ValueError("the plan does not cover every halo cell of every tile")
    if knn_index is None:
        knn_index = np.zeros((total, 0, 1), np.int32)
        knn_weight = np.zeros((total, 0, 1), np.float32)
    return TileHaloPlan(face_size=int(plan.face_size), tile_size=T, tiles_per_dim=tpd, halo_width=h,
                        ne=int(plan.ne), npg=int(plan.npg), world_size=int(plan.world_size),
                        tiles_per_rank=int(plan.tiles_per_rank), tile_to_rank=dict(plan.tile_to_rank),
                        recv_counts=dict(plan.recv_counts), send_sizes=dict(plan.send_sizes),
                        recv_sizes=dict(plan.recv_sizes), halo_positions=pos, src_tile_id=src_tile_id,
                        knn_index=knn_index, knn_weight=knn_weight)


def tile_id_to_tuple(tile_id: int, tiles_per_dim: int) -> tuple:
    """Linear tile id -> (face, ti, tj) (reference _tile_id_to_tuple, :174-181)."""
    face, rem = divmod(int(tile_id), tiles_per_dim * tiles_per_dim)
    return (face, rem // tiles_per_dim, rem % tiles_per_dim)


def tile_tuple_to_id(face: int, ti: int, tj: int, tiles_per_dim: int) -> int:
    return face * tiles_per_dim * tiles_per_dim + ti * tiles_per_dim + tj


def build_tile_to_rank_map(tiles_per_dim: int, world_size: int) -> dict:
    """(face, ti, tj) -> rank: consecutive tile ids in equal shares (reference :189-199)."""
    total = 6 * tiles_per_dim * tiles_per_dim
    per_rank = total // world_size
    return {tile_id_to_tuple(t, tiles_per_dim): t // per_rank for t in range(total)}


def tile_halo_positions(tile_size: int, halo_width: int) -> np.ndarray:
    """Flat row-major positions of the halo cells of a padded tile, ascending (the order in which
    the reference extracts a tile's halo, :262-283, and `_halo_dst_flat_indices_per_face`)."""
    S = tile_size + 2 * halo_width
    ii, jj = np.meshgrid(np.arange(S), np.arange(S), indexing="ij")
    halo = (ii < halo_width) | (ii >= halo_width + tile_size) | \
           (jj < halo_width) | (jj >= halo_width + tile_size)
    return (ii[halo] * S + jj[halo]).astype(np.int64)


def _unit_f32(lon_deg: np.ndarray, lat_deg: np.ndarray) -> np.ndarray:
    """Unit vectors in the precision the reference's assignment step works in (float32 degrees ->
    float32 radians -> float32 components, :126-141 and :319-324)."""
    lo, la = np.deg2rad(lon_deg.astype(np.float32)), np.deg2rad(lat_deg.astype(np.float32))
    return np.stack([np.cos(la) * np.cos(lo), np.cos(la) * np.sin(lo), np.sin(la)], axis=-1)


def _unit_f64(lon_deg: np.ndarray, lat_deg: np.ndarray) -> np.ndarray:
    lo, la = np.radians(lon_deg.astype(np.float64)), np.radians(lat_deg.astype(np.float64))
    return np.stack([np.cos(la) * np.cos(lo), np.cos(la) * np.sin(lo), np.sin(la)], axis=-1)


def padded_lonlat_from_target_grid(grid_tgt: dict, face_size: int, halo_width: int,
                                   num_pg_cells: int) -> np.ndarray:
    """(2, 6, S, S) lon / lat of the padded faces cut out of a padded target grid in element
    order (reference `_padded_lonlat_from_target_grid`, :346-401): the file's faces may carry a
    wider halo than asked for; the centred window of S = face_size + 2*halo_width is taken."""
    lon_t, lat_t = (np.asarray(grid_tgt[k]).astype(np.float32) for k in ("lon", "lat"))
    n_cells = len(lon_t)
    fs_file = int((n_cells / 6) ** 0.5)
    if fs_file * fs_file * 6 != n_cells:
        raise ValueError(f"Target grid has {n_cells} cells, not compatible with 6 square faces")
    ne_file = fs_file // num_pg_cells
    lon_f = unstructured_to_6faces(torch.from_numpy(lon_t), ne=ne_file, npg=num_pg_cells).numpy()
    lat_f = unstructured_to_6faces(torch.from_numpy(lat_t), ne=ne_file, npg=num_pg_cells).numpy()
    hw_file = (fs_file - face_size) // 2
    if halo_width > hw_file:
        raise ValueError(f"Requested halo_width={halo_width} exceeds target grid's "
                         f"halo_width_file={hw_file}")
    i0, i1 = hw_file - halo_width, hw_file + face_size + halo_width
    S = face_size + 2 * halo_width
    out = np.stack([lon_f[:, i0:i1, i0:i1], lat_f[:, i0:i1, i0:i1]], axis=0)
    if out.shape != (2, 6, S, S):
        raise ValueError(f"Expected padded shape (6, {S}, {S}), got {out.shape[1:]}")
    return out


def build_distributed_tile_halo_plan(grid_src: dict, num_elements: int, tile_size: int,
                                     halo_width: int, num_pg_cells: int = 2, k: int = 4,
                                     eps: float = 1e-7, world_size: int = 96,
                                     grid_tgt: dict | None = None) -> TileHaloPlan:
    """Routing plan of the tile-level KNN halo (same arguments and meaning as the reference's
    build_distributed_tile_halo_plan, screamcast/distributed_cubesphere_transforms.py:404-608).

    grid_src: {"lon": (6*N*N,), "lat": (6*N*N,)} degrees, element order. Every halo cell of every
    tile gets a position on the sphere - from `grid_tgt` (a padded grid in element order) when
    given, otherwise from the face-level copy / rot90 / corner padding of the source lon / lat -
    then ONE source tile: the face whose nearest cell is closest (ties: lowest face), and on
    that face the tile holding the nearest cell. Its value is the inverse-distance-weighted mean
    (1 / (chord distance + eps), normalised) of the k nearest cells of THAT tile. The reference
    builds one earth2grid regridder per (source tile, destination tile) pair; here the same
    index / weight lists are kept as dense tables.
    """
    from scipy import spatial
    face_size = num_elements * num_pg_cells
    if face_size % tile_size != 0:
        raise ValueError(f"face_size={face_size} must be divisible by tile_size={tile_size}")
    tpd = face_size // tile_size
    total_tiles = 6 * tpd * tpd
    if total_tiles % world_size != 0:
        raise ValueError(f"total_tiles={total_tiles} must be divisible by world_size={world_size}")
    tiles_per_rank = total_tiles // world_size
    tile_to_rank = build_tile_to_rank_map(tpd, world_size)
    T, h, N = tile_size, halo_width, face_size

    lon_faces, lat_faces = (unstructured_to_6faces(
        torch.from_numpy(np.asarray(grid_src[key]).astype(np.float32)), ne=num_elements,
        npg=num_pg_cells).numpy() for key in ("lon", "lat"))
    if grid_tgt is not None:
        padded = padded_lonlat_from_target_grid(grid_tgt, face_size, halo_width, num_pg_cells)
    else:
        a, b = face_halo_sources(N, h)
        padded = np.stack([apply_face_maps(lon_faces, a, b), apply_face_maps(lat_faces, a, b)])
    padded_lon, padded_lat = padded[0], padded[1]

    face_xyz = _unit_f32(lon_faces, lat_faces).reshape(6, N * N, 3)
    face_trees = [spatial.KDTree(face_xyz[f]) for f in range(6)]
    # One tree over all six faces finds the nearest face of a halo cell in a single query (a
    # nearest-neighbour query against a face on the far side of the sphere walks most of that
    # face's tree, and the reference's six queries per cell are what makes its plan slow). The
    # reference's rule - lowest face among those at the minimum distance - is kept by looking at
    # every neighbour at exactly that distance; the cell inside the face then comes from the
    # face's own tree, as in the reference.
    globe_tree = spatial.cKDTree(face_xyz.reshape(6 * N * N, 3))
    k_face = min(8, 6 * N * N)
    tile_trees: dict = {}

    def tree_of_tile(g: int):
        if g not in tile_trees:
            f, ti, tj = tile_id_to_tuple(g, tpd)
            sl = (f, slice(ti * T, (ti + 1) * T), slice(tj * T, (tj + 1) * T))
            tile_trees[g] = spatial.cKDTree(_unit_f64(lon_faces[sl], lat_faces[sl]).reshape(-1, 3))
        return tile_trees[g]

    pos = tile_halo_positions(T, h)
    n_halo = len(pos)
    S = T + 2 * h
    src_tile_id = np.zeros((total_tiles, n_halo), np.int32)
    knn_index = np.zeros((total_tiles, n_halo, k), np.int32)
    knn_weight = np.zeros((total_tiles, n_halo, k), np.float32)
    recv_counts: dict = {}
    send_sizes = {sr: {dr: 0 for dr in range(world_size)} for sr in range(world_size)}
    for g in range(total_tiles):
        dst_tile = tile_id_to_tuple(g, tpd)
        recv_counts[dst_tile] = {}
        if n_halo == 0:
            continue
        f, ti, tj = dst_tile
        hl_lon = padded_lon[f, ti * T:ti * T + S, tj * T:tj * T + S].reshape(-1)[pos].astype(np.float32)
        hl_lat = padded_lat[f, ti * T:ti * T + S, tj * T:tj * T + S].reshape(-1)[pos].astype(np.float32)
        q32 = _unit_f32(hl_lon, hl_lat)
        gd, gi = globe_tree.query(q32, k=k_face)
        if k_face == 1:
            gd, gi = gd[:, None], gi[:, None]
        cand = np.where(gd == gd[:, :1], gi // (N * N), 6)       # faces of the neighbours at the minimum
        best_face = cand.min(axis=1).astype(np.int64)
        cell = np.zeros(n_halo, np.int64)
        for face_id in np.unique(best_face):
            m = best_face == face_id
            cell[m] = np.asarray(face_trees[face_id].query(q32[m], k=1)[1]).reshape(-1)
        src = best_face * tpd * tpd + (cell // N // T) * tpd + (cell % N) // T
        src_tile_id[g] = src
        q64 = _unit_f64(hl_lon, hl_lat)
        for s in np.unique(src):
            m = src == s
            dist, idx = tree_of_tile(int(s)).query(q64[m], k=k)
            if k == 1:
                dist, idx = dist[:, None], idx[:, None]
            lam = 1.0 / (dist + eps)
            knn_index[g][m] = idx
            knn_weight[g][m] = (lam / lam.sum(axis=1, keepdims=True)).astype(np.float32)
            sr = tile_to_rank[tile_id_to_tuple(int(s), tpd)]
            n = int(m.sum())
            recv_counts[dst_tile][sr] = recv_counts[dst_tile].get(sr, 0) + n
            send_sizes[sr][tile_to_rank[dst_tile]] += n
    recv_sizes = {dr: {sr: send_sizes[sr][dr] for sr in range(world_size)} for dr in range(world_size)}
    return TileHaloPlan(face_size=face_size, tile_size=T, tiles_per_dim=tpd, halo_width=h,
                        ne=num_elements, npg=num_pg_cells, world_size=world_size,
                        tiles_per_rank=tiles_per_rank, tile_to_rank=tile_to_rank,
                        recv_counts=recv_counts, send_sizes=send_sizes, recv_sizes=recv_sizes,
                        halo_positions=pos, src_tile_id=src_tile_id, knn_index=knn_index,
                        knn_weight=knn_weight)


def apply_face_maps(faces: np.ndarray, src_a: np.ndarray, src_b: np.ndarray) -> np.ndarray:
    """(..., 6, N, N) -> (..., 6, N+2p, N+2p) through the face-level source maps of
    `face_halo_sources` (copy, rot90 orientation, corner rule; diagonal cells = mean of two)."""
    lead = faces.shape[:-3]
    flat = faces.reshape(*lead, -1)
    va = flat[..., src_a]
    vb = flat[..., np.where(src_b < 0, 0, src_b)]
    return np.where(src_b < 0, va, (va + vb) / 2).astype(faces.dtype)


def plan_gather_lists(plan: TileHaloPlan, rank: int):
    """The plan as the weighted-gather kernel reads it: (idx int32 [tiles_per_rank*P*P, k] of
    GLOBAL interior cell ids g*T*T + i*T + j, weights float32) for this rank's padded tiles.
    An interior cell is itself with weight 1 (zeros for the other k-1 terms): copied exactly."""
    T, h = plan.tile_size, plan.halo_width
    P = T + 2 * h
    k = plan.knn_index.shape[2]
    tpr = plan.tiles_per_rank
    idx = np.zeros((tpr, P * P, k), np.int64)
    w = np.zeros((tpr, P * P, k), np.float32)
    ii, jj = np.meshgrid(np.arange(T), np.arange(T), indexing="ij")
    inner_pos = ((ii + h) * P + (jj + h)).reshape(-1)
    inner_cell = (ii * T + jj).reshape(-1)
    for n in range(tpr):
        g = rank * tpr + n
        idx[n, inner_pos, :] = (g * T * T + inner_cell)[:, None]
        w[n, inner_pos, 0] = 1.0
        if len(plan.halo_positions):
            idx[n, plan.halo_positions, :] = plan.src_tile_id[g].astype(np.int64)[:, None] * T * T + \
                plan.knn_index[g]
            w[n, plan.halo_positions, :] = plan.knn_weight[g]
    if plan.src_tile_id.shape[0] * T * T >= 2 ** 31:
        raise ValueError("grid too large for 32-bit cell ids")
    return idx.reshape(tpr * P * P, k).astype(np.int32), w.reshape(tpr * P * P, k)
