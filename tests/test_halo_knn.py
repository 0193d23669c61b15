"""k-nearest-neighbour halo weights (host set-up) against a brute-force oracle, and the
properties the reference's tests check for its KNN halo (tests/test_distributed_tile_halo.py:
97-293: interiors preserved, interior-tile halo equals the neighbouring tiles' data to 1e-3)."""
import numpy as np
import pytest

from oracle import halo_oracle as ho
from strata_b200.rollout import equiangular_cubed_sphere_latlon, padded_face_latlon
from strata_b200.topology import TileTopology, knn_adjoint_lists, knn_halo_weights

N, T, H, PW = 16, 4, 2, 4


def _apply(x_all, idx, w):
    """Host evaluation of the weighted gather in the kernel's order (float32, no FMA)."""
    lead = x_all.shape[:-3]
    flat = x_all.reshape(*lead, -1).astype(np.float32)
    acc = np.zeros((*lead, idx.shape[0]), np.float32)
    for j in range(idx.shape[1]):
        acc = (acc + (w[:, j] * flat[..., idx[:, j]]).astype(np.float32)).astype(np.float32)
    return acc


def test_padded_faces_extend_the_face_grid():
    lat, lon = padded_face_latlon(N, PW)
    la0, lo0 = equiangular_cubed_sphere_latlon(N)
    assert np.allclose(lat[:, PW:-PW, PW:-PW], la0) and np.allclose(lon[:, PW:-PW, PW:-PW], lo0)


@pytest.mark.parametrize("world,rank", [(1, 0), (2, 1), (3, 2)])
def test_weights_match_brute_force_and_preserve_interiors(world, rank):
    lat, lon = padded_face_latlon(N, PW)
    topo = TileTopology(world, rank, N, T, H)
    otopo = ho.TileTopology(world, rank, N, T, H)
    full = ho.TileTopology(1, 0, N, T, H)
    idx, w = knn_halo_weights(topo, lon, lat, PW)
    assert np.allclose(w.sum(1), 1.0, atol=1e-6) and (w >= 0).all()
    # smooth field: product lists and brute-force oracle interpolate to the same values (the
    # two searches may break ties between equidistant sources differently)
    la, lo = np.radians(equiangular_cubed_sphere_latlon(N))
    field = (np.sin(la) * np.cos(lo) + 0.3 * np.cos(2 * la)).astype(np.float32)
    tiles = np.stack([field[f, i * T:(i + 1) * T, j * T:(j + 1) * T] for f, i, j in full.global_tiles])
    want, oidx, ow = ho.knn_halo(tiles, otopo, lon, lat, PW)
    got = _apply(tiles, idx, w).reshape(want.shape)
    same = (np.sort(idx, 1) == np.sort(oidx, 1)).all(1)
    assert same.mean() > 0.98
    assert np.array_equal(got.reshape(-1)[same], want.reshape(-1)[same]) or \
        np.allclose(got.reshape(-1)[same], want.reshape(-1)[same], atol=1e-6)
    assert np.allclose(got, want, atol=2e-2)            # tie cells: neighbouring values of a smooth field
    # interiors: the nearest source of an interior cell is the cell itself, with all the weight
    P = T + 2 * H
    s = rank * topo.tiles_per_rank
    own = (np.arange(topo.tiles_per_rank)[:, None, None] + s) * T * T + \
        np.arange(T)[None, :, None] * T + np.arange(T)[None, None, :]
    i0 = idx[:, 0].reshape(topo.tiles_per_rank, P, P)[:, H:-H, H:-H]
    w0 = w[:, 0].reshape(topo.tiles_per_rank, P, P)[:, H:-H, H:-H]
    assert np.array_equal(i0, own) and (w0 > 0.9999).all()


def test_interior_tile_halo_equals_neighbour_data():
    # the reference's own check (test_distributed_tile_halo.py:249-293): pixel-coded payload,
    # tile (face 0, ti 1, tj 1), padded tile == the face window, atol = rtol = 1e-3
    lat, lon = padded_face_latlon(N, PW)
    topo = TileTopology(1, 0, N, T, H)
    idx, w = knn_halo_weights(topo, lon, lat, PW)
    faces = np.zeros((6, N, N), np.float32)
    for f in range(6):
        faces[f] = f * 1000 + np.arange(N)[:, None] * N + np.arange(N)[None, :]
    tiles = np.stack([faces[f, i * T:(i + 1) * T, j * T:(j + 1) * T] for f, i, j in topo.global_tiles])
    P = T + 2 * H
    padded = _apply(tiles, idx, w).reshape(topo.total_tiles, P, P)
    tpd = N // T
    t = 0 * tpd * tpd + 1 * tpd + 1
    want = faces[0, T - H:2 * T + H, T - H:2 * T + H]
    assert np.allclose(padded[t], want, atol=1e-3, rtol=1e-3)


def test_bad_grids_are_rejected():
    lat, lon = padded_face_latlon(N, PW)
    with pytest.raises(ValueError):
        knn_halo_weights(TileTopology(1, 0, N, T, H), lon[:, 1:], lat[:, 1:], PW)
    with pytest.raises(ValueError):
        knn_halo_weights(TileTopology(1, 0, N, T, 6), lon, lat, PW)


def _eval_lists(padded_all, lists, window, P):
    """D_w^-1 A^T (w . y) from the pull lists, in float64 (what the adjoint kernel computes)."""
    off, cell, coef, weights = lists
    flat = padded_all.reshape(*padded_all.shape[:-3], -1).astype(np.float64)
    win = window.reshape(-1).astype(np.float64)
    out = np.zeros((*flat.shape[:-1], off.size - 1))
    for c in range(off.size - 1):
        e = slice(off[c], off[c + 1])
        out[..., c] = (flat[..., cell[e]] * (coef[e].astype(np.float64) * win[cell[e] % (P * P)])).sum(-1)
    with np.errstate(invalid="ignore", divide="ignore"):
        return out / weights.astype(np.float64)


@pytest.mark.parametrize("world", [1, 2, 3])
def test_knn_adjoint_lists_are_the_transpose(world):
    # the reference's un-pad operator is the normalised transpose of the KNN regrid
    # (NormalizedHaloAdjoint, screamcast/distributed_halo.py:330-448)
    lat, lon = padded_face_latlon(N, PW)
    full = TileTopology(1, 0, N, T, H)
    P = T + 2 * H
    idx_all, w_all = knn_halo_weights(full, lon, lat, PW)
    rng = np.random.default_rng(5)
    y = rng.standard_normal((3, full.total_tiles, P, P)).astype(np.float32)
    x = rng.standard_normal((3, full.total_tiles * T * T))
    win = np.outer(np.hanning(P + 2)[1:-1], np.hanning(P + 2)[1:-1]).astype(np.float32) + 0.05
    got = []
    for rank in range(world):
        topo = TileTopology(world, rank, N, T, H)
        lists = knn_adjoint_lists(topo, idx_all, w_all, win)
        out = _eval_lists(y, lists, win, P)
        want = ho.knn_halo_adjoint(y, ho.TileTopology(world, rank, N, T, H), idx_all, w_all, win)
        assert np.allclose(out, want.reshape(out.shape), rtol=1e-5, atol=1e-6, equal_nan=True)
        # un-normalised: <A x, w y> == <x, A^T (w y)>
        off, cell, coef, weights = lists
        aty = out * weights.astype(np.float64)
        got.append(aty)
    aty = np.concatenate(got, axis=-1)
    ax = np.stack([(w_all[:, j].astype(np.float64) * x[:, idx_all[:, j]]) for j in range(idx_all.shape[1])]).sum(0)
    lhs = (ax * (y.reshape(3, -1) * np.tile(win.reshape(-1), full.total_tiles))).sum(-1)
    rhs = (x * aty).sum(-1)
    assert np.allclose(lhs, rhs, rtol=1e-5)
    # constant fields survive pad -> un-pad (reference: tests/distributed/test_distributed_halo.py:61-107)
    const = np.full((1, full.total_tiles, P, P), 3.25, np.float32)
    for rank in range(world):
        topo = TileTopology(world, rank, N, T, H)
        back = _eval_lists(const, knn_adjoint_lists(topo, idx_all, w_all, win), win, P)
        assert np.allclose(back, 3.25, atol=1e-3)
    with pytest.raises(ValueError, match="idx_all"):
        knn_adjoint_lists(full, idx_all[:-1], w_all[:-1])


def test_lists_forward_and_adjoint_equal_the_reference_modules():
    # outputs of the reference's DistributedTileKNNHaloPadding_AllGather and NormalizedHaloAdjoint
    # (screamcast/distributed_halo.py:208-448) at world_size 1, with earth2grid's interpolator
    # replaced by a stand-in of the same interface (tests/golden/make_plan_golden.py): the
    # selection of source and destination points, their order, the regrid and its normalised,
    # windowed transpose are the reference's code
    from pathlib import Path
    gold = np.load(Path(__file__).resolve().parent / "golden" / "knn_allgather_halo.npz")
    n, t, h, pw = (int(gold[k]) for k in ("face_size", "tile", "halo", "pad_width_data"))
    topo = TileTopology(1, 0, n, t, h)
    idx, w = knn_halo_weights(topo, gold["lon_padded"], gold["lat_padded"], pw)
    assert np.array_equal(idx, gold["index"])
    assert np.allclose(w, gold["weight"], rtol=0, atol=1e-7)
    got = _apply(gold["x"], idx, w).reshape(gold["forward"].shape)
    assert np.allclose(got, gold["forward"], rtol=0, atol=1e-6)
    otopo = ho.TileTopology(1, 0, n, t, h)
    for key, window in (("adjoint", None), ("adjoint_windowed", gold["window"])):
        want = gold[key].reshape(gold["padded_in"].shape[:-2] + (t, t))
        adj = ho.knn_halo_adjoint(gold["padded_in"], otopo, idx, w, window)
        assert np.allclose(adj, want, rtol=1e-5, atol=1e-5)
