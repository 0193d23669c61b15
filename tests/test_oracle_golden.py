"""Pins the CPU oracle against fixtures generated from the reference's own in-tree code
(tests/golden/make_golden.py). Integer / index logic must match bit for bit."""
import numpy as np
import pytest

from oracle import halo_oracle as ho
from tests.golden.make_golden import payload


@pytest.fixture(scope="module")
def fp(golden_dir):
    return np.load(golden_dir / "face_padding.npz")


@pytest.mark.parametrize("name", ["n4p2", "n8p3", "n6p1", "n8p8"])
def test_create_padded_faces_bit_exact(fp, name):
    N, p, seed = int(fp[f"{name}_N"]), int(fp[f"{name}_p"]), int(fp[f"{name}_seed"])
    x = payload(3, N, seed)
    got = ho.create_padded_faces(x, p)
    want = fp[f"{name}_out"]
    assert got.dtype == want.dtype and got.shape == want.shape
    assert not np.isnan(got).any()
    assert np.array_equal(got, want)
    assert np.array_equal(ho.halo_dst_flat_indices(N, p), fp[f"{name}_halo_idx"])


def test_halo_cell_count_formula():
    # the reference's own count check: (N*h + h*h) * 4 * 6 halo cells
    for N, h in [(4, 2), (16, 3), (2048 // 64, 1)]:
        assert ho.halo_dst_flat_indices(N, h).size == (N * h + h * h) * 4 * 6


def test_face_reorder_round_trip(fp):
    u = fp["reorder_in"]
    faces = ho.unstructured_to_6faces(u, ne=3, npg=2)
    assert np.array_equal(faces, fp["reorder_faces"])
    assert np.array_equal(ho.faces_to_unstructured(faces, ne=3, npg=2), fp["reorder_back"])
    assert np.array_equal(fp["reorder_back"], u)


def test_tile_topology_known_answer():
    # the known answer held by the reference's tests/test_distributed_halo.py:26-46
    t = ho.TileTopology(world_size=4, rank=1, face_size=8, tile_size=4, halo_width=2)
    assert (t.tiles_per_dim, t.total_tiles, t.tiles_per_rank, t.padded_tile_size) == (2, 24, 6, 8)
    assert t.local_tiles == [(1, 1, 0), (1, 1, 1), (2, 0, 0), (2, 0, 1), (2, 1, 0), (2, 1, 1)]


def test_tile_topology_fixtures(golden_dir):
    g = np.load(golden_dir / "tile_topology.npz")
    for ci, (ws, rk, fs, ts, hw) in enumerate(g["cases"].tolist()):
        t = ho.TileTopology(ws, rk, fs, ts, hw)
        assert np.array_equal(np.array(t.local_tiles), g[f"c{ci}_local_tiles"])
        assert np.array_equal(np.array(t.global_tiles), g[f"c{ci}_global_tiles"])
        assert [t.tiles_per_dim, t.total_tiles, t.tiles_per_rank,
                t.padded_tile_size] == g[f"c{ci}_scalars"].tolist()
        x = payload(2, fs, 10 + ci)
        assert np.array_equal(t.faces_to_local_tiles(x), g[f"c{ci}_local_from_faces"])
        # all tiles of the globe in global order -> this rank's padded tiles
        full = ho.TileTopology(1, 0, fs, ts, hw)
        all_tiles = full.faces_to_local_tiles(x)
        got = ho.padded_local_tiles(all_tiles, t)
        assert np.array_equal(got, g[f"c{ci}_padded_local_tiles"])
        assert np.array_equal(t.crop(got), g[f"c{ci}_cropped"])
        assert np.array_equal(t.crop(got), t.faces_to_local_tiles(x))


def test_topology_rejects_bad_sizes():
    with pytest.raises(ValueError):
        ho.TileTopology(1, 0, 10, 4, 1)
    with pytest.raises(ValueError):
        ho.TileTopology(5, 0, 8, 4, 1)


def test_wind_rotation_and_centre(golden_dir):
    g = np.load(golden_dir / "wind_rotation.npz")
    lat0, lon0 = ho.tile_center(g["lat"], g["lon"])
    np.testing.assert_allclose(lat0, g["lat0"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(lon0, g["lon0"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(ho.mean_longitude(g["lon"], False), g["mean_lon_pm"], atol=1e-6)
    Ul, Vl = ho.forward_uv_to_tile(g["U"], g["V"], g["lat"], g["lon"], g["lat0"], g["lon0"])
    np.testing.assert_allclose(Ul, g["U_loc"], atol=2e-6)
    np.testing.assert_allclose(Vl, g["V_loc"], atol=2e-6)
    Ur, Vr = ho.inverse_tile_to_uv(g["U_loc"], g["V_loc"], g["lat"], g["lon"], g["lat0"], g["lon0"])
    np.testing.assert_allclose(Ur, g["U_rec"], atol=2e-6)
    np.testing.assert_allclose(Vr, g["V_rec"], atol=2e-6)
    np.testing.assert_allclose(Ur, g["U"], atol=1e-4)


def test_rope_length_scale_constant(golden_dir):
    import math
    from oracle import block_oracle as bo
    g = np.load(golden_dir / "wind_rotation.npz")
    for s, want in zip((1, 2, 4), g["rope_scale"].tolist()):
        assert bo.default_rope_length_scale(s) == want == math.sqrt(math.pi * s * s / (3.0 * 1024 ** 2))
