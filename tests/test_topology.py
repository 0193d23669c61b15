"""Host-side tile topology and halo gather maps of the product, against the pinned oracle and
the golden fixtures produced by the reference. Bit-exact."""
import numpy as np
import pytest
import torch

from oracle import halo_oracle as ho
from strata_b200 import topology as tp
from tests.golden.make_golden import payload


def test_known_answer_partition():
    t = tp.TileTopology(world_size=4, rank=1, face_size=8, tile_size=4, halo_width=2)
    assert (t.tiles_per_dim, t.total_tiles, t.tiles_per_rank, t.padded_tile_size) == (2, 24, 6, 8)
    assert t.local_tiles == [(1, 1, 0), (1, 1, 1), (2, 0, 0), (2, 0, 1), (2, 1, 0), (2, 1, 1)]
    assert t.interior_origin((2, 1, 0)) == (4, 0)


def test_invalid_sizes_raise():
    with pytest.raises(ValueError, match="divisible by tile_size"):
        tp.TileTopology(1, 0, 10, 4, 1)
    with pytest.raises(ValueError, match="divisible by"):
        tp.TileTopology(5, 0, 8, 4, 1)


def test_coord_helpers():
    t = tp.TileTopology(world_size=1, rank=0, face_size=4, tile_size=2, halo_width=1)
    base = {"variable": np.array(["A", "B"]), "lead_time": np.array([0])}
    c = t.interior_coords(base, time=np.array([np.datetime64("2020-01-01")]))
    assert list(c) == ["variable", "lead_time", "time", "face", "x", "y"]
    assert len(c["face"]) == 24 and len(c["x"]) == 2
    assert len(t.pad_coords(c)["x"]) == 4 and len(t.crop_coords(t.pad_coords(c))["y"]) == 2


def test_fixtures_from_reference(golden_dir):
    g = np.load(golden_dir / "tile_topology.npz")
    for ci, (ws, rk, fs, ts, hw) in enumerate(g["cases"].tolist()):
        t = tp.TileTopology(ws, rk, fs, ts, hw)
        assert np.array_equal(np.array(t.local_tiles), g[f"c{ci}_local_tiles"])
        x = payload(2, fs, 10 + ci)
        lt = t.faces_to_local_tiles(torch.from_numpy(x)).numpy()
        assert np.array_equal(lt, g[f"c{ci}_local_from_faces"])
        full = tp.TileTopology(1, 0, fs, ts, hw)
        all_tiles = full.faces_to_local_tiles(torch.from_numpy(x)).numpy()
        a, b = tp.halo_source_maps(t)
        got = tp.apply_maps_numpy(all_tiles, a, b)
        assert np.array_equal(got, g[f"c{ci}_padded_local_tiles"])     # reference output
        assert np.array_equal(t.crop(got), g[f"c{ci}_cropped"])


@pytest.mark.parametrize("N,p", [(4, 2), (8, 3), (6, 1), (8, 8), (5, 0)])
def test_face_maps_match_reference_padding(golden_dir, N, p):
    a, b = tp.face_halo_sources(N, p)
    x = payload(3, N, 99)
    flat = x.reshape(3, -1)
    got = np.where(b < 0, flat[:, a], (flat[:, a] + flat[:, np.where(b < 0, 0, b)]) / 2)
    want = ho.create_padded_faces(x, p)
    assert np.array_equal(got.astype(np.float32), want)
    # coverage: every padded cell has a source; interior maps to itself
    assert (a >= 0).all()
    if p:
        assert (b >= 0).sum() == 6 * 4 * p          # one diagonal of length p per corner


@pytest.mark.parametrize("world,fs,ts,hw", [(1, 8, 4, 2), (2, 8, 4, 4), (8, 16, 4, 3), (24, 8, 4, 1),
                                            (6, 12, 4, 6)])
def test_tile_maps_all_ranks(world, fs, ts, hw):
    x = payload(2, fs, 5)
    full_o = ho.TileTopology(1, 0, fs, ts, hw)
    all_tiles = full_o.faces_to_local_tiles(x)
    seen_ranks = set()
    for rank in range(world):
        t = tp.TileTopology(world, rank, fs, ts, hw)
        a, b = tp.halo_source_maps(t)
        got = tp.apply_maps_numpy(all_tiles, a, b)
        want = ho.padded_local_tiles(all_tiles, ho.TileTopology(world, rank, fs, ts, hw))
        assert np.array_equal(got, want)
        seen_ranks |= set((a // (t.tiles_per_rank * ts * ts)).ravel().tolist())
    assert seen_ranks <= set(range(world))


def test_interior_tile_halo_equals_neighbour_data():
    # invariant held by the reference's tests (tests/test_distributed_tile_halo.py:249-293):
    # for a tile strictly inside a face the halo is the neighbouring tiles' data, exactly
    fs, ts, hw = 16, 4, 2
    x = payload(1, fs, 3)[0]                     # (6, 16, 16), integer identity payload
    full = tp.TileTopology(1, 0, fs, ts, hw)
    all_tiles = full.faces_to_local_tiles(torch.from_numpy(x)).numpy()
    a, b = tp.halo_source_maps(full)
    padded = tp.apply_maps_numpy(all_tiles, a, b)
    g = full.global_tiles.index((2, 1, 2))
    want = x[2, 1 * ts - hw:2 * ts + hw, 2 * ts - hw:3 * ts + hw]
    assert np.array_equal(padded[g], want)


def test_element_order_to_face_rasters(golden_dir):
    # outputs of the reference's own functions on a 3-element, 2-point face (bit-exact)
    g = np.load(golden_dir / "face_padding.npz")
    u = torch.from_numpy(g["reorder_in"])
    faces = tp.unstructured_to_6faces(u, ne=3, npg=2)
    assert torch.equal(faces, torch.from_numpy(g["reorder_faces"]))
    back = tp.faces_to_unstructured(faces, ne=3, npg=2)
    assert torch.equal(back, torch.from_numpy(g["reorder_back"])) and torch.equal(back, u)
    one = tp.reorder_cubesphere_to_2d_tensor(u[:, :36], ne=3, npg=2)
    assert torch.equal(one, faces[:, 0])
    assert torch.equal(tp.reorder_2d_tensor_to_cubesphere(one, ne=3, npg=2), u[:, :36])
    with pytest.raises(ValueError, match="must be positive"):
        tp.reorder_cubesphere_to_2d_tensor(u, ne=0, npg=2)
    with pytest.raises(ValueError, match="Expected last dim"):
        tp.unstructured_to_6faces(u[:, :-1], ne=3, npg=2)
    with pytest.raises(ValueError, match="Expected last 3 dims"):
        tp.faces_to_unstructured(faces[:, :5], ne=3, npg=2)


def test_reference_module_names_resolve_to_this_package():
    """`screamcast.distributed_halo`, `.distributed_cubesphere_transforms` and
    `.cubesphere_transforms` each have a module of the same name here that carries the same
    public names (a caller switches by changing the import line)."""
    from strata_b200 import (cubesphere_transforms, distributed_cubesphere_transforms,
                             distributed_halo, halo, topology)
    assert distributed_halo.TileTopology is topology.TileTopology
    assert distributed_halo.DistributedTileKNNHaloPadding_AllGather is halo.DistributedTileKNNHaloPadding
    assert distributed_halo.NormalizedHaloAdjoint is halo.NormalizedHaloAdjoint
    assert hasattr(distributed_halo.DistributedTileKNNHaloPadding_AllGather, "from_padded_face_grid")
    assert distributed_cubesphere_transforms.DistributedTileKNNHaloPadding is halo.DistributedTilePlanHaloPadding
    assert (distributed_cubesphere_transforms.build_distributed_tile_halo_plan
            is topology.build_distributed_tile_halo_plan)
    assert distributed_cubesphere_transforms._tile_id_to_tuple(37, 4) == (2, 1, 1)
    assert distributed_cubesphere_transforms._tile_tuple_to_id(2, 1, 1, 4) == 37
    for name in ("reorder_cubesphere_to_2d_tensor", "reorder_2d_tensor_to_cubesphere",
                 "unstructured_to_6faces", "faces_to_unstructured"):
        assert getattr(cubesphere_transforms, name) is getattr(topology, name)


def test_model_side_reference_module_names_resolve_to_this_package():
    """`screamcast.strata_wrappers`, `.tile_geometry`, `.wind_rotation`, `.dealias` and
    `.checkpoint_compat` have namesakes here with the same public names."""
    from strata_b200 import (checkpoint_compat, dealias, strata, strata_wrappers, tile_geometry,
                             wind_rotation, wrappers)
    assert strata_wrappers.StrataBackboneModel is wrappers.StrataBackboneModel
    assert strata_wrappers.StrataModel is wrappers.StrataModel
    assert strata_wrappers.remap_legacy_state_dict is checkpoint_compat.remap_legacy_state_dict
    assert tile_geometry.TileGeometry is wrappers.TileGeometry
    assert tile_geometry.mean_longitude is wrappers.mean_longitude
    for name in ("local_basis_ENR", "forward_uv_to_tile", "inverse_tile_to_uv"):
        assert getattr(wind_rotation, name) is getattr(wrappers, name)
    assert dealias.DealiasedPatchEmbed3D is strata.DealiasedPatchEmbed3D
