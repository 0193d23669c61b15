"""Plan-based tile KNN halo (build_distributed_tile_halo_plan + the module over it).

Routing - which source tile each halo cell of each tile is interpolated from, in which order a
tile's halo cells are listed, send / receive sizes, tile -> rank - is compared with tables the
reference's own builder produced (tests/golden/make_plan_golden.py; earth2grid's interpolator
replaced there by a stand-in with the inverse-distance weights this repo assumes), and the
module's forward with the reference module's output at world_size 1. The invariants are the
ones of the reference's tests/test_distributed_tile_halo.py:97-330.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import halo_oracle as ho
from strata_b200.rollout import equiangular_cubed_sphere_latlon
from strata_b200.topology import (TileTopology, build_distributed_tile_halo_plan, build_tile_to_rank_map,
                                  faces_to_unstructured, plan_gather_lists, tile_halo_plan_from_reference,
                                  tile_halo_positions, tile_id_to_tuple, tile_tuple_to_id)
from tests.test_halo_knn import _apply

GOLD = Path(__file__).resolve().parent / "golden" / "tile_halo_plan.npz"
NE, NPG, TILE, HALO = 8, 2, 4, 2
FACE = NE * NPG
TPD = FACE // TILE
TOTAL = 6 * TPD * TPD


def _grid(ne=NE, npg=NPG):
    lat, lon = equiangular_cubed_sphere_latlon(ne * npg)
    return {"lon": faces_to_unstructured(torch.from_numpy(lon.astype(np.float32)), ne=ne, npg=npg).numpy(),
            "lat": faces_to_unstructured(torch.from_numpy(lat.astype(np.float32)), ne=ne, npg=npg).numpy()}


@pytest.fixture(scope="module")
def grid_src():
    return _grid()


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


def _cells(plan):
    """One row per halo cell (dst tile, position, src tile, src rank), sorted by (dst, position)."""
    G, n = plan.src_tile_id.shape
    dst = np.repeat(np.arange(G), n)
    pos = np.tile(plan.halo_positions, G)
    src = plan.src_tile_id.reshape(-1).astype(np.int64)
    rank = np.array([plan.tile_to_rank[tile_id_to_tuple(s, plan.tiles_per_dim)] for s in src])
    return np.stack([dst, pos, src, rank], axis=1)


@pytest.mark.parametrize("ws", [1, 2, 6])
def test_routing_equals_the_reference_plan(gold, ws):
    grid = {"lon": gold["grid_lon"], "lat": gold["grid_lat"]}
    plan = build_distributed_tile_halo_plan(grid, int(gold["ne"]), int(gold["tile"]), int(gold["halo"]),
                                            num_pg_cells=int(gold["npg"]), world_size=ws)
    assert np.array_equal(_cells(plan), gold[f"ws{ws}_cells"])
    k = plan.knn_index.shape[2]
    assert np.array_equal(plan.knn_index.reshape(-1, k), gold[f"ws{ws}_index"])
    assert np.allclose(plan.knn_weight.reshape(-1, k), gold[f"ws{ws}_weight"], rtol=0, atol=1e-7)
    send = np.array([[plan.send_sizes[a][b] for b in range(ws)] for a in range(ws)])
    recv = np.array([[plan.recv_sizes[a][b] for b in range(ws)] for a in range(ws)])
    assert np.array_equal(send, gold[f"ws{ws}_send_sizes"]) and np.array_equal(recv, gold[f"ws{ws}_recv_sizes"])
    tpd = plan.tiles_per_dim
    assert [plan.tile_to_rank[tile_id_to_tuple(t, tpd)] for t in range(6 * tpd * tpd)] == \
        gold[f"ws{ws}_tile_to_rank"].tolist()


def test_target_grid_routing_equals_the_reference_plan(gold):
    grid = {"lon": gold["grid_lon"], "lat": gold["grid_lat"]}
    tgt = {"lon": gold["tgt_lon"], "lat": gold["tgt_lat"]}
    plan = build_distributed_tile_halo_plan(grid, int(gold["ne"]), int(gold["tile"]), int(gold["halo"]),
                                            num_pg_cells=int(gold["npg"]), world_size=1, grid_tgt=tgt)
    assert np.array_equal(_cells(plan)[:, :3], gold["tgt_cells"])
    with pytest.raises(ValueError, match="exceeds"):
        build_distributed_tile_halo_plan(grid, int(gold["ne"]), int(gold["tile"]), 8,
                                         num_pg_cells=int(gold["npg"]), world_size=1, grid_tgt=tgt)


def test_forward_equals_the_reference_module(gold):
    grid = {"lon": gold["grid_lon"], "lat": gold["grid_lat"]}
    T, h = int(gold["tile"]), int(gold["halo"])
    plan = build_distributed_tile_halo_plan(grid, int(gold["ne"]), T, h, num_pg_cells=int(gold["npg"]),
                                            world_size=1)
    x, want = gold["ws1_forward_in"], gold["ws1_forward_out"]
    # the gather kernel's arithmetic on the host (float32, neighbour order, no fused multiply-add)
    idx, w = plan_gather_lists(plan, 0)
    got = _apply(x, idx, w).reshape(want.shape)
    assert np.array_equal(got[..., h:-h, h:-h], x)
    assert np.allclose(got, want, rtol=0, atol=1e-6)
    # and the oracle's restatement of the reference forward (NaN fill, per-entry scatter)
    entries = [(tile_tuple_to_id(*e.src_tile, plan.tiles_per_dim), tile_tuple_to_id(*dst, plan.tiles_per_dim),
                e.dst_halo_positions.numpy(), e.regridder_state_dict["index"].numpy(),
                e.regridder_state_dict["weight"].numpy())
               for by_dst in plan.send_plans.values() for dst, es in by_dst.items() for e in es]
    oracle = ho.plan_halo_forward(x, entries, T, h, range(x.shape[-3]))
    assert not np.isnan(oracle).any()
    assert np.allclose(oracle, want, rtol=0, atol=1e-6)
    assert np.array_equal(oracle, got)


@pytest.mark.parametrize("ws", [1, 2, 6, 16, 96])
def test_indices_in_range_coverage_and_symmetry(grid_src, ws):
    plan = build_distributed_tile_halo_plan(grid_src, NE, TILE, HALO, num_pg_cells=NPG, world_size=ws)
    assert plan.knn_index.min() >= 0 and plan.knn_index.max() < TILE * TILE
    assert plan.src_tile_id.min() >= 0 and plan.src_tile_id.max() < TOTAL
    expected = set(tile_halo_positions(TILE, HALO).tolist())
    assert len(expected) == (TILE + 2 * HALO) ** 2 - TILE ** 2
    sp = plan.send_plans
    seen = {}
    for sr, by_dst in sp.items():
        for dst, entries in by_dst.items():
            for e in entries:
                assert plan.tile_to_rank[e.src_tile] == sr
                seen.setdefault(dst, []).extend(e.dst_halo_positions.tolist())
    assert len(seen) == TOTAL
    for dst, positions in seen.items():
        assert len(positions) == len(set(positions)), f"duplicate halo positions for {dst}"
        assert set(positions) == expected, f"halo of {dst} not covered exactly"
    for a in range(ws):
        for b in range(ws):
            assert plan.send_sizes[a][b] == plan.recv_sizes[b][a]
        assert sum(plan.recv_sizes[a].values()) == plan.tiles_per_rank * len(expected)
    for dst, by_rank in plan.recv_counts.items():
        assert sum(by_rank.values()) == len(expected)


def test_interior_tile_halo_is_the_neighbouring_data(grid_src):
    plan = build_distributed_tile_halo_plan(grid_src, NE, TILE, HALO, num_pg_cells=NPG, world_size=1)
    f, i, j = np.meshgrid(np.arange(6), np.arange(FACE), np.arange(FACE), indexing="ij")
    faces = (f * 1000 + i * FACE + j).astype(np.float32)
    tiles = np.stack([faces[fa, ti * TILE:(ti + 1) * TILE, tj * TILE:(tj + 1) * TILE]
                      for fa, ti, tj in TileTopology(1, 0, FACE, TILE, HALO).global_tiles])[None]
    idx, w = plan_gather_lists(plan, 0)
    P = TILE + 2 * HALO
    padded = _apply(tiles, idx, w).reshape(1, TOTAL, P, P)
    assert not np.isnan(padded).any()
    assert np.array_equal(padded[..., HALO:-HALO, HALO:-HALO], tiles)
    g = tile_tuple_to_id(0, 1, 1, TPD)
    want = faces[0, TILE - HALO:2 * TILE + HALO, TILE - HALO:2 * TILE + HALO]
    assert np.allclose(padded[0, g], want, atol=1e-3, rtol=1e-3)


def test_invalid_configurations_and_zero_halo(grid_src):
    with pytest.raises(ValueError, match="divisible"):
        build_distributed_tile_halo_plan(grid_src, NE, 5, HALO, num_pg_cells=NPG, world_size=1)
    with pytest.raises(ValueError, match="divisible"):
        build_distributed_tile_halo_plan(grid_src, NE, TILE, HALO, num_pg_cells=NPG, world_size=7)
    plan = build_distributed_tile_halo_plan(grid_src, NE, TILE, 0, num_pg_cells=NPG, world_size=1)
    assert plan.halo_positions.size == 0 and plan.send_sizes == {0: {0: 0}}
    x = np.random.default_rng(0).standard_normal((2, TOTAL, TILE, TILE)).astype(np.float32)
    idx, w = plan_gather_lists(plan, 0)
    assert np.array_equal(_apply(x, idx, w).reshape(x.shape), x)


def test_tile_helpers():
    for t in range(TOTAL):
        f, ti, tj = tile_id_to_tuple(t, TPD)
        assert 0 <= f < 6 and 0 <= ti < TPD and 0 <= tj < TPD
        assert tile_tuple_to_id(f, ti, tj, TPD) == t
    for ws in (1, 2, 6, 96):
        m = build_tile_to_rank_map(TPD, ws)
        assert len(m) == TOTAL and set(m.values()) == set(range(ws))
        # the same shares as TileTopology.local_tiles
        for r in range(ws):
            assert [t for t, rr in m.items() if rr == r] == TileTopology(ws, r, FACE, TILE, HALO).local_tiles


@pytest.mark.parametrize("ws", [2, 6])
def test_rank_lists_together_equal_the_single_rank_lists(grid_src, ws):
    one = build_distributed_tile_halo_plan(grid_src, NE, TILE, HALO, num_pg_cells=NPG, world_size=1)
    many = build_distributed_tile_halo_plan(grid_src, NE, TILE, HALO, num_pg_cells=NPG, world_size=ws)
    i1, w1 = plan_gather_lists(one, 0)
    parts = [plan_gather_lists(many, r) for r in range(ws)]
    assert np.array_equal(np.concatenate([p[0] for p in parts]), i1)
    assert np.array_equal(np.concatenate([p[1] for p in parts]), w1)


@pytest.mark.parametrize("ws", [1, 6])
def test_plan_in_the_reference_layout_converts_to_the_same_tables(grid_src, ws):
    # a plan handed over in the reference's nested layout (as the reference would build and save
    # it, e.g. with earth2grid's own weights) gives the same dense tables
    import types
    plan = build_distributed_tile_halo_plan(grid_src, NE, TILE, HALO, num_pg_cells=NPG, world_size=ws)
    nested = types.SimpleNamespace(**{k: getattr(plan, k) for k in (
        "face_size", "tile_size", "tiles_per_dim", "halo_width", "ne", "npg", "world_size",
        "tiles_per_rank", "tile_to_rank", "recv_counts", "send_sizes", "recv_sizes")},
        send_plans=plan.send_plans)
    back = tile_halo_plan_from_reference(nested)
    assert np.array_equal(back.src_tile_id, plan.src_tile_id)
    assert np.array_equal(back.knn_index, plan.knn_index)
    assert np.array_equal(back.knn_weight, plan.knn_weight)
    assert np.array_equal(back.halo_positions, plan.halo_positions)
    # entries that miss a halo cell, or list one twice, are refused
    first = next(iter(nested.send_plans[0].values()))
    first.append(first[0])
    with pytest.raises(ValueError, match="twice"):
        tile_halo_plan_from_reference(nested)
    first.pop(); first.pop(0)
    with pytest.raises(ValueError, match="cover"):
        tile_halo_plan_from_reference(nested)
