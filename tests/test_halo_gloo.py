"""Host-side logic of the N > 1 halo path on CPU: two gloo ranks partition the tiles as the
topology says, exchange them with a collective, and each rank's gather maps must rebuild its
padded tiles exactly as the oracle does. Also covers gather_tiles_to_faces over a real group."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    from oracle import halo_oracle as ho
    from strata_b200.topology import TileTopology, apply_maps_numpy, halo_source_maps
    from tests.golden.make_golden import payload
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        fs, ts, hw = 8, 4, 2
        topo = TileTopology(world, rank, fs, ts, hw)
        x = payload(2, fs, 42)
        mine = topo.faces_to_local_tiles(torch.from_numpy(x))
        faces = topo.gather_tiles_to_faces(mine)                  # all_gather over gloo
        ok1 = np.array_equal(faces.numpy(), x)
        parts = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine.contiguous())
        all_tiles = torch.cat(parts, dim=-3).numpy()              # global tile order
        a, b = halo_source_maps(topo)
        got = apply_maps_numpy(all_tiles, a, b)
        want = ho.padded_local_tiles(all_tiles, ho.TileTopology(world, rank, fs, ts, hw))
        ok2 = np.array_equal(got, want)
        owners = set((a // (topo.tiles_per_rank * ts * ts)).ravel().tolist())
        q.put((rank, ok1, ok2, sorted(owners)))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_halo_maps():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 400)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok1, ok2, owners in res:
        assert ok1, f"rank {rank}: gather_tiles_to_faces mismatch"
        assert ok2, f"rank {rank}: halo maps differ from the oracle"
        assert set(owners) == {0, 1}                              # halos do cross ranks


def _knn_worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    from strata_b200.halo import gather_knn_lists
    from strata_b200.rollout import padded_face_latlon
    from strata_b200.topology import TileTopology, knn_adjoint_lists, knn_halo_weights
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        N, T, H, PW = 16, 4, 2, 4
        lat, lon = padded_face_latlon(N, PW)
        topo = TileTopology(world, rank, N, T, H)
        idx, w = knn_halo_weights(topo, lon, lat, PW)            # this rank's padded cells only
        idx_all, w_all = gather_knn_lists(topo, torch.from_numpy(idx), torch.from_numpy(w))
        ref_idx, ref_w = knn_halo_weights(TileTopology(1, 0, N, T, H), lon, lat, PW)
        ok1 = np.array_equal(idx_all, ref_idx) and np.array_equal(w_all, ref_w)
        got = knn_adjoint_lists(topo, idx_all, w_all)
        want = knn_adjoint_lists(topo, ref_idx, ref_w)
        ok2 = all(np.array_equal(a, b) for a, b in zip(got, want))
        # every padded cell that draws on a local interior cell is listed, wherever it lives
        owners = set((got[1] // (topo.tiles_per_rank * (T + 2 * H) ** 2)).tolist())
        q.put((rank, ok1, ok2, sorted(owners)))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_knn_adjoint_lists():
    # set-up of the KNN halo's adjoint (NormalizedHaloAdjoint): the ranks' weight lists are
    # all-gathered, each rank keeps the entries that draw on its own interior cells
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + (os.getpid() % 90)
    procs = [ctx.Process(target=_knn_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok1, ok2, owners in res:
        assert ok1, f"rank {rank}: gathered lists differ from the single-rank lists"
        assert ok2, f"rank {rank}: adjoint lists differ"
        assert set(owners) == {0, 1}


def _plan_worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    from oracle import halo_oracle as ho
    from strata_b200.halo import gather_knn_lists
    from strata_b200.rollout import equiangular_cubed_sphere_latlon
    from strata_b200.topology import (TileTopology, build_distributed_tile_halo_plan, faces_to_unstructured,
                                      plan_gather_lists, tile_tuple_to_id)
    from tests.test_halo_knn import _apply
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ne, npg, T, H = 4, 2, 4, 2
        lat, lon = equiangular_cubed_sphere_latlon(ne * npg)
        grid = {k: faces_to_unstructured(torch.from_numpy(v.astype(np.float32)), ne=ne, npg=npg).numpy()
                for k, v in (("lon", lon), ("lat", lat))}
        plan = build_distributed_tile_halo_plan(grid, ne, T, H, num_pg_cells=npg, world_size=world)
        topo = TileTopology(world, rank, ne * npg, T, H)
        idx, w = plan_gather_lists(plan, rank)
        # this rank's padded tiles from the globe's interiors, as the gather kernel computes them,
        # against the oracle's per-entry scatter restricted to the local tiles
        x = np.random.default_rng(5).standard_normal((2, topo.total_tiles, T, T)).astype(np.float32)
        got = _apply(x, idx, w).reshape(2, topo.tiles_per_rank, T + 2 * H, T + 2 * H)
        tpd = plan.tiles_per_dim
        entries = [(tile_tuple_to_id(*e.src_tile, tpd), tile_tuple_to_id(*dst, tpd), e.dst_halo_positions.numpy(),
                    e.regridder_state_dict["index"].numpy(), e.regridder_state_dict["weight"].numpy())
                   for by_dst in plan.send_plans.values() for dst, es in by_dst.items() for e in es]
        local = range(rank * topo.tiles_per_rank, (rank + 1) * topo.tiles_per_rank)
        ok1 = np.array_equal(got, ho.plan_halo_forward(x, entries, T, H, local))
        # what this rank receives is what the others' plans say they send to it
        recv = sum(plan.recv_sizes[rank].values())
        sent = torch.tensor([plan.send_sizes[rank][r] for r in range(world)])
        parts = [torch.zeros_like(sent) for _ in range(world)]
        dist.all_gather(parts, sent)
        ok2 = recv == int(sum(p[rank] for p in parts))
        # the adjoint's set-up gathers the ranks' lists into the single-rank lists
        idx_all, w_all = gather_knn_lists(topo, torch.from_numpy(idx), torch.from_numpy(w))
        one = build_distributed_tile_halo_plan(grid, ne, T, H, num_pg_cells=npg, world_size=1)
        i1, w1 = plan_gather_lists(one, 0)
        ok3 = np.array_equal(idx_all, i1) and np.array_equal(w_all, w1)
        q.put((rank, ok1, ok2, ok3))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_tile_halo_plan():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() % 90)
    procs = [ctx.Process(target=_plan_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok1, ok2, ok3 in res:
        assert ok1, f"rank {rank}: padded tiles differ from the oracle's scatter"
        assert ok2, f"rank {rank}: receive sizes do not match the senders' send sizes"
        assert ok3, f"rank {rank}: gathered lists differ from the single-rank plan"
