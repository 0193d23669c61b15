"""Multi-GPU halo exchange check, one process per GPU (launched by torch.distributed.run).
Every rank pads its tiles through peer memory and compares with the oracle, bit for bit,
for several steps (exercising the two-slot publication scheme)."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from oracle import halo_oracle as ho  # noqa: E402
from strata_b200.halo import (DistributedTileCopyHaloPadding, DistributedTileKNNHaloPadding,  # noqa: E402
                              NormalizedCopyHaloAdjoint, kbd_window)
from strata_b200.rollout import padded_face_latlon  # noqa: E402
from tests.test_halo_knn import _apply  # noqa: E402
from strata_b200.topology import TileTopology  # noqa: E402
from tests.golden.make_golden import payload  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    fs, ts, hw, D, C = 16, 4, 3, 2, 64
    topo = TileTopology(world, rank, fs, ts, hw)
    topo_o = ho.TileTopology(world, rank, fs, ts, hw)
    full_o = ho.TileTopology(1, 0, fs, ts, hw)
    mod = DistributedTileCopyHaloPadding(topology=topo)
    for step in range(5):
        x = payload(3, fs, 100 + step)                         # (3, 6, N, N), same on every rank
        all_tiles = full_o.faces_to_local_tiles(x)
        mine = topo_o.faces_to_local_tiles(x)
        out = mod(torch.from_numpy(np.ascontiguousarray(mine)).cuda())
        want = ho.padded_local_tiles(all_tiles, topo_o)
        assert np.array_equal(out.cpu().numpy(), want), f"rank {rank} step {step}: field halo differs"
    # token space
    g = torch.Generator().manual_seed(5)
    all_tok = torch.randn(topo.total_tiles, D, ts * ts, C, generator=g).bfloat16()
    s = rank * topo.tiles_per_rank
    out = mod.pad_tokens(all_tok[s:s + topo.tiles_per_rank].cuda(), D)
    mod.check_status()
    a = torch.from_numpy(mod.src_a.cpu().numpy().astype(np.int64))
    b = mod.src_b.cpu().numpy()
    flat = all_tok.permute(1, 3, 0, 2).reshape(D, C, -1)
    va, vb = flat[..., a], flat[..., torch.from_numpy(np.where(b < 0, 0, b).astype(np.int64))]
    want = torch.where(torch.from_numpy(b < 0), va, (va + vb) / 2)
    P = topo.padded_tile_size
    got = out.cpu().reshape(topo.tiles_per_rank, D, P, P, C).permute(1, 4, 0, 2, 3)
    assert torch.equal(got, want), f"rank {rank}: token halo differs"
    # windowed overlap-add un-pad: every rank's padded tiles differ, sources sit on both GPUs
    P = topo.padded_tile_size
    win = kbd_window(P)
    unpad = NormalizedCopyHaloAdjoint(mod, window=win)
    g = torch.Generator().manual_seed(9)
    pad_all = torch.randn(2, topo.total_tiles, P, P, generator=g)
    for step in range(3):
        got = unpad((pad_all[:, s:s + topo.tiles_per_rank] + step).cuda())
        want = ho.halo_adjoint((pad_all + step).numpy(), topo_o, win.numpy())
        assert np.array_equal(got.cpu().numpy(), want), f"rank {rank} step {step}: halo adjoint differs"
    mod.check_status()
    # k-nearest-neighbour halo: sources on both GPUs, weighted gather through peer memory
    lat, lon = padded_face_latlon(fs, hw)
    knn = DistributedTileKNNHaloPadding.from_padded_face_grid(
        topology=topo, lon=torch.from_numpy(lon).float(), lat=torch.from_numpy(lat).float(),
        pad_width_data=hw, device=torch.device("cuda", torch.cuda.current_device()))
    xa = torch.randn(2, topo.total_tiles, ts, ts, generator=torch.Generator().manual_seed(4))
    for step in range(3):
        got = knn((xa[:, s:s + topo.tiles_per_rank] * (step + 1)).cuda())
        want = _apply((xa * (step + 1)).numpy(), knn.knn_idx.cpu().numpy(), knn.knn_weights.cpu().numpy())
        assert np.array_equal(got.cpu().numpy().reshape(want.shape), want), \
            f"rank {rank} step {step}: knn halo differs"
    knn.check_status()
    # plan-based tile halo: each halo cell from ONE assigned source tile, read through peer memory
    from strata_b200.halo import DistributedTilePlanHaloPadding
    from strata_b200.rollout import equiangular_cubed_sphere_latlon
    from strata_b200.topology import build_distributed_tile_halo_plan, faces_to_unstructured
    npg = 2
    la0, lo0 = equiangular_cubed_sphere_latlon(fs)
    grid = {key: faces_to_unstructured(torch.from_numpy(v.astype(np.float32)), ne=fs // npg, npg=npg).numpy()
            for key, v in (("lon", lo0), ("lat", la0))}
    plan = build_distributed_tile_halo_plan(grid, fs // npg, ts, hw, num_pg_cells=npg, world_size=world)
    pm = DistributedTilePlanHaloPadding(plan, rank)
    for step in range(3):
        got = pm((xa[:, s:s + topo.tiles_per_rank] * (step + 1)).cuda())
        want = _apply((xa * (step + 1)).numpy(), pm.knn_idx.cpu().numpy(), pm.knn_weights.cpu().numpy())
        assert np.array_equal(got.cpu().numpy().reshape(want.shape), want), \
            f"rank {rank} step {step}: plan halo differs"
        assert torch.equal(got[..., hw:-hw, hw:-hw].cpu(), xa[:, s:s + topo.tiles_per_rank] * (step + 1))
    pm.check_status()
    dist.barrier()
    pm.close()
    knn.close()
    mod.close()
    if rank == 0:
        print("HALO WORKER OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
