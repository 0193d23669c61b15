"""Per-block K/V halo exchange on several GPUs, one process per GPU (launched by
torch.distributed.run): every rank runs a stack of blocks over its tiles, halos crossing peer
memory in each block, and compares with the CPU oracle evaluated over the whole sphere."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from oracle import block_oracle as bo  # noqa: E402
from strata_b200.halo_block import TiledBlockRunner  # noqa: E402
from strata_b200.topology import TileTopology  # noqa: E402
from tests.test_halo_block_gpu import _grid  # noqa: E402
from tests.util import device_block_weights, rel_max_err  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    face, tile, halo, D, C, heads, kernel, n_blocks = 64, 32, 2, 2, 64, 1, (1, 5, 5), 3
    topo = TileTopology(world, rank, face, tile, halo)
    lat, lon = _grid(face, tile)
    scale = np.radians(90.0 / face)
    run = TiledBlockRunner(topo, depth=D, dim=C, num_heads=heads, kernel=kernel, lat_deg=lat,
                           lon_deg=lon, rope_length_scale=scale)
    params = [bo.init_block_params(C, seed=30 + i, scheme="xavier") for i in range(n_blocks)]
    g = torch.Generator().manual_seed(3)
    x = torch.randn(topo.total_tiles, D * tile * tile, C, generator=g).bfloat16()
    s = rank * topo.tiles_per_rank
    y = x[s:s + topo.tiles_per_rank].cuda()
    ref = x.float()
    for p in params:
        y = run.block_forward(y, device_block_weights(p, "cuda"))
        ref = bo.tiled_block_forward(ref, p, face=face, tile=tile, halo=halo, depth=D,
                                     num_heads=heads, kernel=kernel, lat_deg=lat, lon_deg=lon,
                                     length_scale=scale)
    run.check_status()
    err = rel_max_err(y, ref[s:s + topo.tiles_per_rank])
    assert err < 4e-2, f"rank {rank}: tiled block stack differs from the oracle ({err})"
    dist.barrier()
    run.close()
    if rank == 0:
        print("HALO BLOCK WORKER OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
