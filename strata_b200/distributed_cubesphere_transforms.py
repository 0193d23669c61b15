"""The names of the reference's `screamcast/distributed_cubesphere_transforms.py`, bound to this
package's implementations (one changed import line switches a caller over):

* `TileSendEntry`, `TileHaloPlan` (distributed_cubesphere_transforms.py:49-78),
* `build_distributed_tile_halo_plan(grid_src, num_elements, tile_size, halo_width, num_pg_cells,
  k, eps, world_size, grid_tgt)` (:404-608),
* `DistributedTileKNNHaloPadding(plan, rank, group)` with `forward(data_local[..., tiles_per_rank,
  T, T])` (:611-781) - here the module that reads every halo cell's sources from the owning
  ranks' tiles (no send buffers, no all_to_all),
* the small helpers under the reference's private names (:174-199, :346-401).
Nothing is defined here.
"""
from .halo import DistributedTilePlanHaloPadding as DistributedTileKNNHaloPadding
from .topology import (TileHaloPlan, TileSendEntry, build_distributed_tile_halo_plan,
                       tile_halo_plan_from_reference)
from .topology import build_tile_to_rank_map as _build_tile_to_rank_map
from .topology import padded_lonlat_from_target_grid as _padded_lonlat_from_target_grid
from .topology import tile_id_to_tuple as _tile_id_to_tuple
from .topology import tile_tuple_to_id as _tile_tuple_to_id

__all__ = ["TileSendEntry", "TileHaloPlan", "build_distributed_tile_halo_plan",
           "DistributedTileKNNHaloPadding", "tile_halo_plan_from_reference"]
