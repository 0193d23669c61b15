"""The names of the reference's `screamcast/distributed_halo.py`, bound to this package's
implementations, so that a caller switches by changing one import line:

    from screamcast.distributed_halo import TileTopology, DistributedTileKNNHaloPadding_AllGather, NormalizedHaloAdjoint
    from strata_b200.distributed_halo import TileTopology, DistributedTileKNNHaloPadding_AllGather, NormalizedHaloAdjoint

* `TileTopology` (distributed_halo.py:57-205): same fields, properties and methods.
* `DistributedTileKNNHaloPadding_AllGather` (:208-327): `from_padded_face_grid(topology=, lon=,
  lat=, pad_width_data=, device=)` and `forward(x[..., tiles_per_rank, T, T])`; the halo cells'
  k nearest sources are read from their owners' tiles instead of an all-gathered globe.
* `NormalizedHaloAdjoint` (:330-448): `NormalizedHaloAdjoint(halo_exchange, window=None)`,
  `forward(padded) -> interior`.
Nothing is defined here.
"""
from .halo import DistributedTileKNNHaloPadding as DistributedTileKNNHaloPadding_AllGather
from .halo import NormalizedHaloAdjoint
from .topology import Tile, TileTopology

__all__ = ["Tile", "TileTopology", "DistributedTileKNNHaloPadding_AllGather", "NormalizedHaloAdjoint"]
