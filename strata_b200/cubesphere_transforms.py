"""The element-order functions of the reference's `screamcast/cubesphere_transforms.py:20-146`
under their own names (`reorder_cubesphere_to_2d_tensor`, `reorder_2d_tensor_to_cubesphere`,
`unstructured_to_6faces`, `faces_to_unstructured`), bound to `strata_b200.topology`.

The face-level pad of the same file (`create_padded_faces_batched(faces[..., 6, N, N], pad)`,
:357-445) is the copy halo with one tile per face: `DistributedTileCopyHaloPadding(topology=
TileTopology(1, 0, N, N, pad))(faces)` - see `strata_b200.halo`. Nothing is defined here.
"""
from .topology import (faces_to_unstructured, reorder_2d_tensor_to_cubesphere,
                       reorder_cubesphere_to_2d_tensor, unstructured_to_6faces)

__all__ = ["reorder_cubesphere_to_2d_tensor", "reorder_2d_tensor_to_cubesphere",
           "unstructured_to_6faces", "faces_to_unstructured"]
