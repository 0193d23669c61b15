"""`local_basis_ENR`, `forward_uv_to_tile` and `inverse_tile_to_uv` of the reference's
`screamcast/wind_rotation.py:26-144`, bound to `strata_b200.wrappers` (tensor versions; inside the
model the same rotation runs in the fused pre-/post-processing kernels). Nothing is defined here."""
from .wrappers import forward_uv_to_tile, inverse_tile_to_uv, local_basis_ENR

__all__ = ["local_basis_ENR", "forward_uv_to_tile", "inverse_tile_to_uv"]
