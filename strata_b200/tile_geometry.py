"""`mean_longitude` and `TileGeometry` of the reference's `screamcast/tile_geometry.py:33-170`,
bound to `strata_b200.wrappers`. Nothing is defined here."""
from .wrappers import TileGeometry, mean_longitude

__all__ = ["TileGeometry", "mean_longitude"]
