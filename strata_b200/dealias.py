"""`DealiasedPatchEmbed3D` of the reference's `screamcast/dealias.py:28-143`, bound to
`strata_b200.strata`. Nothing is defined here."""
from .strata import DealiasedPatchEmbed3D

__all__ = ["DealiasedPatchEmbed3D"]
