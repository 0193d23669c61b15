"""The names of the reference's `screamcast/strata_wrappers.py` (`StrataBackboneModel` :252-415,
`StrataModel` :418-680 and the module's helpers), bound to `strata_b200.wrappers`: a caller
switches by changing the package in its import line. Nothing is defined here."""
from .checkpoint_compat import remap_legacy_state_dict
from .wrappers import (StrataBackboneModel, StrataModel, _replace_channels, _resolve_rope_base,
                       _rope_mode, _StrataModelBase, _use_tanh_gelu)

__all__ = ["StrataBackboneModel", "StrataModel", "remap_legacy_state_dict"]
