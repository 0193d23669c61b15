"""torch.library registration of the model boundary, so that `torch.compile(network)` works.

The reference compiles the whole network before a rollout
(screamcast/earth2studio_wrappers.py:412-413, called at scripts/ace/run_screamcast_nudged.py:
639-641) and runs it under `torch.inference_mode()` (:452). The kernels of this package are
reached through ctypes on raw device pointers - nothing a tracing compiler can look into. The
whole network forward is therefore ONE custom operator,

    strata_b200::network_forward(x, lat, lon, handle) -> y

with a fake (shape / dtype only) implementation for tracing: Dynamo records a single opaque
call, `fullgraph=True` holds, Inductor has nothing to fuse across and launches the eager
implementation. `handle` names the module in a registry of live wrapper modules (weak
references); its weights are read from the module when the operator runs, they are not operator
arguments (inference only: there is no backward).

Finer-grained operators over the C ABI (`strata_b200::block_forward`, `::na3d`, `::linear`,
`::layernorm`) are registered the same way for callers that assemble their own graphs.
"""
from __future__ import annotations

import itertools
import weakref
from typing import Optional, Sequence

import torch

_MODULES: "weakref.WeakValueDictionary[int, torch.nn.Module]" = weakref.WeakValueDictionary()
_next_handle = itertools.count(1)


def register_module(module: torch.nn.Module) -> int:
    """Give a wrapper module a handle for `strata_b200::network_forward`."""
    h = next(_next_handle)
    _MODULES[h] = module
    return h


def _module(handle: int) -> torch.nn.Module:
    try:
        return _MODULES[handle]
    except KeyError:
        raise RuntimeError(f"strata_b200::network_forward: no live module with handle {handle}") from None


@torch.library.custom_op("strata_b200::network_forward", mutates_args=())
def network_forward(x: torch.Tensor, lat: torch.Tensor, lon: torch.Tensor, handle: int) -> torch.Tensor:
    return _module(handle)._forward_eager(x, lat, lon)


@network_forward.register_fake
def _network_forward_fake(x, lat, lon, handle):
    m = _module(handle)
    return x.new_empty((x.shape[0], m._out_chans, x.shape[2], x.shape[3], x.shape[4]))


# ------------------------------------------------------------------ operators over the C ABI
@torch.library.custom_op("strata_b200::layernorm", mutates_args=())
def layernorm(x: torch.Tensor, eps: float) -> torch.Tensor:
    from . import ops
    return ops.layernorm(x, eps)


@layernorm.register_fake
def _layernorm_fake(x, eps):
    return torch.empty_like(x)


@torch.library.custom_op("strata_b200::linear", mutates_args=())
def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], epilogue: int,
           aux: Optional[torch.Tensor]) -> torch.Tensor:
    from . import ops
    return ops.linear(x, weight, bias, epilogue, aux)


@linear.register_fake
def _linear_fake(x, weight, bias, epilogue, aux):
    return x.new_empty((*x.shape[:-1], weight.shape[0]))


@torch.library.custom_op("strata_b200::na3d", mutates_args=())
def na3d(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, kernel: Sequence[int]) -> torch.Tensor:
    from . import ops
    return ops.na3d(q, k, v, tuple(kernel))


@na3d.register_fake
def _na3d_fake(q, k, v, kernel):
    return q.new_empty(q.shape)


@torch.library.custom_op("strata_b200::block_forward", mutates_args=())
def block_forward(x: torch.Tensor, weights: Sequence[torch.Tensor], biases: Sequence[torch.Tensor],
                  grid: Sequence[int], num_heads: int, kernel: Sequence[int],
                  rope_cs: Optional[torch.Tensor], qk_norm: bool) -> torch.Tensor:
    """One backbone block. weights / biases: (qkv, proj, fc1, fc2[, gate]) in that order."""
    from . import ops
    names = ("qkv", "proj", "fc1", "fc2", "gate")
    w = {f"w_{n}": t for n, t in zip(names, weights)}
    w.update({f"b_{n}": t for n, t in zip(names, biases)})
    return ops.block_forward(x, w, grid=tuple(grid), num_heads=num_heads, kernel=tuple(kernel),
                             rope_cos=None, rope_sin=None, rope_cs=rope_cs, qk_norm=qk_norm)


@block_forward.register_fake
def _block_forward_fake(x, weights, biases, grid, num_heads, kernel, rope_cs, qk_norm):
    return torch.empty_like(x)
