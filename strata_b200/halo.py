"""Tile halo exchange over peer memory (one process per GPU).

`DistributedTileCopyHaloPadding` has the interface of the reference's halo module
(screamcast/distributed_halo.py:208-327): `forward(x[..., tiles_per_rank, T, T]) ->
[..., tiles_per_rank, T+2h, T+2h]`, attributes `.topology`, `.lat_deg`, `.lon_deg`, the
classmethod `from_padded_face_grid(...)`, wrappable per channel chunk, and `topology.crop`
inverts it. What differs is the mechanism: instead of all-gathering the whole globe to every
rank and regridding, each rank publishes its tiles in a peer-mapped buffer and every GPU's
gather kernel reads just the cells its halos need, directly from the owning GPU over NVLink,
following precomputed copy / rot90 / corner maps (strata_b200/topology.py). Halo values are
COPIES of neighbour cells (exact inside a face, and the reference's own face-padding rule
across face edges), not k-nearest-neighbour interpolants.

`pad_tokens` is the same exchange for bf16 token tensors [tiles_per_rank, D, T*T, C] (per
block, token space).

Synchronisation: a device-side flag barrier on the current stream before the gather (all
ranks have published) — buffers alternate between two slots, so a rank may publish step n+1
while a slower peer still reads step n. Waits are bounded; a peer that never arrives shows up
as device status 105 (`check_status`).
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch
import torch.distributed as dist

from . import _lib
from .topology import (TileTopology, halo_adjoint_lists, halo_source_maps, knn_adjoint_lists,
                       knn_halo_weights, plan_gather_lists)


class _DevPtrTensorView:
    """Exposes raw device memory to torch through __cuda_array_interface__."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


class PeerSharedBuffer:
    """`nbytes` of device memory on every rank, each rank's block mapped into all others.

    ptrs[r] is the pointer through which THIS process reaches rank r's block. Set-up only
    (allocates, exchanges CUDA IPC handles through torch.distributed).
    """

    def __init__(self, nbytes: int, group=None):
        lib = _lib.load()
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.nbytes = int(nbytes)
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        _lib.check(lib.strata_ipc_alloc(self.nbytes, ctypes.byref(ptr), handle), "strata_ipc_alloc")
        self._own = ptr.value
        self.ptrs = [None] * self.world
        self.ptrs[self.rank] = self._own
        self._opened = []
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                p = ctypes.c_void_p()
                _lib.check(lib.strata_ipc_open(ctypes.create_string_buffer(h, 64), ctypes.byref(p)),
                           "strata_ipc_open")
                self.ptrs[r] = p.value
                self._opened.append(p.value)
        self.local = torch.as_tensor(_DevPtrTensorView(self._own, self.nbytes),
                                     device=torch.device("cuda", torch.cuda.current_device()))

    def ptr_array(self, byte_offset: int = 0):
        arr = (ctypes.c_void_p * self.world)()
        for r in range(self.world):
            arr[r] = self.ptrs[r] + byte_offset
        return arr

    def close(self):
        lib = _lib.load()
        if self.world > 1 and dist.is_initialized():
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
        for p in self._opened:
            lib.strata_ipc_close(p)
        self._opened = []
        if self._own:
            self.local = None
            lib.strata_ipc_free(self._own)
            self._own = None


class DistributedTileCopyHaloPadding(torch.nn.Module):
    """Materialise halo-padded local tiles from distributed interior tiles by peer copies."""

    FLAG_BYTES = 256

    def __init__(self, *, topology: TileTopology, lat_deg: torch.Tensor | None = None,
                 lon_deg: torch.Tensor | None = None, device=None, group=None,
                 max_bytes_per_call: int = 0, timeout_ms: int = 2000):
        super().__init__()
        self.topology = topology
        self.group = group
        self.timeout_ms = int(timeout_ms)
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        a, b = halo_source_maps(topology)
        self.register_buffer("src_a", torch.from_numpy(a).to(dev), persistent=False)
        self.register_buffer("src_b", torch.from_numpy(b).to(dev), persistent=False)
        if lat_deg is not None:
            self.register_buffer("lat_deg", lat_deg, persistent=False)
            self.register_buffer("lon_deg", lon_deg, persistent=False)
        self._shared = None
        self._slot_bytes = 0
        self._epoch = 0
        self._stream = None     # the stream every exchange through this module is issued on
        self._max_bytes = int(max_bytes_per_call)
        if topology.world_size > 1:
            if not dist.is_initialized():
                raise RuntimeError("world_size > 1 needs an initialised torch.distributed group")
            if dist.get_world_size(group) != topology.world_size or dist.get_rank(group) != topology.rank:
                raise ValueError("topology world_size / rank do not match the process group")
            if self._max_bytes > 0:
                self._ensure_shared(self._max_bytes)

    @classmethod
    def from_padded_face_grid(cls, *, topology: TileTopology, lon: torch.Tensor, lat: torch.Tensor,
                              pad_width_data: int, device, **kw):
        """Same arguments as the reference's constructor; lon/lat are padded face grids
        [6, N + 2*pad, N + 2*pad] (degrees) from which each local tile's padded window is cut."""
        T, h = topology.tile_size, topology.halo_width

        def cut(g):
            return torch.stack([g[..., f, pad_width_data + ti * T - h:pad_width_data + (ti + 1) * T + h,
                                  pad_width_data + tj * T - h:pad_width_data + (tj + 1) * T + h]
                                for f, ti, tj in topology.local_tiles])
        return cls(topology=topology, lat_deg=cut(lat).to(device), lon_deg=cut(lon).to(device),
                   device=device, **kw)

    # ---------------------------------------------------------------- shared buffers
    def _ensure_shared(self, payload_bytes: int):
        """(Re)allocate the peer-shared buffer: [flags | slot 0 | slot 1]. Collective."""
        slot = (payload_bytes + 255) // 256 * 256
        if self._shared is not None and slot <= self._slot_bytes:
            return
        if self._shared is not None:
            self._shared.close()
        self._slot_bytes = slot
        self._shared = PeerSharedBuffer(self.FLAG_BYTES + 2 * slot, group=self.group)
        self._epoch = 0

    def _publish_and_sync(self, x_flat_bytes: torch.Tensor):
        """Copy this rank's tiles into the current slot, run the flag barrier; returns the
        per-rank source pointer array for the gather."""
        topo = self.topology
        if topo.world_size == 1:
            arr = (ctypes.c_void_p * 1)()
            arr[0] = x_flat_bytes.data_ptr()
            return arr
        # The two alternating slots are safe only while every exchange through this module (the
        # un-pad adjoint shares its buffer) is issued on ONE stream, in the same order on all
        # ranks: a second stream could overwrite a slot a peer is still reading.
        cur = torch.cuda.current_stream().cuda_stream
        if self._stream is None:
            self._stream = cur
        elif self._stream != cur:
            raise RuntimeError("halo exchanges of one module must all be issued on the same CUDA "
                               "stream (first used: %#x, now: %#x)" % (self._stream, cur))
        nbytes = x_flat_bytes.numel()
        if self._shared is None or nbytes > self._slot_bytes:
            # growth re-allocates the peer-shared buffer: a collective (synchronise, barrier,
            # IPC handles) - size it with max_bytes_per_call to keep it out of the steps
            self._ensure_shared(nbytes)
        self._epoch += 1
        off = self.FLAG_BYTES + (self._epoch & 1) * self._slot_bytes
        self._shared.local[off:off + nbytes].copy_(x_flat_bytes, non_blocking=True)
        flags = self._shared.ptr_array(0)
        stream = torch.cuda.current_stream().cuda_stream
        _lib.check(_lib.load().strata_halo_barrier(flags, topo.rank, topo.world_size, self._epoch,
                                                   self.timeout_ms, stream), "strata_halo_barrier")
        return self._shared.ptr_array(off)

    def check_status(self) -> None:
        """Synchronise and raise if a peer never reached a barrier (or any kernel timed out).
        Until this is called (it clears the condition) every padded tile produced after the
        failed barrier is NaN, so a missed poll cannot let a rollout continue on stale halos."""
        st = _lib.device_status()
        if st != 0:
            raise RuntimeError(f"halo exchange failed on the device (status {st}: "
                               f"{'peer flag wait timed out' if st == 105 else 'kernel wait timed out'})")

    # ---------------------------------------------------------------- field space (reference API)
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        topo = self.topology
        *shape, tpr, nx, ny = x.shape
        if tpr != topo.tiles_per_rank:
            raise ValueError(f"Expected {topo.tiles_per_rank} local tiles, got {tpr}")
        if nx != topo.tile_size or ny != topo.tile_size:
            raise ValueError(f"Expected interior tile shape ({topo.tile_size}, {topo.tile_size}), "
                             f"got ({nx}, {ny})")
        if not x.is_cuda:
            raise _lib.StrataLibraryError("halo exchange needs CUDA tensors (no CPU path)")
        if x.dtype != torch.float32:
            raise TypeError(f"field-space halo exchange is float32, got {x.dtype}")
        P = topo.padded_tile_size
        L = int(np.prod(shape)) if shape else 1
        xc = x.contiguous()
        out = torch.empty(*shape, tpr, P, P, dtype=x.dtype, device=x.device)
        if L == 0:
            return out
        with torch.cuda.device(x.device):
            src = self._publish_and_sync(xc.view(-1).view(torch.uint8))
            _lib.check(_lib.load().strata_halo_gather_fields_f32(
                out.data_ptr(), src, topo.world_size, self.src_a.data_ptr(), self.src_b.data_ptr(),
                tpr, topo.tile_size, topo.halo_width, L,
                torch.cuda.current_stream().cuda_stream), "strata_halo_gather_fields_f32")
        return out

    # ---------------------------------------------------------------- token space
    def pad_tokens(self, tokens: torch.Tensor, depth: int, out: torch.Tensor | None = None,
                   only_halo: bool = False) -> torch.Tensor:
        """tokens [tiles_per_rank, depth, T*T, C] bf16 -> [tiles_per_rank, depth, P*P, C]."""
        topo = self.topology
        T, P = topo.tile_size, topo.padded_tile_size
        if tokens.dtype != torch.bfloat16 or not tokens.is_cuda:
            raise TypeError("pad_tokens expects a CUDA bfloat16 tensor")
        if tuple(tokens.shape[:3]) != (topo.tiles_per_rank, depth, T * T):
            raise ValueError(f"expected [{topo.tiles_per_rank}, {depth}, {T * T}, C], "
                             f"got {tuple(tokens.shape)}")
        C = tokens.shape[-1]
        tc = tokens.contiguous()
        if out is None:
            if only_halo:
                raise ValueError("only_halo needs a preallocated `out` holding the interiors")
            out = torch.empty(topo.tiles_per_rank, depth, P * P, C, dtype=torch.bfloat16,
                              device=tokens.device)
        with torch.cuda.device(tokens.device):
            src = self._publish_and_sync(tc.view(-1).view(torch.uint8))
            _lib.check(_lib.load().strata_halo_gather_tokens_bf16(
                out.data_ptr(), src, topo.world_size, self.src_a.data_ptr(), self.src_b.data_ptr(),
                topo.tiles_per_rank, depth, T, topo.halo_width, C, 1 if only_halo else 0,
                torch.cuda.current_stream().cuda_stream), "strata_halo_gather_tokens_bf16")
        return out

    def close(self):
        if self._shared is not None:
            self._shared.close()
            self._shared = None




class DistributedTileKNNHaloPadding(DistributedTileCopyHaloPadding):
    """Halo cells interpolated from their k nearest source cells on the sphere.

    The reference's production halo (DistributedTileKNNHaloPadding_AllGather,
    screamcast/distributed_halo.py:208-327): padded face lon/lat grids give every halo cell its
    true position, and its value is the inverse-distance-weighted mean of the k = 4 nearest
    interior cells of the globe. Same constructor arguments (`from_padded_face_grid`), same
    `forward(x[..., tiles_per_rank, T, T]) -> [..., tiles_per_rank, P, P]`, `.lat_deg`,
    `.lon_deg`, `.topology`. Instead of all-gathering the globe to every rank and applying a
    sparse operator to it, the k sources of every padded cell are read from the tiles of their
    owners (peer memory) by one weighted-gather kernel. The weights are computed here with a
    k-d tree on unit vectors (the reference uses earth2grid's KNNS2Interpolator, which is not
    available; the weight formula 1 / (chord distance + eps), normalised, is its documented
    behaviour as far as known).
    """

    def __init__(self, *, topology: TileTopology, idx: torch.Tensor, weights: torch.Tensor,
                 lat_deg: torch.Tensor, lon_deg: torch.Tensor, device=None, group=None, **kw):
        super().__init__(topology=topology, lat_deg=lat_deg, lon_deg=lon_deg, device=device,
                         group=group, **kw)
        dev = self.src_a.device
        n_out = topology.tiles_per_rank * topology.padded_tile_size ** 2
        if idx.shape != weights.shape or idx.shape[0] != n_out or idx.dim() != 2:
            raise ValueError(f"idx / weights must be [{n_out}, k]")
        self.k = int(idx.shape[1])
        self.register_buffer("knn_idx", idx.to(dev, torch.int32).contiguous(), persistent=False)
        self.register_buffer("knn_weights", weights.to(dev, torch.float32).contiguous(), persistent=False)

    @classmethod
    def from_padded_face_grid(cls, *, topology: TileTopology, lon: torch.Tensor, lat: torch.Tensor,
                              pad_width_data: int, device, k: int = 4, eps: float = 1e-7, **kw):
        T, h = topology.tile_size, topology.halo_width
        idx, w = knn_halo_weights(topology, lon.detach().cpu().numpy(), lat.detach().cpu().numpy(),
                                  pad_width_data, k=k, eps=eps)

        def cut(g):
            return torch.stack([g[..., f, pad_width_data + ti * T - h:pad_width_data + (ti + 1) * T + h,
                                  pad_width_data + tj * T - h:pad_width_data + (tj + 1) * T + h]
                                for f, ti, tj in topology.local_tiles])
        return cls(topology=topology, idx=torch.from_numpy(idx), weights=torch.from_numpy(w),
                   lat_deg=cut(lat).to(device), lon_deg=cut(lon).to(device), device=device, **kw)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        topo = self.topology
        *shape, tpr, nx, ny = x.shape
        if tpr != topo.tiles_per_rank:
            raise ValueError(f"Expected {topo.tiles_per_rank} local tiles, got {tpr}")
        if nx != topo.tile_size or ny != topo.tile_size:
            raise ValueError(f"Expected interior tile shape ({topo.tile_size}, {topo.tile_size}), "
                             f"got ({nx}, {ny})")
        if not x.is_cuda:
            raise _lib.StrataLibraryError("halo exchange needs CUDA tensors (no CPU path)")
        if x.dtype != torch.float32:
            raise TypeError(f"field-space halo exchange is float32, got {x.dtype}")
        P = topo.padded_tile_size
        L = int(np.prod(shape)) if shape else 1
        out = torch.empty(*shape, tpr, P, P, dtype=x.dtype, device=x.device)
        if L == 0:
            return out
        xc = x.contiguous()
        with torch.cuda.device(x.device):
            src = self._publish_and_sync(xc.view(-1).view(torch.uint8))
            _lib.check(_lib.load().strata_halo_gather_knn_fields_f32(
                out.data_ptr(), src, topo.world_size, self.knn_idx.data_ptr(),
                self.knn_weights.data_ptr(), self.k, tpr, topo.tile_size, topo.halo_width, L,
                torch.cuda.current_stream().cuda_stream), "strata_halo_gather_knn_fields_f32")
        return out

class DistributedTilePlanHaloPadding(DistributedTileKNNHaloPadding):
    """The plan-based tile halo: `DistributedTileKNNHaloPadding(plan, rank, group)` of the
    reference's screamcast/distributed_cubesphere_transforms.py:611-781.

    Same constructor arguments (a `TileHaloPlan` from `build_distributed_tile_halo_plan`, this
    rank, an optional process group) and the same `forward(data_local[..., tiles_per_rank, T, T])
    -> [..., tiles_per_rank, T + 2h, T + 2h]`: interiors copied, every halo cell interpolated
    from the k nearest cells of the ONE source tile the plan assigned it to. The reference
    interpolates on the sending rank, packs a send buffer and runs `all_to_all_single`; here
    the receiving rank reads the k source cells of each of its halo cells from their owner's
    tile (local or peer memory) with the weighted-gather kernel, so nothing is packed, sent or
    scattered and the plan's send / receive sizes are bookkeeping only.
    """

    def __init__(self, plan, rank: int, group=None, device=None, **kw):
        topo = TileTopology(plan.world_size, int(rank), plan.face_size, plan.tile_size,
                            plan.halo_width)
        idx, w = plan_gather_lists(plan, int(rank))
        # (the KNN module's own constructor wants the lists of padded face grids; the plan brings its own)
        DistributedTileCopyHaloPadding.__init__(self, topology=topo, device=device, group=group, **kw)
        dev = self.src_a.device
        self.k = int(idx.shape[1])
        self.register_buffer("knn_idx", torch.from_numpy(idx).to(dev).contiguous(), persistent=False)
        self.register_buffer("knn_weights", torch.from_numpy(w).to(dev).contiguous(), persistent=False)
        self.plan = plan
        self.rank = int(rank)
        self.world_size = plan.world_size
        self.tile_size = plan.tile_size
        self.halo_width = plan.halo_width
        self.tiles_per_rank = plan.tiles_per_rank
        self.tiles_per_dim = plan.tiles_per_dim
        self.padded_size = plan.tile_size + 2 * plan.halo_width
        self.my_tiles = list(topo.local_tiles)
        self._send_sizes = [plan.send_sizes[self.rank][r] for r in range(plan.world_size)]
        self._recv_sizes = [plan.recv_sizes[self.rank][r] for r in range(plan.world_size)]

    @classmethod
    def from_padded_face_grid(cls, **kw):
        raise TypeError("the plan-based halo is built from a TileHaloPlan "
                        "(build_distributed_tile_halo_plan), not from padded face grids")


class NormalizedCopyHaloAdjoint(torch.nn.Module):
    """Windowed overlap-add un-pad: D_w^-1 A^T (w . y) for the copy-halo exchange A.

    Interface of the reference's NormalizedHaloAdjoint (screamcast/distributed_halo.py:330-448):
    built from the halo module and an optional [P, P] window, `forward(padded[..., tiles_per_rank,
    P, P]) -> [..., tiles_per_rank, T, T]`, buffers `.window` and `.weights`. With a uniform
    window it is the Shepard normalisation D^-1 A^T y; a Kaiser-Bessel-derived window
    (`kbd_window`) down-weights halo copies against the owning tile's own values, as the rollout
    launcher does (scripts/ace/run_screamcast_nudged.py:622-634).

    Mechanism: each rank publishes its padded tiles in the halo module's peer buffer; after the
    flag barrier a pull kernel lets every interior cell sum the padded cells that were copied
    from it, wherever they live, in a fixed order - no reduce_scatter, no atomics.
    """

    def __init__(self, halo_exchange: DistributedTileCopyHaloPadding, window: torch.Tensor | None = None):
        super().__init__()
        if type(self) is NormalizedCopyHaloAdjoint and isinstance(halo_exchange, DistributedTileKNNHaloPadding):
            raise TypeError("NormalizedCopyHaloAdjoint transposes the copy halo; for a "
                            "DistributedTileKNNHaloPadding module use NormalizedHaloAdjoint")
        self.halo_exchange = halo_exchange
        topo = halo_exchange.topology
        P = topo.padded_tile_size
        dev = halo_exchange.src_a.device
        w = None if window is None else window.detach().to("cpu", torch.float32).numpy()
        offsets, cell, coef, weights = self._lists(halo_exchange, w)
        self.register_buffer("_offsets", torch.from_numpy(offsets).to(dev), persistent=False)
        self._cell = torch.from_numpy(cell).to(dev)
        self._coef = torch.from_numpy(coef).to(dev)
        win = torch.ones(P, P) if window is None else window.detach().to("cpu", torch.float32)
        self.register_buffer("window", win.reshape(-1).to(dev).contiguous(), persistent=False)
        self.register_buffer("weights", torch.from_numpy(weights).to(dev).reshape(
            1, 1, topo.tiles_per_rank, topo.tile_size, topo.tile_size), persistent=False)

    @staticmethod
    def _lists(halo_exchange, window):
        return halo_adjoint_lists(halo_exchange.topology, window)

    def forward(self, padded: torch.Tensor) -> torch.Tensor:
        topo = self.halo_exchange.topology
        P, T = topo.padded_tile_size, topo.tile_size
        *shape, tpr, nx, ny = padded.shape
        if tpr != topo.tiles_per_rank or nx != P or ny != P:
            raise ValueError(f"Expected [..., {topo.tiles_per_rank}, {P}, {P}], got {tuple(padded.shape)}")
        if not padded.is_cuda:
            raise _lib.StrataLibraryError("halo adjoint needs CUDA tensors (no CPU path)")
        if padded.dtype != torch.float32:
            raise TypeError(f"field-space halo adjoint is float32, got {padded.dtype}")
        L = int(np.prod(shape)) if shape else 1
        out = torch.empty(*shape, tpr, T, T, dtype=padded.dtype, device=padded.device)
        if L == 0:
            return out
        pc = padded.contiguous()
        with torch.cuda.device(padded.device):
            src = self.halo_exchange._publish_and_sync(pc.view(-1).view(torch.uint8))
            _lib.check(_lib.load().strata_halo_adjoint_fields_f32(
                out.data_ptr(), src, topo.world_size, self._offsets.data_ptr(), self._cell.data_ptr(),
                self._coef.data_ptr(), self.window.data_ptr(), self.weights.data_ptr(), tpr, T,
                topo.halo_width, L, torch.cuda.current_stream().cuda_stream),
                "strata_halo_adjoint_fields_f32")
        return out


class NormalizedHaloAdjoint(NormalizedCopyHaloAdjoint):
    """D_w^-1 A^T (w . y) for the halo module it is given - the reference's class of that name
    (screamcast/distributed_halo.py:330-448), whose A is the k-nearest-neighbour regrid.

    Given a `DistributedTileKNNHaloPadding` it transposes that module's weighted gather: every
    rank contributes the (index, weight) lists of its padded cells (one all-gather at
    construction, nothing per call), each interior cell keeps the entries that draw on it, and
    the pull kernel of the copy-halo adjoint sums them with coefficient weight * window in a
    fixed order. Given a copy-halo module it behaves as `NormalizedCopyHaloAdjoint`. Same
    constructor, `forward`, `.window` and `.weights` as the reference.
    """

    @staticmethod
    def _lists(halo_exchange, window):
        topo = halo_exchange.topology
        if not isinstance(halo_exchange, DistributedTileKNNHaloPadding):
            return halo_adjoint_lists(topo, window)
        idx_all, w_all = gather_knn_lists(topo, halo_exchange.knn_idx, halo_exchange.knn_weights,
                                          halo_exchange.group)
        return knn_adjoint_lists(topo, idx_all, w_all, window)


def gather_knn_lists(topo: TileTopology, idx: torch.Tensor, weights: torch.Tensor, group=None):
    """All ranks' k-nearest-neighbour (index, weight) lists in global tile order, as numpy arrays
    [total_tiles*P*P, k] (one all-gather; a set-up step of the adjoint, nothing per call)."""
    if topo.world_size > 1:
        backend = dist.get_backend(group)
        dev = idx.device if backend == "nccl" else torch.device("cpu")
        parts_i = [torch.empty(idx.shape, dtype=idx.dtype, device=dev) for _ in range(topo.world_size)]
        parts_w = [torch.empty(weights.shape, dtype=weights.dtype, device=dev) for _ in range(topo.world_size)]
        dist.all_gather(parts_i, idx.to(dev).contiguous(), group=group)
        dist.all_gather(parts_w, weights.to(dev).contiguous(), group=group)
        idx, weights = torch.cat(parts_i), torch.cat(parts_w)
    return idx.cpu().numpy(), weights.cpu().numpy()


def kbd_window(padded_size: int, beta: float = 10 * np.pi) -> torch.Tensor:
    """Separable Kaiser-Bessel-derived window [P, P] (the rollout launcher's choice:
    scripts/ace/run_screamcast_nudged.py:624-630); P must be even."""
    from scipy.signal.windows import kaiser_bessel_derived
    w1 = torch.tensor(kaiser_bessel_derived(padded_size, beta), dtype=torch.float32)
    return w1[None, :] * w1[:, None]

def channel_chunked(fn_or_chunk, chunk: int = 32):
    """Apply a halo module over chunks of dimension 1 and concatenate the results. Both call
    forms work: the reference rollout driver's decorator factory, `channel_chunked(32)(halo)`
    (scripts/ace/run_screamcast_nudged.py:119-134: a chunk <= 0 returns the function itself,
    the wrapper keeps it as `__wrapped__`), and `channel_chunked(halo, 32)`."""
    def decorate(fn, channel_chunk):
        if channel_chunk <= 0:
            return fn

        def wrapped(x: torch.Tensor) -> torch.Tensor:
            return torch.cat([fn(x[:, c:c + channel_chunk])
                              for c in range(0, x.shape[1], channel_chunk)], dim=1)

        wrapped.__wrapped__ = fn
        return wrapped

    if callable(fn_or_chunk):
        return decorate(fn_or_chunk, int(chunk))
    channel_chunk = int(fn_or_chunk)
    return lambda fn: decorate(fn, channel_chunk)
