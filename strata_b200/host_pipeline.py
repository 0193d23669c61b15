"""Block forward for HOST-resident tiles: copies and compute pipelined over chunks of tiles.

A caller whose tokens live in pinned host memory (the end-to-end case: a data loader hands over
host tensors and wants host tensors back) pays two PCIe transfers per block on top of the
compute. Tiles are independent inside a block, so the transfers of one chunk of tiles overlap
with the compute of another: three streams (host->device, compute, device->host) walk a small
ring of device buffers. PCIe is full duplex, so the step time tends to the larger of the two
copy times instead of their sum plus the compute. Consecutive calls can be streamed
(`run(..., join=False)` and one `join()` at the end): the ring carries over, so the first
host->device copy of a call overlaps the last device->host copy of the one before instead of
every call paying the fill and drain of the pipeline.

There is no reference counterpart: the reference feeds device tensors.
"""
from __future__ import annotations

import torch

from . import ops


class HostBlockPipeline:
    """Reusable resources (streams, device ring buffers, workspace) for
    `run(x_host, y_host, ...)`: x_host / y_host [n_tiles, tokens, C] bf16 pinned host tensors."""

    def __init__(self, tokens_per_tile: int, dim: int, hidden: int, device=None, chunk_tiles: int = 1,
                 ring: int = 3):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None \
            else torch.device(device)
        self.tokens, self.dim, self.hidden = int(tokens_per_tile), int(dim), int(hidden)
        self.chunk_tiles, self.ring = int(chunk_tiles), int(ring)
        with torch.cuda.device(self.device):
            self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
            shape = (self.ring, self.chunk_tiles, self.tokens, self.dim)
            self.x_d = torch.empty(shape, dtype=torch.bfloat16, device=self.device)
            self.y_d = torch.empty(shape, dtype=torch.bfloat16, device=self.device)
            self.ws = torch.empty(ops.block_workspace_bytes(self.chunk_tiles * self.tokens, dim, hidden),
                                  dtype=torch.uint8, device=self.device)
        self._computed = [None] * self.ring     # compute of the chunk that last used ring slot b
        self._drained = [None] * self.ring      # its device->host copy
        self._next = 0                          # ring slot of the next chunk
        self._last = None                       # the latest device->host copy

    def join(self) -> None:
        """The current stream waits for every device->host copy issued so far."""
        if self._last is not None:
            torch.cuda.current_stream(self.device).wait_event(self._last)
            self._last = None

    def run(self, x_host: torch.Tensor, y_host: torch.Tensor, weights: dict, *, grid, num_heads: int,
            kernel, rope_cs: torch.Tensor | None = None, qk_norm: bool = False,
            join: bool = True) -> torch.Tensor:
        """join=True: everything is ordered after the work already queued on the current stream,
        and the current stream waits for the last device->host copy - events recorded around
        this call on the current stream time the whole pipeline, and y_host is complete for
        anything queued on that stream afterwards. join=False (streaming): the call returns
        with its device->host copies still in flight and the next call's host->device copies may
        start at once; y_host is complete after `join()` (or a synchronize). x_host must not be
        overwritten by the host before its copies have run."""
        for t, n in ((x_host, "x_host"), (y_host, "y_host")):
            if t.dtype != torch.bfloat16 or t.is_cuda or not t.is_pinned() or not t.is_contiguous():
                raise TypeError(f"{n} must be a contiguous pinned host bfloat16 tensor")
        n_tiles, tokens, C = x_host.shape
        if (tokens, C) != (self.tokens, self.dim) or y_host.shape != x_host.shape:
            raise ValueError("host tensors do not match the pipeline's tile shape")
        main = torch.cuda.current_stream(self.device)
        if self._last is None:
            # nothing of an earlier call is in flight: the copies start after what is queued
            # on the current stream (in streaming mode they only wait for their ring slot)
            start = torch.cuda.Event()
            start.record(main)
            self.s_in.wait_event(start)
            self.s_out.wait_event(start)
        computed, drained = self._computed, self._drained
        last = self._last
        for t0 in range(0, n_tiles, self.chunk_tiles):
            t1 = min(t0 + self.chunk_tiles, n_tiles)
            b, n = self._next, t1 - t0
            self._next = (self._next + 1) % self.ring
            with torch.cuda.stream(self.s_in):
                if computed[b] is not None:
                    self.s_in.wait_event(computed[b])      # x_d[b] has been consumed
                self.x_d[b, :n].copy_(x_host[t0:t1], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(self.s_in)
            main.wait_event(arrived)
            if drained[b] is not None:
                main.wait_event(drained[b])                # y_d[b] has been copied out
            ops.block_forward(self.x_d[b, :n], weights, grid=grid, num_heads=num_heads, kernel=kernel,
                              rope_cos=None, rope_sin=None, qk_norm=qk_norm, workspace=self.ws,
                              out=self.y_d[b, :n],
                              rope_cs=None if rope_cs is None else rope_cs[t0:t1])
            computed[b] = torch.cuda.Event()
            computed[b].record(main)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(computed[b])
                y_host[t0:t1].copy_(self.y_d[b, :n], non_blocking=True)
                drained[b] = torch.cuda.Event()
                drained[b].record(self.s_out)
            last = drained[b]
        self._last = last
        if join:
            self.join()
        return y_host
