"""The allocation-free block entry point (scratch inside the library image) must give the
same result as the ordinary entry point that takes a caller-allocated workspace.

It exists for callers that are handed input/output buffers but cannot obtain device memory
themselves (a plugin inside another program's inference loop, a host whose allocator must
stay untouched). The test drives it through the C ABI directly, twice in a row — the second
call reuses the array with the first call's leftovers in it — and also checks that a problem
beyond the array's 64 MiB limit is refused with the dedicated error code.

Collected last on purpose (file name), so a run that stops at the first failure has already
run everything else.
"""
import ctypes

import pytest
import torch

from oracle import block_oracle as bo
from tests.util import device_block_weights, rel_max_err, tile_latlon

pytestmark = pytest.mark.gpu
TOL_BF16 = 2e-2


def _weights_struct(w):
    from strata_b200 import _lib
    s = _lib.BlockWeights()
    for name in ("qkv", "proj", "gate", "fc1", "fc2"):
        for kind in ("w", "b"):
            t = w.get(f"{kind}_{name}")
            setattr(s, f"{kind}_{name}", None if t is None else t.data_ptr())
    return s


def test_static_scratch_block_matches_workspace_block():
    from strata_b200 import _lib, ops
    lib = _lib.load()
    C, heads, grid, kernel, n_tiles = 128, 2, (4, 16, 16), (3, 7, 7), 2
    D, H, W = grid
    hidden = 4 * C
    p = bo.init_block_params(C, seed=21)
    w = device_block_weights(p, "cuda")
    ws_struct = _weights_struct(w)
    lat, lon = tile_latlon(n_tiles, H, W)
    cos, sin = bo.stereographic_rope_tables(lat, lon, C // heads, 1, bo.default_rope_length_scale(1))
    from strata_b200.rope import pack_rope_tables
    cos, sin = cos.cuda().contiguous(), sin.cuda().contiguous()
    cs = pack_rope_tables(cos, sin)
    stream = torch.cuda.current_stream().cuda_stream

    for call in range(2):                     # two calls in a row share the built-in array
        g = torch.Generator().manual_seed(100 + call)
        x = torch.randn(n_tiles, D * H * W, C, generator=g).bfloat16().cuda().contiguous()
        want = ops.block_forward(x, w, grid=grid, num_heads=heads, kernel=kernel, rope_cos=cos,
                                 rope_sin=sin)
        got = torch.full_like(x, float("nan"))
        if call == 1:
            # The entry point's whole contract: it obtains no device memory. From the second
            # call on (the first one may still load the kernels' code onto the device) neither
            # the driver's free-memory figure nor torch's allocator moves across the call.
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            torch_before = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
        rc = lib.strata_block_forward_static_scratch_bf16(
            x.data_ptr(), got.data_ptr(), n_tiles, D, H, W, C, heads, hidden, *kernel,
            ctypes.byref(ws_struct), cs.data_ptr(), 0, 1e-6, 1e-6, stream)
        assert rc == 0, lib.strata_error_string(rc)
        if call == 1:
            torch.cuda.synchronize()
            assert torch.cuda.mem_get_info()[0] == free_before
            assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == torch_before
        assert _lib.device_status() == 0
        assert not torch.isnan(got).any()
        assert rel_max_err(got, want.float()) < TOL_BF16
        assert torch.equal(got, want)          # same kernels, same order: identical bits


def test_static_scratch_rejects_oversized_problem():
    from strata_b200 import _lib
    lib = _lib.load()
    C, heads, hidden = 512, 8, 2048
    D, H, W, n_tiles = 16, 64, 64, 4           # needs 2.7 GB of scratch: far beyond 64 MiB
    assert lib.strata_block_workspace_bytes(n_tiles * D * H * W, C, hidden) > 64 * 1024 * 1024
    dummy = torch.zeros(8, dtype=torch.bfloat16, device="cuda")
    s = _lib.BlockWeights()
    rc = lib.strata_block_forward_static_scratch_bf16(
        dummy.data_ptr(), dummy.data_ptr(), n_tiles, D, H, W, C, heads, hidden, 3, 9, 9,
        ctypes.byref(s), None, 0, 1e-6, 1e-6, None)
    assert rc == -4
    assert b"64 MiB" in lib.strata_error_string(rc)
