"""Per-block K/V halo exchange (token space, receiver-frame RoPE) against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import block_oracle as bo
from tests.util import device_block_weights, rel_max_err

pytestmark = pytest.mark.gpu
TOL_BF16 = 2e-2


def _grid(face, tile):
    from strata_b200.rollout import equiangular_cubed_sphere_latlon
    from strata_b200.topology import TileTopology
    lat, lon = equiangular_cubed_sphere_latlon(face)
    full = TileTopology(1, 0, face, tile, 0)
    cut = lambda g: np.stack([g[f, i * tile:(i + 1) * tile, j * tile:(j + 1) * tile]
                              for f, i, j in full.global_tiles])
    return cut(lat), cut(lon)


def test_padded_qkv_store_and_region_attention_match_plain_path():
    # halo 0 would be trivial; use a real halo but compare the two building blocks separately
    from strata_b200 import ops
    T, h, D, C, heads, n = 32, 4, 2, 128, 2, 3
    P = T + 2 * h
    g = torch.Generator().manual_seed(0)
    x = torch.randn(n * D * T * T, C, generator=g).bfloat16().cuda()
    w = (torch.randn(3 * C, C, generator=g) * 0.08).bfloat16().cuda()
    b = (torch.randn(3 * C, generator=g) * 0.1).cuda()
    plain = ops.qkv_rope(x, w, b, 64, None, None, D * T * T, T * T)
    out = torch.full((n * D * P * P, 3 * C), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.qkv_rope_padded(x, w, b, 64, None, D * T * T, T * T, out, tile=T, halo=h, depth=D)
    o5 = out.view(n, D, P, P, 3 * C)
    assert torch.equal(o5[:, :, h:h + T, h:h + T].reshape(-1, 3 * C), plain)
    assert torch.isnan(o5[:, :, :h]).all() and torch.isnan(o5[:, :, :, -h:]).all()   # halo untouched
    # region attention == full attention on the padded plane, cropped
    q, k, v = (torch.randn(1, 3, P, P, heads, 64, generator=g).bfloat16().cuda() for _ in range(3))
    full = ops.na3d(q, k, v, (3, 5, 5))
    reg = ops.na3d_region(q, k, v, (3, 5, 5), (h, T, h, T))
    # (query tiles start at the region's origin, so keys are summed in a different order)
    assert rel_max_err(reg, full[:, :, h:h + T, h:h + T].float()) < 1e-2
    # an inner region and four border strips written into one output window give the same
    # tensor (different query tiling, hence only a tolerance)
    r = 2
    o = torch.full((1, 3, T, T, heads, 64), float("nan"), dtype=torch.bfloat16, device="cuda")
    for region in ((h + r, T - 2 * r, h + r, T - 2 * r), (h, r, h, T), (h + T - r, r, h, T),
                   (h + r, T - 2 * r, h, r), (h + r, T - 2 * r, h + T - r, r)):
        ops.na3d_region(q, k, v, (3, 5, 5), region, out=o, out_window=(h, T, h, T))
    assert not torch.isnan(o).any()
    assert rel_max_err(o, reg.float()) < 1e-2
    with pytest.raises(ValueError):   # output window must contain the query region
        ops.na3d_region(q, k, v, (3, 5, 5), (h, T, h, T), out=o[:, :, :T - 1].contiguous(),
                        out_window=(h, T - 1, h, T))


def _setup(halo, kernel, gated=False, seed=12, **runner_kw):
    from strata_b200.halo_block import TiledBlockRunner
    from strata_b200.topology import TileTopology
    face, tile, D, C, heads = 64, 32, 2, 64, 1
    topo = TileTopology(1, 0, face, tile, halo)
    lat, lon = _grid(face, tile)
    p = bo.init_block_params(C, gated=gated, seed=seed, scheme="xavier")
    g = torch.Generator().manual_seed(seed + 1)
    x = torch.randn(topo.total_tiles, D * tile * tile, C, generator=g).bfloat16()
    # a coarse synthetic sphere has huge tokens; pick the length scale so that RoPE angles
    # between neighbouring tokens are O(0.1 - 1) rad, as on the production grid
    scale = np.radians(90.0 / face)
    run = TiledBlockRunner(topo, depth=D, dim=C, num_heads=heads, kernel=kernel, lat_deg=lat,
                           lon_deg=lon, rope_length_scale=scale, **runner_kw)
    okw = dict(face=face, tile=tile, halo=halo, depth=D, num_heads=heads, kernel=kernel,
               lat_deg=lat, lon_deg=lon, length_scale=scale)
    return run, topo, p, x, okw


@pytest.mark.parametrize("qk_norm,kernel,halo", [(False, (1, 5, 5), 2), (True, (2, 7, 7), 4)])
def test_tiled_attention_matches_oracle(qk_norm, kernel, halo):
    from strata_b200 import ops
    run, topo, p, x, okw = _setup(halo, kernel)
    w = device_block_weights(p, "cuda")
    xn = ops.layernorm(x.cuda().reshape(-1, x.shape[-1]))
    o = run.attention(xn, w["w_qkv"], w["b_qkv"], qk_norm=qk_norm).view(x.shape)
    run.check_status()
    ref = bo.tiled_block_forward(x.float(), p, qk_norm=qk_norm, return_attention=True, **okw)
    assert rel_max_err(o, ref) < TOL_BF16
    # the halo (and the frame change of its keys) matters: a tile on its own, or a halo whose
    # keys stay in their owner's RoPE frame, gives visibly different border tokens
    cos, sin = bo.rope_tables_from_coords(*_own_frame_coords(okw), 64, 100.0)
    xn32 = torch.nn.functional.layer_norm(x.float(), (64,), eps=1e-6)
    qkv = torch.nn.functional.linear(xn32, p["attn.qkv.weight"], p["attn.qkv.bias"])
    D, T = 2, 32
    qkv = qkv.reshape(topo.total_tiles, D, T * T, 3, 1, 64)
    q, k, v = qkv[..., 0, :, :], qkv[..., 1, :, :], qkv[..., 2, :, :]
    if qk_norm:
        q, k = bo.rms_norm(q), bo.rms_norm(k)
    q, k = bo.apply_rope(q, cos, sin), bo.apply_rope(k, cos, sin)
    s6 = (topo.total_tiles, D, T, T, 1, 64)
    solo = bo.na3d(q.reshape(s6), k.reshape(s6), v.reshape(s6), kernel).reshape(x.shape)
    assert rel_max_err(solo, ref) > 5 * TOL_BF16


def _own_frame_coords(okw):
    lat = torch.deg2rad(torch.from_numpy(okw["lat_deg"]))
    lon = torch.deg2rad(torch.from_numpy(okw["lon_deg"]))
    lat0, lon0 = bo.spherical_centroid(lat, lon)
    px, py = bo.stereographic_projection(lat, lon, lat0, lon0)
    return (px / okw["length_scale"]).flatten(1), (py / okw["length_scale"]).flatten(1)


@pytest.mark.parametrize("gated,qk_norm,kernel,halo,runner_kw", [
    (False, False, (1, 5, 5), 2, {}), (True, True, (2, 7, 7), 4, {}),
    # token-wise stages in chunks of tiles
    (True, False, (2, 7, 7), 4, {"chunk_tiles": 5}),
    (False, True, (1, 5, 5), 3, {}),
])
def test_tiled_block_matches_oracle(gated, qk_norm, kernel, halo, runner_kw):
    run, topo, p, x, okw = _setup(halo, kernel, gated=gated, **runner_kw)
    y = run.block_forward(x.cuda(), device_block_weights(p, "cuda"), qk_norm=qk_norm)
    run.check_status()
    ref = bo.tiled_block_forward(x.float(), p, qk_norm=qk_norm, gated=gated, **okw)
    assert rel_max_err(y, ref) < TOL_BF16


@pytest.mark.skipif(not (torch.cuda.is_available() and torch.cuda.device_count() >= 2),
                    reason="needs 2 GPUs on one node")
def test_two_rank_tiled_block_stack():
    import os, subprocess, sys
    from pathlib import Path
    worker = Path(__file__).resolve().parent / "halo_block_worker.py"
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                        "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port",
                        "29533", str(worker)], capture_output=True, text=True, timeout=600,
                       env={**os.environ, "NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "HALO BLOCK WORKER OK" in r.stdout
