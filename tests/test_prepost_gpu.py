"""Fused pre-/post-processing kernels against the wind-rotation oracle (pinned to the
reference's wind_rotation.py through tests/golden/wind_rotation.npz) and plain index logic."""
import numpy as np
import pytest
import torch

from oracle import halo_oracle as ho

pytestmark = pytest.mark.gpu


def _geometry(B, H, W, seed):
    g = torch.Generator().manual_seed(seed)
    lat = (torch.linspace(-0.9, 1.1, H).view(1, H, 1) + 0.1 * torch.rand(B, 1, 1, generator=g)).expand(B, H, W)
    lon = (torch.linspace(0.2, 1.4, W).view(1, 1, W) + 3.0 * torch.rand(B, 1, 1, generator=g)).expand(B, H, W)
    lat, lon = lat.contiguous(), lon.contiguous()
    lat0, lon0 = ho.tile_center(lat.numpy(), lon.numpy())
    return lat, lon, torch.from_numpy(np.asarray(lat0, np.float32)).reshape(B), \
        torch.from_numpy(np.asarray(lon0, np.float32)).reshape(B)


@pytest.mark.parametrize("patch,wind,concat", [((1, 1, 1), (1, 3), True), ((2, 4, 4), (0, 2), True),
                                               ((1, 2, 2), None, False), ((2, 1, 1), (2, 0), False)])
def test_preprocess_patches(patch, wind, concat):
    from strata_b200 import ops
    B, C, D, H, W = 2, 4, 4, 8, 12
    g = torch.Generator().manual_seed(5)
    x = torch.randn(B, C, D, H, W, generator=g) * 10
    lat, lon, lat0, lon0 = _geometry(B, H, W, 1)
    a = ops.preprocess_patches(x.cuda(), lat.cuda(), lon.cuda(), lat0.cuda(), lon0.cuda(), wind=wind,
                               concat_lat=concat, patch=patch)
    # the same on the host: rotate (oracle), append, gather patches in (c, dv, dh, dw) order
    xr = x.clone().numpy()
    if wind is not None:
        u, v = ho.forward_uv_to_tile(xr[:, wind[0]], xr[:, wind[1]], lat.numpy(), lon.numpy(),
                                     lat0.numpy().reshape(B, 1, 1), lon0.numpy().reshape(B, 1, 1))
        xr[:, wind[0]], xr[:, wind[1]] = u, v
    xr = torch.from_numpy(xr)
    if concat:
        le = lat[:, None, None].expand(B, 1, D, H, W)
        xr = torch.cat([xr, torch.cos(le), torch.sin(le)], dim=1)
    pv, ph, pw = patch
    cin = xr.shape[1]
    want = xr.view(B, cin, D // pv, pv, H // ph, ph, W // pw, pw).permute(0, 2, 4, 6, 1, 3, 5, 7)
    want = want.reshape(-1, cin * pv * ph * pw)
    K = want.shape[1]
    got = a.float().cpu()
    assert got.shape == (want.shape[0], (K + 7) // 8 * 8)
    assert torch.all(got[:, K:] == 0)
    # bf16 rounding of values that agree to fp32 accuracy: at most one bf16 step apart
    assert torch.allclose(got[:, :K], want.bfloat16().float(), rtol=2 ** -7, atol=1e-6)
    exact = (got[:, :K] == want.bfloat16().float()).float().mean()
    assert exact > 0.999


@pytest.mark.parametrize("patch,wind", [((1, 1, 1), (0, 1)), ((2, 2, 2), (3, 1)), ((1, 4, 4), None)])
def test_postprocess_fields(patch, wind):
    from strata_b200 import ops
    B, C, D, H, W = 2, 5, 4, 8, 8
    pv, ph, pw = patch
    g = torch.Generator().manual_seed(8)
    fields = (torch.randn(B, C, D, H, W, generator=g) * 5).bfloat16().float()   # local-frame winds
    lat, lon, lat0, lon0 = _geometry(B, H, W, 2)
    y = fields.view(B, C, D // pv, pv, H // ph, ph, W // pw, pw).permute(0, 2, 4, 6, 3, 5, 7, 1)
    y = y.reshape(-1, pv * ph * pw * C)
    ypad = torch.zeros(y.shape[0], (y.shape[1] + 7) // 8 * 8)
    ypad[:, :y.shape[1]] = y
    got = ops.postprocess_fields(ypad.bfloat16().cuda(), (B, C, D, H, W), lat.cuda(), lon.cuda(),
                                 lat0.cuda(), lon0.cuda(), wind=wind, patch=patch).cpu()
    want = fields.clone().numpy()
    if wind is not None:
        u, v = ho.inverse_tile_to_uv(want[:, wind[0]], want[:, wind[1]], lat.numpy(), lon.numpy(),
                                     lat0.numpy().reshape(B, 1, 1), lon0.numpy().reshape(B, 1, 1))
        want[:, wind[0]], want[:, wind[1]] = u, v
    assert np.allclose(got.numpy(), want, rtol=2e-5, atol=2e-5)
    if wind is None:
        assert np.array_equal(got.numpy(), want)


def test_argument_errors():
    from strata_b200 import ops
    x = torch.zeros(1, 3, 4, 8, 8, device="cuda")
    with pytest.raises(ValueError):
        ops.preprocess_patches(x, None, None, patch=(3, 1, 1))
    with pytest.raises(ValueError):   # rotation without tile centres
        ops.preprocess_patches(x, torch.zeros(1, 8, 8, device="cuda"), torch.zeros(1, 8, 8, device="cuda"),
                               wind=(0, 1))
