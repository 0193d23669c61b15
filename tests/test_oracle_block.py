"""Self-consistency of the block oracle: the gather-based and the mask-based restatements of
neighbourhood attention agree, windows clamp as documented, RoPE is a rotation."""
import pytest
import torch

from oracle import block_oracle as bo


def test_window_starts_clamp():
    assert bo.window_starts(8, 3).tolist() == [0, 0, 1, 2, 3, 4, 5, 5]
    assert bo.window_starts(9, 9).tolist() == [0] * 9
    assert bo.window_starts(10, 7).tolist() == [0, 0, 0, 0, 1, 2, 3, 3, 3, 3]
    with pytest.raises(ValueError):
        bo.window_starts(4, 5)


@pytest.mark.parametrize("shape,kernel", [((1, 3, 6, 7, 2, 8), (3, 3, 5)), ((2, 4, 5, 5, 1, 4), (1, 5, 3)),
                                          ((1, 2, 9, 4, 1, 8), (2, 7, 3))])
def test_na3d_gather_equals_masked(shape, kernel):
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(*shape, generator=g) for _ in range(3))
    a = bo.na3d(q, k, v, kernel)
    b = bo.na3d_masked(q, k, v, kernel)
    torch.testing.assert_close(a, b, atol=1e-5, rtol=1e-5)


def test_na3d_full_window_is_dense_attention():
    g = torch.Generator().manual_seed(4)
    q, k, v = (torch.randn(1, 2, 3, 3, 1, 8, generator=g) for _ in range(3))
    a = bo.na3d(q, k, v, (2, 3, 3))
    qf, kf, vf = (t.reshape(18, 8) for t in (q, k, v))
    ref = torch.softmax(qf @ kf.T * 8 ** -0.5, -1) @ vf
    torch.testing.assert_close(a.reshape(18, 8), ref, atol=1e-5, rtol=1e-5)


def test_rope_is_norm_preserving_and_relative():
    cos, sin = bo.axial_rope_tables(4, 5, 16)
    assert cos.shape == (1, 20, 8)
    g = torch.Generator().manual_seed(5)
    t = torch.randn(1, 2, 20, 3, 16, generator=g)
    r = bo.apply_rope(t, cos, sin)
    torch.testing.assert_close(r.norm(dim=-1), t.norm(dim=-1), atol=1e-5, rtol=1e-5)
    # table length = H*W, shared over depth (reference: tests/test_dit_3d.py:99-101)
    torch.testing.assert_close(bo.apply_rope(t[:, :1], cos, sin), r[:, :1])


def test_stereographic_tables_shape_and_centre():
    H = W = 8
    lat = torch.linspace(0.2, 0.7, H).view(1, H, 1).expand(1, H, W)
    lon = torch.linspace(0.1, 0.6, W).view(1, 1, W).expand(1, H, W)
    cos, sin = bo.stereographic_rope_tables(lat, lon, 64, 4, bo.default_rope_length_scale(1) * 4)
    assert cos.shape == (1, 4, 32) and sin.shape == (1, 4, 32)
    lat0, lon0 = bo.spherical_centroid(lat.double(), lon.double())
    x, y = bo.stereographic_projection(lat0[:, None, None], lon0[:, None, None], lat0, lon0)
    assert abs(float(x)) < 1e-12 and abs(float(y)) < 1e-12


def test_block_forward_runs_and_bf16_emulation_is_close():
    C, heads, grid, kernel = 64, 2, (2, 4, 4), (1, 3, 3)
    p = bo.init_block_params(C, gated=True, seed=1)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(1, 32, C, generator=g)
    cos, sin = bo.axial_rope_tables(4, 4, C // heads)
    y = bo.block_forward(x, p, grid=grid, num_heads=heads, kernel=kernel, rope_cos=cos,
                         rope_sin=sin, gated=True)
    yb = bo.block_forward(x, p, grid=grid, num_heads=heads, kernel=kernel, rope_cos=cos,
                          rope_sin=sin, gated=True, emulate_bf16=True)
    assert y.shape == x.shape and torch.isfinite(y).all()
    assert (y - yb).abs().max() / y.abs().max() < 2e-2
    assert bo.block_flops_per_token(512, (3, 9, 9)) == 6789120
