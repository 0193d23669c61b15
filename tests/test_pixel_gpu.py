"""Pixel stage (two-stage model) on the GPU against oracle/pixel_oracle.py: the row kernel
(gated residual + LayerNorm + modulate), the q/k RMS norm, the bilinear + depthwise-conv + GELU
conditioning kernel, one AdaLN pixel block, and the whole two-stage wrapper. Tolerances are
max-abs relative errors of bf16 arithmetic (2e-2, as for the backbone block)."""
import pytest
import torch
import torch.nn.functional as F

from oracle import block_oracle as bo
from oracle import pixel_oracle as po
from tests.util import rel_max_err, tile_latlon

pytestmark = pytest.mark.gpu
TOL_BF16 = 2e-2


def _bf(t):
    return t.to(device="cuda", dtype=torch.bfloat16).contiguous()


@pytest.mark.parametrize("M,C", [(1000, 128), (37, 64), (513, 1024), (5, 2048)])
def test_adaln_rows_matches_formula(M, C):
    from strata_b200 import ops
    g = torch.Generator().manual_seed(M + C)
    x, y = torch.randn(M, C, generator=g), torch.randn(M, C, generator=g)
    mod = torch.randn(M, 6 * C, generator=g) * 0.5
    xb, yb, mb = _bf(x), _bf(y), _bf(mod)
    xf, yf, mf = xb.float().cpu(), yb.float().cpu(), mb.float().cpu()
    sh, sc, gt = mf[:, :C], mf[:, C:2 * C], mf[:, 2 * C:3 * C]
    # LN + modulate only
    out = ops.adaln_rows(xb.clone(), shift=mb[:, :C], scale=mb[:, C:2 * C])
    want = F.layer_norm(xf, (C,), eps=1e-6) * (1 + sc) + sh
    assert rel_max_err(out, want) < 1e-2
    # plain LN equals the LayerNorm kernel bit for bit
    assert torch.equal(ops.adaln_rows(xb.clone()), ops.layernorm(xb))
    # gated residual + LN + modulate; the residual stream is updated in place
    x2 = xb.clone()
    out2 = ops.adaln_rows(x2, y=yb, gate=mb[:, 2 * C:3 * C], shift=mb[:, :C], scale=mb[:, C:2 * C])
    x_new = (xf + gt * yf).bfloat16()
    assert torch.equal(x2.cpu(), x_new)
    want2 = F.layer_norm(x_new.float(), (C,), eps=1e-6) * (1 + sc) + sh
    assert rel_max_err(out2, want2) < 1e-2
    # residual only, no gate
    x3 = xb.clone()
    assert ops.adaln_rows(x3, y=yb, norm=False) is None
    assert torch.equal(x3.cpu(), (xf + yf).bfloat16())
    with pytest.raises(ValueError):
        ops.adaln_rows(xb, norm=False)


def test_qk_norm_rows():
    from strata_b200 import ops
    M, C = 777, 128
    qkv = _bf(torch.randn(M, 3 * C, generator=torch.Generator().manual_seed(3)) * 3)
    ref = qkv.float().cpu().reshape(M, 3, C // 64, 64).clone()
    ref[:, :2] = bo.rms_norm(ref[:, :2])
    got = ops.qk_norm_rows_(qkv.clone(), C)
    assert torch.equal(got[:, 2 * C:], qkv[:, 2 * C:])          # v untouched
    assert rel_max_err(got, ref.reshape(M, 3 * C)) < 1e-2


@pytest.mark.parametrize("shape,factor,ks", [((1, 2, 5, 6, 64), 4, 5), ((2, 1, 4, 4, 128), 2, 5),
                                             ((1, 3, 3, 7, 64), 4, 3), ((1, 2, 6, 5, 64), 1, 5),
                                             ((2, 2, 9, 11, 1024), 4, 5), ((1, 1, 5, 4, 96), 8, 5),
                                             ((1, 2, 4, 6, 72), 4, 5)])
def test_adaln_cond_matches_oracle(shape, factor, ks):
    from strata_b200 import ops
    g = torch.Generator().manual_seed(sum(shape) + factor)
    tok = _bf(torch.randn(shape, generator=g))
    Cb = shape[-1]
    w = torch.randn(Cb, ks, ks, generator=g) * 0.3
    b = torch.randn(Cb, generator=g) * 0.1
    want = po.adaln_cond(tok.float().cpu(), w, b, factor).reshape(-1, Cb)
    got = ops.adaln_cond(tok, w.cuda(), b.cuda(), factor)
    assert got.shape == want.shape
    assert rel_max_err(got, want) < 1e-2
    # the tap-by-tap evaluation (the only one for small factors) agrees as well
    direct = ops.adaln_cond(tok, w.cuda(), b.cuda(), factor, direct=True)
    assert rel_max_err(direct, want) < 1e-2
    # a row range gives the same rows
    part = ops.adaln_cond(tok, w.cuda(), b.cuda(), factor, row0=17, n_rows=40)
    assert torch.equal(part, got[17:57])
    # without bias
    got0 = ops.adaln_cond(tok, w.cuda(), None, factor)
    assert rel_max_err(got0, po.adaln_cond(tok.float().cpu(), w, None, factor).reshape(-1, Cb)) < 1e-2


def _two_stage(**over):
    from strata_b200.wrappers import StrataModel
    kw = dict(depth=4, height=32, width=32, n_layers=2, patch_size_vert=1, patch_size_horiz=4,
              in_chans=5, base_out_chans=5, embed_dim=128, num_heads=2, attn_kernel=3,
              do_rope_2d_stereographic=True, index_is_latlon=True, do_bf16_mixed=True,
              gated_attention=True, qk_norm=True, embed_dim_pixel=128, n_layers_pixel=2,
              attn_kernel_pixel=(3, 5, 5), qk_norm_pixel=True, do_bf16_mixed_pixel=True,
              use_bilinear_dw_gelu_project_adaln_pixel=True)
    kw.update(over)
    torch.manual_seed(0)
    return StrataModel(**kw).cuda().eval()


def _randomise(m, seed=5):
    """Seeded default initialisation, random biases, and a non-zero AdaLN projection (a fresh
    one is zero, which would leave the modulation path untested)."""
    with torch.no_grad():
        g = torch.Generator().manual_seed(seed)
        for n, p in m.named_parameters():
            if n.endswith(".bias"):
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)
            if n.endswith("adaln_bilinear_dw_proj.weight") or n.endswith("adaln_pixel_proj.1.weight"):
                p.copy_(torch.randn(p.shape, generator=g) * (0.5 / p.shape[1] ** 0.5))
    return m


def test_pixel_block_matches_oracle():
    m = _randomise(_two_stage())
    blk = m.strata.pixel_blocks[0]
    B, D, H, W, C, Cb, f = 1, 4, 16, 16, 128, 128, 4
    g = torch.Generator().manual_seed(1)
    x = torch.randn(B, D * H * W, C, generator=g)
    s = torch.randn(B, D, H // f, W // f, Cb, generator=g)
    with torch.inference_mode():
        mod = blk.modulation(_bf(s), f)
        got = blk(_bf(x).view(-1, C), (D, H, W), mod, B).view(B, -1, C)
    p = {k: v.detach().cpu() for k, v in blk.state_dict().items()}
    sb = _bf(s).float().cpu()
    cond = po.adaln_cond(sb, p["adaln_bilinear_dw_conv.weight"].reshape(Cb, 5, 5),
                         p["adaln_bilinear_dw_conv.bias"], f)
    for emulate in (False, True):
        want = po.pixel_block_forward(_bf(x).float().cpu(), po.modulation(cond, p, emulate), p,
                                      grid=(D, H, W), num_heads=2, kernel=(3, 5, 5), qk_norm=True,
                                      emulate_bf16=emulate)
        err = rel_max_err(got, want)
        print(f"pixel block vs oracle (emulate_bf16={emulate}): {err:.4f}")
        assert err < TOL_BF16


def test_fresh_pixel_blocks_are_identity():
    # adaLN-zero: with the projection at its zero initialisation every gate is 0
    m = _two_stage()
    blk = m.strata.pixel_blocks[0]
    x = _bf(torch.randn(4 * 16 * 16, 128, generator=torch.Generator().manual_seed(2)))
    s = _bf(torch.randn(1, 4, 4, 4, 128, generator=torch.Generator().manual_seed(3)))
    with torch.inference_mode():
        y = blk(x.clone(), (4, 16, 16), blk.modulation(s, 4), 1)
    assert torch.equal(y, x)


@pytest.mark.parametrize("wind,first_only,extra", [
    (False, False, {}),
    (True, True, {}),
    (False, False, dict(do_rope_2d_stereographic_pixel=True)),
    (True, False, dict(do_rope_2d_pixel=True, qk_norm_pixel=False)),
    (False, False, dict(use_bilinear_dw_gelu_project_adaln_pixel=False)),
    (False, True, dict(use_bilinear_dw_gelu_project_adaln_pixel=False, patch_size_vert=2,
                       attn_kernel=(1, 3, 3))),
])
def test_two_stage_model_matches_oracle(wind, first_only, extra):
    over = dict(first_block_only_adaln_pixel=first_only, **extra)
    if wind:
        over.update(do_rotate_wind=True, wind_channel_indices=(0, 1))
    m = _randomise(_two_stage(**over))
    names = [n for n, _ in m.named_parameters()]
    assert any(n.startswith("strata.pixel_blocks.1.adaln_") for n in names) == (not first_only)
    assert not any(n.startswith("strata.backbone.final_layer") for n in names)
    B, H, W = 2, 32, 32
    x = torch.randn(B, 5, 4, H, W, generator=torch.Generator().manual_seed(0))
    lat, lon = tile_latlon(B, H, W)
    with torch.inference_mode():
        y = m(x.cuda(), {"lat": lat.cuda(), "lon": lon.cuda()})
    assert y.shape == x.shape and torch.isfinite(y).all()
    state = {k: v.detach().cpu() for k, v in m.state_dict().items()}
    rope_px = ("stereographic" if extra.get("do_rope_2d_stereographic_pixel")
               else "axial" if extra.get("do_rope_2d_pixel") else "none")
    kw = dict(patch=(extra.get("patch_size_vert", 1), 4, 4), num_heads=2,
              kernel=extra.get("attn_kernel", 3), num_layers=2,
              num_heads_pixel=2, kernel_pixel=(3, 5, 5), num_layers_pixel=2, lat=lat, lon=lon,
              qk_norm=True, gated=True, qk_norm_pixel=extra.get("qk_norm_pixel", True),
              wind_channels=(0, 1) if wind else None, rope_mode_pixel=rope_px)
    for emulate in (False, True):
        ref = po.two_stage_forward(x, state, emulate_bf16=emulate, **kw)
        err = rel_max_err(y, ref)
        print(f"two-stage model vs oracle (emulate_bf16={emulate}, {extra}): {err:.4f}")
        assert err < TOL_BF16


def test_two_stage_wrapper_contract():
    from strata_b200.wrappers import StrataModel
    m = _two_stage()
    assert (m._depth, m._height, m._width, m._out_chans) == (4, 32, 32, 5)
    m.set_tile_size(16, 48)
    assert (m._height, m._width, m.strata.backbone.height) == (16, 48, 16)
    m.set_rope_length_scale(1e-2)
    assert m.strata.backbone.rope_length_scale == 4e-2
    m.disable_activation_checkpointing()
    ax = _two_stage(do_rope_2d_pixel=True)
    assert ax.strata._rope_cos_pixel.shape[-2] == 4 * 32 * 32     # tests/test_dit_3d_pixel.py:200
    ax.set_tile_size(16, 48)
    assert ax.strata._rope_cos_pixel.shape[-2] == 4 * 16 * 48 and ax.strata._rope_cos_pixel.is_cuda
    st = _two_stage(do_rope_2d_stereographic_pixel=True)
    st.set_rope_length_scale(1e-2)
    assert st.strata.rope_length_scale_pixel == 1e-2 and st.strata.backbone.rope_length_scale == 4e-2
    with pytest.raises(ValueError, match="patch_size_vert=1"):
        _two_stage(patch_size_vert=2, depth=4)
    with pytest.raises(TypeError, match="Unsupported legacy DiT kwargs"):
        _two_stage(no_such_option=1)
    with pytest.raises(ValueError, match="both"):
        StrataModel(do_rope_2d_pixel=True, do_rope_2d_stereographic_pixel=True, depth=4, height=32,
                    width=32, in_chans=5, base_out_chans=5)
    x = torch.randn(1, 5, 4, 16, 48, device="cuda")
    lat, lon = tile_latlon(1, 16, 48)
    with torch.inference_mode():
        y = m(x, {"lat": lat.cuda(), "lon": lon.cuda()})
    assert y.shape == x.shape


def test_sphere_stepper_runs_the_two_stage_model():
    from strata_b200.rollout import TiledSphereStepper
    from strata_b200.topology import TileTopology
    topo = TileTopology(1, 0, face_size=32, tile_size=16, halo_width=8)
    net = _randomise(_two_stage(height=32, width=32, in_chans=3, base_out_chans=3, n_layers=1,
                                n_layers_pixel=1))
    step = TiledSphereStepper(net, topo)
    x = torch.randn(3, 4, topo.tiles_per_rank, 16, 16, device="cuda",
                    generator=torch.Generator("cuda").manual_seed(1))
    y = step(x)
    assert y.shape == x.shape and torch.isfinite(y).all()
    padded = step.halo(x).permute(2, 0, 1, 3, 4).contiguous()
    with torch.inference_mode():
        want = topo.crop(net(padded, {"lat": step.lat_rad, "lon": step.lon_rad})).permute(1, 2, 0, 3, 4)
    assert torch.equal(y, want)
    step.halo.check_status()
