"""Module-level behaviour of the drop-in wrappers on the GPU: the shape / structure contract the
reference's own model tests check (tests/test_dit_3d.py, tests/test_dit_3d_pixel.py), and
numerical parity of the whole single-stage model with the CPU oracle."""
import math

import pytest
import torch

from oracle import block_oracle as bo
from tests.util import rel_max_err, tile_latlon

pytestmark = pytest.mark.gpu
TOL_BF16 = 2e-2


def _model(**over):
    from strata_b200.wrappers import StrataBackboneModel
    kw = dict(depth=4, height=32, width=32, n_layers=2, patch_size_vert=1, patch_size_horiz=4,
              in_chans=5, base_out_chans=5, embed_dim=128, num_heads=2, attn_kernel=3,
              do_rope_2d_stereographic=True, index_is_latlon=True, do_bf16_mixed=True)
    kw.update(over)
    torch.manual_seed(0)
    return StrataBackboneModel(**kw).cuda().eval()


def _fill_deterministic(model):
    # the reference's characterisation recipe (tests/test_characterization_inference.py:95-109)
    with torch.no_grad():
        for idx, (_n, p) in enumerate(sorted(model.named_parameters(), key=lambda kv: kv[0])):
            ramp = torch.arange(p.numel(), dtype=torch.float32, device=p.device)
            p.copy_((torch.sin(ramp * 0.013 + idx * 0.7) * 0.02).reshape(p.shape))
    return model


def _index(B, H, W):
    lat, lon = tile_latlon(B, H, W)
    return {"lat": lat.cuda(), "lon": lon.cuda()}, lat, lon


def test_forward_shape_and_finite():
    m = _model()
    x = torch.randn(2, 5, 4, 32, 32, device="cuda")
    idx, _, _ = _index(2, 32, 32)
    with torch.inference_mode():
        y = m(x, idx)
    assert y.shape == x.shape and torch.isfinite(y).all()


def test_gated_wind_axial_variants_run():
    for over in (dict(gated_attention=True, qk_norm=True),
                 dict(do_rotate_wind=True, wind_channel_indices=(0, 1)),
                 dict(do_rope_2d_stereographic=False, do_rope_2d=True),
                 dict(do_alt_depthwise_attn=True, attn_kernel=3)):
        m = _model(**over)
        x = torch.randn(1, 5, 4, 32, 32, device="cuda")
        idx, _, _ = _index(1, 32, 32)
        with torch.inference_mode():
            y = m(x, idx)
        assert y.shape == x.shape and torch.isfinite(y).all(), over


def test_set_tile_size_equals_fresh_construction():
    # reference: tests/test_dit_3d.py:107-142 (bit-exact)
    a = _fill_deterministic(_model(height=32, width=32))
    a.set_tile_size(16, 48)
    b = _fill_deterministic(_model(height=16, width=48))
    x = torch.randn(1, 5, 4, 16, 48, device="cuda", generator=torch.Generator("cuda").manual_seed(0))
    idx, _, _ = _index(1, 16, 48)
    with torch.inference_mode():
        assert torch.equal(a(x, idx), b(x, idx))
    assert (a._height, a._width, a._depth, a._out_chans) == (16, 48, 4, 5)


def test_rope_unit_system_and_errors():
    from strata_b200.wrappers import StrataBackboneModel
    m = _model()
    assert m.strata.rope_length_scale == math.sqrt(math.pi * 16 / (3.0 * 1024 ** 2))
    m.set_rope_length_scale(1e-2)
    assert m.strata.rope_length_scale == 4e-2
    with pytest.raises(ValueError, match="must be positive"):
        _model(rope_length_scale=-1.0)
    with pytest.raises(ValueError, match="stereographic"):
        _model(do_rope_2d_stereographic=False, do_rope_2d=True).set_rope_length_scale(1e-2)
    with pytest.raises(ValueError, match="both"):
        StrataBackboneModel(do_rope_2d=True, do_rope_2d_stereographic=True)
    with pytest.raises(ValueError, match="wind_channel_indices"):
        StrataBackboneModel(do_rotate_wind=True)
    m.disable_activation_checkpointing()
    assert m._activation_checkpointing_ratio == 0.0


def test_mlp_gelu_is_tanh_everywhere():
    from strata_b200.strata import Mlp
    m = _model()
    acts = [mod.layers[1] for mod in m.modules() if isinstance(mod, Mlp)]
    assert acts and all(a.approximate == "tanh" for a in acts)


def test_state_dict_order_matches_manifest_shape():
    m = _model(gated_attention=True, n_layers=3)
    names = [n for n, _ in m.named_parameters()]
    per_block = ["attn.qkv.weight", "attn.qkv.bias", "attn.proj.weight", "attn.proj.bias",
                 "attn.gate_proj.weight", "attn.gate_proj.bias", "mlp.layers.0.weight",
                 "mlp.layers.0.bias", "mlp.layers.2.weight", "mlp.layers.2.bias"]
    want = ["strata.patch_embed.proj.weight", "strata.patch_embed.proj.bias"]
    for i in range(3):
        want += [f"strata.blocks.{i}.{s}" for s in per_block]
    want += ["strata.final_layer.linear.weight", "strata.final_layer.linear.bias"]
    assert names == want
    assert not any("lat_radians" in k or "rope" in k for k in m.state_dict())   # buffers not persisted


@pytest.mark.parametrize("wind,gated", [(False, False), (True, True)])
def test_whole_model_matches_oracle(wind, gated):
    over = dict(gated_attention=gated, qk_norm=gated, attn_kernel=(3, 5, 5))
    if wind:
        over.update(do_rotate_wind=True, wind_channel_indices=(0, 1))
    # Seeded default initialisation plus random biases. (The sin-ramp fill of the reference's
    # characterisation test gives strongly correlated channels; the final LayerNorm then
    # amplifies single-ulp bf16 differences of the tokens and the comparison measures that
    # amplification instead of the kernels.)
    m = _model(**over)
    with torch.no_grad():
        g = torch.Generator().manual_seed(5)
        for n, p in m.named_parameters():
            if n.endswith(".bias"):
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)
    B, H, W = 2, 32, 32
    x = torch.randn(B, 5, 4, H, W, generator=torch.Generator().manual_seed(0))
    idx, lat, lon = _index(B, H, W)
    with torch.inference_mode():
        y = m(x.cuda(), idx)
    state = {k: v.detach().cpu() for k, v in m.state_dict().items()}
    kw = dict(patch=(1, 4, 4), num_heads=2, kernel=(3, 5, 5), num_layers=2, lat=lat, lon=lon,
              qk_norm=gated, gated=gated, wind_channels=(0, 1) if wind else None)
    ref = bo.backbone_forward(x, state, **kw)
    ref_bf16 = bo.backbone_forward(x, state, emulate_bf16=True, **kw)
    err_fp32, err_bf16 = rel_max_err(y, ref), rel_max_err(y, ref_bf16)
    print(f"whole model: vs fp32 oracle {err_fp32:.4f}, vs bf16-rounding oracle {err_bf16:.4f}")
    assert err_fp32 < TOL_BF16
    assert err_bf16 < TOL_BF16


def test_sphere_stepper_is_pad_network_crop():
    from strata_b200.rollout import TiledSphereStepper
    from strata_b200.topology import TileTopology
    topo = TileTopology(1, 0, face_size=32, tile_size=16, halo_width=8)
    net = _fill_deterministic(_model(height=32, width=32, patch_size_horiz=1, embed_dim=64,
                                     num_heads=1, in_chans=3, base_out_chans=3, n_layers=1))
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


def test_sphere_stepper_overlap_add_unpad():
    # un-pad by windowed overlap-add instead of the crop: with a network that returns its input,
    # every interior cell becomes a weighted mean of copies of itself - the input comes back
    # (up to rounding; cells that feed a corner mean also receive that mean back)
    from strata_b200.rollout import TiledSphereStepper
    from strata_b200.topology import TileTopology

    class Identity(torch.nn.Module):
        def forward(self, x, index):
            return x
    topo = TileTopology(1, 0, face_size=32, tile_size=16, halo_width=4)
    step = TiledSphereStepper(Identity(), topo, unpad="adjoint", window="kbd")
    x = torch.randn(2, 3, topo.tiles_per_rank, 16, 16, device="cuda",
                    generator=torch.Generator("cuda").manual_seed(2))
    y = step(x)
    assert y.shape == x.shape
    away = torch.ones(16, 16, dtype=torch.bool)      # cells that no corner mean draws from
    for r in (slice(0, 4), slice(12, 16)):
        for c in (slice(0, 4), slice(12, 16)):
            away[r, c] = False
    assert torch.allclose(y[..., away], x[..., away], rtol=1e-5, atol=1e-6)
    assert (y - x).abs().max() < 4.0                 # corner cells: a mean of nearby values
    step.halo.check_status()
    with pytest.raises(ValueError):
        TiledSphereStepper(Identity(), topo, unpad="average")
