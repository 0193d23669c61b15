"""De-aliased patch embedding: the oracle against golden outputs of the reference's own module
(tests/golden/dealias_patch_embed.npz, made by tests/golden/make_golden.py from
screamcast/dealias.py run in fp32), the filtered-patch form the CUDA path uses against the
same goldens, and - on the GPU - the kernel + GEMM and the wrapper option."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import block_oracle as bo

GOLD = np.load(Path(__file__).parent / "golden" / "dealias_patch_embed.npz")
CASES = ("p144", "p222", "p133")


def _case(n):
    t = lambda k: torch.from_numpy(GOLD[f"{n}_{k}"])
    return t("x"), t("w"), t("b"), tuple(int(v) for v in GOLD[n + "_patch"]), GOLD[n + "_filter"].tolist(), t("y")


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_reference_golden(name):
    x, w, b, patch, filt, y = _case(name)
    got = bo.dealiased_patch_embed(x, w, b, patch, filt)
    assert got.shape == y.shape
    assert torch.allclose(got, y, atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("name", CASES)
def test_filtered_patch_form_matches_reference_golden(name):
    """token = bias + W . (sum_k f[k] * patch at clamp(t * p + k - (K-1)//2, 0, S - p)): the
    arithmetic of dealias_patches_kernel followed by the GEMM, in float64 loops."""
    x, w, b, patch, filt, y = _case(name)
    x, w, b = x.double(), w.double(), b.double()
    B, C, D, H, W = x.shape
    pd, ph, pw = patch
    f = torch.tensor(filt, dtype=torch.float64)
    taps = [(f / f.sum()) if p > 1 else torch.ones(1, dtype=torch.float64) for p in patch]
    out = torch.zeros(B, w.shape[0], D // pd, H // ph, W // pw, dtype=torch.float64)
    for td in range(D // pd):
        for th in range(H // ph):
            for tw in range(W // pw):
                acc = torch.zeros(B, C, pd, ph, pw, dtype=torch.float64)
                for i, fd in enumerate(taps[0]):
                    sd = min(max(td * pd + i - (len(taps[0]) - 1) // 2, 0), D - pd)
                    for j, fh in enumerate(taps[1]):
                        sh = min(max(th * ph + j - (len(taps[1]) - 1) // 2, 0), H - ph)
                        for k, fw in enumerate(taps[2]):
                            sw = min(max(tw * pw + k - (len(taps[2]) - 1) // 2, 0), W - pw)
                            acc += fd * fh * fw * x[:, :, sd:sd + pd, sh:sh + ph, sw:sw + pw]
                out[:, :, td, th, tw] = torch.einsum("bcvyx,ecvyx->be", acc, w) + b
    assert torch.allclose(out.float(), y, atol=2e-5, rtol=1e-5)


def test_module_contract_on_cpu():
    from strata_b200.strata import DealiasedPatchEmbed3D
    from strata_b200.wrappers import StrataBackboneModel
    m = DealiasedPatchEmbed3D(4, 8, 8, patch_size=(1, 4, 4), in_chans=3, embed_dim=16,
                              resample_filter=(1, 4, 6, 4, 1))
    assert list(m.state_dict()) == ["proj.weight", "proj.bias"]          # filter not persisted
    assert m.dealias_filter.shape == (1, 1, 1, 5, 5) and abs(float(m.dealias_filter.sum()) - 1) < 1e-6
    assert m.num_patches == 4 * 2 * 2 and m.proj.stride == (1, 1, 1)
    with pytest.raises(ValueError, match="Height"):
        DealiasedPatchEmbed3D(4, 9, 8, patch_size=(1, 4, 4))
    net = StrataBackboneModel(depth=4, height=16, width=16, n_layers=1, patch_size_vert=1,
                              patch_size_horiz=4, in_chans=3, base_out_chans=3, embed_dim=64,
                              num_heads=1, use_dealiased_patch_embed=True)
    assert isinstance(net.strata.patch_embed, DealiasedPatchEmbed3D)
    assert not net.strata.patch_embed.proj.bias.any()
    assert [k for k in net.state_dict()][:2] == ["strata.patch_embed.proj.weight", "strata.patch_embed.proj.bias"]


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_gpu_module_matches_reference_golden(name):
    from strata_b200.strata import DealiasedPatchEmbed3D
    x, w, b, patch, filt, y = _case(name)
    B, C, D, H, W = x.shape
    m = DealiasedPatchEmbed3D(D, H, W, patch_size=patch, in_chans=C, embed_dim=w.shape[0],
                              resample_filter=filt).cuda()
    with torch.no_grad():
        m.proj.weight.copy_(w)
        m.proj.bias.copy_(b)
        got = m(x.cuda())
    assert got.shape == y.shape
    err = float((got.float().cpu() - y).abs().max() / y.abs().max())
    print(f"dealias {name}: max-abs relative error vs the reference's fp32 output {err:.4f}")
    assert err < 2e-2        # bf16 operands, fp32 accumulation


@pytest.mark.gpu
def test_gpu_whole_model_with_dealiased_embed_matches_oracle():
    from strata_b200.wrappers import StrataBackboneModel
    from tests.util import rel_max_err, tile_latlon
    torch.manual_seed(0)
    net = StrataBackboneModel(depth=4, height=32, width=32, n_layers=2, patch_size_vert=1,
                              patch_size_horiz=4, in_chans=5, base_out_chans=5, embed_dim=128,
                              num_heads=2, attn_kernel=3, do_rope_2d_stereographic=True,
                              index_is_latlon=True, do_bf16_mixed=True, do_rotate_wind=True,
                              wind_channel_indices=(0, 1), use_dealiased_patch_embed=True).cuda().eval()
    B, H, W = 2, 32, 32
    x = torch.randn(B, 5, 4, H, W, generator=torch.Generator().manual_seed(0))
    lat, lon = tile_latlon(B, H, W)
    with torch.inference_mode():
        y = net(x.cuda(), {"lat": lat.cuda(), "lon": lon.cuda()})
    state = {k: v.detach().cpu() for k, v in net.state_dict().items()}
    ref = bo.backbone_forward(x, state, patch=(1, 4, 4), num_heads=2, kernel=3, num_layers=2, lat=lat,
                              lon=lon, wind_channels=(0, 1), dealias_filter=(1, 4, 6, 4, 1))
    assert rel_max_err(y, ref) < 2e-2
    plain = bo.backbone_forward(x, state, patch=(1, 4, 4), num_heads=2, kernel=3, num_layers=2,
                                lat=lat, lon=lon, wind_channels=(0, 1))
    assert rel_max_err(y, plain) > 5e-2          # the filter is really applied
