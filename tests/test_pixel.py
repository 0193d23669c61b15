"""CPU checks of the pixel stage: the two-stage module tree against the reference's parameter
manifest (tests/golden/two_stage_param_names.txt, copied from the reference's
tests/regression_data/pixeldit_*.param_order.txt by tests/golden/make_golden.py), and the
oracle's conventions (adaLN-zero identity; the bilinear + depthwise-conv index arithmetic that
the CUDA kernel uses, restated with explicit loops, against torch's interpolate + conv2d)."""
import math
from pathlib import Path

import pytest
import torch

from oracle import block_oracle as bo
from oracle import pixel_oracle as po

GOLDEN = Path(__file__).parent / "golden"


def _two_stage(**over):
    from strata_b200.wrappers import StrataModel
    kw = dict(depth=4, height=32, width=32, n_layers=24, patch_size_vert=1, patch_size_horiz=4,
              in_chans=5, base_out_chans=5, embed_dim=128, num_heads=2, attn_kernel=3,
              do_rope_2d_stereographic=True, index_is_latlon=True, gated_attention=True,
              qk_norm=True, embed_dim_pixel=128, n_layers_pixel=4, attn_kernel_pixel=9,
              qk_norm_pixel=True, use_bilinear_dw_gelu_project_adaln_pixel=True)
    kw.update(over)
    return StrataModel(**kw)


def test_parameter_names_and_order_match_the_reference_manifest():
    want = (GOLDEN / "two_stage_param_names.txt").read_text().split()
    got = [n for n, _ in _two_stage().named_parameters()]
    assert got == want


def test_structure_contract():
    # reference: tests/test_dit_3d_pixel.py:108-145, 229-279, 375-393
    from strata_b200.pixel import StrataPixel3DBlock
    from strata_b200.strata import Mlp
    m = _two_stage(n_layers=2, n_layers_pixel=3, first_block_only_adaln_pixel=True)
    blocks = m.strata.pixel_blocks
    assert isinstance(blocks[0], StrataPixel3DBlock) and blocks[0].has_adaln
    for b in blocks[1:]:
        assert not hasattr(b, "adaln_bilinear_dw_proj") and not hasattr(b, "adaln_pixel_proj")
    assert m.strata.adaln_mode == "bilinear_dw" and m.strata.rope_mode_pixel == "none"
    assert m.strata.backbone.rope_mode == "stereographic"
    assert all(hasattr(b.attn, "gate_proj") for b in m.strata.backbone.blocks)
    acts = [mod.layers[1] for mod in m.modules() if isinstance(mod, Mlp)]
    assert len(acts) == 5 and all(a.approximate == "tanh" for a in acts)
    assert m.strata.backbone.rope_length_scale == math.sqrt(math.pi * 16 / (3.0 * 1024 ** 2))
    # adaLN-zero initialisation
    assert not blocks[0].adaln_bilinear_dw_proj.weight.any()
    assert not blocks[0].adaln_bilinear_dw_proj.bias.any()
    # default AdaLN mode: one projection per block, Sequential ending in the zero-initialised Linear
    d = _two_stage(n_layers=2, n_layers_pixel=2, use_bilinear_dw_gelu_project_adaln_pixel=False)
    assert d.strata.adaln_mode == "pixel_proj"
    last = d.strata.pixel_blocks[1].adaln_pixel_proj[-1]
    assert last.out_features == 16 * 6 * 128 and not last.weight.any() and not last.bias.any()
    assert not hasattr(d.strata.pixel_blocks[0], "adaln_bilinear_dw_proj")
    with pytest.raises(RuntimeError, match="CUDA"):
        m(torch.zeros(1, 5, 4, 32, 32), {"lat": torch.zeros(1, 32, 32), "lon": torch.zeros(1, 32, 32)})


def _tap(p, factor, n):
    s = max((p + 0.5) / factor - 0.5, 0.0)
    i0 = min(int(s), n - 1)
    i1 = min(i0 + 1, n - 1)
    return i0, i1, 1.0 - (s - i0), s - i0


@pytest.mark.parametrize("h,w,factor,ks", [(3, 4, 4, 5), (2, 3, 2, 3), (4, 2, 1, 5), (3, 3, 3, 5)])
def test_conditioning_index_arithmetic(h, w, factor, ks):
    g = torch.Generator().manual_seed(h * 10 + w)
    Cb = 3
    tok = torch.randn(1, 2, h, w, Cb, generator=g, dtype=torch.float64)
    wd = torch.randn(Cb, ks, ks, generator=g, dtype=torch.float64)
    bd = torch.randn(Cb, generator=g, dtype=torch.float64)
    H, W, r = h * factor, w * factor, ks // 2
    want = torch.zeros(1, 2, H, W, Cb, dtype=torch.float64)
    for d in range(2):
        for y in range(H):
            for x in range(W):
                acc = bd.clone()
                for dy in range(-r, r + 1):
                    for dx in range(-r, r + 1):
                        py, px = y + dy, x + dx
                        if not (0 <= py < H and 0 <= px < W):
                            continue
                        r0, r1, a0, a1 = _tap(py, factor, h)
                        c0, c1, b0, b1 = _tap(px, factor, w)
                        u = (a0 * (b0 * tok[0, d, r0, c0] + b1 * tok[0, d, r0, c1])
                             + a1 * (b0 * tok[0, d, r1, c0] + b1 * tok[0, d, r1, c1]))
                        acc = acc + wd[:, dy + r, dx + r] * u
                want[0, d, y, x] = torch.nn.functional.gelu(acc, approximate="tanh")
    got = po.adaln_cond(tok.float(), wd.float(), bd.float(), factor)
    assert torch.allclose(got, want.reshape(1, -1, Cb).float(), atol=2e-5, rtol=1e-5)


def test_oracle_block_is_identity_at_zero_modulation_and_plain_without():
    C, grid = 64, (2, 4, 4)
    p = bo.init_block_params(C, seed=1)
    x = torch.randn(1, 32, C, generator=torch.Generator().manual_seed(0))
    zero = torch.zeros(1, 32, 6 * C)
    assert torch.equal(po.pixel_block_forward(x, zero, p, grid=grid, num_heads=1, kernel=(1, 3, 3)), x)
    # a block without AdaLN parameters is the plain pre-norm block of the backbone
    plain = po.pixel_block_forward(x, None, p, grid=grid, num_heads=1, kernel=(1, 3, 3))
    ref = bo.block_forward(x, p, grid=grid, num_heads=1, kernel=(1, 3, 3), rope_cos=None, rope_sin=None)
    assert torch.allclose(plain, ref, atol=1e-5, rtol=1e-5)
