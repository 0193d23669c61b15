"""Legacy checkpoint key translation against outputs of the reference's own remap
(tests/golden/checkpoint_remap.json, made by tests/golden/make_golden.py from
screamcast/checkpoint_compat.py), and the load pre-hook on the wrapper classes (direct load,
load as a submodule, wrapper-prefixed checkpoints) as the reference tests it
(tests/test_checkpoint_compat.py)."""
import json
from pathlib import Path

import pytest
import torch
import torch.nn as nn

from strata_b200.checkpoint_compat import remap_legacy_state_dict

CASES = json.loads((Path(__file__).parent / "golden" / "checkpoint_remap.json").read_text())


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_remap_matches_reference(case):
    sd = {k: torch.zeros(1) for k in case["input"]}
    if "raises" in case:
        with pytest.raises(ValueError) as exc:
            remap_legacy_state_dict(sd)
        assert str(exc.value).startswith(case["raises"])
        return
    new, rep = remap_legacy_state_dict(sd)
    assert list(new) == case["output"]                      # names AND order
    assert rep.was_legacy == case["was_legacy"]
    assert rep.dropped == case["dropped"] and rep.passthrough == case["passthrough"]
    again, rep2 = remap_legacy_state_dict(new)              # idempotent
    assert list(again) == list(new) and not rep2.was_legacy


def _small(**over):
    from strata_b200.wrappers import StrataModel
    kw = dict(depth=2, height=8, width=8, n_layers=2, patch_size_vert=1, patch_size_horiz=4,
              in_chans=3, base_out_chans=3, embed_dim=64, num_heads=1, gated_attention=True,
              embed_dim_pixel=64, n_layers_pixel=1, use_bilinear_dw_gelu_project_adaln_pixel=True)
    kw.update(over)
    return StrataModel(**kw)


def _legacy(sd):
    out = {}
    for k, v in sd.items():
        k = k[len("strata."):]
        k = k.replace(".attn.gate_proj.", ".attn.gated_attention_map.")
        k = k.replace(".mlp.layers.0.", ".mlp.fwd.0.").replace(".mlp.layers.2.", ".mlp.fwd.3.")
        for new, old in (("backbone.patch_embed.", "semantic._patch_emb."),
                         ("backbone.blocks.", "semantic._blocks."),
                         ("pixel_patch_embed.", "_pixel_patch_emb."), ("pixel_blocks.", "_pixel_blocks."),
                         ("pixel_final_layer.", "_pixel_final_layer.")):
            if k.startswith(new):
                k = old + k[len(new):]
                break
        out[k] = v
    return out


def test_pre_hook_translates_on_every_load_path():
    torch.manual_seed(0)
    src = _small()
    with torch.no_grad():
        for p in src.parameters():
            p.normal_()
    want = {k: v.clone() for k, v in src.state_dict().items()}
    legacy = _legacy(want)
    assert all(not k.startswith("strata.") for k in legacy)
    # direct load, strict
    a = _small()
    a.load_state_dict(legacy, strict=True)
    assert all(torch.equal(a.state_dict()[k], want[k]) for k in want)
    # compiled-era checkpoint: every key prefixed
    b = _small()
    b.load_state_dict({"_orig_mod." + k: v for k, v in legacy.items()}, strict=True)
    assert all(torch.equal(b.state_dict()[k], want[k]) for k in want)
    # the wrapper as a submodule of the module being loaded
    outer = nn.Module()
    outer.net = _small()
    outer.load_state_dict({"net." + k: v for k, v in legacy.items()}, strict=True)
    assert all(torch.equal(outer.net.state_dict()[k], want[k]) for k in want)
    # migrated checkpoints pass through; coverage check against a target model
    c = _small()
    c.load_state_dict(want, strict=True)
    new, rep = remap_legacy_state_dict(legacy, target_model=c)
    assert rep.was_legacy and not rep.missing_in_target and not rep.unexpected_in_target
    bad = dict(legacy)
    bad.pop(next(iter(bad)))
    with pytest.raises(ValueError, match="does not match the target model"):
        remap_legacy_state_dict(bad, target_model=c)
    wrong = dict(legacy)
    k0 = next(iter(wrong))
    wrong[k0] = torch.zeros(3)
    with pytest.raises(ValueError, match="Shape mismatch"):
        remap_legacy_state_dict(wrong, target_model=c)
