"""Legacy checkpoint keys -> the `strata.*` names of the wrapper classes (reference:
screamcast/checkpoint_compat.py:15-206 and the load pre-hook of
screamcast/strata_wrappers.py:110-131, registered at :193-199).

Checkpoints written before the reference moved to the physicsnemo module tree name the
backbone `semantic._blocks...` / `_blocks...`, the pixel stage `_pixel_blocks...`, the MLP
`mlp.fwd.{0,3}` and the attention gate `attn.gated_attention_map`; they may also carry the
prefixes torch.compile, DDP and lightning add. `remap_legacy_state_dict` rewrites such a state
dict (network weights only; parameter ORDER is unchanged, so index-based optimiser state still
lines up) and leaves an already-migrated one alone, so it can run on every load.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass, field

logger = logging.getLogger(__name__)

WRAPPER_PREFIXES = ("_orig_mod.", "module.", "_forward_module.")
# a state dict is legacy iff a (wrapper-stripped) key starts with one of these
LEGACY_HEADS = ("semantic.", "_pixel_patch_emb.", "_pixel_blocks.", "_pixel_final_layer.",
                "_patch_emb.", "_blocks.", "_final_layer.", "_concat_skip_linear.")
# head of the key -> new head; the first match wins (two-stage heads before the bare ones)
HEAD_RENAMES = (("semantic._patch_emb.", "backbone.patch_embed."),
                ("semantic._blocks.", "backbone.blocks."),
                ("semantic.", "backbone."),
                ("_pixel_patch_emb.", "pixel_patch_embed."),
                ("_pixel_blocks.", "pixel_blocks."),
                ("_pixel_final_layer.", "pixel_final_layer."),
                ("_patch_emb.", "patch_embed."),
                ("_blocks.", "blocks."),
                ("_final_layer.", "final_layer."))
# renames inside a module path, at any depth (legacy Mlp: Sequential(fc1, act, drop, fc2, drop))
INNER_RENAMES = ((".attn.gated_attention_map.", ".attn.gate_proj."),
                 (".mlp.fwd.0.", ".mlp.layers.0."),
                 (".mlp.fwd.3.", ".mlp.layers.2."))
# legacy keys without a home in the wrappers (unused concat-skip head; the two-stage model's
# backbone has no output head)
DROPPED_HEADS = ("_concat_skip_linear.", "semantic._final_layer.")


@dataclass
class RemapReport:
    was_legacy: bool = False
    renamed: dict = field(default_factory=dict)
    dropped: list = field(default_factory=list)
    passthrough: int = 0
    missing_in_target: list = field(default_factory=list)
    unexpected_in_target: list = field(default_factory=list)


def _strip_wrapper_prefixes(key: str) -> str:
    while key.startswith(WRAPPER_PREFIXES):
        for p in WRAPPER_PREFIXES:
            if key.startswith(p):
                key = key[len(p):]
    return key


def _new_name(key: str):
    """New name of one wrapper-stripped legacy key, or None when the key is dropped."""
    if key.startswith(DROPPED_HEADS):
        return None
    for old, new in HEAD_RENAMES:
        if key.startswith(old):
            key = new + key[len(old):]
            break
    for old, new in INNER_RENAMES:
        key = key.replace(old, new)
    return "strata." + key


def remap_legacy_state_dict(state_dict: dict, target_model=None):
    """-> (new_state_dict, RemapReport). Raises ValueError for keys that collide after the
    wrapper prefixes are stripped, for a mix of legacy and migrated keys, for a remap collision
    and - when `target_model` is given and no LoRA adapter keys are present - for a key set or
    a shape that does not match the model."""
    report = RemapReport()
    bare = {_strip_wrapper_prefixes(k): v for k, v in state_dict.items()}
    if len(bare) != len(state_dict):
        raise ValueError("Duplicate keys after stripping wrapper prefixes — refusing to remap")
    legacy = [k for k in bare if k.startswith(LEGACY_HEADS)]
    report.was_legacy = bool(legacy)
    if legacy and len(legacy) != len(bare):
        others = sorted(set(bare) - set(legacy))[:5]
        raise ValueError("State dict mixes legacy and non-legacy keys; cannot remap safely. "
                         f"Non-legacy examples: {others}")
    if not legacy:
        report.passthrough = len(bare)
        out = bare
    else:
        out = {}
        for key, value in bare.items():
            name = _new_name(key)
            if name is None:
                report.dropped.append(key)
                logger.warning("checkpoint remap: dropping legacy key %s", key)
            elif name in out:
                raise ValueError(f"Remap collision: {key} -> {name}")
            else:
                report.renamed[key] = name
                out[name] = value
        logger.info("checkpoint remap: translated %d legacy keys (%d dropped)",
                    len(report.renamed), len(report.dropped))
    if target_model is not None:
        want = target_model.state_dict()
        report.missing_in_target = sorted(set(out) - set(want))
        report.unexpected_in_target = sorted(set(want) - set(out))
        lora = any(".lora_A." in k or ".lora_B." in k for k in out)
        if not lora and (report.missing_in_target or report.unexpected_in_target):
            raise ValueError("Remapped state dict does not match the target model.\n"
                             f"  keys not in model (first 5): {report.missing_in_target[:5]}\n"
                             f"  model keys not in ckpt (first 5): {report.unexpected_in_target[:5]}")
        for k in out.keys() & want.keys():
            if out[k].shape != want[k].shape:
                raise ValueError(f"Shape mismatch for {k}: checkpoint {tuple(out[k].shape)} "
                                 f"vs model {tuple(want[k].shape)}")
    return out, report


def remap_legacy_pre_hook(module, state_dict, prefix, *args) -> None:
    """load_state_dict pre-hook of the wrapper classes: rewrites, in place, the keys under
    `prefix` (this wrapper's position in the outer module tree). Being a hook it also fires when
    the wrapper is loaded as a submodule of a compiled / DDP / fabric module."""
    mine = [k for k in state_dict if k.startswith(prefix)]
    if not mine:
        return
    bare = {k[len(prefix):]: state_dict[k] for k in mine}
    new, report = remap_legacy_state_dict(bare)
    if not report.was_legacy and new.keys() == bare.keys():
        return
    for k in mine:
        del state_dict[k]
    for k, v in new.items():
        state_dict[prefix + k] = v
