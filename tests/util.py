"""Shared helpers of the GPU parity tests."""
import torch

from oracle import block_oracle as bo


def rel_max_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """max|got - want| / max|want| — the 'max-abs relative error' the tolerances are stated in."""
    return float((got.float().cpu() - want.float().cpu()).abs().max() / want.float().abs().max())


def rel_rms_err(got: torch.Tensor, want: torch.Tensor) -> float:
    d = got.float().cpu() - want.float().cpu()
    return float(d.pow(2).mean().sqrt() / want.float().pow(2).mean().sqrt())


def tile_latlon(n_tiles: int, H: int, W: int):
    """Smooth synthetic tiles: the lat/lon recipe of the reference's characterisation test
    (tests/test_characterization_inference.py:151-165) with a per-tile offset."""
    lat = torch.linspace(0.2, 0.7, H).view(1, H, 1) - 0.35 * torch.arange(n_tiles).view(-1, 1, 1)
    lon = torch.linspace(0.1, 0.6, W).view(1, 1, W) + 0.8 * torch.arange(n_tiles).view(-1, 1, 1)
    return lat.expand(n_tiles, H, W).contiguous(), lon.expand(n_tiles, H, W).contiguous()


def device_block_weights(p: dict, device):
    out = {}
    for short, name in (("qkv", "attn.qkv"), ("proj", "attn.proj"), ("gate", "attn.gate_proj"),
                        ("fc1", "mlp.layers.0"), ("fc2", "mlp.layers.2")):
        if f"{name}.weight" in p:
            out[f"w_{short}"] = p[f"{name}.weight"].to(device=device, dtype=torch.bfloat16).contiguous()
            out[f"b_{short}"] = p[f"{name}.bias"].to(device=device, dtype=torch.float32).contiguous()
    return out
