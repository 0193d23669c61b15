"""Generates the golden fixtures under tests/golden/ from the reference's own in-tree code.

Run once, in a container where the reference checkout is available, as

    python tests/golden/make_golden.py /path/to/reference

It imports the reference modules that run without third-party packages
(screamcast.cubesphere_transforms, screamcast.distributed_halo, screamcast.wind_rotation,
screamcast.tile_geometry static helpers) with `earth2grid` / `xarray` stubbed (they are only
needed by code paths not exercised here), feeds them seeded inputs and stores inputs'
recipes + outputs as small .npz files. The tests never import the reference.
"""
import sys
import types
from pathlib import Path

import numpy as np
import torch

OUT = Path(__file__).resolve().parent


def _stub(name, **attrs):
    m = types.ModuleType(name)
    for k, v in attrs.items():
        setattr(m, k, v)
    sys.modules[name] = m
    return m


def import_reference(ref_root: str):
    sys.path.insert(0, ref_root)

    class _KNN:  # placeholder for earth2grid.KNNS2Interpolator (not exercised)
        def __init__(self, *a, **k):
            raise RuntimeError("stub")

    e2g = _stub("earth2grid", KNNS2Interpolator=_KNN)
    e2g.healpix = _stub("earth2grid.healpix")
    _stub("earth2grid._regrid", Regridder=object)
    if "xarray" not in sys.modules:
        try:
            import xarray  # noqa: F401
        except Exception:
            _stub("xarray")
    import screamcast.cubesphere_transforms as ct
    import screamcast.distributed_halo as dh
    import screamcast.wind_rotation as wr
    import screamcast.tile_geometry as tg
    return ct, dh, wr, tg


def payload(n_lead, N, seed):
    """Integer-valued channel (face*1e6 + i*N + j) followed by seeded N(0,1) channels."""
    f, i, j = np.meshgrid(np.arange(6), np.arange(N), np.arange(N), indexing="ij")
    ident = (f * 1_000_000 + i * N + j).astype(np.float32)
    rng = np.random.default_rng(seed)
    rest = rng.standard_normal((n_lead - 1, 6, N, N)).astype(np.float32)
    return np.concatenate([ident[None], rest], axis=0)


def main(ref_root):
    ct, dh, wr, tg = import_reference(ref_root)

    # ---- face padding (copy + rot90 + diagonal-rule corners)
    pad_cases = {}
    for name, (N, p, seed) in {"n4p2": (4, 2, 1), "n8p3": (8, 3, 2), "n6p1": (6, 1, 3),
                               "n8p8": (8, 8, 4)}.items():
        x = payload(3, N, seed)
        y = ct.create_padded_faces_batched(torch.from_numpy(x), pad_width=p).numpy()
        pad_cases[f"{name}_N"] = np.int64(N)
        pad_cases[f"{name}_p"] = np.int64(p)
        pad_cases[f"{name}_seed"] = np.int64(seed)
        pad_cases[f"{name}_out"] = y
        pad_cases[f"{name}_halo_idx"] = ct.halo_dst_flat_indices(N, p)
    # element <-> raster reorder
    ne, npg = 3, 2
    u = np.arange(5 * 6 * ne * ne * npg * npg, dtype=np.float32).reshape(5, -1)
    faces = ct.unstructured_to_6faces(torch.from_numpy(u), ne=ne, npg=npg)
    pad_cases["reorder_in"] = u
    pad_cases["reorder_faces"] = faces.numpy()
    pad_cases["reorder_back"] = ct.faces_to_unstructured(faces, ne=ne, npg=npg).numpy()
    np.savez_compressed(OUT / "face_padding.npz", **pad_cases)

    # ---- tile topology
    topo = {}
    cases = [(4, 1, 8, 4, 2), (1, 0, 4, 2, 1), (8, 3, 8, 4, 2), (8, 7, 16, 4, 2), (2, 1, 8, 2, 1),
             (6, 4, 8, 8, 3)]
    topo["cases"] = np.array(cases, dtype=np.int64)
    for ci, (ws, rk, fs, ts, hw) in enumerate(cases):
        t = dh.TileTopology(world_size=ws, rank=rk, face_size=fs, tile_size=ts, halo_width=hw)
        topo[f"c{ci}_local_tiles"] = np.array(t.local_tiles, dtype=np.int64)
        topo[f"c{ci}_global_tiles"] = np.array(t.global_tiles, dtype=np.int64)
        topo[f"c{ci}_scalars"] = np.array([t.tiles_per_dim, t.total_tiles, t.tiles_per_rank,
                                           t.padded_tile_size], dtype=np.int64)
        x = payload(2, fs, 10 + ci)
        lt = t.faces_to_local_tiles(torch.from_numpy(x))
        topo[f"c{ci}_local_from_faces"] = lt.numpy()
        padded_faces = ct.create_padded_faces_batched(torch.from_numpy(x), pad_width=hw)
        sel = torch.stack([dh._select_padded_tile(padded_faces, tile, tile_size=ts, halo_width=hw,
                                                  pad_width_data=hw) for tile in t.local_tiles],
                          dim=-3)
        topo[f"c{ci}_padded_local_tiles"] = sel.numpy()
        topo[f"c{ci}_cropped"] = t.crop(sel).numpy()
    np.savez_compressed(OUT / "tile_topology.npz", **topo)

    # ---- wind rotation + tile centre + rope length scale
    g = torch.Generator().manual_seed(7)
    B, D, H, W = 2, 3, 6, 5
    U = torch.randn(B, D, H, W, generator=g)
    V = torch.randn(B, D, H, W, generator=g)
    lat = (torch.linspace(0.2, 0.7, H).view(1, H, 1) + torch.tensor([0.0, -0.9]).view(B, 1, 1)
           ).expand(B, H, W).contiguous()
    lon = (torch.linspace(0.1, 0.6, W).view(1, 1, W) + torch.tensor([0.0, 5.9]).view(B, 1, 1)
           ).expand(B, H, W).contiguous()
    lat0, lon0 = tg.TileGeometry.tile_center(lat, lon)
    Ul, Vl = wr.forward_uv_to_tile(U, V, lat, lon, lat0, lon0)
    Ur, Vr = wr.inverse_tile_to_uv(Ul, Vl, lat, lon, lat0, lon0)
    np.savez_compressed(
        OUT / "wind_rotation.npz", U=U.numpy(), V=V.numpy(), lat=lat.numpy(), lon=lon.numpy(),
        lat0=lat0.numpy(), lon0=lon0.numpy(), U_loc=Ul.numpy(), V_loc=Vl.numpy(), U_rec=Ur.numpy(),
        V_rec=Vr.numpy(),
        mean_lon_pm=tg.mean_longitude(lon, return_0_2pi=False).numpy(),
        rope_scale=np.array([tg.TileGeometry.default_rope_length_scale(s) for s in (1, 2, 4)]))
    # ---- de-aliased patch embedding (reference module run in fp32 on seeded inputs)
    import screamcast.dealias as dl
    cases = {}
    for name, (shape, patch, cin, cout, filt, seed) in {
            "p144": ((2, 3, 8, 12), (1, 4, 4), 3, 8, (1, 4, 6, 4, 1), 11),
            "p222": ((1, 4, 6, 4), (2, 2, 2), 2, 16, (1, 1), 12),
            "p133": ((1, 2, 6, 9), (1, 3, 3), 4, 8, (1, 2, 1), 13)}.items():
        torch.manual_seed(seed)
        B, D, H, W = shape
        mod = dl.DealiasedPatchEmbed3D(D, H, W, patch_size=patch, in_chans=cin, embed_dim=cout,
                                       resample_filter=filt)
        x = torch.randn(B, cin, D, H, W)
        with torch.no_grad():
            y = mod(x)
        cases[name + "_x"] = x.numpy()
        cases[name + "_w"] = mod.proj.weight.detach().numpy()
        cases[name + "_b"] = mod.proj.bias.detach().numpy()
        cases[name + "_y"] = y.numpy()
        cases[name + "_patch"] = np.array(patch)
        cases[name + "_filter"] = np.array(filt, dtype=np.float32)
    np.savez_compressed(OUT / "dealias_patch_embed.npz", **cases)

    # parameter names of the two-stage model, in order (names only; the manifest holds no values)
    manifest = next(Path(ref_root, "tests", "regression_data").glob("pixeldit_*param_order.txt"))
    names = [ln.strip() for ln in manifest.read_text().splitlines() if ln.strip()]
    (OUT / "two_stage_param_names.txt").write_text("\n".join(names) + "\n")
    # ---- legacy checkpoint key translation: the reference's remap run on legacy spellings of
    # the manifest's names (built here by the inverse renames), on wrapper-prefixed variants, on
    # keys it drops and on inputs it rejects
    import json
    import screamcast.checkpoint_compat as cc

    def legacy_of(n, two_stage):
        n = n[len("strata."):]
        n = n.replace(".attn.gate_proj.", ".attn.gated_attention_map.")
        n = n.replace(".mlp.layers.0.", ".mlp.fwd.0.").replace(".mlp.layers.2.", ".mlp.fwd.3.")
        for new, old in (("backbone.patch_embed.", "semantic._patch_emb."),
                         ("backbone.blocks.", "semantic._blocks."),
                         ("pixel_patch_embed.", "_pixel_patch_emb."), ("pixel_blocks.", "_pixel_blocks."),
                         ("pixel_final_layer.", "_pixel_final_layer."), ("patch_embed.", "_patch_emb."),
                         ("blocks.", "_blocks."), ("final_layer.", "_final_layer.")):
            if n.startswith(new):
                return old + n[len(new):]
        return n

    single = next(Path(ref_root, "tests", "regression_data").glob("sweep1_*param_order.txt"))
    single_names = [ln.strip() for ln in single.read_text().splitlines() if ln.strip()]
    inputs = {
        "two_stage": [legacy_of(n, True) for n in names],
        "single_stage": [legacy_of(n, False) for n in single_names],
        "compiled": ["_orig_mod." + legacy_of(n, True) for n in names[:40]],
        "ddp_over_compiled": ["module._orig_mod." + legacy_of(n, False) for n in single_names[:20]],
        "migrated_with_prefix": ["_orig_mod." + n for n in names[:30]],
        "migrated": list(names[:30]),
        "with_dropped": [legacy_of(n, True) for n in names[:12]]
                        + ["semantic._final_layer.linear.weight", "_concat_skip_linear.weight"],
        "mixed": [legacy_of(names[0], True), names[1]],
        "duplicate_after_strip": ["_orig_mod." + names[0], names[0]],
    }
    cases = []
    for cname, keys in inputs.items():
        sd = {k: torch.zeros(1) for k in keys}
        try:
            new_sd, rep = cc.remap_legacy_state_dict(sd)
            cases.append(dict(name=cname, input=keys, output=list(new_sd), was_legacy=rep.was_legacy,
                              dropped=rep.dropped, passthrough=rep.passthrough))
        except ValueError as exc:
            cases.append(dict(name=cname, input=keys, raises=str(exc)[:40]))
    (OUT / "checkpoint_remap.json").write_text(json.dumps(cases, indent=0))
    print("wrote", sorted(p.name for p in OUT.glob("*.npz")), "two_stage_param_names.txt",
          "checkpoint_remap.json")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference>")
    main(sys.argv[1])
