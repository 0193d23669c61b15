"""Generates tests/golden/tile_halo_plan.npz (plan-based tile halo) and
tests/golden/knn_allgather_halo.npz (all-gather KNN halo and its normalised adjoint) from the
reference's own code.

    python tests/golden/make_plan_golden.py /path/to/reference

screamcast/distributed_cubesphere_transforms.py needs earth2grid (KNNS2Interpolator, Regridder),
which is not available. Both are replaced here by small stand-ins that follow the interface the
reference uses (constructor (src_lon, src_lat, dst_lon, dst_lat, k, eps), state_dict with
"index" / "weight", Regridder.from_state_dict, forward(x[..., n_src]) -> [..., n_dst]) and
compute inverse-distance weights 1 / (chord distance + eps), normalised, over the k nearest
source points. Everything else - halo cell extraction, assignment of halo cells to source
faces and tiles, grouping into send entries, send / receive sizes, and the module's forward
(interior fill, per-entry interpolation, scatter) at world_size 1 - is the reference's code.
The second file runs screamcast/distributed_halo.py's DistributedTileKNNHaloPadding_AllGather
(source / destination point selection, all-gather, regrid) and NormalizedHaloAdjoint (vjp of the
regrid, window, normalisation) at world_size 1 with the same stand-in interpolator.
The tests never import the reference.
"""
import sys
import types
from pathlib import Path

import numpy as np
import torch
from scipy.spatial import cKDTree

OUT = Path(__file__).resolve().parent
NE, NPG, TILE, HALO = 4, 2, 4, 2


class _Regridder(torch.nn.Module):
    def __init__(self, index, weight):
        super().__init__()
        self.register_buffer("index", index)
        self.register_buffer("weight", weight)

    @classmethod
    def from_state_dict(cls, sd):
        return cls(sd["index"], sd["weight"])

    def forward(self, x):
        acc = torch.zeros(*x.shape[:-1], self.index.shape[0], dtype=x.dtype)
        for j in range(self.index.shape[1]):
            acc = acc + self.weight[:, j].to(x.dtype) * x[..., self.index[:, j]]
        return acc


def _unit(lon, lat):
    lo, la = np.radians(np.asarray(lon, np.float64)), np.radians(np.asarray(lat, np.float64))
    return np.stack([np.cos(la) * np.cos(lo), np.cos(la) * np.sin(lo), np.sin(la)], axis=-1)


class _KNN(_Regridder):
    def __init__(self, src_lon, src_lat, dst_lon, dst_lat, k=4, eps=1e-7):
        dist, idx = cKDTree(_unit(src_lon.numpy(), src_lat.numpy())).query(
            _unit(dst_lon.numpy(), dst_lat.numpy()), k=k)
        if k == 1:
            dist, idx = dist[:, None], idx[:, None]
        lam = 1.0 / (dist + eps)
        w = (lam / lam.sum(axis=1, keepdims=True)).astype(np.float32)
        super().__init__(torch.from_numpy(idx.astype(np.int64)), torch.from_numpy(w))


def _stub(name, **attrs):
    m = types.ModuleType(name)
    for key, v in attrs.items():
        setattr(m, key, v)
    sys.modules[name] = m
    return m


def equiangular_faces(N):
    """lon / lat (degrees) of an equiangular gnomonic cubed sphere, [6, N, N] face rasters."""
    a = (np.arange(N) + 0.5) / N * (np.pi / 2) - np.pi / 4
    x, y = np.meshgrid(np.tan(a), np.tan(a), indexing="ij")
    one = np.ones_like(x)
    faces = [(one, x, y), (-x, one, y), (-one, -x, y), (x, -one, y), (-y, x, one), (y, x, -one)]
    lon, lat = [], []
    for X, Y, Z in faces:
        r = np.sqrt(X * X + Y * Y + Z * Z)
        lon.append(np.degrees(np.arctan2(Y, X)) % 360.0)
        lat.append(np.degrees(np.arcsin(Z / r)))
    return np.stack(lon).astype(np.float32), np.stack(lat).astype(np.float32)


def main(ref_root):
    sys.path.insert(0, ref_root)
    e2g = _stub("earth2grid", KNNS2Interpolator=_KNN)
    e2g.healpix = _stub("earth2grid.healpix")
    _stub("earth2grid._regrid", Regridder=_Regridder)
    import screamcast.cubesphere_transforms as ct
    import screamcast.distributed_cubesphere_transforms as dct

    N = NE * NPG
    lon_f, lat_f = equiangular_faces(N)
    grid = {"lon": ct.faces_to_unstructured(torch.from_numpy(lon_f), ne=NE, npg=NPG).numpy(),
            "lat": ct.faces_to_unstructured(torch.from_numpy(lat_f), ne=NE, npg=NPG).numpy()}
    out = {"ne": np.int64(NE), "npg": np.int64(NPG), "tile": np.int64(TILE), "halo": np.int64(HALO),
           "lon_faces": lon_f, "lat_faces": lat_f, "grid_lon": grid["lon"], "grid_lat": grid["lat"]}
    tpd = N // TILE
    for ws in (1, 2, 6):
        plan = dct.build_distributed_tile_halo_plan(grid, NE, TILE, HALO, num_pg_cells=NPG, world_size=ws)
        rows = []       # one row per halo cell: dst tile, position, src tile, src rank, index[k], weight[k]
        for sr, by_dst in plan.send_plans.items():
            for dst_tile, entries in by_dst.items():
                d = dct._tile_tuple_to_id(*dst_tile, tpd)
                for e in entries:
                    s = dct._tile_tuple_to_id(*e.src_tile, tpd)
                    idx = e.regridder_state_dict["index"].numpy()
                    w = e.regridder_state_dict["weight"].numpy()
                    for n, ppos in enumerate(e.dst_halo_positions.numpy()):
                        rows.append((d, int(ppos), s, sr, *idx[n].tolist(), *w[n].tolist()))
        rows.sort(key=lambda r: (r[0], r[1]))
        arr = np.array(rows, dtype=np.float64)
        out[f"ws{ws}_cells"] = arr[:, :4].astype(np.int64)
        out[f"ws{ws}_index"] = arr[:, 4:8].astype(np.int64)
        out[f"ws{ws}_weight"] = arr[:, 8:12].astype(np.float32)
        out[f"ws{ws}_send_sizes"] = np.array([[plan.send_sizes[a][b] for b in range(ws)] for a in range(ws)])
        out[f"ws{ws}_recv_sizes"] = np.array([[plan.recv_sizes[a][b] for b in range(ws)] for a in range(ws)])
        out[f"ws{ws}_tile_to_rank"] = np.array([plan.tile_to_rank[dct._tile_id_to_tuple(t, tpd)]
                                               for t in range(6 * tpd * tpd)])
        if ws == 1:
            g = torch.Generator().manual_seed(11)
            x = torch.randn(2, 3, 6 * tpd * tpd, TILE, TILE, generator=g)
            mod = dct.DistributedTileKNNHaloPadding(plan, rank=0)
            out["ws1_forward_in"] = x.numpy()
            out["ws1_forward_out"] = mod(x).numpy()
    # the padded target grid path ("duo padding"): a wider padded grid in element order
    from_tgt = 3
    ne_t = (N + 2 * from_tgt * NPG) // NPG
    Nt = ne_t * NPG
    a = (np.arange(Nt) + 0.5 - from_tgt * NPG) / N * (np.pi / 2) - np.pi / 4
    x_, y_ = np.meshgrid(np.tan(a), np.tan(a), indexing="ij")
    one = np.ones_like(x_)
    faces = [(one, x_, y_), (-x_, one, y_), (-one, -x_, y_), (x_, -one, y_), (-y_, x_, one), (y_, x_, -one)]
    lon_t = np.stack([np.degrees(np.arctan2(Y, X)) % 360.0 for X, Y, Z in faces]).astype(np.float32)
    lat_t = np.stack([np.degrees(np.arcsin(Z / np.sqrt(X * X + Y * Y + Z * Z))) for X, Y, Z in faces]).astype(np.float32)
    tgt = {"lon": ct.faces_to_unstructured(torch.from_numpy(lon_t), ne=ne_t, npg=NPG).numpy(),
           "lat": ct.faces_to_unstructured(torch.from_numpy(lat_t), ne=ne_t, npg=NPG).numpy()}
    plan = dct.build_distributed_tile_halo_plan(grid, NE, TILE, HALO, num_pg_cells=NPG, world_size=1, grid_tgt=tgt)
    rows = []
    for sr, by_dst in plan.send_plans.items():
        for dst_tile, entries in by_dst.items():
            d = dct._tile_tuple_to_id(*dst_tile, tpd)
            for e in entries:
                s = dct._tile_tuple_to_id(*e.src_tile, tpd)
                for ppos in e.dst_halo_positions.numpy():
                    rows.append((d, int(ppos), s))
    rows.sort()
    out["tgt_lon"], out["tgt_lat"] = tgt["lon"], tgt["lat"]
    out["tgt_cells"] = np.array(rows, dtype=np.int64)
    np.savez_compressed(OUT / "tile_halo_plan.npz", **out)
    print("wrote", OUT / "tile_halo_plan.npz", {k: v.shape for k, v in out.items() if hasattr(v, "shape")})

    # ---- all-gather KNN halo + normalised adjoint (screamcast/distributed_halo.py:208-448)
    import os
    import torch.distributed as dist
    import screamcast.distributed_halo as dh
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT="29655")
    dist.init_process_group("gloo", rank=0, world_size=1)
    pw, T, h = from_tgt * NPG, TILE, HALO       # the padded faces built above: N + 2*pw per side
    topo = dh.TileTopology(world_size=1, rank=0, face_size=N, tile_size=T, halo_width=h)
    mod = dh.DistributedTileKNNHaloPadding_AllGather.from_padded_face_grid(
        topology=topo, lon=torch.from_numpy(lon_t), lat=torch.from_numpy(lat_t), pad_width_data=pw,
        device=torch.device("cpu"))
    g = torch.Generator().manual_seed(12)
    x = torch.randn(2, 3, topo.tiles_per_rank, T, T, generator=g)
    y = mod(x)
    P = T + 2 * h
    win1 = torch.sin((torch.arange(P) + 0.5) / P * np.pi) ** 2
    window = (win1[:, None] * win1[None, :]).float()
    yp = torch.randn(2, topo.tiles_per_rank, P, P, generator=g)
    adj = dh.NormalizedHaloAdjoint(mod)(yp)
    adj_w = dh.NormalizedHaloAdjoint(mod, window=window)(yp)
    knn = {"face_size": np.int64(N), "tile": np.int64(T), "halo": np.int64(h), "pad_width_data": np.int64(pw),
           "lon_padded": lon_t, "lat_padded": lat_t, "x": x.numpy(), "forward": y.numpy(),
           "index": mod.regrid.index.numpy(), "weight": mod.regrid.weight.numpy(),
           "lat_deg": mod.lat_deg.numpy(), "lon_deg": mod.lon_deg.numpy(),
           "padded_in": yp.numpy(), "window": window.numpy(), "adjoint": adj.numpy(),
           "adjoint_windowed": adj_w.numpy()}
    dist.destroy_process_group()
    np.savez_compressed(OUT / "knn_allgather_halo.npz", **knn)
    print("wrote", OUT / "knn_allgather_halo.npz", {k: v.shape for k, v in knn.items() if hasattr(v, "shape")})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_plan_golden.py /path/to/reference")
    main(sys.argv[1])
