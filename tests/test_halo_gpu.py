"""GPU halo gather (world_size 1: every source is local) against the pinned oracle. Bit-exact:
halo exchange is index logic plus the corner mean in the storage type's arithmetic."""
import numpy as np
import pytest
import torch

from oracle import halo_oracle as ho
from tests.golden.make_golden import payload

pytestmark = pytest.mark.gpu


def _topos(fs, ts, hw):
    from strata_b200.topology import TileTopology
    return TileTopology(1, 0, fs, ts, hw), ho.TileTopology(1, 0, fs, ts, hw)


@pytest.mark.parametrize("fs,ts,hw,lead", [(8, 4, 2, (3,)), (16, 4, 3, (2, 5)), (8, 8, 8, (1,)),
                                           (12, 4, 1, ()), (8, 4, 0, (2,))])
def test_field_halo_bit_exact(fs, ts, hw, lead):
    from strata_b200.halo import DistributedTileCopyHaloPadding
    t, to = _topos(fs, ts, hw)
    n_lead = int(np.prod(lead)) if lead else 1
    x = payload(max(n_lead, 2), fs, 7)[:n_lead]                       # (L, 6, N, N)
    tiles = to.faces_to_local_tiles(x).reshape(*lead, t.tiles_per_rank, ts, ts)
    mod = DistributedTileCopyHaloPadding(topology=t)
    out = mod(torch.from_numpy(np.ascontiguousarray(tiles)).cuda())
    mod.check_status()
    want = ho.padded_local_tiles(tiles, to)
    assert out.shape == want.shape
    assert np.array_equal(out.cpu().numpy(), want)
    assert np.array_equal(t.crop(out).cpu().numpy(), tiles)           # crop(pad(x)) == x


def test_field_halo_golden_from_reference(golden_dir):
    from strata_b200.halo import DistributedTileCopyHaloPadding
    from strata_b200.topology import TileTopology
    g = np.load(golden_dir / "tile_topology.npz")
    for ci, (ws, rk, fs, ts, hw) in enumerate(g["cases"].tolist()):
        if ws != 1:
            continue
        t = TileTopology(ws, rk, fs, ts, hw)
        x = payload(2, fs, 10 + ci)
        tiles = t.faces_to_local_tiles(torch.from_numpy(x)).cuda()
        out = DistributedTileCopyHaloPadding(topology=t)(tiles)
        assert np.array_equal(out.cpu().numpy(), g[f"c{ci}_padded_local_tiles"])


def test_token_halo_bit_exact_bf16():
    from strata_b200.halo import DistributedTileCopyHaloPadding
    fs, ts, hw, D, C = 8, 4, 2, 3, 64
    t, to = _topos(fs, ts, hw)
    g = torch.Generator().manual_seed(3)
    tok = torch.randn(t.tiles_per_rank, D, ts * ts, C, generator=g).bfloat16()
    mod = DistributedTileCopyHaloPadding(topology=t)
    out = mod.pad_tokens(tok.cuda(), D)
    mod.check_status()
    # oracle in bf16 arithmetic: channels/depth become leading dims of the (tile, i, j) layout
    lead = tok.permute(1, 3, 0, 2).reshape(D, C, t.tiles_per_rank, ts, ts)
    want = torch.from_numpy(ho.padded_local_tiles(lead.float().numpy(), to))
    # the corner mean must round like bf16 arithmetic: (a + b) rounded, then halved
    a, b = mod.src_a.cpu().numpy(), mod.src_b.cpu().numpy()
    flat = lead.reshape(D, C, -1)
    va = flat[..., torch.from_numpy(a.astype(np.int64))]
    vb = flat[..., torch.from_numpy(np.where(b < 0, 0, b).astype(np.int64))]
    want_bf16 = torch.where(torch.from_numpy(b < 0), va, (va + vb) / 2)        # bf16 tensor math
    P = t.padded_tile_size
    got = out.cpu().reshape(t.tiles_per_rank, D, P, P, C).permute(1, 4, 0, 2, 3)
    assert torch.equal(got, want_bf16)
    assert (got.float() - want).abs().max() <= 2 ** -7 * want.abs().max()     # and close to fp32


def test_token_halo_only_halo_keeps_interior():
    from strata_b200.halo import DistributedTileCopyHaloPadding
    fs, ts, hw, D, C = 8, 4, 2, 2, 32
    t, _ = _topos(fs, ts, hw)
    P = t.padded_tile_size
    tok = torch.randn(t.tiles_per_rank, D, ts * ts, C, generator=torch.Generator().manual_seed(1)).bfloat16().cuda()
    mod = DistributedTileCopyHaloPadding(topology=t)
    full = mod.pad_tokens(tok, D)
    out = torch.full_like(full, 7.0)
    mod.pad_tokens(tok, D, out=out, only_halo=True)
    o5 = out.view(t.tiles_per_rank, D, P, P, C)
    f5 = full.view(t.tiles_per_rank, D, P, P, C)
    assert (o5[:, :, hw:-hw, hw:-hw] == 7.0).all()
    o5[:, :, hw:-hw, hw:-hw] = f5[:, :, hw:-hw, hw:-hw]
    assert torch.equal(o5, f5)


def test_shape_validation():
    from strata_b200.halo import DistributedTileCopyHaloPadding
    t, _ = _topos(8, 4, 2)
    mod = DistributedTileCopyHaloPadding(topology=t)
    with pytest.raises(ValueError, match="local tiles"):
        mod(torch.zeros(1, 5, 4, 4, device="cuda"))
    with pytest.raises(ValueError, match="interior tile shape"):
        mod(torch.zeros(1, 24, 5, 4, device="cuda"))



def test_halo_modules_under_inference_mode_with_channel_chunks():
    """The rollout loop pads, runs the network and un-pads under torch.inference_mode(), the halo
    modules wrapped in channel chunks (scripts/ace/run_screamcast_nudged.py:452-477, 612-639)."""
    from strata_b200.halo import (DistributedTileCopyHaloPadding, NormalizedCopyHaloAdjoint,
                                  channel_chunked, kbd_window)
    fs, ts, hw = 16, 8, 2
    t, to = _topos(fs, ts, hw)
    x = torch.randn(2, 7, t.tiles_per_rank, ts, ts, generator=torch.Generator().manual_seed(5)).cuda()
    mod = DistributedTileCopyHaloPadding(topology=t)
    unpad = NormalizedCopyHaloAdjoint(mod, window=kbd_window(t.padded_tile_size))
    want_pad = mod(x)
    want_unpad = unpad(want_pad)
    with torch.inference_mode():
        got_pad = channel_chunked(3)(mod)(x)
        got_unpad = channel_chunked(3)(unpad)(got_pad)
        sliced = channel_chunked(mod, 2)(x[:, 1:6])            # a non-contiguous channel slice
    mod.check_status()
    assert torch.equal(got_pad, want_pad) and torch.equal(got_unpad, want_unpad)
    assert torch.equal(sliced, want_pad[:, 1:6])
    assert np.array_equal(want_pad.cpu().numpy(), ho.padded_local_tiles(x.cpu().numpy(), to))


@pytest.mark.parametrize("window", ["ones", "kbd"])
def test_halo_adjoint_bit_exact(window):
    from strata_b200.halo import DistributedTileCopyHaloPadding, NormalizedCopyHaloAdjoint, kbd_window
    from strata_b200.topology import TileTopology
    fs, ts, hw = 16, 8, 3
    topo = TileTopology(1, 0, fs, ts, hw)
    otopo = ho.TileTopology(1, 0, fs, ts, hw)
    P = topo.padded_tile_size
    win = None if window == "ones" else kbd_window(P)
    pad_mod = DistributedTileCopyHaloPadding(topology=topo)
    unpad = NormalizedCopyHaloAdjoint(pad_mod, window=win)
    g = torch.Generator().manual_seed(11)
    y = torch.randn(2, 3, topo.tiles_per_rank, P, P, generator=g)
    got = unpad(y.cuda())
    pad_mod.check_status()
    want = ho.halo_adjoint(y.numpy(), otopo, None if win is None else win.numpy())
    assert np.array_equal(got.cpu().numpy(), want)
    # constant round trip through the real exchange (reference: tests/distributed/
    # test_distributed_halo.py:105) and crop(pad(x)) == x for the uniform window on
    # consistent tiles away from the corner means
    c = torch.full((1, topo.tiles_per_rank, ts, ts), 1.75, device="cuda")
    assert torch.allclose(unpad(pad_mod(c)), c, rtol=1e-6, atol=0)
    with pytest.raises(ValueError):
        unpad(torch.zeros(1, topo.tiles_per_rank, P, P - 1, device="cuda"))


def test_knn_halo_bit_exact_against_host_evaluation():
    from strata_b200.halo import DistributedTileKNNHaloPadding
    from strata_b200.rollout import padded_face_latlon
    from strata_b200.topology import TileTopology
    from tests.test_halo_knn import _apply
    N, T, H, PW = 16, 4, 2, 4
    lat, lon = padded_face_latlon(N, PW)
    topo = TileTopology(1, 0, N, T, H)
    mod = DistributedTileKNNHaloPadding.from_padded_face_grid(
        topology=topo, lon=torch.from_numpy(lon).float(), lat=torch.from_numpy(lat).float(),
        pad_width_data=PW, device="cuda")
    assert mod.lat_deg.shape == (topo.tiles_per_rank, T + 2 * H, T + 2 * H)
    g = torch.Generator().manual_seed(21)
    x = torch.randn(3, 2, topo.tiles_per_rank, T, T, generator=g)
    got = mod(x.cuda())
    mod.check_status()
    want = _apply(x.numpy(), mod.knn_idx.cpu().numpy(), mod.knn_weights.cpu().numpy())
    assert np.array_equal(got.cpu().numpy().reshape(want.shape), want)
    # interiors preserved to the reference's tolerance, topology.crop inverts the padding
    assert torch.allclose(topo.crop(got).cpu(), x, atol=1e-3, rtol=1e-3)
    with pytest.raises(TypeError):
        mod(x.cuda().double())

def test_knn_halo_and_adjoint_equal_the_reference_modules(golden_dir):
    # the reference's DistributedTileKNNHaloPadding_AllGather / NormalizedHaloAdjoint outputs at
    # world_size 1 (tests/golden/make_plan_golden.py: the reference's modules, earth2grid's
    # interpolator replaced by a stand-in of the same interface)
    from strata_b200.halo import DistributedTileKNNHaloPadding, NormalizedHaloAdjoint
    from strata_b200.topology import TileTopology
    gold = np.load(golden_dir / "knn_allgather_halo.npz")
    n, t, h, pw = (int(gold[k]) for k in ("face_size", "tile", "halo", "pad_width_data"))
    topo = TileTopology(1, 0, n, t, h)
    mod = DistributedTileKNNHaloPadding.from_padded_face_grid(
        topology=topo, lon=torch.from_numpy(gold["lon_padded"]), lat=torch.from_numpy(gold["lat_padded"]),
        pad_width_data=pw, device="cuda")
    assert torch.equal(mod.lat_deg.cpu(), torch.from_numpy(gold["lat_deg"]))
    assert torch.equal(mod.lon_deg.cpu(), torch.from_numpy(gold["lon_deg"]))
    got = mod(torch.from_numpy(gold["x"]).cuda())
    assert np.allclose(got.cpu().numpy(), gold["forward"], rtol=0, atol=1e-6)
    yp = torch.from_numpy(gold["padded_in"]).cuda()
    for key, window in (("adjoint", None), ("adjoint_windowed", torch.from_numpy(gold["window"]))):
        want = gold[key].reshape(yp.shape[:-2] + (t, t))
        out = NormalizedHaloAdjoint(mod, window=window)(yp)
        assert np.allclose(out.cpu().numpy(), want, rtol=1e-5, atol=1e-5)
    mod.check_status()


def test_plan_halo_equals_the_reference_module(golden_dir):
    # plan-based tile halo (reference DistributedTileKNNHaloPadding(plan, rank, group)): the
    # reference module's own output at world_size 1 (tests/golden/make_plan_golden.py)
    from strata_b200.halo import DistributedTilePlanHaloPadding, NormalizedHaloAdjoint
    from strata_b200.topology import build_distributed_tile_halo_plan
    from tests.test_halo_knn import _apply
    gold = np.load(golden_dir / "tile_halo_plan.npz")
    T, h = int(gold["tile"]), int(gold["halo"])
    plan = build_distributed_tile_halo_plan({"lon": gold["grid_lon"], "lat": gold["grid_lat"]}, int(gold["ne"]),
                                            T, h, num_pg_cells=int(gold["npg"]), world_size=1)
    mod = DistributedTilePlanHaloPadding(plan, rank=0)
    assert (mod.tile_size, mod.halo_width, mod.padded_size, mod.tiles_per_rank) == (T, h, T + 2 * h, 24)
    x = torch.from_numpy(gold["ws1_forward_in"])
    got = mod(x.cuda())
    mod.check_status()
    assert got.shape == gold["ws1_forward_out"].shape
    assert not torch.isnan(got).any()
    assert torch.equal(got[..., h:-h, h:-h].cpu(), x)                      # interiors copied exactly
    assert np.allclose(got.cpu().numpy(), gold["ws1_forward_out"], rtol=0, atol=1e-6)
    want = _apply(x.numpy(), mod.knn_idx.cpu().numpy(), mod.knn_weights.cpu().numpy())
    assert np.array_equal(got.cpu().numpy().reshape(want.shape), want)
    # one leading dimension, none, and a halo of width zero (tiles come back unchanged)
    assert torch.equal(mod(x[0].cuda()), got[0]) and torch.equal(mod(x[1, 2].cuda()), got[1, 2])
    plan0 = build_distributed_tile_halo_plan({"lon": gold["grid_lon"], "lat": gold["grid_lat"]}, int(gold["ne"]),
                                             T, 0, num_pg_cells=int(gold["npg"]), world_size=1)
    assert torch.equal(DistributedTilePlanHaloPadding(plan0, rank=0)(x.cuda()).cpu(), x)
    # its normalised adjoint un-pads constant fields to themselves
    unpad = NormalizedHaloAdjoint(mod)
    c = torch.full((1, 24, T, T), 2.5, device="cuda")
    assert torch.allclose(unpad(mod(c)), c, rtol=1e-5, atol=0)
    with pytest.raises(TypeError):
        DistributedTilePlanHaloPadding.from_padded_face_grid(topology=None)


def test_knn_halo_adjoint_matches_oracle():
    # the reference's un-pad operator proper: D_w^-1 A^T (w . y) with A the KNN regrid
    # (NormalizedHaloAdjoint, screamcast/distributed_halo.py:330-448)
    from strata_b200.halo import (DistributedTileKNNHaloPadding, NormalizedCopyHaloAdjoint,
                                  NormalizedHaloAdjoint, kbd_window)
    from strata_b200.rollout import padded_face_latlon
    from strata_b200.topology import TileTopology
    N, T, H, PW = 16, 4, 2, 4
    lat, lon = padded_face_latlon(N, PW)
    topo = TileTopology(1, 0, N, T, H)
    P = topo.padded_tile_size
    mod = DistributedTileKNNHaloPadding.from_padded_face_grid(
        topology=topo, lon=torch.from_numpy(lon).float(), lat=torch.from_numpy(lat).float(),
        pad_width_data=PW, device="cuda")
    with pytest.raises(TypeError, match="NormalizedHaloAdjoint"):
        NormalizedCopyHaloAdjoint(mod)                      # the copy transpose refuses a KNN module
    for win in (None, kbd_window(P)):
        unpad = NormalizedHaloAdjoint(mod, window=win)
        g = torch.Generator().manual_seed(31)
        y = torch.randn(2, 3, topo.tiles_per_rank, P, P, generator=g)
        got = unpad(y.cuda())
        mod.check_status()
        want = ho.knn_halo_adjoint(y.numpy(), ho.TileTopology(1, 0, N, T, H),
                                   mod.knn_idx.cpu().numpy(), mod.knn_weights.cpu().numpy(),
                                   None if win is None else win.numpy())
        assert np.allclose(got.cpu().numpy(), want, rtol=2e-5, atol=2e-6)
        # constant fields survive pad -> un-pad to the reference's tolerance
        # (tests/distributed/test_distributed_halo.py:61-107)
        c = torch.full((1, topo.tiles_per_rank, T, T), 1.75, device="cuda")
        assert torch.allclose(unpad(mod(c)), c, rtol=1e-3, atol=0)
    # on a copy-halo module the class is the copy transpose
    from strata_b200.halo import DistributedTileCopyHaloPadding
    cp = DistributedTileCopyHaloPadding(topology=topo)
    y = torch.randn(1, topo.tiles_per_rank, P, P, generator=torch.Generator().manual_seed(3)).cuda()
    assert torch.equal(NormalizedHaloAdjoint(cp)(y), NormalizedCopyHaloAdjoint(cp)(y))


def test_failed_barrier_poisons_the_padded_tiles():
    # failure made on the host side of the protocol (a partner flag nobody sets, a 20 ms limit):
    # the gathers that follow on the stream must not hand back plausible numbers
    import ctypes
    from strata_b200 import _lib
    from strata_b200.halo import DistributedTileCopyHaloPadding, NormalizedCopyHaloAdjoint
    from strata_b200.topology import TileTopology
    lib = _lib.load()
    topo = TileTopology(1, 0, 8, 4, 2)
    mod = DistributedTileCopyHaloPadding(topology=topo)
    unpad = NormalizedCopyHaloAdjoint(mod)
    x = torch.ones(2, topo.tiles_per_rank, 4, 4, device="cuda")
    assert torch.isfinite(mod(x)).all()
    flags = torch.zeros(2, 64, dtype=torch.int32, device="cuda")
    ptrs = (ctypes.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.strata_halo_barrier(ptrs, 0, 2, 1, 20, stream), "strata_halo_barrier")
    padded = mod(x)                                 # issued behind the failed barrier
    assert torch.isnan(padded).all()
    assert torch.isnan(unpad(torch.ones(2, topo.tiles_per_rank, 8, 8, device="cuda"))).all()
    tok = torch.ones(topo.tiles_per_rank, 2, 16, 8, dtype=torch.bfloat16, device="cuda")
    assert torch.isnan(mod.pad_tokens(tok, 2).float()).all()
    with pytest.raises(RuntimeError, match="status 105"):
        mod.check_status()                          # reports and clears
    assert torch.equal(mod(x)[..., 2:-2, 2:-2], x)  # the next exchange is clean again
    assert _lib.device_status() == 0
    # exchanges of one module stay on one stream
    with torch.cuda.stream(torch.cuda.Stream()):
        if topo.world_size > 1:
            with pytest.raises(RuntimeError, match="same CUDA stream"):
                mod(x)


def _two_gpus():
    return torch.cuda.is_available() and torch.cuda.device_count() >= 2


@pytest.mark.skipif(not _two_gpus(), reason="needs 2 GPUs on one node")
def test_two_rank_peer_halo():
    import subprocess, sys
    from pathlib import Path
    worker = Path(__file__).resolve().parent / "halo_worker.py"
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                        "--nproc-per-node", "2", "--master-addr", "127.0.0.1", "--master-port",
                        "29531", str(worker)], capture_output=True, text=True, timeout=600,
                       env={**__import__("os").environ, "NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "HALO WORKER OK" in r.stdout


def test_barrier_wait_runs_out_and_reports():
    # failure detection without a fault: a two-rank barrier whose partner never publishes (its
    # flag word is never written). The wait has a short limit; the kernel returns by itself,
    # the status word says "peer flag wait timed out", the context stays usable and the status
    # can be cleared.
    import ctypes
    from strata_b200 import _lib
    lib = _lib.load()
    assert _lib.device_status() == 0
    flags = torch.zeros(2, 64, dtype=torch.int32, device="cuda")   # [rank][slot]
    ptrs = (ctypes.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.strata_halo_barrier(ptrs, 0, 2, 1, 20, stream), "strata_halo_barrier")
    assert _lib.device_status() == 105          # reported ...
    assert _lib.device_status() == 0            # ... and cleared by the read
    assert flags[1, 0].item() == 1 and flags[0, 0].item() == 1   # our own publication happened
    # the same barrier completes at once when the partner's slot carries the epoch
    flags[0, 1] = 2
    _lib.check(lib.strata_halo_barrier(ptrs, 0, 2, 2, 20, stream), "strata_halo_barrier")
    assert _lib.device_status() == 0
    x = torch.ones(8, device="cuda")
    assert float((x * 2).sum()) == 16.0         # context still alive
