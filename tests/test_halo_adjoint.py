"""Windowed overlap-add un-pad (normalised halo adjoint): host lists against the oracle, and the
properties the reference's tests rely on (tests/distributed/test_distributed_halo.py:61,105:
crop(pad(x)) ~ x and the constant round trip)."""
import numpy as np
import pytest

from oracle import halo_oracle as ho
from strata_b200.topology import TileTopology, apply_maps_numpy, halo_adjoint_lists, halo_source_maps


def _kbd(P):
    from scipy.signal.windows import kaiser_bessel_derived
    w = kaiser_bessel_derived(P, 10 * np.pi).astype(np.float32)
    return w[None, :] * w[:, None]


def _apply_lists(pad_all, topo, window):
    """The kernel's loop on the host: entry by entry, float32, no fused multiply-add."""
    P = topo.padded_tile_size
    off, cell, coef, weights = halo_adjoint_lists(topo, window)
    w = np.ones(P * P, np.float32) if window is None else np.asarray(window, np.float32).reshape(-1)
    lead = pad_all.shape[:-3]
    y = pad_all.reshape(*lead, -1).astype(np.float32)
    out = np.zeros((*lead, len(weights)), np.float32)
    for c in range(len(weights)):
        acc = np.zeros(lead, np.float32)
        for e in range(off[c], off[c + 1]):
            wy = (w[cell[e] % (P * P)] * y[..., cell[e]]).astype(np.float32)
            acc = (acc + (coef[e] * wy).astype(np.float32)).astype(np.float32)
        out[..., c] = acc / weights[c]
    return out.reshape(*lead, topo.tiles_per_rank, topo.tile_size, topo.tile_size)


@pytest.mark.parametrize("world,face,tile,halo,window", [(2, 16, 4, 3, "ones"), (1, 8, 4, 1, "kbd"),
                                                          (3, 8, 4, 2, "kbd"), (1, 4, 4, 2, "ones")])
def test_lists_match_oracle_bit_exactly(world, face, tile, halo, window):
    full = ho.TileTopology(1, 0, face, tile, halo)
    win = None if window == "ones" else _kbd(tile + 2 * halo)
    rng = np.random.default_rng(face + halo)
    x = rng.standard_normal((2, full.total_tiles, tile, tile)).astype(np.float32)
    pad_all = ho.padded_local_tiles(x, full) + rng.standard_normal(
        (2, full.total_tiles, tile + 2 * halo, tile + 2 * halo)).astype(np.float32)
    for rank in range(world):
        got = _apply_lists(pad_all, TileTopology(world, rank, face, tile, halo), win)
        want = ho.halo_adjoint(pad_all, ho.TileTopology(world, rank, face, tile, halo), win)
        assert np.array_equal(got, want)


def test_transpose_identity_and_round_trips():
    face, tile, halo = 16, 8, 3
    topo = TileTopology(1, 0, face, tile, halo)
    a, b = halo_source_maps(topo)
    rng = np.random.default_rng(3)
    x = rng.standard_normal((topo.total_tiles, tile, tile))
    y = rng.standard_normal(a.shape)
    off, cell, coef, weights = halo_adjoint_lists(topo)
    aty = np.array([(coef[off[c]:off[c + 1]] * y.reshape(-1)[cell[off[c]:off[c + 1]]]).sum()
                    for c in range(len(weights))])
    assert np.isclose((apply_maps_numpy(x, a, b) * y).sum(), (x.reshape(-1) * aty).sum(), rtol=1e-10)
    # every padded cell is handed back exactly once in total
    assert np.isclose(weights.sum(), a.size)
    otopo = ho.TileTopology(1, 0, face, tile, halo)
    const = np.full((topo.total_tiles, tile, tile), -3.25, np.float32)
    for win in (None, _kbd(tile + 2 * halo)):
        back = ho.halo_adjoint(ho.padded_local_tiles(const, otopo), otopo, win)
        assert np.allclose(back, -3.25, rtol=1e-6, atol=0)
    # consistent padded tiles (every halo cell equals its source, no corner means): un-pad == crop
    xs = rng.standard_normal((topo.total_tiles, tile, tile)).astype(np.float32)
    win0 = np.zeros((tile + 2 * halo,) * 2, np.float32)
    win0[halo:-halo, halo:-halo] = 1.0
    pad = ho.padded_local_tiles(xs, otopo)
    assert np.array_equal(ho.halo_adjoint(pad, otopo, win0), xs)


def test_window_shape_is_checked():
    with pytest.raises(ValueError):
        halo_adjoint_lists(TileTopology(1, 0, 8, 4, 1), np.ones((5, 5), np.float32))


def test_channel_chunked_accepts_both_call_forms():
    """`channel_chunked(32)(halo)` is the reference rollout driver's form
    (scripts/ace/run_screamcast_nudged.py:119-134, 621); `channel_chunked(halo, 32)` the short one."""
    import torch
    from strata_b200.halo import channel_chunked
    calls = []

    def fn(x):
        calls.append(x.shape[1])
        return x * 2

    x = torch.arange(2 * 7 * 3, dtype=torch.float32).reshape(2, 7, 3)
    for wrapped in (channel_chunked(3)(fn), channel_chunked(fn, 3)):
        calls.clear()
        assert torch.equal(wrapped(x), x * 2)
        assert calls == [3, 3, 1]
        assert wrapped.__wrapped__ is fn
    assert channel_chunked(0)(fn) is fn and channel_chunked(fn, -1) is fn
