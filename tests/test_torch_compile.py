"""The module boundary under torch.compile (the reference compiles the whole network before a
rollout: screamcast/earth2studio_wrappers.py:412-413, scripts/ace/run_screamcast_nudged.py:639-641,
and runs it under torch.inference_mode(), :452).

CPU: the wrappers trace as ONE registered operator with fullgraph=True (fake tensors only - no
kernel runs). GPU: the compiled network returns the eager network's bits.
"""
import pytest
import torch


def _small_backbone(**kw):
    from strata_b200.wrappers import StrataBackboneModel
    cfg = dict(depth=4, height=16, width=16, n_layers=2, in_chans=5, base_out_chans=5,
               embed_dim=128, num_heads=2, attn_kernel=(3, 5, 5), do_rope_2d_stereographic=True,
               index_is_latlon=True, patch_size_horiz=2, do_rotate_wind=True,
               wind_channel_indices=(0, 1))
    cfg.update(kw)
    return StrataBackboneModel(**cfg)


def _tracing_backend(graphs):
    """A compile backend that records the graph and 'runs' it on fake tensors only."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    def backend(gm, example_inputs):
        graphs.append(gm)

        def run(*args):
            with FakeTensorMode(allow_non_fake_inputs=True) as mode:
                fake = [mode.from_tensor(a) if isinstance(a, torch.Tensor) else a for a in args]
                out = gm(*fake)
            return [torch.zeros(o.shape, dtype=o.dtype) for o in out]
        return run
    return backend


def _ops_of(graphs):
    return [str(n.target) for g in graphs for n in g.graph.nodes if n.op == "call_function"]


def test_backbone_wrapper_traces_as_one_operator():
    m = _small_backbone()
    graphs = []
    cm = torch.compile(m, backend=_tracing_backend(graphs), fullgraph=True)
    x = torch.randn(3, 5, 4, 16, 16)
    idx = {"lat": torch.rand(1, 16, 16), "lon": torch.rand(1, 16, 16)}
    with torch.inference_mode():
        y = cm(x, idx)
    assert y.shape == (3, 5, 4, 16, 16) and y.dtype == torch.float32
    assert _ops_of(graphs) == ["strata_b200.network_forward"]


def test_integer_index_lookup_stays_in_the_graph():
    m = _small_backbone(index_is_latlon=False, do_rotate_wind=False, wind_channel_indices=None)
    m.geometry.set_lookup_tables(torch.linspace(-1, 1, 1000), torch.linspace(0, 6, 1000))
    graphs = []
    cm = torch.compile(m, backend=_tracing_backend(graphs), fullgraph=True)
    x = torch.randn(2, 5, 4, 16, 16)
    idx = torch.randint(0, 1000, (2, 16, 16))
    y = cm(x, idx)
    assert y.shape == (2, 5, 4, 16, 16)
    ops = _ops_of(graphs)
    assert ops[-1] == "strata_b200.network_forward" and len(ops) > 1   # gathers + the operator


def test_two_stage_wrapper_traces_and_copies_get_their_own_handle():
    import copy
    from strata_b200.wrappers import StrataModel
    m = StrataModel(depth=2, height=16, width=16, n_layers=1, in_chans=4, base_out_chans=4,
                    embed_dim=128, num_heads=2, attn_kernel=3, patch_size_horiz=4,
                    index_is_latlon=True, embed_dim_pixel=64, n_layers_pixel=1, num_heads_pixel=1,
                    attn_kernel_pixel=3, use_bilinear_dw_gelu_project_adaln_pixel=True)
    m2 = copy.deepcopy(m)
    assert m2._op_handle != m._op_handle
    graphs = []
    cm = torch.compile(m2, backend=_tracing_backend(graphs), fullgraph=True)
    y = cm(torch.randn(1, 4, 2, 16, 16), {"lat": torch.rand(1, 16, 16), "lon": torch.rand(1, 16, 16)})
    assert y.shape == (1, m2._out_chans, 2, 16, 16)
    assert _ops_of(graphs) == ["strata_b200.network_forward"]


def test_fine_grained_operators_have_fake_implementations():
    import strata_b200.torch_ops  # noqa: F401  (registers the operators)
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        x = torch.empty(64, 128, dtype=torch.bfloat16)
        w = torch.empty(256, 128, dtype=torch.bfloat16)
        assert torch.ops.strata_b200.linear(x, w, None, 0, None).shape == (64, 256)
        assert torch.ops.strata_b200.layernorm(x, 1e-6).shape == (64, 128)
        q = torch.empty(1, 2, 8, 8, 2, 64, dtype=torch.bfloat16)
        assert torch.ops.strata_b200.na3d(q, q, q, [1, 3, 3]).shape == q.shape
        xb = torch.empty(1, 128, 128, dtype=torch.bfloat16)
        ws = [torch.empty(384, 128), torch.empty(128, 128), torch.empty(512, 128), torch.empty(128, 512)]
        bs = [torch.empty(384), torch.empty(128), torch.empty(512), torch.empty(128)]
        assert torch.ops.strata_b200.block_forward(xb, ws, bs, [2, 8, 8], 2, [1, 3, 3], None,
                                                   False).shape == xb.shape


@pytest.mark.gpu
@pytest.mark.parametrize("backend,fullgraph", [("eager", True), ("inductor", False)])
def test_compiled_network_equals_eager(backend, fullgraph):
    torch.manual_seed(0)
    m = _small_backbone().cuda().eval()
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.05)
    x = torch.randn(3, 5, 4, 16, 16, device="cuda")
    idx = {"lat": torch.rand(1, 16, 16, device="cuda") * 0.5,
           "lon": torch.rand(1, 16, 16, device="cuda") * 0.5 + 1.0}
    with torch.inference_mode():
        want = m(x, idx)
        cm = torch.compile(m, backend=backend, fullgraph=fullgraph)
        got = cm(x, idx)
        got2 = cm(x + 1.0, idx)
        want2 = m(x + 1.0, idx)
    assert torch.isfinite(want).all()
    assert torch.equal(got, want) and torch.equal(got2, want2)
    # the operators over the C ABI, called directly
    from strata_b200 import ops
    xb = torch.randn(256, 128, device="cuda").bfloat16()
    w = (torch.randn(64, 128, device="cuda") * 0.05).bfloat16()
    assert torch.equal(torch.ops.strata_b200.linear(xb, w, None, 0, None), ops.linear(xb, w))
