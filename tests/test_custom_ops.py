"""The torch.library registration of the operator (CPU part: schema and fake implementations)."""
import pytest
import torch


def _ops():
    from gtr_b200 import custom_ops
    return custom_ops


def test_operators_are_registered_with_mutable_workspace_and_output():
    co = _ops()
    for op, n_args in ((torch.ops.gtr_b200.chunk_gla, 11), (torch.ops.gtr_b200.chunk_gla_gated, 14)):
        schema = op.default._schema
        assert len(schema.arguments) == n_args
        mutated = {a.name for a in schema.arguments if a.alias_info is not None and a.alias_info.is_write}
        assert mutated == {"ws", "out"}
        assert len(schema.returns) == 0
    assert co.chunk_gla is torch.ops.gtr_b200.chunk_gla


def test_fake_implementations_run_without_a_device():
    _ops()
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        B, T, H = 2, 128, 3
        q = torch.empty(B, T, H, 64, dtype=torch.float16, device="cuda")
        ws = torch.empty(1024, dtype=torch.float32, device="cuda")
        out = torch.empty_like(q)
        w = torch.empty(64, dtype=torch.float16, device="cuda")
        assert torch.ops.gtr_b200.chunk_gla(q, q, q, q, 0.125, ws, out, 0.0, 0, 0, 0) is None
        assert torch.ops.gtr_b200.chunk_gla_gated(q, q, q, q, q, w, 0.125, 1e-5, ws, out, 16.0, 2, 8, 16) is None


def test_cpu_tensors_are_refused_loudly():
    """The real implementation has no CPU path: calling it with CPU tensors raises, it does not fall back."""
    _ops()
    q = torch.zeros(1, 64, 1, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError):
        torch.ops.gtr_b200.chunk_gla(q, q, q, q, 0.125, torch.zeros(16), torch.zeros_like(q), 0.0, 0, 0, 0)


@pytest.mark.gpu
def test_custom_op_equals_direct_call_and_traces_without_graph_breaks():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import gtr_b200 as G
    from oracle import gla_ref
    _ops()
    B, T, H = 2, 320, 3
    q, k, v, g = (x.cuda() for x in gla_ref.make_inputs(B, T, H, seed=3))
    ws = G.make_workspace(B, T, H, "cuda")
    ref = torch.empty(B, T, H, 64, dtype=torch.float16, device="cuda")
    G.chunk_gla_run(q, k, v, g, 0.125, ws, ref, direction=3, grid_hw=(16, 20))

    def f(q, k, v, g, ws):
        out = torch.empty_like(q)
        torch.ops.gtr_b200.chunk_gla(q, k, v, g, 0.125, ws, out, 0.0, 3, 16, 20)
        return out * 2.0

    got = f(q, k, v, g, ws)
    assert torch.equal(got, ref * 2.0)
    traced = torch.compile(f, backend="eager", fullgraph=True)   # Dynamo only: no graph break at the operator
    assert torch.equal(traced(q, k, v, g, ws), ref * 2.0)
