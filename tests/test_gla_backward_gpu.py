"""Parity of the CUDA gradient kernels (through the C ABI and through autograd) against the CPU gradient oracle.

Tolerances: dq, dk, dv are fp16 outputs of fp32 arithmetic -> relative L2 error <= 1e-3 against the float64 oracle on
the same fp16 inputs; dg and the state gradient are fp32 -> <= 1e-4."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

REL_HALF = 1e-3
REL_FLOAT = 1e-4
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def G():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import gtr_b200
    return gtr_b200


def _rel(ref, got):
    ref, got = ref.detach().double().cpu().flatten(), got.detach().double().cpu().flatten()
    assert bool(torch.isfinite(got).all())
    return float((got - ref).norm() / ref.norm().clamp_min(1e-30))


def _compare(want, got, states, q=None, k=None):
    names = ("dq", "dk", "dv", "dg", "dh0")
    for i, n in enumerate(names[: 5 if states else 4]):
        tol = REL_HALF if i < 3 else REL_FLOAT
        if i == 3 and q is not None:
            # dg is a running sum of differences q dq - k dk that cancel (exactly, for a lone token): its error is
            # measured against the running sum of the terms' magnitudes
            mag = ((q.double() * want[0]).abs() + (k.double() * want[1]).abs()).flip(1).cumsum(1).flip(1)
            err = (got[3].double().cpu() - want[3]).norm()
            assert bool(torch.isfinite(got[3]).all()) and float(err) <= tol * float(want[3].norm()) + 1e-6 * float(mag.norm()), n
            continue
        assert _rel(want[i], got[i]) <= tol, (n, _rel(want[i], got[i]))


def _inputs(B, T, H, K, seed, gate=("ls", 0.0, 1.0, 16.0), states=False):
    from oracle import gla_ref
    q, k, v, g = gla_ref.make_inputs(B, T, H, K=K, seed=seed, gate=gate)
    gen = torch.Generator().manual_seed(seed + 100)
    do = (torch.randn(v.shape, generator=gen) / 8).half()
    s0 = torch.randn(B, H, K, 64, generator=gen) / 8 if states else None
    dht = torch.randn(B, H, K, 64, generator=gen) / 8 if states else None
    return q, k, v, g, do, s0, dht


@pytest.mark.parametrize("B,T,H,K", [(2, 1, 2, 64), (1, 31, 1, 64), (2, 32, 3, 64), (1, 33, 2, 64), (2, 100, 3, 64),
                                     (1, 257, 2, 32), (1, 640, 2, 64), (3, 70, 2, 32),
                                     (1, 1000, 2, 64), (1, 600, 2, 32), (1, 2048, 1, 64)])   # cut into 3, 2 and 8 segments
@pytest.mark.parametrize("states", [False, True])
def test_gradients_against_the_oracle(G, B, T, H, K, states):
    from oracle import gla_bwd_ref
    q, k, v, g, do, s0, dht = _inputs(B, T, H, K, seed=T + K, states=states)
    want = gla_bwd_ref.recurrent_gla_backward(q, k, v, g, do, initial_state=s0, d_final_state=dht)
    dev = "cuda"
    got = G.chunk_gla_backward(q.to(dev), k.to(dev), v.to(dev), g.to(dev), do.to(dev), None,
                               None if s0 is None else s0.to(dev), None if dht is None else dht.to(dev), states)
    torch.cuda.synchronize()
    _compare(want, got, states, q, k)


@pytest.mark.parametrize("gate", [("ls", -4.0, 2.0, 1.0), ("ls", 3.0, 1.0, 1.0)])
def test_strong_and_open_gates(G, gate):
    from oracle import gla_bwd_ref
    q, k, v, g, do, s0, dht = _inputs(1, 200, 2, 64, seed=9, gate=gate, states=True)
    want = gla_bwd_ref.recurrent_gla_backward(q, k, v, g, do, initial_state=s0, d_final_state=dht)
    got = G.chunk_gla_backward(*(x.cuda() for x in (q, k, v, g, do)), None, s0.cuda(), dht.cuda(), True)
    _compare(want, got, True, q, k)


@pytest.mark.parametrize("K", [64, 32])
@pytest.mark.parametrize("gates", ["weak", "strong"])
def test_committed_vectors_of_the_reference_recurrence(G, K, gates):
    F = np.load(os.path.join(GOLDEN, "recurrence_backward.npz"))
    tag = f"k{K}_{gates}"
    q, k, v, g, do = (torch.from_numpy(F[f"{tag}_{n}"]).cuda() for n in ("q", "k", "v", "g", "do"))
    got = G.chunk_gla_backward(q, k, v, g, do)
    want = [torch.from_numpy(F[f"{tag}_{n}"]) for n in ("dq", "dk", "dv", "dg")]
    _compare(want, got, False)


def test_autograd_through_chunk_gla(G):
    from oracle import gla_bwd_ref, c_oracle
    q, k, v, g, do, s0, dht = _inputs(2, 150, 2, 64, seed=4, states=True)
    leaves = [x.cuda().requires_grad_(True) for x in (q, k, v, g, s0)]
    o, hT = G.chunk_gla(*leaves[:4], initial_state=leaves[4], output_final_state=True)
    ref_o, ref_h = c_oracle.forward(q, k, v, g, initial_state=s0, output_final_state=True)
    assert _rel(ref_o, o) <= 1e-3 and _rel(ref_h, hT) <= 1e-3
    ((o.float() * do.cuda().float()).sum() + (hT * dht.cuda()).sum()).backward()
    want = gla_bwd_ref.recurrent_gla_backward(q, k, v, g, do, initial_state=s0, d_final_state=dht)
    got = [x.grad for x in leaves]
    assert got[3].dtype == torch.float16
    for i, n in enumerate(("dq", "dk", "dv", "dg", "dh0")):
        assert _rel(want[i], got[i]) <= (REL_HALF if i < 4 else REL_FLOAT), n      # dg is cast to the gate's fp16 here
    # without a final state, and with no gradient wanted for the state
    q2, k2 = q.cuda().requires_grad_(True), k.cuda()
    o2, none = G.fused_recurrent_gla(q2, k2, v.cuda(), g.cuda())
    assert none is None
    (o2.float() * do.cuda().float()).sum().backward()
    want2 = gla_bwd_ref.recurrent_gla_backward(q, k, v, g, do)
    assert _rel(want2[0], q2.grad) <= REL_HALF


def test_autograd_with_packed_sequences(G):
    from oracle import gla_bwd_ref
    lens = [40, 1, 130, 64]
    T = sum(lens)
    q, k, v, g, do, _, _ = _inputs(1, T, 2, 64, seed=21)
    gen = torch.Generator().manual_seed(5)
    s0 = torch.randn(len(lens), 2, 64, 64, generator=gen) / 8
    offs = [0]
    for n in lens:
        offs.append(offs[-1] + n)
    leaves = [x.cuda().requires_grad_(True) for x in (q, k, v, g, s0)]
    o, hT = G.chunk_gla(*leaves[:4], initial_state=leaves[4], output_final_state=True,
                        cu_seqlens=torch.tensor(offs, dtype=torch.int32))
    dht = torch.randn(hT.shape, generator=gen) / 8
    ((o.float() * do.cuda().float()).sum() + (hT * dht.cuda()).sum()).backward()
    for i, (a, b) in enumerate(zip(offs, offs[1:])):
        want = gla_bwd_ref.recurrent_gla_backward(q[:, a:b], k[:, a:b], v[:, a:b], g[:, a:b], do[:, a:b],
                                                  initial_state=s0[i:i + 1], d_final_state=dht[i:i + 1])
        for j in range(4):
            assert _rel(want[j], leaves[j].grad[:, a:b]) <= REL_HALF * (3 if b - a == 1 else 1), (i, j)
        assert _rel(want[4], leaves[4].grad[i:i + 1]) <= REL_FLOAT


def test_long_sequence_at_bench_width(G):
    """The bench's head layout (12 heads) at a length of many chunks: gradients against the oracle on one sequence."""
    from oracle import gla_bwd_ref
    q, k, v, g, do, _, _ = _inputs(1, 1600, 12, 64, seed=2)
    want = gla_bwd_ref.recurrent_gla_backward(q, k, v, g, do)
    got = G.chunk_gla_backward(*(x.cuda() for x in (q, k, v, g, do)))
    _compare(want, got, False)


def test_argument_errors(G):
    from gtr_b200 import _lib
    q, k, v, g, do, _, _ = _inputs(1, 8, 1, 64, seed=0)
    with pytest.raises(RuntimeError):
        G.chunk_gla_backward(q.cuda().float(), k.cuda(), v.cuda(), g.cuda(), do.cuda())
    a = _lib.BwdArgs()
    assert _lib.lib().gla_b200_backward(None, None) == -1
    a.B, a.T, a.H, a.K, a.V = 1, 8, 1, 48, 64
    assert _lib.lib().gla_b200_backward(a, None) == -2
    a.K = 64
    assert _lib.lib().gla_b200_backward(a, None) == -1          # pointers missing


@pytest.mark.parametrize("direction", [1, 2, 3])
def test_autograd_in_the_other_scan_directions(G, direction):
    """The gradient of a column / reversed scan is the row-major gradient of the tokens gathered into scan order."""
    from oracle import gla_bwd_ref, gla_ref
    grid = (9, 14)
    q, k, v, g, do, s0, dht = _inputs(2, grid[0] * grid[1], 2, 64, seed=30 + direction, states=True)
    leaves = [x.cuda().requires_grad_(True) for x in (q, k, v, g, s0)]
    o, hT = G.chunk_gla(*leaves[:4], initial_state=leaves[4], output_final_state=True, direction=direction, grid_hw=grid)
    ((o.float() * do.cuda().float()).sum() + (hT * dht.cuda()).sum()).backward()
    perm = gla_ref.scan_order(direction, *grid)
    want = gla_bwd_ref.recurrent_gla_backward(q[:, perm], k[:, perm], v[:, perm], g[:, perm], do[:, perm],
                                              initial_state=s0, d_final_state=dht)
    for i, n in enumerate(("dq", "dk", "dv", "dg")):
        back = torch.empty_like(want[i])
        back[:, perm] = want[i]
        assert _rel(back, leaves[i].grad) <= REL_HALF, n
    assert _rel(want[4], leaves[4].grad) <= REL_FLOAT


def test_autograd_with_raw_gate_logits(G):
    """gk_normalizer > 0: the operator takes logits x and uses logsigmoid(x) / normalizer; dx = dg * sigmoid(-x) / normalizer."""
    from oracle import gla_bwd_ref
    q, k, v, _, do, _, _ = _inputs(1, 300, 2, 64, seed=40)
    x = (torch.randn(1, 300, 2, 64, generator=torch.Generator().manual_seed(41)) * 2).half()
    leaves = [t.cuda().requires_grad_(True) for t in (q, k, v, x)]
    o, _ = G.chunk_gla(*leaves, gk_normalizer=16.0)
    (o.float() * do.cuda().float()).sum().backward()
    g = torch.nn.functional.logsigmoid(x.double()) / 16
    want = gla_bwd_ref.recurrent_gla_backward(q, k, v, g, do)
    dx = want[3] * torch.sigmoid(-x.double()) / 16
    for i, (n, w) in enumerate(zip(("dq", "dk", "dv", "dx"), (want[0], want[1], want[2], dx))):
        assert _rel(w, leaves[i].grad) <= 2e-3, n                 # the gates reach the gradient kernels rounded to fp16
