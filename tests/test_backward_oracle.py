"""The gradient oracle (oracle/gla_bwd_ref.py) against autograd: through the reference's own float64 recurrence
(committed vectors, tests/golden/make_golden.py), through the third-party pure-PyTorch recurrence, and through a
differentiable restatement with states."""
import os

import numpy as np
import pytest
import torch

from oracle import gla_bwd_ref, gla_ref

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
NAMES = ("dq", "dk", "dv", "dg")


def _t(a):
    return torch.from_numpy(np.asarray(a))


@pytest.mark.parametrize("K", [64, 32])
@pytest.mark.parametrize("gates", ["weak", "strong"])
def test_gradients_match_autograd_of_the_reference_recurrence(K, gates):
    G = np.load(os.path.join(GOLDEN, "recurrence_backward.npz"))
    tag = f"k{K}_{gates}"
    q, k, v, g, do = (_t(G[f"{tag}_{n}"]) for n in ("q", "k", "v", "g", "do"))
    got = gla_bwd_ref.recurrent_gla_backward(q, k, v, g, do)
    for n, x in zip(NAMES, got):
        want = _t(G[f"{tag}_{n}"]).double()
        assert torch.allclose(x, want, rtol=1e-5, atol=1e-6 * float(want.abs().max())), n


def test_gradients_match_third_party_naive_recurrence_with_states():
    naive = pytest.importorskip("fla.ops.gla.naive").naive_recurrent_gla
    q, k, v, g = gla_ref.make_inputs(2, 70, 2, dtype=torch.float32, seed=5)
    gen = torch.Generator().manual_seed(3)
    do, s0, dht = torch.randn(v.shape, generator=gen), torch.randn(2, 2, 64, 64, generator=gen), torch.randn(2, 2, 64, 64, generator=gen)
    leaves = [x.double().requires_grad_(True) for x in (q, k, v, g, s0)]
    o, h = naive(*leaves[:4], initial_state=leaves[4], output_final_state=True)
    want = torch.autograd.grad((o.double() * do.double()).sum() + (h.double() * dht.double()).sum(), leaves)
    got = gla_bwd_ref.recurrent_gla_backward(q, k, v, g, do, initial_state=s0, d_final_state=dht)
    for n, x, w in zip(NAMES + ("dh0",), got, want):          # the third-party code keeps its state in fp32
        assert torch.allclose(x, w, rtol=1e-4, atol=1e-5 * float(w.abs().max())), n


@pytest.mark.parametrize("K,T,states", [(64, 1, True), (64, 45, False), (32, 33, True)])
def test_hand_derivation_equals_autograd(K, T, states):
    q, k, v, g = gla_ref.make_inputs(1, T, 2, K=K, dtype=torch.float32, seed=T, gate=("ls", 1.0, 2.0, 1.0))
    gen = torch.Generator().manual_seed(T)
    do = torch.randn(v.shape, generator=gen)
    s0 = torch.randn(1, 2, K, 64, generator=gen) if states else None
    dht = torch.randn(1, 2, K, 64, generator=gen) if states else None
    a = gla_bwd_ref.recurrent_gla_backward(q, k, v, g, do, scale=0.3, initial_state=s0, d_final_state=dht)
    b = gla_bwd_ref.autograd_backward(q, k, v, g, do, scale=0.3, initial_state=s0, d_final_state=dht)
    for n, x, y in zip(NAMES + ("dh0",), a, b):
        assert torch.allclose(x, y, rtol=1e-10, atol=1e-12), n
