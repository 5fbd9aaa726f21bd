"""The CPU oracle against vectors produced by the reference's own code (tests/golden/make_golden.py)
and against the third-party pure-PyTorch recurrence the reference depends on."""
import os

import numpy as np
import pytest
import torch

from oracle import c_oracle, gla_ref


GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _t(a):
    return torch.from_numpy(np.asarray(a))


@pytest.mark.parametrize("K", [64, 32])
@pytest.mark.parametrize("gates", ["weak", "strong", "bursts"])
def test_recurrence_matches_reference_fp64(golden_recurrence, K, gates):
    G = golden_recurrence
    q, k, v, g = (_t(G[f"k{K}_{gates}_{n}"]) for n in "qkvg")
    want = _t(G[f"k{K}_{gates}_o"])
    got, _ = gla_ref.recurrent_gla(q, k, v, g, dtype=torch.float64)
    assert torch.allclose(got.float(), want, rtol=1e-6, atol=1e-7)
    got_c, _ = c_oracle.forward(q, k, v, g, acc64=True)
    assert torch.allclose(got_c, want, rtol=1e-6, atol=1e-7)
    # the fp32 recurrence (what the tolerances are stated against) stays within 1e-5 relative
    got32, _ = c_oracle.forward(q, k, v, g)
    m = gla_ref.error_metrics(want, got32)
    assert m["rel_l2"] < 1e-5 and m["finite"]


@pytest.mark.parametrize("K", [64, 32])
@pytest.mark.parametrize("gate", [10.5, 12.0])
@pytest.mark.parametrize("j", [0, 7, 23, 63])
def test_single_term_history_rows(golden_recurrence, K, gate, j):
    want = _t(golden_recurrence[f"k{K}_hist_{gate:g}_{j}_row"])
    T = 192
    q = torch.zeros(1, T, 1, K, dtype=torch.float16)
    k = q.clone()
    v = torch.zeros(1, T, 1, 64, dtype=torch.float16)
    g = torch.full_like(q, -0.08)
    q[0, j + 1, 0, 0], k[0, j, 0, 0], v[0, j] = 16.0, 16.0, 4.0
    g[0, j + 1, 0, 0] = -gate
    for fn in (lambda: gla_ref.recurrent_gla(q, k, v, g, dtype=torch.float64)[0],
               lambda: c_oracle.forward(q, k, v, g, acc64=True)[0],
               lambda: gla_ref.chunk_gla(q, k, v, g, dtype=torch.float64)[0]):
        got = fn()[0, j + 1, 0].float()
        assert torch.allclose(got, want, rtol=1e-5, atol=0)


@pytest.mark.parametrize("K", [64, 32])
def test_all_gates_minus_1000(golden_recurrence, K):
    G = golden_recurrence
    q, k, v = (_t(G[f"k{K}_m1000_{n}"]) for n in "qkv")
    g = torch.full_like(q, -1000.0)
    want = _t(G[f"k{K}_m1000_o"])
    for got in (c_oracle.forward(q, k, v, g)[0], gla_ref.chunk_gla(q, k, v, g)[0]):
        assert torch.isfinite(got).all()
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-6)


def test_scan_orders_match_reference_backbone(golden_scan_order):
    for gs in (4, 6):
        want = golden_scan_order[f"order_gs{gs}"]
        for layer in range(4):
            got = gla_ref.scan_order(layer % 4, gs, gs).numpy()
            assert (got == want[layer]).all(), (gs, layer)


def test_scan_order_rectangular_grid():
    hg, wg = 3, 5
    col = gla_ref.scan_order("col", hg, wg)
    # step p = c*hg + r reads token r*wg + c
    for c in range(wg):
        for r in range(hg):
            assert col[c * hg + r] == r * wg + c
    assert (gla_ref.scan_order("col_rev", hg, wg) == col.flip(0)).all()
    assert (gla_ref.scan_order("row_rev", hg, wg) == torch.arange(15).flip(0)).all()


def test_against_third_party_naive_recurrence():
    naive = pytest.importorskip("fla.ops.gla.naive").naive_recurrent_gla
    q, k, v, g = gla_ref.make_inputs(2, 96, 3, dtype=torch.float32, seed=3)
    s0 = torch.randn(2, 3, 64, 64, generator=torch.Generator().manual_seed(1))
    want, want_s = naive(q, k, v, g, initial_state=s0, output_final_state=True)
    got, got_s = c_oracle.forward(q, k, v, g, initial_state=s0, output_final_state=True)
    assert torch.allclose(got, want.float(), rtol=1e-4, atol=1e-5)
    assert torch.allclose(got_s, want_s.float(), rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("direction", [0, 1, 2, 3])
def test_c_oracle_equals_python_oracle_all_directions(direction):
    q, k, v, g = gla_ref.make_inputs(1, 6 * 11, 2, dtype=torch.float32, seed=direction)
    s0 = torch.randn(1, 2, 64, 64, generator=torch.Generator().manual_seed(2))
    a, sa = gla_ref.gla_scan(q, k, v, g, direction=direction, grid_hw=(6, 11), initial_state=s0,
                             output_final_state=True)
    b, sb = c_oracle.forward(q, k, v, g, direction=direction, grid_hw=(6, 11), initial_state=s0,
                             output_final_state=True)
    assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)
    assert torch.allclose(sa, sb, rtol=1e-5, atol=1e-6)


def test_chunk_formulation_equals_recurrence():
    q, k, v, g = gla_ref.make_inputs(1, 200, 2, std=3.0, gate=("ls", 4.0, 2.0, 1.0), dtype=torch.float32)
    a, sa = gla_ref.recurrent_gla(q, k, v, g, dtype=torch.float64, output_final_state=True)
    b, sb = gla_ref.chunk_gla(q, k, v, g, dtype=torch.float64, output_final_state=True)
    assert torch.allclose(a, b, rtol=1e-9, atol=1e-9)
    assert torch.allclose(sa, sb, rtol=1e-9, atol=1e-9)


def test_empty_and_bad_arguments():
    q = torch.zeros(1, 0, 2, 64)
    o, _ = c_oracle.forward(q, q, q, q)
    assert o.shape == (1, 0, 2, 64)
    with pytest.raises(ValueError):
        gla_ref.direction_id(7)


def _backbone_fixture(tag):
    z = np.load(os.path.join(GOLDEN, "backbone_small.npz"))
    sd = {k[len(tag) + 4:]: torch.from_numpy(z[k]).float() for k in z.files if k.startswith(tag + "_sd/")}
    img = torch.from_numpy(z[tag + "_img"]).float()
    outs = [torch.from_numpy(z[f"{tag}_out{i}"]) for i in range(3)]
    return sd, img, outs


@pytest.mark.parametrize("tag,expand_k", [("k64", 1.0), ("k32", 0.5)])
def test_backbone_oracle_matches_the_reference_backbone(tag, expand_k):
    """oracle/backbone_ref.py against outputs of the reference's own ViTAdapterSpatialSwiGLU (four blocks, dim 128,
    two heads with V = 64 and K = 64 or 32, ffn_ratio 6; recorded by tests/golden/make_golden.py): pins the stem, the BatchNorm
    folding, the gate normaliser, norm_eps, the hidden-size rule, the per-block scan orders and the orientation of
    the depthwise kernels, through the product's load_reference_state_dict."""
    from gtr_b200.backbone import GTRBackbone
    from oracle import backbone_ref
    sd, img, outs = _backbone_fixture(tag)
    m = GTRBackbone(embed_dim=128, depth=4, num_heads=2, mlp_ratio=6, return_layers=(1, 2, 3),
                    expand_k=expand_k).eval().float()
    m.load_reference_state_dict(sd)
    got = backbone_ref.forward(m, img)
    assert len(got) == 3
    for ref, o in zip(outs, got):
        o = o.transpose(1, 2).reshape(ref.shape)                 # the reference returns [B, C, H, W] maps
        e = gla_ref.error_metrics(ref, o)
        assert e["finite"] and e["rel_l2"] < 5e-6 and e["max_abs"] < 5e-6, e
