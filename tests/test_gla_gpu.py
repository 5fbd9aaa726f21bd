"""Parity of the CUDA operator (called through the C ABI) against the CPU oracle.

Tolerances are the ones the operator is specified with: relative L2 error <= 1e-3 against the
fp32 token recurrence, no non-finite values, and max-abs error <= 2e-3.  For the stress
config (inputs ~N(0,3), outputs of magnitude several hundred) an fp16 output cannot resolve
2e-3 absolute, so there the max-abs bound is applied relative to the largest reference value.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

REL_L2 = 1e-3
MAX_ABS = 2e-3


@pytest.fixture(scope="module")
def G():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import gtr_b200
    return gtr_b200


def _run(G, q, k, v, g, *, scale=None, direction=0, grid_hw=None, segments=0, s0=None, final=False,
         gk_normalizer=0.0, poison=True):
    dev = "cuda"
    B, T, H, K = q.shape
    scale = K ** -0.5 if scale is None else scale
    qd, kd, vd, gd = (x.to(dev) for x in (q, k, v, g))
    ws = G.make_workspace(B, T, H, dev)
    if segments and 0 < segments < 4:   # the advertised size covers segments of >= 4 chunks
        ws = torch.zeros(ws.numel() * 4, dtype=torch.float32, device=dev)
    o = torch.full((B, T, H, 64), float("nan"), dtype=torch.float16, device=dev) if poison else \
        torch.empty(B, T, H, 64, dtype=torch.float16, device=dev)
    fs = torch.full((B, H, K, 64), float("nan"), dtype=torch.float32, device=dev) if final else None
    G.chunk_gla_run(qd, kd, vd, gd, scale, ws, o, gk_normalizer, direction=direction, grid_hw=grid_hw,
                    segments=segments, initial_state=None if s0 is None else s0.to(dev), final_state=fs)
    G.check_status(ws)
    return o.float().cpu(), (fs.cpu() if final else None)


def _check(ref, got, rel=REL_L2, relative_abs=False):
    from oracle import gla_ref
    m = gla_ref.error_metrics(ref, got)
    assert m["finite"], m
    assert m["rel_l2"] <= rel, m
    bound = MAX_ABS * max(1.0, m["ref_max"]) if relative_abs else MAX_ABS
    assert m["max_abs"] <= bound, m
    return m


@pytest.mark.parametrize("T", [1, 17, 63, 64, 65, 100, 127, 128, 256, 640, 1000])
def test_lengths_including_ragged(G, T):
    from oracle import c_oracle, gla_ref
    q, k, v, g = gla_ref.make_inputs(2, T, 3, seed=T)
    ref, _ = c_oracle.forward(q, k, v, g)
    got, _ = _run(G, q, k, v, g)
    _check(ref, got)


@pytest.mark.parametrize("direction", [0, 1, 2, 3])
@pytest.mark.parametrize("grid", [(40, 40), (7, 13), (64, 5), (3, 70)])
def test_scan_orders(G, direction, grid):
    from oracle import c_oracle, gla_ref
    hg, wg = grid
    q, k, v, g = gla_ref.make_inputs(2, hg * wg, 2, seed=direction)
    ref, _ = c_oracle.forward(q, k, v, g, direction=direction, grid_hw=grid)
    got, _ = _run(G, q, k, v, g, direction=direction, grid_hw=grid)
    _check(ref, got)


@pytest.mark.parametrize("segments", [1, 2, 3, 5, 64])
@pytest.mark.parametrize("direction", [0, 3])
def test_segmented_sequences_with_states(G, segments, direction):
    """Every split of a sequence into work items gives the same result, incoming state included."""
    from oracle import c_oracle, gla_ref
    B, H, grid = 2, 3, (25, 28)           # T = 700: 11 chunks, the last one ragged
    q, k, v, g = gla_ref.make_inputs(B, 700, H, seed=5)
    s0 = torch.randn(B, H, 64, 64, generator=torch.Generator().manual_seed(9))
    ref, ref_s = c_oracle.forward(q, k, v, g, direction=direction, grid_hw=grid, initial_state=s0,
                                  output_final_state=True)
    got, got_s = _run(G, q, k, v, g, direction=direction, grid_hw=grid, segments=segments, s0=s0, final=True)
    _check(ref, got, relative_abs=True)
    assert torch.isfinite(got_s).all()
    assert ((got_s - ref_s).norm() / ref_s.norm()).item() < 5e-4   # fp32 carry; the increments come from fp16 operands


def test_config2_all_four_scan_orders(G):
    from oracle import c_oracle, gla_ref
    q, k, v, g = gla_ref.config_inputs("c2")
    for d in range(4):
        ref, _ = c_oracle.forward(q, k, v, g, direction=d, grid_hw=(40, 40))
        got, _ = _run(G, q, k, v, g, direction=d, grid_hw=(40, 40))
        _check(ref, got)


@pytest.mark.parametrize("direction", [0, 1, 2, 3])
def test_config3_high_resolution(G, direction):
    """The throughput point of the benchmark (B4 H12 T6400 on an 80 x 80 grid), every scan order it cycles through."""
    from oracle import c_oracle, gla_ref
    q, k, v, g = gla_ref.config_inputs("c3")
    ref, _ = c_oracle.forward(q, k, v, g, direction=direction, grid_hw=(80, 80))
    got, _ = _run(G, q, k, v, g, direction=direction, grid_hw=(80, 80))
    _check(ref, got)


@pytest.mark.parametrize("direction", [0, 1, 2, 3])
def test_config5_numerical_stress(G, direction):
    """B2 H8 T8192 on a 64 x 128 grid, inputs ~N(0,3), near-zero decay over long spans, every scan order."""
    from oracle import c_oracle, gla_ref
    q, k, v, g = gla_ref.config_inputs("c5")
    ref, _ = c_oracle.forward(q, k, v, g, direction=direction, grid_hw=(64, 128))
    got, _ = _run(G, q, k, v, g, direction=direction, grid_hw=(64, 128))
    m = gla_ref.error_metrics(ref, got)
    print(f"config 5 direction {direction}: max_abs {m['max_abs']:.4g} at ref_max {m['ref_max']:.4g}, "
          f"rel_l2 {m['rel_l2']:.3g}")
    assert m["finite"] and m["rel_l2"] <= REL_L2, m
    # Outputs reach several hundred here and fp16 values of that size are 0.25 to 0.5 apart, so no fp16 output
    # can be within 2e-3 of the reference in absolute terms: the bound is applied relative to the largest
    # reference value, and the absolute error is required to stay below one fp16 spacing at that magnitude.
    assert m["max_abs"] <= MAX_ABS * m["ref_max"], \
        f"max-abs {m['max_abs']:.4g} exceeds 2e-3 x the largest reference value {m['ref_max']:.4g} (relative reading)"
    assert m["max_abs"] / m["ref_max"] <= 1e-3, m
    assert m["max_abs"] <= 2.0 ** (np.floor(np.log2(m["ref_max"])) - 10), \
        f"absolute max-abs {m['max_abs']:.4g} exceeds one fp16 spacing at {m['ref_max']:.4g}"


@pytest.mark.parametrize("direction", [0, 1, 2, 3])
def test_the_backbone_blocks_call_at_full_length(G, direction):
    """The call a backbone block makes on 1024 x 2048 images (64 x 128 patch grid, T = 8192, 12 heads): q, k, v,
    the raw gate logits (normaliser 16) and the output gate are strided views of one packed projection buffer,
    and RMSNorm * w * silu(gate) is fused into the operator."""
    from oracle import c_oracle, gla_ref
    B, H, grid = 2, 12, (64, 128)
    T, D = grid[0] * grid[1], 12 * 64
    gen = torch.Generator().manual_seed(40 + direction)
    packed = torch.randn(B, T, 5 * D, generator=gen)
    packed[..., :2 * D] *= 0.125                                  # q, k ~ N(0,1)/8
    packed = packed.half()
    w = (torch.rand(64, generator=gen) + 0.5).half()
    view = lambda i: packed[..., i * D:(i + 1) * D].unflatten(-1, (H, 64))
    q, k, v, gate, logits = (view(i) for i in range(5))
    # the reference hands its kernel fp16 log gates (vit_adapter.py:506-509 on an fp16 tensor); the kernel here
    # rounds its own logsigmoid(x)/16 to fp16 as well
    g = gla_ref.gate_from_logits(logits.float(), 16.0).half()
    o_ref, _ = c_oracle.forward(q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous(), direction=direction,
                                grid_hw=grid)
    y_ref = gla_ref.rmsnorm_swish_gate(o_ref, gate.contiguous(), w, 1e-5)
    pd = packed.cuda()
    dview = lambda i: pd[..., i * D:(i + 1) * D].unflatten(-1, (H, 64))
    ws = G.make_workspace(B, T, H, "cuda")
    y = torch.full((B, T, H, 64), float("nan"), dtype=torch.float16, device="cuda")
    G.chunk_gla_run_gated(dview(0), dview(1), dview(2), dview(4), dview(3), w.cuda(), 0.125, 1e-5, ws, y, 16.0,
                          direction=direction, grid_hw=grid)
    G.check_status(ws)
    m = gla_ref.error_metrics(y_ref, y.float().cpu())
    # the normalised output is of order one: fp16 rounding of y alone is 2^-11 relative per element
    assert m["finite"] and m["rel_l2"] <= 1.5e-3 and m["max_abs"] <= 2e-2, m


def test_matches_reference_fp64_vectors(G, golden_recurrence):
    """Vectors computed by the reference's own fp64 recurrence on its own seeded inputs (K = 64)."""
    Gd = golden_recurrence
    for gates, rel in (("weak", REL_L2), ("strong", REL_L2), ("bursts", REL_L2)):
        q, k, v, g = (torch.from_numpy(np.asarray(Gd[f"k64_{gates}_{n}"])) for n in "qkvg")
        ref = torch.from_numpy(np.asarray(Gd[f"k64_{gates}_o"]))
        got, _ = _run(G, q, k, v, g)
        from oracle import gla_ref
        m = gla_ref.error_metrics(ref, got)
        assert m["finite"] and m["rel_l2"] <= rel, (gates, m)


@pytest.mark.parametrize("gate", [10.5, 12.0])
@pytest.mark.parametrize("j", [0, 7, 23, 63])
def test_single_term_through_a_strong_gate(G, golden_recurrence, gate, j):
    """One key/value at row j read at row j+1 through a gate of -10.5 / -12 (reference exact_cases):
    within 2% of the fp64 value, as the reference demands; here it is far tighter."""
    want = torch.from_numpy(np.asarray(golden_recurrence[f"k64_hist_{gate:g}_{j}_row"]))
    T = 192
    q = torch.zeros(1, T, 1, 64, dtype=torch.float16)
    k = q.clone()
    v = torch.zeros(1, T, 1, 64, dtype=torch.float16)
    g = torch.full_like(q, -0.08)
    q[0, j + 1, 0, 0], k[0, j, 0, 0], v[0, j] = 16.0, 16.0, 4.0
    g[0, j + 1, 0, 0] = -gate
    got, _ = _run(G, q, k, v, g)
    row = got[0, j + 1, 0]
    assert torch.isfinite(got).all()
    assert ((row - want).norm() / want.norm()).item() <= 2e-3


def test_all_gates_minus_1000_is_finite_and_exact(G, golden_recurrence):
    Gd = golden_recurrence
    q, k, v = (torch.from_numpy(np.asarray(Gd[f"k64_m1000_{n}"])) for n in "qkv")
    g = torch.full_like(q, -1000.0)
    ref = torch.from_numpy(np.asarray(Gd["k64_m1000_o"]))
    got, _ = _run(G, q, k, v, g)
    from oracle import gla_ref
    m = gla_ref.error_metrics(ref, got)
    assert m["finite"] and m["rel_l2"] <= REL_L2, m


def test_subnormal_operands_on_block_boundaries(G):
    """Reference exact_cases: one factor of the product is 2^-24, the other 32768, gates -8.7 / -9.5."""
    from oracle import c_oracle
    for gate in (-8.7, -9.5):
        for row in (7, 8, 23, 24, 39, 40, 55, 56):
            q = torch.zeros(1, 128, 1, 64, dtype=torch.float16)
            k = q.clone()
            v = torch.zeros(1, 128, 1, 64, dtype=torch.float16)
            g = torch.full_like(q, gate)
            tiny_q = row % 16 == 7
            q[0, row, 0, 0] = 2.0 ** -24 if tiny_q else 32768.0
            k[0, row, 0, 0] = 32768.0 if tiny_q else 2.0 ** -24
            v[0, row] = 1.0
            ref, _ = c_oracle.forward(q, k, v, g, acc64=True)
            got, _ = _run(G, q, k, v, g)
            assert torch.isfinite(got).all()
            r, w = got[0, row, 0], ref[0, row, 0]
            assert ((r - w).norm() / w.norm()).item() <= 0.02, (gate, row)


def test_raw_logit_gates(G):
    """gk_normalizer > 0: the kernel applies logsigmoid(x)/normalizer itself."""
    from oracle import c_oracle, gla_ref
    gen = torch.Generator().manual_seed(3)
    q, k, v, _ = gla_ref.make_inputs(1, 300, 2, seed=3)
    raw = (torch.randn(1, 300, 2, 64, generator=gen) * 3).half()
    ref, _ = c_oracle.forward(q, k, v, gla_ref.gate_from_logits(raw, 16.0))
    got, _ = _run(G, q, k, v, raw, gk_normalizer=16.0)
    _check(ref, got)


def test_strided_views_of_a_packed_projection(G):
    """q, k, g, v taken as views of one [B, T, 4*H*64] buffer (no contiguous copies)."""
    from oracle import c_oracle, gla_ref
    B, T, H = 2, 200, 3
    q, k, v, g = gla_ref.make_inputs(B, T, H, seed=11)
    packed = torch.cat([x.reshape(B, T, H * 64) for x in (q, k, v, g)], dim=-1).cuda()
    views = [packed[..., i * H * 64:(i + 1) * H * 64].view(B, T, H, 64) for i in range(4)]
    assert not views[1].is_contiguous()
    ws = G.make_workspace(B, T, H, "cuda")
    o = torch.empty(B, T, H, 64, dtype=torch.float16, device="cuda")
    G.chunk_gla_run(views[0], views[1], views[2], views[3], 0.125, ws, o)
    ref, _ = c_oracle.forward(q, k, v, g)
    _check(ref, o.float().cpu())


def test_repeated_calls_are_bit_identical_and_reuse_the_workspace(G):
    from oracle import gla_ref
    q, k, v, g = (x.cuda() for x in gla_ref.make_inputs(2, 1600, 6, seed=2))
    ws = G.make_workspace(2, 1600, 6, "cuda")
    outs = []
    for _ in range(3):
        o = torch.full((2, 1600, 6, 64), float("nan"), dtype=torch.float16, device="cuda")
        G.chunk_gla_run(q, k, v, g, 0.125, ws, o, direction=2, grid_hw=(40, 40))
        outs.append(o)
    G.check_status(ws)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_fla_style_call_returns_final_state(G):
    from oracle import c_oracle, gla_ref
    q, k, v, g = gla_ref.make_inputs(1, 500, 2, seed=4)
    ref, ref_s = c_oracle.forward(q, k, v, g, output_final_state=True)
    o, s = G.chunk_gla(q.cuda(), k.cuda(), v.cuda(), g.cuda(), output_final_state=True)
    _check(ref, o.float().cpu())
    assert ((s.cpu() - ref_s).norm() / ref_s.norm()).item() < 5e-4


def test_round_trip_property_at_full_size(G):
    """Size-independent property at the benchmark shape: running the reversed scan on the
    token-reversed inputs gives the token-reversed output of the forward scan (the two runs sum
    the same products in a different order, so they agree to rounding, not bit for bit)."""
    from oracle import gla_ref
    q, k, v, g = (x.cuda() for x in gla_ref.config_inputs("c3"))
    B, T, H, _ = q.shape
    ws = G.make_workspace(B, T, H, "cuda")
    o1 = torch.empty(B, T, H, 64, dtype=torch.float16, device="cuda")
    o2 = torch.empty_like(o1)
    G.chunk_gla_run(q, k, v, g, 0.125, ws, o1, direction=0)
    G.chunk_gla_run(q.flip(1).contiguous(), k.flip(1).contiguous(), v.flip(1).contiguous(),
                    g.flip(1).contiguous(), 0.125, ws, o2, direction=1)
    G.check_status(ws)
    from oracle import gla_ref as R
    m = R.error_metrics(o1.float(), o2.flip(1).float())
    assert m["finite"] and m["rel_l2"] <= 3e-4 and m["max_abs"] <= 1e-4, m


def test_rmsnorm_gated(G):
    from oracle import gla_ref
    gen = torch.Generator().manual_seed(1)
    x = torch.randn(3, 77, 6, 64, generator=gen).half()
    g = torch.randn(3, 77, 6, 64, generator=gen).half()
    w = (torch.randn(64, generator=gen).abs() + 0.5).half()
    ref = gla_ref.rmsnorm_swish_gate(x, g, w, 1e-5)
    xd, gd, wd = x.cuda(), g.cuda(), w.cuda()
    y = torch.empty_like(xd)
    G.rmsnorm_gated(xd, gd, wd, y, 1e-5)
    m = gla_ref.error_metrics(ref, y.float().cpu())
    assert m["finite"] and m["rel_l2"] < 1e-3
    G.rmsnorm_gated(xd, gd, wd, xd, 1e-5)         # in place, as the backbone calls it
    assert torch.equal(xd, y)


def test_trt_enqueue_shape(G):
    """The plugin-shaped entry point: pointer arrays in, 0 / -1 out."""
    import ctypes
    from gtr_b200 import _lib
    from oracle import c_oracle, gla_ref
    q, k, v, g = gla_ref.make_inputs(1, 256, 2, seed=8)
    qd, kd, vd, gd = (x.cuda() for x in (q, k, v, g))
    o = torch.empty(1, 256, 2, 64, dtype=torch.float16, device="cuda")
    ws = G.make_workspace(1, 256, 2, "cuda")
    ins = (ctypes.c_void_p * 4)(qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), gd.data_ptr())
    outs = (ctypes.c_void_p * 1)(o.data_ptr())
    dims = (ctypes.c_int64 * 4)(1, 256, 2, 64)
    stream = torch.cuda.current_stream().cuda_stream
    rc = _lib.lib().gla_b200_trt_enqueue(ins, 4, outs, dims, 0.125, 0.0, 0.0, ws.data_ptr(),
                                         ws.numel() * 4, ctypes.c_void_p(stream))
    assert rc == 0
    ref, _ = c_oracle.forward(q, k, v, g)
    _check(ref, o.float().cpu())
    assert _lib.lib().gla_b200_trt_enqueue(ins, 5, outs, dims, 0.125, 0.0, 0.0, ws.data_ptr(),
                                           ws.numel() * 4, ctypes.c_void_p(stream)) == -1


@pytest.mark.parametrize("direction,grid,T", [(0, None, 300), (3, (20, 23), 460), (2, (40, 40), 1600)])
def test_fused_rmsnorm_swish_gate_epilogue(G, direction, grid, T):
    """chunk_gla_run_gated == RMSNorm(GLA) * w * silu(gate) (reference: chunk_gla_run_gated, test_gla.py:102-119)."""
    from oracle import c_oracle, gla_ref
    B, H = 2, 3
    q, k, v, g = gla_ref.make_inputs(B, T, H, seed=21 + direction)
    gen = torch.Generator().manual_seed(5)
    gate = torch.randn(B, T, H, 64, generator=gen).half()
    w = (torch.randn(64, generator=gen).abs() + 0.5).half()
    o_ref, _ = c_oracle.forward(q, k, v, g, direction=direction, grid_hw=grid)
    y_ref = gla_ref.rmsnorm_swish_gate(o_ref, gate, w, 1e-5)
    ws = G.make_workspace(B, T, H, "cuda")
    y = torch.full((B, T, H, 64), float("nan"), dtype=torch.float16, device="cuda")
    G.chunk_gla_run_gated(q.cuda(), k.cuda(), v.cuda(), g.cuda(), gate.cuda(), w.cuda(), 0.125, 1e-5, ws, y,
                          direction=direction, grid_hw=grid)
    G.check_status(ws)
    m = gla_ref.error_metrics(y_ref, y.float().cpu())
    assert m["finite"] and m["rel_l2"] <= REL_L2, m
    # unfused: plain operator followed by the standalone kernel gives the same result to rounding
    o = torch.empty_like(y)
    G.chunk_gla_run(q.cuda(), k.cuda(), v.cuda(), g.cuda(), 0.125, ws, o, direction=direction, grid_hw=grid)
    G.rmsnorm_gated(o, gate.cuda(), w.cuda(), o, 1e-5)
    m2 = gla_ref.error_metrics(y_ref, o.float().cpu())
    assert m2["finite"] and m2["rel_l2"] <= 2 * REL_L2, m2


@pytest.mark.parametrize("scale", [1.0, 0.037, 3.5, -0.25, 0.0])
def test_output_scales(G, scale):
    """Positive scales ride in q's exponent inside the kernel, zero and negative ones are multiplied in at the
    end: both must equal scale * (unscaled recurrence).  The final state never carries the scale."""
    from oracle import c_oracle, gla_ref
    q, k, v, g = gla_ref.make_inputs(2, 333, 3, seed=77)
    ref, st_ref = c_oracle.forward(q, k, v, g, scale=scale, output_final_state=True)
    got, st = _run(G, q, k, v, g, scale=scale, final=True, segments=2)
    if scale == 0.0:
        assert torch.isfinite(got).all() and float(got.abs().max()) == 0.0
    else:
        _check(ref, got)
    assert ((st - st_ref).norm() / st_ref.norm()).item() < 5e-4   # increments come from fp16 operands


@pytest.mark.parametrize("scale", [0.125, -0.5])
def test_fused_epilogue_with_scales(G, scale):
    from oracle import c_oracle, gla_ref
    B, T, H = 1, 200, 2
    q, k, v, g = gla_ref.make_inputs(B, T, H, seed=31)
    gen = torch.Generator().manual_seed(6)
    gate = torch.randn(B, T, H, 64, generator=gen).half()
    w = (torch.randn(64, generator=gen).abs() + 0.5).half()
    o_ref, _ = c_oracle.forward(q, k, v, g, scale=scale)
    y_ref = gla_ref.rmsnorm_swish_gate(o_ref, gate, w, 1e-5)
    ws = G.make_workspace(B, T, H, "cuda")
    y = torch.full((B, T, H, 64), float("nan"), dtype=torch.float16, device="cuda")
    G.chunk_gla_run_gated(q.cuda(), k.cuda(), v.cuda(), g.cuda(), gate.cuda(), w.cuda(), scale, 1e-5, ws, y)
    G.check_status(ws)
    m = gla_ref.error_metrics(y_ref, y.float().cpu())
    assert m["finite"] and m["rel_l2"] <= REL_L2, m


@pytest.mark.parametrize("direction", [0, 1])
def test_strong_gates_across_segments(G, direction):
    """Chunks on the exact-score path (decay beyond the tf32 path's range) mixed with ordinary ones, with the
    sequence cut into segments so that both passes and the look-back see them."""
    from oracle import c_oracle, gla_ref
    B, T, H = 1, 640, 2
    q, k, v, g = gla_ref.make_inputs(B, T, H, seed=41)
    g = g.clone()
    g[:, 100:260] = -2.0          # 64 tokens x -2 = e^-128 per chunk: exact path
    g[:, 400:410, :, :8] = -30.0  # a burst in a few channels
    ref, st_ref = c_oracle.forward(q, k, v, g, direction=direction, output_final_state=True)
    got, st = _run(G, q, k, v, g, direction=direction, segments=3, final=True)
    _check(ref, got)
    assert ((st - st_ref).norm() / st_ref.norm()).item() < 5e-4


def test_unsegmented_sequences_need_only_the_control_words(G):
    """One work item per sequence exchanges no states between items: 512 bytes of scratch are enough."""
    from oracle import c_oracle, gla_ref
    B, T, H = 2, 640, 3
    q, k, v, g = gla_ref.make_inputs(B, T, H, seed=51)
    ref, _ = c_oracle.forward(q, k, v, g)
    ws = torch.zeros(128, dtype=torch.float32, device="cuda")
    o = torch.full((B, T, H, 64), float("nan"), dtype=torch.float16, device="cuda")
    G.chunk_gla_run(q.cuda(), k.cuda(), v.cuda(), g.cuda(), 0.125, ws, o, segments=T)
    G.check_status(ws)
    _check(ref, o.float().cpu())
    with pytest.raises(Exception):      # three segments per sequence do not fit in it
        G.chunk_gla_run(q.cuda(), k.cuda(), v.cuda(), g.cuda(), 0.125, ws, o, segments=4)


def test_bounded_waits_time_out_cleanly(G):
    """A wait that nothing satisfies gives up after its limit, sets the status word, and the context
    stays usable (no trap, no hang): the operator runs correctly right afterwards."""
    import ctypes
    from gtr_b200 import _lib
    from oracle import c_oracle, gla_ref
    ws = G.make_workspace(1, 256, 2, "cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = _lib.lib().gla_b200_selftest_wait_timeout(ws.data_ptr(), ws.numel() * 4, 20000, stream)   # 20 ms
    assert rc == 0
    with pytest.raises(_lib.GlaError) as err:
        G.check_status(ws)
    assert err.value.code == _lib.ERR_TIMEOUT
    assert int(ws.view(torch.int32)[2].item()) == 1
    q, k, v, g = gla_ref.make_inputs(1, 256, 2, seed=1)
    o = torch.empty(1, 256, 2, 64, dtype=torch.float16, device="cuda")
    G.chunk_gla_run(q.cuda(), k.cuda(), v.cuda(), g.cuda(), 0.125, ws, o)
    G.check_status(ws)                                     # cleared by the new launch
    ref, _ = c_oracle.forward(q, k, v, g)
    _check(ref, o.float().cpu())


# ---------------------------------------------------------------------------------------------------------
# K = 32 key heads, V = 64: the reference extension's only shape (gla_chunk.cuh:14-16) and the released models'.

def test_k32_matches_reference_fp64_vectors(G, golden_recurrence):
    """The reference's own fp64 recurrence on its own seeded inputs at its own head size."""
    from oracle import gla_ref
    Gd = golden_recurrence
    for gates in ("weak", "strong", "bursts"):
        q, k, v, g = (torch.from_numpy(np.asarray(Gd[f"k32_{gates}_{n}"])) for n in "qkvg")
        assert q.shape[-1] == 32 and v.shape[-1] == 64
        ref = torch.from_numpy(np.asarray(Gd[f"k32_{gates}_o"]))
        got, _ = _run(G, q, k, v, g)
        m = gla_ref.error_metrics(ref, got)
        assert m["finite"] and m["rel_l2"] <= REL_L2, (gates, m)


@pytest.mark.parametrize("gate", [10.5, 12.0])
@pytest.mark.parametrize("j", [0, 7, 23, 63])
def test_k32_single_term_through_a_strong_gate(G, golden_recurrence, gate, j):
    want = torch.from_numpy(np.asarray(golden_recurrence[f"k32_hist_{gate:g}_{j}_row"]))
    T = 192
    q = torch.zeros(1, T, 1, 32, dtype=torch.float16)
    k = q.clone()
    v = torch.zeros(1, T, 1, 64, dtype=torch.float16)
    g = torch.full_like(q, -0.08)
    q[0, j + 1, 0, 0], k[0, j, 0, 0], v[0, j] = 16.0, 16.0, 4.0
    g[0, j + 1, 0, 0] = -gate
    got, _ = _run(G, q, k, v, g)
    assert torch.isfinite(got).all()
    row = got[0, j + 1, 0]
    assert ((row - want).norm() / want.norm()).item() <= 0.02


def test_k32_all_gates_minus_1000(G, golden_recurrence):
    Gd = golden_recurrence
    q, k, v = (torch.from_numpy(np.asarray(Gd[f"k32_m1000_{n}"])) for n in "qkv")
    ref = torch.from_numpy(np.asarray(Gd["k32_m1000_o"]))
    got, _ = _run(G, q, k, v, torch.full_like(q, -1000.0))
    from oracle import gla_ref
    m = gla_ref.error_metrics(ref, got)
    assert m["finite"] and m["rel_l2"] <= 2e-3, m


@pytest.mark.parametrize("direction,grid,segments", [(0, (1, 700), 0), (1, (25, 28), 3), (2, (25, 28), 0),
                                                     (3, (25, 28), 2), (3, (40, 40), 0)])
def test_k32_scan_orders_segments_and_states(G, direction, grid, segments):
    from oracle import c_oracle, gla_ref
    B, H = 2, 3
    T = grid[0] * grid[1]
    q, k, v, g = gla_ref.make_inputs(B, T, H, K=32, seed=30 + direction)
    s0 = torch.randn(B, H, 32, 64, generator=torch.Generator().manual_seed(3))
    ref, ref_s = c_oracle.forward(q, k, v, g, direction=direction, grid_hw=grid, initial_state=s0,
                                  output_final_state=True)
    got, got_s = _run(G, q, k, v, g, direction=direction, grid_hw=grid, segments=segments, s0=s0, final=True)
    _check(ref, got, relative_abs=True)
    assert got_s.shape == (B, H, 32, 64) and torch.isfinite(got_s).all()
    assert ((got_s - ref_s).norm() / ref_s.norm()).item() < 5e-4


def test_k32_released_model_call(G):
    """What a released GTR block hands the operator (dim 192, 3 heads: q, k and the raw gate logits 32 wide, v and
    the output gate 64 wide, all views of one packed projection), with the fused RMSNorm * w * silu(gate)."""
    from oracle import c_oracle, gla_ref
    B, H, grid, direction = 2, 3, (40, 40), 2
    T = 1600
    gen = torch.Generator().manual_seed(77)
    widths = (H * 32, H * 32, H * 64, H * 64, H * 32)             # q, k, v, output gate, gate logits
    packed = torch.randn(B, T, sum(widths), generator=gen)
    packed[..., :2 * H * 32] *= 0.18
    packed = packed.half()
    w = (torch.rand(64, generator=gen) + 0.5).half()

    def views(t):
        out, at = [], 0
        for wd in widths:
            out.append(t[..., at:at + wd].unflatten(-1, (H, -1)))
            at += wd
        return out

    q, k, v, gate, logits = views(packed)
    g = gla_ref.gate_from_logits(logits.float(), 16.0).half()
    o_ref, _ = c_oracle.forward(q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous(), direction=direction,
                                grid_hw=grid)
    y_ref = gla_ref.rmsnorm_swish_gate(o_ref, gate.contiguous(), w, 1e-5)
    dq, dk, dv, dgate, dlogits = views(packed.cuda())
    ws = G.make_workspace(B, T, H, "cuda")
    y = torch.full((B, T, H, 64), float("nan"), dtype=torch.float16, device="cuda")
    G.chunk_gla_run_gated(dq, dk, dv, dlogits, dgate, w.cuda(), 32 ** -0.5, 1e-5, ws, y, 16.0, direction=direction,
                          grid_hw=grid)
    G.check_status(ws)
    m = gla_ref.error_metrics(y_ref, y.float().cpu())
    assert m["finite"] and m["rel_l2"] <= 1.5e-3, m


def test_stream_probe_reports_a_plausible_rate(G):
    """The loader-only diagnostic runs, none of its bounded waits gives up, and the rate is that of a B200's memory."""
    for ctas, tiles in ((144, 4), (96, 3)):
        r = G.stream_probe(ctas=ctas, tiles=tiles, chunks=33)
        assert r["bytes"] == ctas * 33 * tiles * 8192
        assert 500.0 < r["GBs"] < 9000.0, r


@pytest.mark.parametrize("B,H,T,direction,grid", [
    (1, 1, 16384, 0, None),          # one long sequence: many segments, a look-back over many aggregates
    (1, 2, 12000, 3, (100, 120)),    # the same on a reversed column scan with a ragged last chunk
    (40, 8, 100, 1, None),           # more sequences than SMs, two chunks each: several work items per CTA
    (25, 4, 2000, 2, (40, 50)),      # segmented sequences and several work items per CTA (pre-pass and output pass each)
    (3, 5, 1000, 0, None),           # odd counts
])
def test_work_decompositions(G, B, H, T, direction, grid):
    """Shapes that drive the work decomposition to its corners, with incoming and outgoing states."""
    from oracle import c_oracle, gla_ref
    q, k, v, g = gla_ref.make_inputs(B, T, H, seed=B + T)
    s0 = torch.randn(B, H, 64, 64, generator=torch.Generator().manual_seed(T)) * 0.5
    ref, ref_s = c_oracle.forward(q, k, v, g, direction=direction, grid_hw=grid, initial_state=s0,
                                  output_final_state=True)
    got, got_s = _run(G, q, k, v, g, direction=direction, grid_hw=grid, s0=s0, final=True)
    _check(ref, got, relative_abs=True)
    assert torch.isfinite(got_s).all()
    assert ((got_s - ref_s).norm() / ref_s.norm()).item() < 5e-4


@pytest.mark.parametrize("B,H,T,direction,grid,K", [
    (2, 8, 64 * 40 + 17, 0, None, 64),         # 16 sequences on 148 SMs: nine CTAs each, ten unequal segments
    (2, 8, 2560, 3, (40, 64), 64),             # the same count on a reversed column scan
    (1, 70, 64 * 13, 1, None, 64),             # two CTAs per sequence: three segments, reversed
    (4, 12, 15 * 87, 2, (15, 87), 32),         # three CTAs per sequence, K = 32, ragged column scan (T = 1305)
    (1, 37, 64 * 24, 0, None, 64),             # four CTAs per sequence
    (13, 12, 2078, 1, None, 64),               # more sequences than CTAs: two relayed halves, no pre-pass, reversed
    (10, 16, 48 * 48, 3, (48, 48), 32),        # the same in thirds, K = 32, reversed column scan
    (8, 12, 64 * 30 + 7, 0, None, 64),         # 96 sequences: the second and third thirds wait for the first
])
def test_staggered_segment_plans(G, B, H, T, direction, grid, K):
    """Few sequences: a short first segment that runs at once and hands its state on, pre-passed middle segments, a
    last segment taken by the first free CTA.  Many sequences: equal segments that hand their state on, no pre-pass.
    (Automatic segmentation, with incoming and outgoing states.)"""
    from oracle import c_oracle, gla_ref
    q, k, v, g = gla_ref.make_inputs(B, T, H, K=K, seed=B + T + K)
    s0 = torch.randn(B, H, K, 64, generator=torch.Generator().manual_seed(T)) * 0.5
    ref, ref_s = c_oracle.forward(q, k, v, g, direction=direction, grid_hw=grid, initial_state=s0,
                                  output_final_state=True)
    got, got_s = _run(G, q, k, v, g, direction=direction, grid_hw=grid, s0=s0, final=True)
    _check(ref, got, relative_abs=True)
    assert torch.isfinite(got_s).all()
    assert ((got_s - ref_s).norm() / ref_s.norm()).item() < 5e-4
    again, _ = _run(G, q, k, v, g, direction=direction, grid_hw=grid, s0=s0, final=True)
    # which CTA takes the last segment, and whether a look-back finds a ready-made state or sums the pieces itself,
    # varies from run to run: the results agree to the rounding of the fp32 state sums
    assert (got - again).abs().max().item() <= 1e-3 * ref.abs().max().item()


def test_many_launches_never_reach_the_wait_limit(G):
    """The barrier protocol under the timing the staggered plan creates (pre-passes next to output passes, tiles that
    come in late): 3000 launches of the benchmark's shape, the status word read after every one.  With two-deep rings
    for the barriers the three teams share, about one launch in a hundred ran into the bounded waits here."""
    from oracle import gla_ref
    q, k, v, g = (x.cuda() for x in gla_ref.config_inputs("c3"))
    B, T, H, _ = q.shape
    ws = G.make_workspace(B, T, H, "cuda")
    o = torch.empty(B, T, H, 64, dtype=torch.float16, device="cuda")
    status = ws.view(torch.int32)
    sets = [(q, k, v, g), tuple(x.clone() for x in (q, k, v, g))]
    for it in range(3000):
        G.chunk_gla_run(*sets[it % 2], 0.125, ws, o, direction=it % 4, grid_hw=(80, 80), wait_limit=100000)
        torch.cuda.synchronize()
        assert int(status[1]) == 0, f"launch {it}: a bounded wait expired (status {int(status[1])})"


def test_packed_variable_length_sequences(G):
    """cu_seqlens (the FLA convention the reference block passes through): one row, sequences back to back."""
    from oracle import c_oracle, gla_ref
    lens = [130, 1, 64, 700, 65]
    offs = [0]
    for n in lens:
        offs.append(offs[-1] + n)
    H = 3
    q, k, v, g = gla_ref.make_inputs(1, offs[-1], H, seed=21)
    s0 = torch.randn(len(lens), H, 64, 64, generator=torch.Generator().manual_seed(5)) * 0.5
    o, s = G.chunk_gla(q.cuda(), k.cuda(), v.cuda(), g.cuda(), initial_state=s0.cuda(), output_final_state=True,
                       cu_seqlens=torch.tensor(offs, dtype=torch.int32))
    torch.cuda.synchronize()
    assert s.shape == (len(lens), H, 64, 64)
    for i, (a, b) in enumerate(zip(offs, offs[1:])):
        ref, ref_s = c_oracle.forward(q[:, a:b].contiguous(), k[:, a:b].contiguous(), v[:, a:b].contiguous(),
                                      g[:, a:b].contiguous(), initial_state=s0[i:i + 1], output_final_state=True)
        _check(ref, o[:, a:b].float().cpu(), relative_abs=True)
        assert ((s[i:i + 1].cpu() - ref_s).norm() / ref_s.norm()).item() < 5e-4
    with pytest.raises(ValueError):
        G.chunk_gla(q.cuda(), k.cuda(), v.cuda(), g.cuda(), cu_seqlens=[0, 10, 5, offs[-1]])


def test_short_sequences_and_decoding_with_a_carried_state(G):
    """The block's `fused_recurrent` call (at most 64 tokens, state cached between calls): pieces of a sequence run one
    after the other with the state handed on give the outputs and the final state of the whole sequence."""
    from oracle import c_oracle, gla_ref
    H, T = 2, 130
    q, k, v, g = gla_ref.make_inputs(2, T, H, seed=33)
    ref, ref_s = c_oracle.forward(q, k, v, g, output_final_state=True)
    qd, kd, vd, gd = (x.cuda() for x in (q, k, v, g))
    state, outs, a = None, [], 0
    for n in (64, 1, 1, 37, 27):
        o, state = G.fused_recurrent_gla(qd[:, a:a + n], kd[:, a:a + n], vd[:, a:a + n], gd[:, a:a + n],
                                         initial_state=state, output_final_state=True)
        outs.append(o)
        a += n
    torch.cuda.synchronize()
    _check(ref, torch.cat(outs, dim=1).float().cpu())
    assert ((state.cpu() - ref_s).norm() / ref_s.norm()).item() < 5e-4
