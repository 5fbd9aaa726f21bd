"""gla_b200_forward_static: the entry point for hosts that cannot allocate device memory when they
call the operator (a serving process whose pool owns the GPU, a plugin without a workspace).  Its
scratch is an array inside the library, so the caller passes inputs and outputs only.

Called through the C ABI twice in a row on different inputs and compared with the regular entry
point (which gets a caller-owned workspace): the array keeps the first call's contents, so the second
call shows that stale scratch does no harm.  The file sorts last so that a failure here cannot hide
another test's result in a run that stops at the first failure.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(_lib, q, k, v, g, o, direction, grid):
    a = _lib.Args()
    a.q, a.k, a.v, a.g, a.o = (t.data_ptr() for t in (q, k, v, g, o))
    a.B, a.T, a.H = q.shape[0], q.shape[1], q.shape[2]
    a.K = a.V = 64
    a.grid_h, a.grid_w = grid
    a.direction = direction
    a.scale = 0.125
    return a


def test_static_scratch_entry_point_matches_regular_one_twice():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import gtr_b200
    from gtr_b200 import _lib
    from oracle import gla_ref
    L = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    B, H, grid = 2, 3, (30, 32)                  # T = 960: 15 chunks, split into several segments
    T = grid[0] * grid[1]
    for call, (seed, direction) in enumerate(((11, 0), (12, 3))):
        q, k, v, g = (x.cuda() for x in gla_ref.make_inputs(B, T, H, seed=seed))
        want = torch.empty(B, T, H, 64, dtype=torch.float16, device="cuda")
        ws = gtr_b200.make_workspace(B, T, H, "cuda")
        gtr_b200.chunk_gla_run(q, k, v, g, 0.125, ws, want, direction=direction, grid_hw=grid)
        got = torch.full_like(want, float("nan"))
        a = _args(_lib, q, k, v, g, got, direction, grid)          # workspace stays NULL
        rc = L.gla_b200_forward_static(ctypes.byref(a), stream)
        assert rc == 0, L.gla_b200_strerror(rc).decode()
        torch.cuda.synchronize()
        m = gla_ref.error_metrics(want.float(), got.float())
        assert m["finite"] and m["rel_l2"] <= 1e-3 and m["max_abs"] <= 2e-3, (call, m)


def test_static_scratch_rejects_oversized_segmentation():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from gtr_b200 import _lib
    L = _lib.lib()
    B, T, H = 16, 8192, 16                       # one-chunk segments: 32768 slots of 33 KB, far beyond 24 MiB
    q = torch.zeros(B, T, H, 64, dtype=torch.float16, device="cuda")
    o = torch.empty_like(q)
    a = _args(_lib, q, q, q, q, o, 0, (0, 0))
    a.segments = 1
    rc = L.gla_b200_forward_static(ctypes.byref(a), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -10
    assert b"built-in" in L.gla_b200_strerror(rc)


def test_static_scratch_automatic_split_never_exceeds_the_array():
    """160 sequences of 100 chunks: the split the cost model would like best needs about 50 MiB of scratch; with
    the 24 MiB array the policy must settle for a coarser one and still give the regular entry point's result."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import gtr_b200
    from gtr_b200 import _lib
    from oracle import gla_ref
    L = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    B, T, H = 10, 6400, 16
    q, k, v, g = (x.cuda() for x in gla_ref.make_inputs(B, T, H, seed=5))
    want = torch.empty(B, T, H, 64, dtype=torch.float16, device="cuda")
    ws = gtr_b200.make_workspace(B, T, H, "cuda")
    gtr_b200.chunk_gla_run(q, k, v, g, 0.125, ws, want)
    got = torch.full_like(want, float("nan"))
    a = _args(_lib, q, k, v, g, got, 0, (0, 0))
    rc = L.gla_b200_forward_static(ctypes.byref(a), stream)
    assert rc == 0, L.gla_b200_strerror(rc).decode()
    torch.cuda.synchronize()
    assert L.gla_b200_check_status(None, stream) == 0
    m = gla_ref.error_metrics(want.float(), got.float())
    assert m["finite"] and m["rel_l2"] <= 1e-3 and m["max_abs"] <= 2e-3, m


def test_static_scratch_reports_a_timeout_and_the_next_call_clears_it():
    """The status word of the built-in array is read with a NULL workspace: a wait that runs out there (the
    self-test's, 20 ms) must show up, and the next forward must start from a clean status."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from gtr_b200 import _lib
    from oracle import gla_ref
    L = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.gla_b200_selftest_wait_timeout(None, 0, 20000, stream) == 0
    assert L.gla_b200_check_status(None, stream) == -8
    B, T, H = 1, 256, 2
    q, k, v, g = (x.cuda() for x in gla_ref.make_inputs(B, T, H, seed=6))
    o = torch.empty(B, T, H, 64, dtype=torch.float16, device="cuda")
    a = _args(_lib, q, k, v, g, o, 0, (0, 0))
    assert L.gla_b200_forward_static(ctypes.byref(a), stream) == 0
    assert L.gla_b200_check_status(None, stream) == 0
    assert torch.isfinite(o).all()
