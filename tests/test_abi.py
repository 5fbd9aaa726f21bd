"""The C-ABI library: loads, exports every symbol the header declares, and rejects bad
arguments with the documented codes before it touches a device (runs without a GPU)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from gtr_b200 import build, _lib
    build.build()
    return _lib.lib()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "gla_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gla_b200_[a-z_0-9]+)\s*\(", text)))


def test_header_symbols_are_exported(L):
    names = declared_functions()
    assert "gla_b200_forward" in names and "gla_b200_workspace_bytes" in names
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/gla_b200.h but not exported"
    from gtr_b200 import _lib
    assert set(_lib.EXPORTS) == set(names)


def test_version_and_strerror(L):
    assert L.gla_b200_version() == 1
    assert L.gla_b200_strerror(0) == b"ok"
    for code in range(-9, 0):
        assert len(L.gla_b200_strerror(code)) > 4
    assert b"unknown" in L.gla_b200_strerror(-99)


def test_args_struct_matches_header_size():
    # 10 pointers + size_t + 18 int64 + 9 int32 + 3 float + 1 uint32, padded to 8
    from gtr_b200 import _lib
    raw = 10 * 8 + 8 + 18 * 8 + 9 * 4 + 3 * 4 + 4
    assert ctypes.sizeof(_lib.Args) == (raw + 7) // 8 * 8


def test_workspace_bytes(L):
    assert L.gla_b200_workspace_bytes(4, 6400, 12, 64, 64) > 0
    assert L.gla_b200_workspace_bytes(4, 6400, 12, 32, 64) > 0       # the reference extension's own head size
    assert L.gla_b200_workspace_bytes(4, 6400, 12, 48, 64) == 0
    assert L.gla_b200_workspace_bytes(-1, 64, 1, 64, 64) == 0
    small = L.gla_b200_workspace_bytes(1, 64, 1, 64, 64)
    big = L.gla_b200_workspace_bytes(8, 8192, 12, 64, 64)
    assert 0 < small < big
    assert small % 256 == 0 and big % 256 == 0


def _args(**kw):
    from gtr_b200 import _lib
    a = _lib.Args()
    a.B, a.T, a.H, a.K, a.V = 1, 128, 2, 64, 64
    a.scale = 0.125
    fake = 0x10000
    a.q = a.k = a.v = a.g = a.o = fake
    a.workspace, a.workspace_bytes = fake, 1 << 30
    for k, v in kw.items():
        setattr(a, k, v)
    return a


@pytest.mark.parametrize("kw,code", [
    (dict(K=48), -2), (dict(K=16), -2), (dict(V=128), -2), (dict(V=32), -2), (dict(B=-1), -2),
    (dict(direction=4), -4), (dict(direction=-1), -4),
    (dict(direction=2), -2),                       # column scan without a grid
    (dict(grid_h=10, grid_w=10), -2),              # grid does not cover T
    (dict(q=None), -1), (dict(o=None), -1),
    (dict(q=0x10008), -3),                         # misaligned
    (dict(segments=-1), -9),
    (dict(gk_normalizer=-1.0), -9),
    (dict(scale=float("nan")), -9),
])
def test_forward_rejects_bad_arguments_without_a_device(L, kw, code):
    a = _args(**kw)
    assert L.gla_b200_forward(ctypes.byref(a), None) == code


def test_forward_null_args_and_empty_problem(L):
    assert L.gla_b200_forward(None, None) == -1
    a = _args(T=0)
    assert L.gla_b200_forward(ctypes.byref(a), None) == 0          # nothing to do, nothing launched
    a = _args(B=0)
    assert L.gla_b200_forward(ctypes.byref(a), None) == 0


def test_bad_strides(L):
    from gtr_b200 import _lib
    a = _args()
    a.q_stride = (ctypes.c_int64 * 3)(128 * 2 * 64, 2 * 64 + 4, 64)   # token stride not a multiple of 8
    assert L.gla_b200_forward(ctypes.byref(a), None) == -3
    a = _args()
    a.q_stride = (ctypes.c_int64 * 3)(128 * 2 * 64, 2 * 64, 32)       # heads overlap
    assert L.gla_b200_forward(ctypes.byref(a), None) == -9


def test_rmsnorm_and_enqueue_argument_checks(L):
    assert L.gla_b200_rmsnorm_gated(None, None, None, None, 0, 64, 1e-5, None) == 0
    assert L.gla_b200_rmsnorm_gated(None, None, None, None, 4, 64, 1e-5, None) == -1
    assert L.gla_b200_rmsnorm_gated(0x100, 0x100, 0x100, 0x100, 4, 32, 1e-5, None) == -2
    assert L.gla_b200_trt_enqueue(None, 4, None, None, 1.0, 0.0, 0.0, None, 0, None) == -1
    # a NULL workspace means the library's built-in scratch array on the current device: without a device the
    # lookup fails with a CUDA error, with one it reports that array's status word
    import torch
    rc = L.gla_b200_check_status(None, None)
    assert rc in ((0, -8) if torch.cuda.is_available() else (-7, -6))


def test_python_front_end_rejects_cpu_tensors():
    import torch
    import gtr_b200
    q = torch.zeros(1, 64, 1, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA"):
        gtr_b200.chunk_gla_run(q, q, q, q, 0.125, torch.zeros(16), q)
    with pytest.raises(ValueError):
        gtr_b200.ops._direction_id("diagonal")


def test_backward_args_struct_and_argument_checks(L):
    """gla_b200_bwd_args as ctypes sees it: nine tensor pointers, three state pointers, workspace, sizes, scale."""
    from gtr_b200 import _lib
    assert ctypes.sizeof(_lib.BwdArgs) == 13 * 8 + 8 + 5 * 4 + 4
    per = 4 * 6400 * 12 * 64 * 4
    need = L.gla_b200_backward_workspace_bytes(4, 6400, 12, 64, 64)
    assert need >= 2 * per + 4 * 12 * 64 * 4                  # the two product arrays and the last-token term
    assert need <= 2 * per + (64 << 20)                       # plus per-segment states: a few MB
    many = L.gla_b200_backward_workspace_bytes(32, 2048, 12, 64, 64)     # many sequences: no segments
    assert many < 2 * (32 * 2048 * 12 * 64 * 4) + (1 << 20)
    assert L.gla_b200_backward_workspace_bytes(4, 6400, 12, 48, 64) == 0
    assert L.gla_b200_backward(None, None) == -1
    a = _lib.BwdArgs()
    a.B, a.T, a.H, a.K, a.V = 1, 64, 1, 64, 32
    assert L.gla_b200_backward(ctypes.byref(a), None) == -2
    a.V = 64
    assert L.gla_b200_backward(ctypes.byref(a), None) == -1   # pointers missing
    a.T = 0
    assert L.gla_b200_backward(ctypes.byref(a), None) == 0    # an empty problem is a no-op
    fake = 0x10000
    a.T = 64
    a.q = a.k = a.v = a.g = a.d_o = a.dq = a.dk = a.dv = a.dg = fake
    a.q = fake + 2
    assert L.gla_b200_backward(ctypes.byref(a), None) == -3   # misaligned
    a.q = fake
    assert L.gla_b200_backward(ctypes.byref(a), None) == -5   # no workspace
