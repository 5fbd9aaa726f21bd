"""ctypes binding of libgla_b200.so (the C ABI in include/gla_b200.h).

There is no fallback: if the shared library is missing or was built for another
architecture the import of any operator fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes
import os

PKG = os.path.dirname(os.path.abspath(__file__))
# GTR_B200_LIB selects another build of the same library (e.g. one compiled with different tile parameters)
LIB_PATH = os.environ.get("GTR_B200_LIB") or os.path.join(PKG, "libgla_b200.so")

OK = 0
ERR_TIMEOUT = -8


class Args(ctypes.Structure):
    """Mirror of `gla_b200_args`."""
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("g", ctypes.c_void_p),
        ("o", ctypes.c_void_p),
        ("out_gate", ctypes.c_void_p), ("rms_weight", ctypes.c_void_p),
        ("initial_state", ctypes.c_void_p), ("final_state", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
        ("q_stride", ctypes.c_int64 * 3), ("k_stride", ctypes.c_int64 * 3), ("v_stride", ctypes.c_int64 * 3),
        ("g_stride", ctypes.c_int64 * 3), ("o_stride", ctypes.c_int64 * 3), ("gate_stride", ctypes.c_int64 * 3),
        ("B", ctypes.c_int32), ("T", ctypes.c_int32), ("H", ctypes.c_int32), ("K", ctypes.c_int32),
        ("V", ctypes.c_int32),
        ("grid_h", ctypes.c_int32), ("grid_w", ctypes.c_int32),
        ("direction", ctypes.c_int32), ("segments", ctypes.c_int32),
        ("scale", ctypes.c_float), ("gk_normalizer", ctypes.c_float), ("rms_eps", ctypes.c_float),
        ("wait_limit", ctypes.c_uint32),
    ]


class BwdArgs(ctypes.Structure):
    """Mirror of `gla_b200_bwd_args`."""
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("g", ctypes.c_void_p),
        ("d_o", ctypes.c_void_p),
        ("dq", ctypes.c_void_p), ("dk", ctypes.c_void_p), ("dv", ctypes.c_void_p), ("dg", ctypes.c_void_p),
        ("initial_state", ctypes.c_void_p), ("d_final_state", ctypes.c_void_p), ("d_initial_state", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_size_t),
        ("B", ctypes.c_int32), ("T", ctypes.c_int32), ("H", ctypes.c_int32), ("K", ctypes.c_int32),
        ("V", ctypes.c_int32),
        ("scale", ctypes.c_float),
    ]


EXPORTS = (
    "gla_b200_forward", "gla_b200_workspace_bytes", "gla_b200_check_status", "gla_b200_rmsnorm_gated",
    "gla_b200_trt_enqueue", "gla_b200_strerror", "gla_b200_last_cuda_error", "gla_b200_version",
    "gla_b200_forward_static", "gla_b200_selftest_wait_timeout", "gla_b200_swiglu_dwconv", "gla_b200_layernorm",
    "gla_b200_stream_probe", "gla_b200_backward", "gla_b200_backward_workspace_bytes",
)

_lib = None


class GlaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"gla_b200 error {code}: {message}")
        self.code = code


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m gtr_b200.build` (needs nvcc, targets sm_100a). "
            "gtr_b200 has no CPU or PyTorch fallback.")
    L = ctypes.CDLL(LIB_PATH)
    L.gla_b200_forward.argtypes = [ctypes.POINTER(Args), ctypes.c_void_p]
    L.gla_b200_forward.restype = ctypes.c_int
    L.gla_b200_forward_static.argtypes = [ctypes.POINTER(Args), ctypes.c_void_p]
    L.gla_b200_forward_static.restype = ctypes.c_int
    L.gla_b200_selftest_wait_timeout.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint32, ctypes.c_void_p]
    L.gla_b200_selftest_wait_timeout.restype = ctypes.c_int
    L.gla_b200_stream_probe.argtypes = [ctypes.c_void_p, ctypes.c_int64] + [ctypes.c_int32] * 4 + [ctypes.c_void_p] * 2
    L.gla_b200_stream_probe.restype = ctypes.c_int
    L.gla_b200_backward.argtypes = [ctypes.POINTER(BwdArgs), ctypes.c_void_p]
    L.gla_b200_backward.restype = ctypes.c_int
    L.gla_b200_backward_workspace_bytes.argtypes = [ctypes.c_int32] * 5
    L.gla_b200_backward_workspace_bytes.restype = ctypes.c_size_t
    L.gla_b200_workspace_bytes.argtypes = [ctypes.c_int32] * 5
    L.gla_b200_workspace_bytes.restype = ctypes.c_size_t
    L.gla_b200_check_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    L.gla_b200_check_status.restype = ctypes.c_int
    L.gla_b200_rmsnorm_gated.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64, ctypes.c_int32, ctypes.c_float,
                                                                 ctypes.c_void_p]
    L.gla_b200_rmsnorm_gated.restype = ctypes.c_int
    L.gla_b200_swiglu_dwconv.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int32] * 4 + [ctypes.c_void_p]
    L.gla_b200_swiglu_dwconv.restype = ctypes.c_int
    L.gla_b200_layernorm.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int64, ctypes.c_int32, ctypes.c_float, ctypes.c_void_p]
    L.gla_b200_layernorm.restype = ctypes.c_int
    L.gla_b200_trt_enqueue.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int32,
                                       ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_int64),
                                       ctypes.c_float, ctypes.c_float, ctypes.c_float, ctypes.c_void_p,
                                       ctypes.c_size_t, ctypes.c_void_p]
    L.gla_b200_trt_enqueue.restype = ctypes.c_int32
    L.gla_b200_strerror.argtypes = [ctypes.c_int]
    L.gla_b200_strerror.restype = ctypes.c_char_p
    L.gla_b200_last_cuda_error.restype = ctypes.c_char_p
    L.gla_b200_version.restype = ctypes.c_int
    _lib = L
    return L


def check(code: int) -> None:
    if code == OK:
        return
    L = lib()
    msg = L.gla_b200_strerror(code).decode()
    detail = L.gla_b200_last_cuda_error().decode()
    if code in (-6, -7) and detail:
        msg = f"{msg} [{detail}]"
    raise GlaError(code, msg)
