"""ctypes front end of oracle/gla_oracle.c (the fast CPU recurrence).  Test infrastructure only."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build as _build
from .gla_ref import direction_id, scan_order

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_build.build())
        _lib.gla_oracle_forward.restype = ctypes.c_int
        _lib.gla_oracle_threads.restype = ctypes.c_int
    return _lib


def threads() -> int:
    return int(lib().gla_oracle_threads())


def _f32(x):
    return x.detach().to("cpu", torch.float32).contiguous()


def forward(q, k, v, g, scale: Optional[float] = None, initial_state=None,
            output_final_state: bool = False, direction=0, grid_hw=None, acc64: bool = False):
    """fp32 (or fp64-accumulated) recurrence over [B,T,H,*] tensors; returns (o fp32, final state or None)."""
    q, k, v, g = map(_f32, (q, k, v, g))
    B, T, H, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    o = torch.empty(B, T, H, V, dtype=torch.float32)
    s0 = _f32(initial_state) if initial_state is not None else None
    sT = torch.empty(B, H, K, V, dtype=torch.float32) if output_final_state else None
    d = direction_id(direction)
    perm = None
    if d != 0:
        hg, wg = grid_hw if grid_hw is not None else (1, T)
        assert hg * wg == T
        perm = scan_order(d, hg, wg).to(torch.int32).contiguous()
    p = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)
    rc = lib().gla_oracle_forward(p(q), p(k), p(v), p(g), p(o), p(s0), p(sT), B, T, H, K, V,
                                  ctypes.c_float(scale), p(perm), int(acc64))
    if rc != 0:
        raise ValueError("gla_oracle_forward rejected its arguments")
    return o, sT
