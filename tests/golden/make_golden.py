"""Generate tests/golden/*.npz by running the reference's OWN CPU code for the GLA path.

Only runs where the reference checkout is present (pass its root as argv[1]); the produced
vectors are committed so that tests never need the checkout.

What is executed from the reference (imported, never copied):
  * engine/gtr/backbone/csrc/test_gla.py : `_inputs` (seeded input generator, gates "weak",
    "strong", "bursts"), `_blank` and `_recurrence_fp64` (float64 token recurrence).
    The module imports a CUDA extension and Triton kernels at the top, so stand-in modules
    are registered for `gla_torch_ext`, `fla.ops.gla` and `fla.modules` first; none of their
    attributes is called except the constants kK / kV.
  * engine/gtr/backbone/vit_adapter_spatial_swiglu.py : `_apply_bid_scan` is applied to an
    index sequence to record the token order each of the first four layers sees.

    python tests/golden/make_golden.py /path/to/GTR
"""
from __future__ import annotations

import importlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


class _Anything(types.ModuleType):
    """Stand-in module: any attribute that was not given resolves to a do-nothing callable."""

    def __getattr__(self, item):
        if item.startswith("__"):
            raise AttributeError(item)
        return lambda *a, **k: None


def _stub(name, **attrs):
    m = _Anything(name)
    m.__dict__.update(attrs)
    sys.modules[name] = m
    if "." in name:
        parent, child = name.rsplit(".", 1)
        if parent in sys.modules:
            setattr(sys.modules[parent], child, m)
    return m


def load_reference_test_module(ref_root: str, K: int, V: int = 64):
    for name in ("test_gla", "gla_torch_ext"):
        sys.modules.pop(name, None)
    _stub("gla_torch_ext", kK=K, kV=V, kBT=64)
    if "fla" not in sys.modules:
        _stub("fla")
        _stub("fla.ops")
        _stub("fla.ops.gla", chunk_gla=None)
        _stub("fla.modules", FusedRMSNormGated=None)
    sys.path.insert(0, os.path.join(ref_root, "engine/gtr/backbone/csrc"))
    try:
        mod = importlib.import_module("test_gla")
    finally:
        sys.path.pop(0)
    mod.DEVICE = "cpu"
    return mod


def recurrence_cases(ref_root: str):
    out = {}
    for K in (64, 32):
        ref = load_reference_test_module(ref_root, K)
        for gates, (B, T, H) in (("weak", (1, 130, 2)), ("strong", (1, 70, 1)), ("bursts", (1, 70, 1))):
            q, k, v, g = ref._inputs(B, T, H, seed=0, gates=gates)
            o = ref._recurrence_fp64(q, k, v, g)
            tag = f"k{K}_{gates}"
            for n, x in (("q", q), ("k", k), ("v", v), ("g", g)):
                out[f"{tag}_{n}"] = x.numpy()
            out[f"{tag}_o"] = o.float().numpy()
        # single-term constructions of the reference's exact_cases(): one key/value at row j,
        # read at row j+1 through a strong gate
        ref.T_EXACT = 192
        for gate in (-10.5, -12.0):
            for j in (0, 7, 23, 63):
                q, k, v, g = ref._blank(-0.08)
                q[0, j + 1, 0, 0], k[0, j, 0, 0], v[0, j] = 16.0, 16.0, 4.0
                g[0, j + 1, 0, 0] = gate
                o = ref._recurrence_fp64(q, k, v, g)
                tag = f"k{K}_hist_{abs(gate):g}_{j}"
                out[f"{tag}_row"] = o[0, j + 1, 0].float().numpy()
        # all gates -1000: every output row is its own q.k product only
        torch.manual_seed(0)
        ref.T_EXACT = 130
        q, k, v, g = ref._blank(-1000.0)
        q.normal_(), k.normal_(), v.normal_()
        o = ref._recurrence_fp64(q, k, v, g)
        for n, x in (("q", q), ("k", k), ("v", v)):
            out[f"k{K}_m1000_{n}"] = x.numpy()
        out[f"k{K}_m1000_o"] = o.float().numpy()
    return out


def scan_order_cases(ref_root: str):
    """Token order seen by blocks 0..3 of the CLS-free backbone on a square grid."""
    for name in [n for n in sys.modules if n == "fla" or n.startswith("fla.")]:
        if isinstance(sys.modules[name], _Anything):
            del sys.modules[name]          # the backbone imports the real flash-linear-attention
    sys.path.insert(0, ref_root)
    for name in ("faster_coco_eval", "faster_coco_eval.core", "faster_coco_eval.core.mask", "calflops"):
        if name not in sys.modules:
            _stub(name, COCO=object, COCOeval_faster=object, calculate_flops=None)
    try:
        mod = importlib.import_module("engine.gtr.backbone.vit_adapter_spatial_swiglu")
    finally:
        sys.path.pop(0)
    cls = mod.VisionTransformerSpatialSwiGLU
    fake = types.SimpleNamespace(if_quad_dir=True)
    out = {}
    for gs in (4, 6):
        x = torch.arange(gs * gs, dtype=torch.float32).view(1, gs * gs, 1)
        orders = [x.flatten().long().numpy().copy()]
        for layer in range(3):
            x = cls._apply_bid_scan(fake, x, layer)
            orders.append(x.flatten().long().numpy().copy())
        out[f"order_gs{gs}"] = np.stack(orders)   # [4, L]: order seen by block 0,1,2,3
    return out


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python make_golden.py <path to a checkout of the GTR reference>")
    ref_root = sys.argv[1]
    np.savez_compressed(os.path.join(HERE, "recurrence_fp64.npz"), **recurrence_cases(ref_root))
    try:
        np.savez_compressed(os.path.join(HERE, "scan_order.npz"), **scan_order_cases(ref_root))
    except Exception as e:  # the backbone module has heavier imports; report, do not hide
        print("scan-order fixture not generated:", repr(e))
        raise


if __name__ == "__main__":
    main()
