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

  * engine/gtr/backbone/vit_adapter_spatial_swiglu.py : `ViTAdapterSpatialSwiGLU` itself (four blocks, dim 128,
    two heads, ffn_ratio 6, `multi_layer_same_res`), in eval mode on the CPU in fp32, once with expand_k = 1.0
    (head K = 64) and once with expand_k = 0.5 (head K = 32, what the released configs use).  Two names that the
    reference binds to Triton kernels are re-bound first, because Triton does not run on a CPU:
    `vit_adapter.chunk_gla` to the reference's own float64 recurrence (`test_gla._recurrence_fp64`), and
    `FusedRMSNormGated.forward` to x * rsqrt(mean(x^2) + eps) * w * silu(g) (what test_gla.py:138-139 and
    tensorrt_plugin/gtr_onnx_patches.py:94-96 state).  Weights are random, rounded to fp16 so that the fixture can
    store them in half the space; the fixture holds the state dict, the input and the three returned feature maps.

  * engine/gtr/backbone/csrc/test_gla.py : `_recurrence_fp64` once more, under torch autograd, for the gradients of
    the recurrence (recurrence_backward.npz; `--backward-only` regenerates just that file).

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


def backward_cases(ref_root: str):
    """Gradients of the reference's own float64 recurrence (`test_gla._recurrence_fp64`) by torch autograd: the
    reference trains through a third-party operator's autograd, so the gradient of its own statement of the
    recurrence is the vector to hold the backward kernels to."""
    out = {}
    for K in (64, 32):
        ref = load_reference_test_module(ref_root, K)
        for gates, (B, T, H) in (("weak", (1, 70, 2)), ("strong", (1, 40, 1))):
            q, k, v, g = ref._inputs(B, T, H, seed=1, gates=gates)
            do = torch.randn(v.shape, generator=torch.Generator().manual_seed(7)).to(v.dtype)
            leaves = [x.detach().double().requires_grad_(True) for x in (q, k, v, g)]
            o = ref._recurrence_fp64(*leaves)
            grads = torch.autograd.grad((o * do.double()).sum(), leaves)
            tag = f"k{K}_{gates}"
            for n, x in (("q", q), ("k", k), ("v", v), ("g", g), ("do", do)):
                out[f"{tag}_{n}"] = x.numpy()
            for n, x in zip(("dq", "dk", "dv", "dg"), grads):
                out[f"{tag}_{n}"] = x.float().numpy()
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


def backbone_cases(ref_root: str, expand_k: float):
    """Run the reference backbone on the CPU; returns {name: array} with weights (fp16), input and outputs."""
    head_k = int(128 * expand_k) // 2
    ref_test = load_reference_test_module(ref_root, head_k)      # K, V constants of its recurrence
    recurrence = ref_test._recurrence_fp64
    for name in [n for n in sys.modules if n == "fla" or n.startswith("fla.")]:
        if isinstance(sys.modules[name], _Anything):
            del sys.modules[name]
    sys.path.insert(0, ref_root)
    for name in ("faster_coco_eval", "faster_coco_eval.core", "faster_coco_eval.core.mask", "calflops"):
        if name not in sys.modules:
            _stub(name, COCO=object, COCOeval_faster=object, calculate_flops=None)
    try:
        va = importlib.import_module("engine.gtr.backbone.vit_adapter")
        mod = importlib.import_module("engine.gtr.backbone.vit_adapter_spatial_swiglu")
    finally:
        sys.path.pop(0)

    def chunk_gla_cpu(q, k, v, g, initial_state=None, output_final_state=False, cu_seqlens=None, **kw):
        assert initial_state is None and cu_seqlens is None
        return recurrence(q, k, v, g).to(q.dtype), None

    def norm_gate_cpu(self, x, g, residual=None, prenorm=False, residual_in_fp32=False):
        y = x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + self.eps)
        return y * self.weight * torch.nn.functional.silu(g)

    va.chunk_gla = chunk_gla_cpu
    va.FusedRMSNormGated.forward = norm_gate_cpu
    torch.manual_seed(0)
    model = mod.ViTAdapterSpatialSwiGLU(interaction_indexes=[1, 2, 3], embed_dim=128, num_heads=2, expand_k=expand_k,
                                        ffn_ratio=6, depth=4, multi_layer_same_res=True, skip_weights_warning=True)
    model.eval()
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for name, t in model.state_dict().items():
            if name.endswith("num_batches_tracked"):
                continue
            if name.endswith("running_var") or name.endswith("g_norm_swish_gate.weight") or ".norm.weight" in name:
                t.copy_(torch.rand(t.shape, generator=g) + 0.5)
            elif name.endswith("running_mean") or name.endswith(".bias"):
                t.copy_(torch.randn(t.shape, generator=g) * (1.0 if "gk_proj" in name else 0.1))
            t.copy_(t.half().float())                        # the fixture stores fp16
    img = torch.rand(2, 3, 192, 192, generator=g).half().float()
    with torch.no_grad():
        outs = model(img)
    tag = f"k{head_k}"
    out = {f"{tag}_img": img.half().numpy()}
    for i, o in enumerate(outs):
        out[f"{tag}_out{i}"] = o.float().numpy()
    for name, t in model.state_dict().items():
        if not name.endswith("num_batches_tracked"):
            out[f"{tag}_sd/{name}"] = t.half().numpy()
    return out


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python make_golden.py <path to a checkout of the GTR reference>")
    ref_root = sys.argv[1]
    np.savez_compressed(os.path.join(HERE, "recurrence_backward.npz"), **backward_cases(ref_root))
    if "--backward-only" in sys.argv:
        return
    np.savez_compressed(os.path.join(HERE, "recurrence_fp64.npz"), **recurrence_cases(ref_root))
    try:
        np.savez_compressed(os.path.join(HERE, "scan_order.npz"), **scan_order_cases(ref_root))
    except Exception as e:  # the backbone module has heavier imports; report, do not hide
        print("scan-order fixture not generated:", repr(e))
        raise
    bb = {}
    for expand_k in (1.0, 0.5):
        bb.update(backbone_cases(ref_root, expand_k))
    np.savez_compressed(os.path.join(HERE, "backbone_small.npz"), **bb)


if __name__ == "__main__":
    main()
