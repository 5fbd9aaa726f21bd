"""CPU oracle for the gated-linear-attention (GLA) forward path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package may import this module: it exists so that tests, the smoke
check and the benchmark's CPU-baseline leg can compare the CUDA operator with a plain
restatement of the reference algorithm.

Each function names the reference code it restates (paths are relative to the GTR project
root):

* ``recurrent_gla``      engine/gtr/backbone/csrc/test_gla.py:124-132 (``_recurrence_fp64``),
                         generalised with an initial state and a final-state output as in
                         the FLA call the backbone makes (engine/gtr/backbone/vit_adapter.py:566-568).
* ``scan_order``         engine/gtr/backbone/vit_adapter_spatial_swiglu.py:88-94 and
                         engine/gtr/backbone/vit_adapter.py:798-803 (flip, then transpose the
                         square grid on odd layers), generalised to an Hg x Wg grid.
* ``gate_from_logits``   engine/gtr/backbone/vit_adapter.py:506-509 (``logsigmoid(x)/normalizer``).
* ``rmsnorm_swish_gate`` engine/gtr/backbone/csrc/test_gla.py:138-139 and
                         tensorrt_plugin/gtr_onnx_patches.py:94-96 (RMSNorm * w * silu(gate)).
* ``chunk_gla``          the 64-token chunk formulation the reference kernels implement
                         (engine/gtr/backbone/csrc/gla_chunk.cuh:718-890 state pass,
                         :343-716 output pass), written with exact fp32/fp64 arithmetic.

Parity pin: ``recurrent_gla`` is checked in tests against vectors produced by running the
reference's own ``_recurrence_fp64`` (tests/golden/make_golden.py) and against the
third-party ``fla.ops.gla.naive.naive_recurrent_gla`` (flash-linear-attention, pinned 0.5.0
by the reference's requirements.txt:9).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

DIRECTIONS = ("row", "row_rev", "col", "col_rev")
CHUNK = 64


def direction_id(direction) -> int:
    if isinstance(direction, str):
        return DIRECTIONS.index(direction)
    d = int(direction)
    if not 0 <= d < 4:
        raise ValueError(f"direction must be 0..3 or one of {DIRECTIONS}")
    return d


def scan_order(direction, hg: int, wg: int) -> torch.Tensor:
    """perm[p] = index (row-major over the hg x wg grid) of the token read at sequence step p.

    Layer i of the reference backbone sees order ``DIRECTIONS[i % 4]``: block 0 reads the
    canonical row-major sequence; after every block the sequence is flipped, and after odd
    blocks the grid is also transposed.
    """
    d = direction_id(direction)
    n = hg * wg
    idx = torch.arange(n).reshape(hg, wg)
    if d >= 2:
        idx = idx.t()
    perm = idx.reshape(-1)
    if d & 1:
        perm = perm.flip(0)
    return perm.contiguous()


def gate_from_logits(x: torch.Tensor, normalizer: float) -> torch.Tensor:
    return F.logsigmoid(x.float()) / float(normalizer)


def recurrent_gla(q, k, v, g, scale: Optional[float] = None, initial_state=None,
                  output_final_state: bool = False, dtype=torch.float32
                  ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Token-by-token recurrence.  q,k,g: [B,T,H,K]; v: [B,T,H,V]; state [B,H,K,V].

    S_t = exp(g_t)[:,None] * S_{t-1} + k_t v_t^T ;  o_t = scale * q_t^T S_t
    """
    q, k, v, g = (x.detach().to("cpu", dtype) for x in (q, k, v, g))
    B, T, H, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    S = torch.zeros(B, H, K, V, dtype=dtype)
    if initial_state is not None:
        S = initial_state.detach().to("cpu", dtype).clone()
    o = torch.empty(B, T, H, V, dtype=dtype)
    for t in range(T):
        S = g[:, t].exp().unsqueeze(-1) * S + k[:, t].unsqueeze(-1) * v[:, t].unsqueeze(-2)
        o[:, t] = scale * (q[:, t].unsqueeze(-1) * S).sum(-2)
    return o, (S if output_final_state else None)


def gla_scan(q, k, v, g, direction=0, grid_hw=None, **kw):
    """Recurrence along one of the four 2-D scan orders; output is returned in token order."""
    B, T = q.shape[:2]
    d = direction_id(direction)
    if d == 0:
        return recurrent_gla(q, k, v, g, **kw)
    if grid_hw is None:
        if d >= 2:
            raise ValueError("column scans need grid_hw")
        grid_hw = (1, T)
    hg, wg = grid_hw
    assert hg * wg == T
    perm = scan_order(d, hg, wg)
    o_p, S = recurrent_gla(q[:, perm], k[:, perm], v[:, perm], g[:, perm], **kw)
    o = torch.empty_like(o_p)
    o[:, perm] = o_p
    return o, S


def chunk_gla(q, k, v, g, scale: Optional[float] = None, initial_state=None,
              output_final_state: bool = False, dtype=torch.float32, chunk: int = CHUNK):
    """Chunkwise formulation (exact arithmetic in `dtype`), used as a second opinion and as
    the timed pure-PyTorch chunk baseline.  Inside a chunk with inclusive gate cumsum G:
        A[i,j] = sum_c q[i,c] k[j,c] exp(G[i,c]-G[j,c])   (j <= i)
        o      = scale * (A v + (q*exp(G)) S_in)
        S_out  = exp(G_last)[:,None]*S_in + (k*exp(G_last-G))^T v
    The pairwise exponent is formed before exponentiation, so any gate strength is safe.
    """
    q, k, v, g = (x.detach().to("cpu", dtype) for x in (q, k, v, g))
    B, T, H, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    S = torch.zeros(B, H, K, V, dtype=dtype)
    if initial_state is not None:
        S = initial_state.detach().to("cpu", dtype).clone()
    o = torch.empty(B, T, H, V, dtype=dtype)
    for s in range(0, T, chunk):
        e = min(T, s + chunk)
        qc, kc, vc, gc = (x[:, s:e].transpose(1, 2) for x in (q, k, v, g))  # [B,H,C,*]
        G = gc.cumsum(2)
        C = e - s
        diff = G.unsqueeze(3) - G.unsqueeze(2)                       # [B,H,i,j,K]
        mask = torch.tril(torch.ones(C, C, dtype=torch.bool))
        w = torch.where(mask[None, None, :, :, None], diff, torch.full_like(diff, -float("inf"))).exp()
        A = torch.einsum("bhic,bhjc,bhijc->bhij", qc, kc, w)
        oc = A @ vc + (qc * G.exp()) @ S
        o[:, s:e] = (scale * oc).transpose(1, 2)
        Gl = G[:, :, -1]
        S = Gl.exp().unsqueeze(-1) * S + (kc * (Gl.unsqueeze(2) - G).exp()).transpose(2, 3) @ vc
    return o, (S if output_final_state else None)


def rmsnorm_swish_gate(o, gate, w, eps: float):
    """y = o * rsqrt(mean(o^2) + eps) * w * silu(gate), computed in fp32 over the last dim."""
    o, gate, w = o.float(), gate.float(), w.float()
    return o * torch.rsqrt(o.square().mean(-1, keepdim=True) + eps) * w * F.silu(gate)


# Seeded synthetic inputs live in gtr_b200/workloads.py (shared with the benchmark); re-exported for the tests.
from gtr_b200.workloads import CONFIGS, config_inputs, make_inputs  # noqa: E402,F401


def error_metrics(ref: torch.Tensor, got: torch.Tensor):
    ref = ref.detach().double().flatten().cpu()
    got = got.detach().double().flatten().cpu()
    d = got - ref
    return dict(
        max_abs=d.abs().max().item(),
        rel_l2=(d.norm() / ref.norm().clamp_min(1e-30)).item(),
        ref_max=ref.abs().max().item(),
        finite=bool(torch.isfinite(got).all()),
        cos=F.cosine_similarity(ref, got, dim=0).item(),
    )
