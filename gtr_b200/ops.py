"""Python face of the B200 GLA operator (forward, and its gradient for training).

Two call styles are kept so the operator drops in where the reference calls its own:

* the extension style of the reference's ``gla_torch_ext`` module
  (engine/gtr/backbone/csrc/gla_torch_ext.cu:263-293): ``chunk_gla_run``,
  ``chunk_gla_run_gated``, ``chunk_gla_with_ws``, ``workspace_floats``, ``make_workspace``,
  ``rmsnorm_gated`` and the constants ``kK``, ``kV``, ``kBT`` -- caller-owned workspace and
  output, nothing allocated, returns None;
* the FLA style the backbone falls back to (engine/gtr/backbone/vit_adapter.py:566-568):
  ``chunk_gla(q, k, v, g, scale=None, initial_state=None, output_final_state=False)``
  returning ``(o, final_state)``.

Both take two extra keywords the reference expresses by physically permuting tokens between
blocks (engine/gtr/backbone/vit_adapter_spatial_swiglu.py:88-94): ``direction`` (0 row, 1 row
reversed, 2 column, 3 column reversed; or the names) and ``grid_hw``.  Inputs and outputs
always stay in canonical token order.

Everything here runs through libgla_b200.so; there is no PyTorch or CPU fallback.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib

kK = 64                 # widest key head; SUPPORTED_K lists every key head size served
kV = 64
kBT = 64
SUPPORTED_K = (32, 64)  # the reference extension's own head is K = 32 (gla_chunk.cuh:14); its FLA path takes any K

DIRECTIONS = ("row", "row_rev", "col", "col_rev")


def _direction_id(direction) -> int:
    if isinstance(direction, str):
        if direction not in DIRECTIONS:
            raise ValueError(f"direction must be one of {DIRECTIONS} or 0..3, got {direction!r}")
        return DIRECTIONS.index(direction)
    return int(direction)


def _check_tensor(x: torch.Tensor, name: str, last: int, like: Optional[torch.Tensor] = None) -> None:
    if not isinstance(x, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not x.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if x.dtype != torch.float16:
        raise RuntimeError(f"{name} must be float16, got {x.dtype}")
    if x.dim() != 4:
        raise RuntimeError(f"{name} must be [B, T, H, D], got {tuple(x.shape)}")
    if x.shape[-1] != last:
        raise RuntimeError(f"{name}: last dim must be {last}, got {x.shape[-1]}")
    if x.numel() and x.stride(-1) != 1:
        raise RuntimeError(f"{name}: innermost dimension must be dense")
    if like is not None and (x.shape[:3] != like.shape[:3] or x.device != like.device):
        raise RuntimeError(f"{name}: shape/device {tuple(x.shape)}/{x.device} does not match q "
                           f"{tuple(like.shape)}/{like.device}")


def _strides(x: torch.Tensor):
    return (ctypes.c_int64 * 3)(x.stride(0), x.stride(1), x.stride(2))


def workspace_bytes(B: int, T: int, H: int) -> int:
    """Bytes of scratch one forward of this shape needs (reference: workspace_floats)."""
    return int(_lib.lib().gla_b200_workspace_bytes(B, T, H, kK, kV))


def workspace_floats(B: int, T: int, H: int) -> int:
    return (workspace_bytes(B, T, H) + 3) // 4


def make_workspace(B: int, T: int, H: int, device) -> torch.Tensor:
    """fp32 scratch tensor for (B, T, H); reusable across calls of that shape or smaller."""
    return torch.zeros(max(workspace_floats(B, T, H), 64), dtype=torch.float32, device=device)


def _forward(q, k, v, gk, o, ws, scale, gk_normalizer, direction, grid_hw, initial_state, final_state,
             out_gate=None, rms_w=None, eps=0.0, segments=0, wait_limit=0) -> None:
    K = q.shape[-1] if isinstance(q, torch.Tensor) and q.dim() == 4 else kK
    if K not in SUPPORTED_K:
        raise RuntimeError(f"q: last dim must be one of {SUPPORTED_K}, got {K}")
    _check_tensor(q, "q", K)
    _check_tensor(k, "k", K, q)
    _check_tensor(gk, "gk", K, q)
    _check_tensor(v, "v", kV, q)
    _check_tensor(o, "o", kV, q)
    B, T, H, _ = q.shape
    a = _lib.Args()
    a.q, a.k, a.v, a.g, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), gk.data_ptr(), o.data_ptr()
    a.q_stride, a.k_stride, a.v_stride = _strides(q), _strides(k), _strides(v)
    a.g_stride, a.o_stride = _strides(gk), _strides(o)
    if out_gate is not None or rms_w is not None:
        if out_gate is None or rms_w is None:
            raise RuntimeError("the fused epilogue needs both the output gate and the RMSNorm weight")
        _check_tensor(out_gate, "g", kV, q)
        if rms_w.dtype != torch.float16 or rms_w.numel() != kV or not rms_w.is_contiguous() or rms_w.device != q.device:
            raise RuntimeError("rms_w must be a contiguous float16 vector of 64 elements on q's device")
        a.out_gate, a.rms_weight, a.rms_eps = out_gate.data_ptr(), rms_w.data_ptr(), float(eps)
        a.gate_stride = _strides(out_gate)
    for name, s in (("initial_state", initial_state), ("final_state", final_state)):
        if s is None:
            continue
        if (s.dtype != torch.float32 or tuple(s.shape) != (B, H, K, kV) or not s.is_contiguous()
                or s.device != q.device):
            raise RuntimeError(f"{name} must be a contiguous float32 [B, H, {K}, {kV}] tensor on q's device")
    a.initial_state = initial_state.data_ptr() if initial_state is not None else None
    a.final_state = final_state.data_ptr() if final_state is not None else None
    if not isinstance(ws, torch.Tensor) or not ws.is_cuda or ws.device != q.device or not ws.is_contiguous():
        raise RuntimeError("ws must be a contiguous CUDA tensor on q's device (see make_workspace)")
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel() * ws.element_size()
    a.B, a.T, a.H, a.K, a.V = B, T, H, K, kV
    if grid_hw is not None:
        a.grid_h, a.grid_w = int(grid_hw[0]), int(grid_hw[1])
    a.direction = _direction_id(direction)
    a.segments = int(segments)
    a.scale = float(scale)
    a.gk_normalizer = float(gk_normalizer)
    a.wait_limit = int(wait_limit)
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream(q.device).cuda_stream
        _lib.check(_lib.lib().gla_b200_forward(ctypes.byref(a), ctypes.c_void_p(stream)))


def chunk_gla_run(q, k, v, gk, scale, ws, o, gk_normalizer: float = 0.0, *, direction=0, grid_hw=None,
                  initial_state=None, final_state=None, segments: int = 0, wait_limit: int = 0) -> None:
    """o <- GLA(q, k, v, gk) on the current stream.  Reference: ext.chunk_gla_run (gla_torch_ext.cu:40-90)."""
    _forward(q, k, v, gk, o, ws, scale, gk_normalizer, direction, grid_hw, initial_state, final_state,
             segments=segments, wait_limit=wait_limit)


def chunk_gla_run_gated(q, k, v, gk, g, rms_w, scale, eps, ws, y, gk_normalizer: float = 0.0, *, direction=0,
                        grid_hw=None, initial_state=None, final_state=None, segments: int = 0) -> None:
    """y <- RMSNorm(GLA(q,k,v,gk)) * rms_w * silu(g).  Reference: ext.chunk_gla_run_gated (gla_torch_ext.cu:92-154)."""
    _forward(q, k, v, gk, y, ws, scale, gk_normalizer, direction, grid_hw, initial_state, final_state,
             out_gate=g, rms_w=rms_w, eps=eps, segments=segments)


def chunk_gla_with_ws(q, k, v, gk, scale, ws, **kw) -> torch.Tensor:
    """Allocates the output only.  Reference: ext.chunk_gla_with_ws (gla_torch_ext.cu:222-226)."""
    o = torch.empty(*q.shape[:3], kV, dtype=torch.float16, device=q.device)
    chunk_gla_run(q, k, v, gk, scale, ws, o, **kw)
    return o


def _sequence_bounds(cu_seqlens, B: int, T: int):
    if B != 1:
        raise ValueError("cu_seqlens needs a batch of one row, as in FLA")
    offs = [int(x) for x in (cu_seqlens.tolist() if hasattr(cu_seqlens, "tolist") else cu_seqlens)]
    if len(offs) < 2 or offs[0] != 0 or offs[-1] != T or any(b < a for a, b in zip(offs, offs[1:])):
        raise ValueError("cu_seqlens must rise from 0 to the row's length")
    return offs


def _chunk_gla_forward(q, k, v, g, scale: Optional[float] = None, initial_state: Optional[torch.Tensor] = None,
                       output_final_state: bool = False, cu_seqlens=None, *, direction=0, grid_hw=None,
                       gk_normalizer: float = 0.0, segments: int = 0) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """FLA-style call: returns (o, final_state).  Allocates output, workspace and final state.

    `cu_seqlens` (the FLA convention the reference block passes through, vit_adapter.py:448-451,566-568): a batch of
    one row holding N sequences back to back, `cu_seqlens` their N + 1 cumulative offsets.  Every sequence is one
    launch on its slice of the row (the operator takes strided views, so nothing is copied); states are [N, H, K, 64]."""
    B, T, H, K = q.shape
    if scale is None:
        scale = K ** -0.5
    o = torch.empty(B, T, H, kV, dtype=torch.float16, device=q.device)
    if cu_seqlens is not None:
        if direction != 0 or grid_hw is not None:
            raise ValueError("cu_seqlens describes plain forward scans")
        offs = _sequence_bounds(cu_seqlens, B, T)
        n = len(offs) - 1
        if initial_state is not None and initial_state.shape[0] != n:
            raise ValueError("initial_state needs one state per sequence")
        final = torch.empty(n, H, K, kV, dtype=torch.float32, device=q.device) if output_final_state else None
        ws = make_workspace(1, max(b - a for a, b in zip(offs, offs[1:])), H, q.device)
        for i, (a, b) in enumerate(zip(offs, offs[1:])):
            chunk_gla_run(q[:, a:b], k[:, a:b], v[:, a:b], g[:, a:b], scale, ws, o[:, a:b], gk_normalizer,
                          initial_state=None if initial_state is None else initial_state[i:i + 1],
                          final_state=None if final is None else final[i:i + 1], segments=segments)
        return o, final
    ws = make_workspace(B, T, H, q.device)
    final = torch.empty(B, H, K, kV, dtype=torch.float32, device=q.device) if output_final_state else None
    chunk_gla_run(q, k, v, g, scale, ws, o, gk_normalizer, direction=direction, grid_hw=grid_hw,
                  initial_state=initial_state, final_state=final, segments=segments)
    return o, final


def backward_workspace_bytes(B: int, T: int, H: int, K: int = kK) -> int:
    return int(_lib.lib().gla_b200_backward_workspace_bytes(B, T, H, K, kV))


def chunk_gla_backward(q, k, v, g, do, scale: Optional[float] = None, initial_state: Optional[torch.Tensor] = None,
                       d_final_state: Optional[torch.Tensor] = None, want_d_initial_state: bool = False):
    """Gradients of `chunk_gla` (row-major scan, log-space gates): returns (dq, dk, dv, dg, d_initial_state) with
    dq, dk, dv in fp16, dg and the state gradient in fp32.  The reference gets these from FLA's autograd
    (vit_adapter.py:441,560-568)."""
    B, T, H, K = q.shape
    if K not in SUPPORTED_K:
        raise RuntimeError(f"K must be one of {SUPPORTED_K}")
    if scale is None:
        scale = K ** -0.5
    q, k, v, g, do = (x.contiguous() for x in (q, k, v, g, do))
    for x, name in ((q, "q"), (k, "k"), (g, "g")):
        if x.dtype != torch.float16 or not x.is_cuda or tuple(x.shape) != (B, T, H, K):
            raise RuntimeError(f"{name} must be a CUDA fp16 tensor of shape [B,T,H,K]")
    for x, name in ((v, "v"), (do, "do")):
        if x.dtype != torch.float16 or not x.is_cuda or tuple(x.shape) != (B, T, H, kV):
            raise RuntimeError(f"{name} must be a CUDA fp16 tensor of shape [B,T,H,{kV}]")
    for x, name in ((initial_state, "initial_state"), (d_final_state, "d_final_state")):
        if x is not None and (x.dtype != torch.float32 or tuple(x.shape) != (B, H, K, kV) or not x.is_contiguous()):
            raise RuntimeError(f"{name} must be a contiguous fp32 tensor of shape [B,H,K,{kV}]")
    dev = q.device
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    dg = torch.empty(B, T, H, K, dtype=torch.float32, device=dev)
    dh0 = torch.empty(B, H, K, kV, dtype=torch.float32, device=dev) if want_d_initial_state else None
    if B == 0 or T == 0:
        if dh0 is not None:
            dh0.copy_(d_final_state) if d_final_state is not None else dh0.zero_()
        return dq, dk, dv, dg, dh0
    ws = torch.empty(backward_workspace_bytes(B, T, H, K), dtype=torch.uint8, device=dev)
    a = _lib.BwdArgs()
    a.q, a.k, a.v, a.g, a.d_o = (x.data_ptr() for x in (q, k, v, g, do))
    a.dq, a.dk, a.dv, a.dg = dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr()
    a.initial_state = initial_state.data_ptr() if initial_state is not None else None
    a.d_final_state = d_final_state.data_ptr() if d_final_state is not None else None
    a.d_initial_state = dh0.data_ptr() if dh0 is not None else None
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.B, a.T, a.H, a.K, a.V = B, T, H, K, kV
    a.scale = float(scale)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        _lib.check(_lib.lib().gla_b200_backward(ctypes.byref(a), ctypes.c_void_p(stream)))
    return dq, dk, dv, dg, dh0


def _scan_order(direction: int, grid_hw, T: int, device) -> torch.Tensor:
    """perm[p] = canonical (row-major) index of the token the scan reads at step p
    (vit_adapter_spatial_swiglu.py:88-94: flip after every block, transpose the grid after odd ones)."""
    hg, wg = (1, T) if grid_hw is None else (int(grid_hw[0]), int(grid_hw[1]))
    idx = torch.arange(hg * wg, device=device).reshape(hg, wg)
    if direction >= 2:
        idx = idx.t()
    perm = idx.reshape(-1)
    return perm.flip(0) if direction & 1 else perm.contiguous()


class _ChunkGLA(torch.autograd.Function):
    """`chunk_gla` with a gradient: forward and backward are both this library's kernels."""

    @staticmethod
    def forward(ctx, q, k, v, g, initial_state, scale, output_final_state, offs, segments, direction, grid_hw,
                gk_normalizer):
        o, final = _chunk_gla_forward(q, k, v, g, scale, initial_state, output_final_state, offs, direction=direction,
                                      grid_hw=grid_hw, gk_normalizer=gk_normalizer, segments=segments)
        ctx.save_for_backward(q, k, v, g, initial_state)
        ctx.scale, ctx.offs, ctx.direction, ctx.grid_hw, ctx.gk_normalizer = scale, offs, direction, grid_hw, gk_normalizer
        if final is None:
            final = q.new_empty(0, dtype=torch.float32)
            ctx.mark_non_differentiable(final)
        return o, final

    @staticmethod
    def backward(ctx, do, d_final):
        q, k, v, g, s0 = ctx.saved_tensors
        if d_final is not None and d_final.numel() == 0:
            d_final = None
        want_s0 = s0 is not None and ctx.needs_input_grad[4]
        if d_final is not None:
            d_final = d_final.float().contiguous()
        do = do.to(torch.float16)
        logits = None
        if ctx.gk_normalizer > 0.0:          # the forward kernel turned raw logits into log-space gates itself
            logits = g.float()
            g = (torch.nn.functional.logsigmoid(logits) / ctx.gk_normalizer).to(torch.float16)
        inverse = None
        if ctx.direction != 0:               # the gradient kernels walk tokens in memory order: put them in scan order
            perm = _scan_order(ctx.direction, ctx.grid_hw, q.shape[1], q.device)
            inverse = torch.empty_like(perm)
            inverse[perm] = torch.arange(perm.numel(), device=perm.device)
            q, k, v, g, do = (x.index_select(1, perm) for x in (q, k, v, g, do))
        if ctx.offs is None:
            dq, dk, dv, dg, ds0 = chunk_gla_backward(q, k, v, g, do, ctx.scale, s0, d_final, want_s0)
        else:
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            dg = torch.empty(q.shape, dtype=torch.float32, device=q.device)
            ds0 = torch.empty_like(s0) if want_s0 else None
            for i, (a, b) in enumerate(zip(ctx.offs, ctx.offs[1:])):
                part = chunk_gla_backward(q[:, a:b], k[:, a:b], v[:, a:b], g[:, a:b], do[:, a:b], ctx.scale,
                                          None if s0 is None else s0[i:i + 1].contiguous(),
                                          None if d_final is None else d_final[i:i + 1], want_s0)
                dq[:, a:b], dk[:, a:b], dv[:, a:b], dg[:, a:b] = part[:4]
                if want_s0:
                    ds0[i:i + 1] = part[4]
        if inverse is not None:
            dq, dk, dv, dg = (x.index_select(1, inverse) for x in (dq, dk, dv, dg))
        if logits is not None:               # d logsigmoid(x) / dx = sigmoid(-x)
            dg = dg * torch.sigmoid(-logits) / ctx.gk_normalizer
        return dq, dk, dv, dg.to(ctx.saved_tensors[3].dtype), ds0, None, None, None, None, None, None, None


def chunk_gla(q, k, v, g, scale: Optional[float] = None, initial_state: Optional[torch.Tensor] = None,
              output_final_state: bool = False, cu_seqlens=None, *, direction=0, grid_hw=None,
              gk_normalizer: float = 0.0, segments: int = 0) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """FLA-style call (vit_adapter.py:566-568): returns (o, final_state); `_chunk_gla_forward` documents the arguments.
    When gradients are enabled and an input requires one, the call is recorded for autograd and its backward runs
    `chunk_gla_backward` -- as FLA's operator does for the reference in training.  The gradient kernels serve the
    row-major scan with log-space gates (what FLA's signature expresses); for the other scan directions the backward
    gathers the tokens into scan order around them, and for raw gate logits it applies logsigmoid's derivative."""
    tensors = [x for x in (q, k, v, g, initial_state) if x is not None]
    if not (torch.is_grad_enabled() and any(x.requires_grad for x in tensors)):
        return _chunk_gla_forward(q, k, v, g, scale, initial_state, output_final_state, cu_seqlens, direction=direction,
                                  grid_hw=grid_hw, gk_normalizer=gk_normalizer, segments=segments)
    B, T, H, K = q.shape
    if scale is None:
        scale = K ** -0.5
    offs = None if cu_seqlens is None else _sequence_bounds(cu_seqlens, B, T)
    o, final = _ChunkGLA.apply(q, k, v, g, initial_state, float(scale), bool(output_final_state), offs, int(segments),
                               _direction_id(direction), grid_hw, float(gk_normalizer))
    return o, (final if output_final_state else None)


def fused_recurrent_gla(q, k, v, gk, scale: Optional[float] = None, initial_state: Optional[torch.Tensor] = None,
                        output_final_state: bool = False, cu_seqlens=None):
    """The call the reference block makes for sequences of at most 64 tokens and for decoding with a cached state
    (FLA's fused_recurrent_gla, vit_adapter.py:441,560-562).  The chunkwise kernel serves any length from one token
    up -- a short sequence is one ragged chunk -- and carries the state in fp32 from call to call, so this is the same
    operator under the name the block expects."""
    return chunk_gla(q, k, v, gk, scale, initial_state, output_final_state, cu_seqlens)


def check_status(ws: torch.Tensor) -> None:
    """Synchronise the current stream and raise if a bounded wait expired inside the last forward using `ws`."""
    with torch.cuda.device(ws.device):
        stream = torch.cuda.current_stream(ws.device).cuda_stream
        _lib.check(_lib.lib().gla_b200_check_status(ctypes.c_void_p(ws.data_ptr()), ctypes.c_void_p(stream)))


def stream_probe(ctas: int = 144, tiles: int = 4, chunks: int = 33, heads: int = 12, repeats: int = 5, device="cuda"):
    """What the forward kernel's loading scheme alone streams on this GPU: `ctas` CTAs, each filling a ring of five
    stages of `tiles` 64-row x 128-byte tiles by TMA from a [rows, heads, 64] fp16 tensor (one head per CTA, rows
    strided by heads * 128 B as in the operator's inputs) and handing every stage back as soon as it has landed.
    The L2 is flushed before every repeat.  Returns GB/s (best repeat, CUDA events around the launch, so start-up
    and tail are included, as they are in the operator's own timing) and microseconds."""
    dev = torch.device(device)
    with torch.cuda.device(dev):
        regions = -(-ctas // heads)
        rows = tiles * (regions + 1) * chunks * 64
        buf = torch.zeros(rows, heads, 64, dtype=torch.float16, device=dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        best = None
        for r in range(repeats + 1):
            flush.fill_(r)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _lib.check(_lib.lib().gla_b200_stream_probe(ctypes.c_void_p(buf.data_ptr()), rows, heads, ctas, tiles, chunks,
                                                        ctypes.c_void_p(status.data_ptr()), ctypes.c_void_p(stream)))
            e1.record()
            torch.cuda.synchronize(dev)
            us = e0.elapsed_time(e1) * 1e3
            if r > 0 and (best is None or us < best):
                best = us
        if int(status.item()) != 0:
            raise RuntimeError("gla_b200_stream_probe: a bounded wait gave up")
        nbytes = ctas * chunks * tiles * 8192
        return {"GBs": nbytes / best / 1e3, "us": best, "bytes": nbytes, "ctas": ctas, "tiles_per_chunk": tiles,
                "chunks_per_cta": chunks, "stages": 5}


def rmsnorm_gated(x, g, w, y, eps: float) -> None:
    """y <- x * rsqrt(mean(x^2) + eps) * w * silu(g), rows of 64.  Reference: ext.rmsnorm_gated
    (gla_torch_ext.cu:228-261; kernel gla_norm_gate.cuh:13-75).  y may alias x."""
    for t, name in ((x, "x"), (g, "g"), (y, "y")):
        if not t.is_cuda or t.dtype != torch.float16 or not t.is_contiguous() or t.shape[-1] != kV:
            raise RuntimeError(f"{name} must be a contiguous float16 CUDA tensor with last dim {kV}")
    if g.shape != x.shape or y.shape != x.shape:
        raise RuntimeError("x, g and y must have the same shape")
    if w.dtype != torch.float16 or w.numel() != kV or not w.is_contiguous() or w.device != x.device:
        raise RuntimeError("w must be a contiguous float16 vector of 64 elements on x's device")
    rows = x.numel() // kV
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream(x.device).cuda_stream
        _lib.check(_lib.lib().gla_b200_rmsnorm_gated(x.data_ptr(), g.data_ptr(), w.data_ptr(), y.data_ptr(),
                                                     rows, kV, float(eps), ctypes.c_void_p(stream)))


def swiglu_dwconv(gate: torch.Tensor, y: torch.Tensor, weight_taps: torch.Tensor, bias: Optional[torch.Tensor],
                  grid_hw: Tuple[int, int], out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = silu(gate) * (bias + depthwise 3x3 conv of y on the patch grid), tokens in [B, L, C] layout.

    The middle of the reference's SpatialSwiGLU in deploy form (vit_adapter_spatial_swiglu.py:50-60) as one kernel.
    ``weight_taps`` is the depthwise weight as fp16 [3, 3, C] (``conv.weight[:, 0].permute(1, 2, 0)``), already
    oriented for the canonical grid."""
    hg, wg = int(grid_hw[0]), int(grid_hw[1])
    for t, name in ((gate, "gate"), (y, "y")):
        if not t.is_cuda or t.dtype != torch.float16 or t.dim() != 3 or not t.is_contiguous():
            raise RuntimeError(f"{name} must be a contiguous float16 CUDA tensor [B, L, C]")
    B, L, C = y.shape
    if gate.shape != y.shape or L != hg * wg or C % 8:
        raise RuntimeError(f"gate/y shapes {tuple(gate.shape)}/{tuple(y.shape)} do not fit a {hg}x{wg} grid "
                           "(C must be a multiple of 8)")
    if weight_taps.dtype != torch.float16 or tuple(weight_taps.shape) != (3, 3, C) or not weight_taps.is_contiguous() \
            or weight_taps.device != y.device:
        raise RuntimeError("weight_taps must be a contiguous float16 [3, 3, C] tensor on y's device")
    if bias is not None and (bias.dtype != torch.float16 or bias.numel() != C or not bias.is_contiguous()
                             or bias.device != y.device):
        raise RuntimeError("bias must be a contiguous float16 vector of C elements on y's device")
    if out is None:
        out = torch.empty_like(y)
    elif out.shape != y.shape or out.dtype != torch.float16 or not out.is_contiguous() or out.device != y.device:
        raise RuntimeError("out must match y")
    with torch.cuda.device(y.device):
        stream = torch.cuda.current_stream(y.device).cuda_stream
        _lib.check(_lib.lib().gla_b200_swiglu_dwconv(gate.data_ptr(), y.data_ptr(), weight_taps.data_ptr(),
                                                     bias.data_ptr() if bias is not None else None, out.data_ptr(),
                                                     B, hg, wg, C, ctypes.c_void_p(stream)))
    return out


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """LayerNorm over the last dimension of a contiguous float16 CUDA tensor (fp32 statistics); the backbone block's
    norm1 / norm2 (vit_adapter.py:608-642) in one read and one write.  ``out`` may be ``x``."""
    if not x.is_cuda or x.dtype != torch.float16 or not x.is_contiguous():
        raise RuntimeError("x must be a contiguous float16 CUDA tensor")
    D = x.shape[-1]
    for t, name in ((weight, "weight"), (bias, "bias")):
        if t is not None and (t.dtype != torch.float16 or t.numel() != D or not t.is_contiguous() or t.device != x.device):
            raise RuntimeError(f"{name} must be a contiguous float16 vector of {D} elements on x's device")
    if out is None:
        out = torch.empty_like(x)
    elif out.shape != x.shape or out.dtype != torch.float16 or not out.is_contiguous() or out.device != x.device:
        raise RuntimeError("out must match x")
    rows = x.numel() // D if D else 0
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream(x.device).cuda_stream
        _lib.check(_lib.lib().gla_b200_layernorm(x.data_ptr(), weight.data_ptr(),
                                                 bias.data_ptr() if bias is not None else None, out.data_ptr(),
                                                 rows, D, float(eps), ctypes.c_void_p(stream)))
    return out
