"""CPU oracle for the gradient of the gated-linear-attention operator.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package may import this module.

The GTR reference trains through the third-party FLA operator (``fla.ops.gla.chunk_gla`` /
``fused_recurrent_gla``, flash-linear-attention pinned 0.5.0 by the reference's requirements.txt:9;
call sites engine/gtr/backbone/vit_adapter.py:441,560-568); its own CUDA extension is forward-only.
FLA's source is not part of the reference tree, so this file restates the published recurrence

    S_t = exp(g_t)[:, None] * S_{t-1} + k_t v_t^T ,   o_t = scale * q_t^T S_t

and differentiates it by hand, token by token:

    dS_t  = exp(g_{t+1})[:, None] * dS_{t+1} + scale * q_t do_t^T          (dS_T starts from d final_state)
    dq_t  = scale * S_t do_t          dk_t = dS_t v_t          dv_t = dS_t^T k_t
    dG_t  = q_t * dq_t - k_t * dk_t   (+ sum_v d final_state * final_state at the last token)
    dg_t  = sum_{s >= t} dG_s         d initial_state = exp(g_1)[:, None] * dS_1

Parity pin: tests check it against autograd through the third-party
``fla.ops.gla.naive.naive_recurrent_gla`` and through ``oracle.gla_ref.recurrent_gla``'s own arithmetic
re-expressed in differentiable torch, and against the committed vectors made from the former
(tests/golden/make_golden.py).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def recurrent_gla_backward(q, k, v, g, do, scale: Optional[float] = None, initial_state=None, d_final_state=None,
                           dtype=torch.float64) -> Tuple[torch.Tensor, ...]:
    """q, k, g: [B,T,H,K]; v, do: [B,T,H,V]; states [B,H,K,V].  Returns (dq, dk, dv, dg, d_initial_state)."""
    q, k, v, g, do = (x.detach().to("cpu", dtype) for x in (q, k, v, g, do))
    B, T, H, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    S = torch.zeros(B, H, K, V, dtype=dtype) if initial_state is None else initial_state.detach().to("cpu", dtype).clone()
    dq = torch.empty_like(q)
    for t in range(T):                                       # forward sweep: the state each query saw
        S = torch.exp(g[:, t])[..., None] * S + k[:, t][..., None] * v[:, t][..., None, :]
        dq[:, t] = scale * torch.einsum("bhkv,bhv->bhk", S, do[:, t])
    dS = torch.zeros(B, H, K, V, dtype=dtype) if d_final_state is None else d_final_state.detach().to("cpu", dtype).clone()
    dG_last = (dS * S).sum(-1)                               # the final state's own dependence on the last cumulative gate
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    for t in range(T - 1, -1, -1):                           # backward sweep
        dS = dS + scale * q[:, t][..., None] * do[:, t][..., None, :]
        dk[:, t] = torch.einsum("bhkv,bhv->bhk", dS, v[:, t])
        dv[:, t] = torch.einsum("bhkv,bhk->bhv", dS, k[:, t])
        dS = torch.exp(g[:, t])[..., None] * dS
    dG = q * dq - k * dk
    if T > 0:
        dG[:, T - 1] += dG_last
    dg = dG.flip(1).cumsum(1).flip(1)
    return dq, dk, dv, dg, dS


def autograd_backward(q, k, v, g, do, scale: Optional[float] = None, initial_state=None, d_final_state=None,
                      dtype=torch.float64):
    """The same gradients by torch autograd through the plain recurrence (the checker's checker)."""
    q, k, v, g = (x.detach().to("cpu", dtype).requires_grad_(True) for x in (q, k, v, g))
    do = do.detach().to("cpu", dtype)
    B, T, H, K = q.shape
    V = v.shape[-1]
    if scale is None:
        scale = K ** -0.5
    s0 = torch.zeros(B, H, K, V, dtype=dtype) if initial_state is None else initial_state.detach().to("cpu", dtype)
    s0 = s0.clone().requires_grad_(True)
    S = s0
    loss = torch.zeros((), dtype=dtype)
    for t in range(T):
        S = torch.exp(g[:, t])[..., None] * S + k[:, t][..., None] * v[:, t][..., None, :]
        loss = loss + (scale * torch.einsum("bhkv,bhk->bhv", S, q[:, t]) * do[:, t]).sum()
    if d_final_state is not None:
        loss = loss + (S * d_final_state.detach().to("cpu", dtype)).sum()
    grads = torch.autograd.grad(loss, (q, k, v, g, s0))
    return grads
