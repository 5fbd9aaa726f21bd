"""The operator's two entry points as ``torch.library`` custom operators.

The reference registers its extension calls the same way (engine/gtr/backbone/vit_adapter.py:59-93,
``gtr::chunk_gla`` and ``gtr::chunk_gla_gated``) so that Dynamo traces through the twelve GLA calls of
the backbone instead of breaking the graph at each.  Here the operators are

    torch.ops.gtr_b200.chunk_gla(q, k, v, gk, scale, ws, out, gk_norm, direction, grid_h, grid_w)
    torch.ops.gtr_b200.chunk_gla_gated(q, k, v, gk, g, w, scale, eps, ws, out, gk_norm, direction, grid_h, grid_w)

with the reference's argument order followed by the scan order (``direction`` 0..3 and the patch grid;
``grid_h = grid_w = 0`` means one row of T tokens).  Both write ``out`` and use ``ws`` as scratch, return
nothing, and have a fake (meta) implementation, so they can be traced, exported and captured without
running.  The real implementations are the calls of ``gtr_b200.ops`` -- no fallback.
"""
from __future__ import annotations

import torch

from . import ops

_NS = "gtr_b200"


def _grid(grid_h: int, grid_w: int):
    return (grid_h, grid_w) if grid_h > 0 and grid_w > 0 else None


@torch.library.custom_op(f"{_NS}::chunk_gla", mutates_args={"ws", "out"})
def chunk_gla_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gk: torch.Tensor, scale: float,
                 ws: torch.Tensor, out: torch.Tensor, gk_norm: float, direction: int, grid_h: int,
                 grid_w: int) -> None:
    ops.chunk_gla_run(q, k, v, gk, scale, ws, out, gk_norm, direction=direction, grid_hw=_grid(grid_h, grid_w))


@chunk_gla_op.register_fake
def _(q, k, v, gk, scale, ws, out, gk_norm, direction, grid_h, grid_w):
    return None


@torch.library.custom_op(f"{_NS}::chunk_gla_gated", mutates_args={"ws", "out"})
def chunk_gla_gated_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gk: torch.Tensor, g: torch.Tensor,
                       w: torch.Tensor, scale: float, eps: float, ws: torch.Tensor, out: torch.Tensor,
                       gk_norm: float, direction: int, grid_h: int, grid_w: int) -> None:
    ops.chunk_gla_run_gated(q, k, v, gk, g, w, scale, eps, ws, out, gk_norm, direction=direction,
                            grid_hw=_grid(grid_h, grid_w))


@chunk_gla_gated_op.register_fake
def _(q, k, v, gk, g, w, scale, eps, ws, out, gk_norm, direction, grid_h, grid_w):
    return None


chunk_gla = torch.ops.gtr_b200.chunk_gla
chunk_gla_gated = torch.ops.gtr_b200.chunk_gla_gated
