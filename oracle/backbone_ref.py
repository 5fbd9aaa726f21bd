"""CPU restatement of the reference backbone forward, for parity tests.  TEST INFRASTRUCTURE ONLY.

Follows the reference's own data flow, not the product's: the token sequence is physically
flipped after every block and the (square) grid transposed after odd blocks
(engine/gtr/backbone/vit_adapter_spatial_swiglu.py:88-94, :96-127), the GLA of every block is
then a plain forward scan (engine/gtr/backbone/vit_adapter.py:435-605 with the fp32 token
recurrence in place of the Triton kernel), the depthwise convolution runs on the grid as
permuted (vit_adapter_spatial_swiglu.py:52-61), and returned features are brought back to
canonical order through the tracked permutation.  Weights are read from a
gtr_b200.backbone.GTRBackbone (fp32 copy on the CPU); its depthwise kernels are stored in the
canonical orientation, so they are turned back into the reference's orientation here.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import gla_ref


def _attn(att, x):
    B, T, _ = x.shape
    H = att.num_heads
    fused = att.qkv_g_gkl_proj(x)
    q, k, v, g, gkl = fused.split(att.split, dim=-1)
    gk = gla_ref.gate_from_logits(att.gk_high_proj(gkl), att.gate_logit_normalizer)
    r = lambda t: t.reshape(B, T, H, -1)
    o, _ = gla_ref.chunk_gla(r(q), r(k), r(v), r(gk), scale=att.scale)
    y = gla_ref.rmsnorm_swish_gate(o, r(g), att.g_norm_weight, att.norm_eps)
    return att.o_proj(y.reshape(B, T, -1))


def _mlp(mlp, x, gs, w_ref):
    B, L, _ = x.shape
    gate = F.linear(x, mlp.gate_w)
    y = F.linear(x, mlp.value_w)
    y = y.transpose(1, 2).reshape(B, -1, gs, gs)
    y = F.conv2d(y, w_ref, mlp.dwconv.bias, padding=1, groups=y.shape[1]).flatten(2).transpose(1, 2)
    return mlp.down_proj(F.silu(gate) * y)


@torch.no_grad()
def forward(model, img):
    """model: GTRBackbone in fp32 on the CPU.  Square patch grids only, like the reference."""
    from gtr_b200.backbone import oriented_dwconv_weight
    x = model.patch_embed(img)
    L = x.shape[1]
    gs = int(round(L ** 0.5))
    assert gs * gs == L, "the reference backbone handles square grids only"
    perm = torch.arange(L)
    outs = []
    for i, blk in enumerate(model.blocks):
        w_ref = oriented_dwconv_weight(blk.mlp.dwconv.weight, i % 4)     # the transform is its own inverse
        x = x + _attn(blk.attn, blk.norm1(x))
        x = x + _mlp(blk.mlp, blk.norm2(x), gs, w_ref)
        x = x.flip(1)
        perm = perm.flip(0)
        if i % 2 == 1:
            x = x.reshape(x.shape[0], gs, gs, -1).transpose(1, 2).flatten(1, 2)
            perm = perm.reshape(gs, gs).t().reshape(-1)
        if i in model.return_layers:
            outs.append(x[:, torch.argsort(perm), :])
    return outs
