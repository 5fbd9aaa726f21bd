"""The GTR backbone pieces that sit either side of the GLA operator, in deploy form.

Mirrors, for inference only, the reference's

* ``GatedLinearAttention`` after ``convert_to_deploy`` (engine/gtr/backbone/vit_adapter.py:338-418
  fused q/k/v/g/gk_low projection, :435-605 forward): one fused GEMM, the low-rank gate head,
  the GLA operator with the RMSNorm * w * silu(g) epilogue, ``o_proj``;
* ``SpatialSwiGLU`` in its split-GEMM deploy form (engine/gtr/backbone/vit_adapter_spatial_swiglu.py:21-70), with the
  depthwise convolution, bias, silu(gate) and the product fused into one kernel (``ops.swiglu_dwconv``);
* ``Block`` (vit_adapter.py:608-642) and the CLS-free ``VisionTransformerSpatialSwiGLU`` forward
  (vit_adapter_spatial_swiglu.py:96-127) on top of the conv-pyramid patch-16 stem
  (vit_adapter.py:188-204).

What is different by design: the reference physically permutes the token sequence after every
block (flip, and a grid transpose after odd blocks, vit_adapter_spatial_swiglu.py:88-94) so that
block i scans the grid in order ``DIRECTIONS[i % 4]``.  Here tokens never move: block i passes
``direction = i % 4`` to the operator, which folds the order into its tile coordinates, and the
3x3 depthwise convolution of the MLP uses the kernel the reference's permuted grid implies
(``oriented_dwconv_weight``).  q, k, v and the output gate are strided views of the fused GEMM
output -- no contiguous copies -- and the gate logits go to the kernel raw (gk_normalizer).

There is no fallback path: fp16 CUDA tensors, key heads of 32 or 64 channels (expand_k 0.5 or 1 at 64 channels
per value head) and value heads of 64.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops

HEAD_DIM = 64


def oriented_dwconv_weight(w: torch.Tensor, direction: int) -> torch.Tensor:
    """Depthwise 3x3 kernel to apply on the canonical grid so that the result equals the
    reference's convolution on the grid as block ``direction`` sees it: reversed scans view the
    grid rotated by 180 degrees, column scans view it transposed."""
    d = ops._direction_id(direction)
    if d >= 2:
        w = w.transpose(-1, -2)
    if d & 1:
        w = w.flip(-1, -2)
    return w.contiguous()


# (B, T, heads, device) -> (operator workspace, operator output), shared by every attention module of the process
_GLA_BUFFERS: dict = {}


class GatedLinearAttention(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, expand_k: float = 1.0, expand_v: float = 1.0,
                 gate_low_rank_dim: int = 16, gate_logit_normalizer: float = 16.0, norm_eps: float = 1e-5):
        super().__init__()
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.key_dim, self.value_dim = int(hidden_size * expand_k), int(hidden_size * expand_v)
        self.head_k_dim = self.key_dim // num_heads
        if (self.key_dim != num_heads * self.head_k_dim or self.head_k_dim not in ops.SUPPORTED_K
                or self.value_dim != num_heads * HEAD_DIM):
            raise ValueError(f"gtr_b200 serves key heads of {ops.SUPPORTED_K} and value heads of 64 channels "
                             f"(got K = {self.key_dim / num_heads:g}, V = {self.value_dim / num_heads:g})")
        self.split = (self.key_dim, self.key_dim, self.value_dim, self.value_dim, gate_low_rank_dim)
        self.qkv_g_gkl_proj = nn.Linear(hidden_size, sum(self.split), bias=False)
        self.gk_high_proj = nn.Linear(gate_low_rank_dim, self.key_dim, bias=True)
        self.g_norm_weight = nn.Parameter(torch.ones(HEAD_DIM))
        self.o_proj = nn.Linear(self.value_dim, hidden_size, bias=False)
        self.gate_logit_normalizer = float(gate_logit_normalizer)
        self.norm_eps = float(norm_eps)
        self.scale = self.head_k_dim ** -0.5
        self._ws_key = None
        self._ws = self._out = None
        self._folded = False

    def _gla_buffers(self, B: int, T: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        """Workspace and output are kept per shape so that captured graphs see stable pointers
        (reference: _get_or_make_gla_ws, vit_adapter.py:420-433).  All attention modules of a process share one pair
        per (B, T, heads, device): the blocks run back to back on one stream, the operator clears its control words
        at the start of every call and a block's output is consumed by its o_proj before the next block's operator
        runs, so twelve blocks need one worst-case workspace (hundreds of MB at the backbone's shape), not twelve."""
        key = (B, T, self.num_heads, str(device))
        if self._ws_key != key:
            if key not in _GLA_BUFFERS:
                _GLA_BUFFERS[key] = (ops.make_workspace(B, T, self.num_heads, device),
                                     torch.empty(B, T, self.num_heads, HEAD_DIM, dtype=torch.float16, device=device))
            self._ws, self._out = _GLA_BUFFERS[key]
            self._ws_key = key
        return self._ws, self._out

    @torch.no_grad()
    def fold_gate_head(self) -> None:
        """Deploy-time weight folding: gk = (x W_low^T) W_high^T + b = x (W_high W_low)^T + b becomes key_dim more
        columns of the fused projection, with the bias in that GEMM's epilogue.  The low-rank form saves FLOPs that
        a B200 does not miss; it costs a K = 16 GEMM that is bound by writing its output, a separate bias kernel and
        a strided read of the 16 low-rank columns per block."""
        if self._folded:
            return
        W = self.qkv_g_gkl_proj.weight
        main = sum(self.split[:4])
        w_gk = (self.gk_high_proj.weight.float() @ W[main:].float()).to(W.dtype)
        self.fused_w = nn.Parameter(torch.cat([W[:main], w_gk], dim=0).contiguous(), requires_grad=False)
        self.fused_b = nn.Parameter(torch.cat([torch.zeros(main, dtype=W.dtype, device=W.device),
                                               self.gk_high_proj.bias.to(W.dtype)]).contiguous(), requires_grad=False)
        self._folded = True

    def forward(self, x: torch.Tensor, direction: int = 0, grid_hw: Optional[Tuple[int, int]] = None,
                residual: Optional[torch.Tensor] = None, keep_residual: bool = True):
        if not x.is_cuda or x.dtype != torch.float16:
            raise RuntimeError("gtr_b200.GatedLinearAttention runs fp16 on CUDA only (no fallback path)")
        B, T, _ = x.shape
        H = self.num_heads
        if self._folded:
            q, k, v, g, gk = F.linear(x, self.fused_w, self.fused_b).split(self.split[:4] + (self.key_dim,), dim=-1)
        else:
            fused = self.qkv_g_gkl_proj(x)
            q, k, v, g, gkl = fused.split(self.split, dim=-1)
            gk = self.gk_high_proj(gkl)                           # raw gate logits [B, T, key_dim]
        view = lambda t: t.unflatten(-1, (H, -1))                 # strided views, no copies
        ws, out = self._gla_buffers(B, T, x.device)
        ops.chunk_gla_run_gated(view(q), view(k), view(v), view(gk), view(g), self.g_norm_weight, self.scale,
                                self.norm_eps, ws, out, self.gate_logit_normalizer, direction=direction,
                                grid_hw=grid_hw)
        return _project_add(out.flatten(-2), self.o_proj.weight, residual, keep_residual)


def _project_add(inp: torch.Tensor, weight: torch.Tensor, residual: Optional[torch.Tensor],
                 keep_residual: bool) -> torch.Tensor:
    """``residual + inp @ weight.T`` (or the plain projection without a residual).  With ``keep_residual=False``
    and autograd off, the sum is the GEMM's own epilogue, accumulated into ``residual`` in place (beta = 1): the
    residual stream is then read once by the GEMM instead of passing through a separate elementwise add."""
    if residual is None:
        return F.linear(inp, weight)
    if keep_residual or torch.is_grad_enabled() or not residual.is_contiguous():
        return residual + F.linear(inp, weight)
    residual.view(-1, residual.shape[-1]).addmm_(inp.reshape(-1, inp.shape[-1]), weight.t())
    return residual


class SpatialSwiGLU(nn.Module):
    """SwiGLU whose value branch passes a 3x3 depthwise convolution on the patch grid."""

    def __init__(self, hidden_size: int, hidden_ratio: int = 4, direction: int = 0):
        super().__init__()
        inter = int(hidden_size * hidden_ratio * 2 / 3)
        inter = 256 * ((inter + 255) // 256)                      # vit_adapter_spatial_swiglu.py:28-30
        self.intermediate_size = inter
        self.direction = ops._direction_id(direction)
        self.gate_w = nn.Parameter(torch.empty(inter, hidden_size))
        self.value_w = nn.Parameter(torch.empty(inter, hidden_size))
        self.dwconv = nn.Conv2d(inter, inter, 3, padding=1, groups=inter)
        self.down_proj = nn.Linear(inter, hidden_size, bias=False)
        nn.init.normal_(self.gate_w, std=0.02)
        nn.init.normal_(self.value_w, std=0.02)

    def load_reference_dwconv(self, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> None:
        """Take the reference's depthwise weight (applied there on the permuted grid)."""
        with torch.no_grad():
            self.dwconv.weight.copy_(oriented_dwconv_weight(weight, self.direction))
            if bias is not None:
                self.dwconv.bias.copy_(bias)

    def _taps(self) -> torch.Tensor:
        """The depthwise weight as [3, 3, C] (tap-major), rebuilt when the parameter changes."""
        w = self.dwconv.weight
        key = (w.data_ptr(), w._version, w.device, w.dtype)
        if getattr(self, "_taps_key", None) != key:
            self._taps_cache = w.detach()[:, 0].permute(1, 2, 0).contiguous()
            self._taps_key = key
        return self._taps_cache

    def forward(self, x: torch.Tensor, grid_hw: Tuple[int, int], residual: Optional[torch.Tensor] = None,
                keep_residual: bool = True) -> torch.Tensor:
        gate = F.linear(x, self.gate_w)
        y = F.linear(x, self.value_w)                              # [B, L, C]
        # depthwise 3x3 conv on the patch grid, bias, silu(gate) and the product in one pass over memory, on
        # tokens in place (the reference views y as a channels-last image for cuDNN and back)
        z = ops.swiglu_dwconv(gate, y, self._taps(), self.dwconv.bias, grid_hw)
        return _project_add(z, self.down_proj.weight, residual, keep_residual)


class Block(nn.Module):
    def __init__(self, dim: int, num_heads: int, mlp_ratio: int, direction: int, expand_k: float = 1.0):
        super().__init__()
        self.direction = ops._direction_id(direction)
        self.norm1 = nn.LayerNorm(dim, eps=1e-6)
        self.attn = GatedLinearAttention(dim, num_heads, expand_k=expand_k)
        self.norm2 = nn.LayerNorm(dim, eps=1e-6)
        self.mlp = SpatialSwiGLU(dim, hidden_ratio=mlp_ratio, direction=direction)

    def forward(self, x: torch.Tensor, grid_hw: Tuple[int, int], keep_input: bool = True) -> torch.Tensor:
        """``keep_input=False`` lets the block overwrite ``x`` with its result (inference only)."""
        n1, n2 = self.norm1, self.norm2
        x = self.attn(ops.layernorm(x, n1.weight, n1.bias, n1.eps), self.direction, grid_hw, residual=x,
                      keep_residual=keep_input)
        # x now is this block's own tensor (or the caller's, given up with keep_input=False)
        return self.mlp(ops.layernorm(x, n2.weight, n2.bias, n2.eps), grid_hw, residual=x,
                        keep_residual=keep_input and torch.is_grad_enabled())


class ConvPyramidPatchEmbed(nn.Module):
    """Patch-16 stem: three stride-2 3x3 conv + ReLU stages (BatchNorm folded, as after the
    reference's convert_to_deploy) and a stride-2 projection."""

    def __init__(self, embed_dim: int):
        super().__init__()
        chans = [embed_dim // 8, embed_dim // 4, embed_dim // 2]
        self.convs = nn.ModuleList(nn.Conv2d(i, o, 3, 2, padding=1, bias=True) for i, o in zip([3] + chans[:-1], chans))
        self.proj = nn.Conv2d(chans[-1], embed_dim, 3, 2, padding=1)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        # channels-last through the stem: the convolutions then run without layout conversions around them and
        # the projection's output already is the dense [B, L, C] token tensor
        x = x.contiguous(memory_format=torch.channels_last)
        for conv in self.convs:
            if x.is_cuda:
                # cuDNN's fused convolution + bias + ReLU: otherwise the bias and the ReLU are two more passes over
                # the stem's large early feature maps (a strided add and a clamp per stage)
                x = torch.cudnn_convolution_relu(x, conv.weight, conv.bias, conv.stride, conv.padding, conv.dilation,
                                                 conv.groups)
            else:
                x = F.relu(conv(x))
        # tokens as a dense [B, L, C] tensor: a transposed view here would hand its strides on to every
        # residual sum of the backbone (strided adds, a copy in front of each LayerNorm)
        return self.proj(x).flatten(2).transpose(1, 2).contiguous()


class GTRBackbone(nn.Module):
    """Stem + `depth` blocks; block i scans in order DIRECTIONS[i % 4] (vit_adapter.py:896-898)."""

    def __init__(self, embed_dim: int = 768, depth: int = 12, num_heads: int = 12, mlp_ratio: int = 6,
                 return_layers: Sequence[int] = (3, 7, 11), patch_size: int = 16, expand_k: float = 1.0):
        super().__init__()
        if patch_size != 16:
            raise ValueError("the conv-pyramid stem is patch-16")
        self.embed_dim, self.depth, self.patch_size = embed_dim, depth, patch_size
        self.return_layers = tuple(return_layers)
        self.patch_embed = ConvPyramidPatchEmbed(embed_dim)
        self.blocks = nn.ModuleList(Block(embed_dim, num_heads, mlp_ratio, i % 4, expand_k) for i in range(depth))
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, nn.Linear):                               # vit_adapter.py:745-751
            nn.init.normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.zeros_(m.bias)

    @torch.no_grad()
    def load_reference_state_dict(self, sd, prefix: str = "backbone._model.") -> "GTRBackbone":
        """Take the weights of the reference's ``ViTAdapterSpatialSwiGLU`` (its ``state_dict()``; the ViT sits under
        ``backbone._model.``), in training form or after its ``convert_to_deploy``:

        * stem: ``convs.i.conv`` + ``convs.i.norm`` (BatchNorm, folded here like
          engine/gtr/backbone/vit_adapter.py:145-152) or the already folded ``convs.i.conv_bn_fused``;
        * attention: ``q_proj, k_proj, v_proj, g_proj, gk_proj.0`` are stacked into the fused projection
          (vit_adapter.py:338-374), ``gk_proj.1`` is the gate head, ``g_norm_swish_gate.weight`` the norm weight;
        * MLP: ``gate_proj`` is split into its gate and value halves (vit_adapter_spatial_swiglu.py:36-48) and the
          depthwise kernel, which the reference applies on the grid as block i sees it, is re-oriented for the
          canonical grid (``oriented_dwconv_weight``)."""
        get = lambda name: torch.as_tensor(sd[prefix + name])
        has = lambda name: (prefix + name) in sd
        dst = self.state_dict()

        def put(name, value):
            dst[name].copy_(value.to(dst[name].dtype))

        for i in range(len(self.patch_embed.convs)):
            base = f"patch_embed.convs.{i}."
            if has(base + "conv_bn_fused.weight"):
                w, b = get(base + "conv_bn_fused.weight"), get(base + "conv_bn_fused.bias")
            else:
                w = get(base + "conv.weight").float()
                gamma, beta = get(base + "norm.weight").float(), get(base + "norm.bias").float()
                mean, var = get(base + "norm.running_mean").float(), get(base + "norm.running_var").float()
                std = (var + 1e-5).sqrt()
                w, b = w * (gamma / std).reshape(-1, 1, 1, 1), beta - mean * gamma / std
            put(f"patch_embed.convs.{i}.weight", w)
            put(f"patch_embed.convs.{i}.bias", b)
        put("patch_embed.proj.weight", get("patch_embed.proj.weight"))
        put("patch_embed.proj.bias", get("patch_embed.proj.bias"))
        for i, blk in enumerate(self.blocks):
            b = f"blocks.{i}."
            for n in ("norm1.weight", "norm1.bias", "norm2.weight", "norm2.bias", "attn.o_proj.weight",
                      "mlp.down_proj.weight"):
                put(b + n, get(b + n))
            a = b + "attn."
            if has(a + "qkv_g_gkl_proj.weight"):
                put(a + "qkv_g_gkl_proj.weight", get(a + "qkv_g_gkl_proj.weight"))
                put(a + "gk_high_proj.weight", get(a + "gk_high_proj.weight"))
                put(a + "gk_high_proj.bias", get(a + "gk_high_proj.bias"))
            else:
                put(a + "qkv_g_gkl_proj.weight", torch.cat([get(a + n + ".weight") for n in
                                                           ("q_proj", "k_proj", "v_proj", "g_proj", "gk_proj.0")]))
                put(a + "gk_high_proj.weight", get(a + "gk_proj.1.weight"))
                put(a + "gk_high_proj.bias", get(a + "gk_proj.1.bias"))
            put(a + "g_norm_weight", get(a + "g_norm_swish_gate.weight"))
            m = b + "mlp."
            if has(m + "gate_proj.weight"):
                gate_w, value_w = get(m + "gate_proj.weight").chunk(2, dim=0)
            else:
                gate_w, value_w = get(m + "gate_w"), get(m + "value_w")
            put(m + "gate_w", gate_w)
            put(m + "value_w", value_w)
            blk.mlp.load_reference_dwconv(get(m + "dwconv.weight").to(blk.mlp.dwconv.weight),
                                          get(m + "dwconv.bias").to(blk.mlp.dwconv.bias))
            blk.attn._folded = False
        return self

    def convert_to_deploy(self) -> "GTRBackbone":
        """Inference-time weight transforms (call after the weights are loaded and moved to their device and dtype):
        folds the low-rank gate head of every block into its fused projection."""
        for blk in self.blocks:
            blk.attn.fold_gate_head()
        self.patch_embed.to(memory_format=torch.channels_last)
        return self

    def forward(self, img: torch.Tensor) -> List[torch.Tensor]:
        hg, wg = img.shape[-2] // self.patch_size, img.shape[-1] // self.patch_size
        x = self.patch_embed(img)
        outs = []
        for i, blk in enumerate(self.blocks):
            # a block may overwrite its input unless that input is one of the returned layers
            x = blk(x, (hg, wg), keep_input=(i - 1) in self.return_layers)
            if i in self.return_layers:
                outs.append(x)                                     # canonical token order at every layer
        return outs


class GraphedBackbone:
    """Replays one captured CUDA graph per input shape (the reference benchmarks its model the same
    way, tools/benchmark/torch_speed_fullgraph.py:134-158).  The operator's launches (a memset and one
    kernel per block) are captured like any other stream work."""

    def __init__(self, model: GTRBackbone):
        self.model = model.eval()
        self._graphs = {}

    @torch.no_grad()
    def __call__(self, img: torch.Tensor) -> List[torch.Tensor]:
        key = (tuple(img.shape), img.device)
        if key not in self._graphs:
            static_in = img.clone()
            side = torch.cuda.Stream(device=img.device)
            side.wait_stream(torch.cuda.current_stream(img.device))
            with torch.cuda.stream(side):
                for _ in range(2):                                  # warm-up: allocations, tensor-map cache
                    self.model(static_in)
            torch.cuda.current_stream(img.device).wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_out = self.model(static_in)
            self._graphs[key] = (graph, static_in, static_out)
        graph, static_in, static_out = self._graphs[key]
        static_in.copy_(img, non_blocking=True)
        graph.replay()
        return static_out
