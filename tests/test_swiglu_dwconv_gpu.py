"""The fused depthwise-conv + SwiGLU kernel against the reference's own formulation of that step
(engine/gtr/backbone/vit_adapter_spatial_swiglu.py:50-60) evaluated with PyTorch in fp32."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _reference(gate, y, conv_w, bias, hg, wg):
    B, L, C = y.shape
    img = y.float().view(B, hg, wg, C).permute(0, 3, 1, 2)
    z = F.conv2d(img, conv_w.float(), None if bias is None else bias.float(), padding=1, groups=C)
    z = z.permute(0, 2, 3, 1).reshape(B, L, C)
    return F.silu(gate.float()) * z


@pytest.mark.parametrize("B,hg,wg,C,with_bias", [(2, 8, 8, 64, True), (1, 5, 37, 256, True), (3, 17, 3, 128, False),
                                                 (1, 1, 1, 8, True), (1, 64, 128, 512, True), (2, 9, 18, 200, True),
                                                 (1, 16, 32, 392, False)])
def test_matches_conv_silu_product(B, hg, wg, C, with_bias):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import gtr_b200 as G
    gen = torch.Generator().manual_seed(hg * 131 + wg)
    L = hg * wg
    gate = (torch.randn(B, L, C, generator=gen) * 1.5).half().cuda()
    y = torch.randn(B, L, C, generator=gen).half().cuda()
    conv_w = (torch.randn(C, 1, 3, 3, generator=gen) * 0.3).half().cuda()
    bias = (torch.randn(C, generator=gen) * 0.1).half().cuda() if with_bias else None
    taps = conv_w[:, 0].permute(1, 2, 0).contiguous()
    out = torch.full_like(y, float("nan"))
    G.swiglu_dwconv(gate, y, taps, bias, (hg, wg), out=out)
    ref = _reference(gate, y, conv_w, bias, hg, wg)
    err = (out.float() - ref).norm() / ref.norm().clamp_min(1e-30)
    assert torch.isfinite(out).all()
    assert err.item() < 1e-3, err.item()          # fp16 output rounding plus the 2^-11 tanh approximation
    assert (out.float() - ref).abs().max().item() <= 2e-3 * max(1.0, ref.abs().max().item())


def test_rejects_aliasing_and_bad_shapes():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import gtr_b200 as G
    y = torch.zeros(1, 16, 64, dtype=torch.float16, device="cuda")
    taps = torch.zeros(3, 3, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(Exception):
        G.swiglu_dwconv(y, y, taps, None, (4, 4), out=y)           # in place is not possible: neighbours are read later
    with pytest.raises(RuntimeError):
        G.swiglu_dwconv(y, y, taps, None, (4, 5))                  # grid does not match L
    with pytest.raises(RuntimeError):
        G.swiglu_dwconv(y.float(), y, taps, None, (4, 4))


@pytest.mark.parametrize("rows,D,with_bias", [(1, 8, True), (37, 768, True), (1000, 128, False), (5, 2048, True), (64, 264, True)])
def test_layernorm_rows(rows, D, with_bias):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import gtr_b200 as G
    gen = torch.Generator().manual_seed(rows + D)
    x = (torch.randn(rows, D, generator=gen) * 2.0 + 0.5).half().cuda()
    w = (torch.randn(D, generator=gen) * 0.2 + 1.0).half().cuda()
    b = (torch.randn(D, generator=gen) * 0.1).half().cuda() if with_bias else None
    ref = F.layer_norm(x.float(), (D,), w.float(), None if b is None else b.float(), 1e-6)
    y = G.layernorm(x, w, b, 1e-6)
    assert torch.isfinite(y).all()
    assert ((y.float() - ref).norm() / ref.norm()).item() < 5e-4          # fp16 output rounding
    G.layernorm(x, w, b, 1e-6, out=x)                                     # in place
    assert torch.equal(x, y)
    with pytest.raises(Exception):
        G.layernorm(torch.zeros(4, 4096, dtype=torch.float16, device="cuda"), torch.ones(4096, dtype=torch.float16, device="cuda"),
                    None, 1e-6)
