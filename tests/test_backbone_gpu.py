"""The backbone that keeps tokens in place and passes scan directions to the operator, against a
CPU restatement of the reference's forward that physically permutes tokens between blocks."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def small_model():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from gtr_b200.backbone import GTRBackbone
    torch.manual_seed(0)
    m = GTRBackbone(embed_dim=128, depth=4, num_heads=2, mlp_ratio=6, return_layers=(1, 2, 3)).eval()
    with torch.no_grad():                        # keep gates and norm weights away from trivial values
        for blk in m.blocks:
            blk.attn.g_norm_weight.uniform_(0.5, 1.5)
            blk.attn.gk_high_proj.bias.normal_(0, 1.0)
    return m


def test_backbone_matches_reference_style_forward(small_model):
    from oracle import backbone_ref, gla_ref
    img = torch.rand(2, 3, 192, 192, generator=torch.Generator().manual_seed(1))      # 12 x 12 patch grid
    want = backbone_ref.forward(copy.deepcopy(small_model).float(), img)
    dev = copy.deepcopy(small_model).half().cuda()
    with torch.no_grad():
        got = dev(img.half().cuda())
    assert len(got) == len(want) == 3
    for w, g in zip(want, got):
        m = gla_ref.error_metrics(w, g.float().cpu())
        # an fp16 model (weights, GEMMs, LayerNorm, conv) against an fp32 one: a few 1e-3; a wrong scan
        # order or a wrongly oriented depthwise kernel shows up as an error of order one
        assert m["finite"] and m["rel_l2"] < 1.5e-2, m


@pytest.mark.parametrize("tag,expand_k", [("k64", 1.0), ("k32", 0.5)])
@pytest.mark.parametrize("deploy", [False, True])
def test_backbone_matches_recorded_outputs_of_the_reference_backbone(deploy, tag, expand_k):
    """The fp16 CUDA backbone, loaded with the reference's own state dict, against feature maps the reference's
    ViTAdapterSpatialSwiGLU produced for the same weights and input (tests/golden/backbone_small.npz, recorded by
    tests/golden/make_golden.py from the reference run in fp32 on a CPU), with key heads of 64 channels
    (expand_k = 1) and of 32 (expand_k = 0.5, the released GTR configurations)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import os
    import numpy as np
    from gtr_b200.backbone import GTRBackbone
    from oracle import gla_ref
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "backbone_small.npz"))
    sd = {k[len(tag) + 4:]: torch.from_numpy(z[k]).float() for k in z.files if k.startswith(tag + "_sd/")}
    m = GTRBackbone(embed_dim=128, depth=4, num_heads=2, mlp_ratio=6, return_layers=(1, 2, 3),
                    expand_k=expand_k).eval()
    m.load_reference_state_dict(sd)
    m = m.half().cuda()
    if deploy:
        m.convert_to_deploy()
    with torch.no_grad():
        got = m(torch.from_numpy(z[tag + "_img"]).cuda())
    for i, g in enumerate(got):
        ref = torch.from_numpy(z[f"{tag}_out{i}"])
        e = gla_ref.error_metrics(ref, g.float().cpu().transpose(1, 2).reshape(ref.shape))
        # fp16 weights, GEMMs, LayerNorm and convolutions against the reference in fp32
        assert e["finite"] and e["rel_l2"] < 1.5e-2, (i, e)


def test_deploy_form_matches_reference_style_forward(small_model):
    """convert_to_deploy folds the low-rank gate head into the fused projection: same function, other rounding."""
    from oracle import backbone_ref, gla_ref
    img = torch.rand(2, 3, 224, 224, generator=torch.Generator().manual_seed(4))      # 14 x 14 patch grid
    want = backbone_ref.forward(copy.deepcopy(small_model).float(), img)
    dev = copy.deepcopy(small_model).half().cuda().convert_to_deploy()
    assert all(blk.attn._folded for blk in dev.blocks)
    with torch.no_grad():
        got = dev(img.half().cuda())
    for w, g in zip(want, got):
        m = gla_ref.error_metrics(w, g.float().cpu())
        assert m["finite"] and m["rel_l2"] < 1.5e-2, m


def test_wrong_scan_order_is_detected(small_model):
    """Negative control for the tolerance above."""
    from oracle import backbone_ref, gla_ref
    img = torch.rand(1, 3, 192, 192, generator=torch.Generator().manual_seed(2))
    want = backbone_ref.forward(copy.deepcopy(small_model).float(), img)
    dev = copy.deepcopy(small_model).half().cuda()
    dev.blocks[1].direction = 0                               # should be 1 (row reversed)
    with torch.no_grad():
        got = dev(img.half().cuda())
    assert gla_ref.error_metrics(want[-1], got[-1].float().cpu())["rel_l2"] > 0.1


def test_graph_replay_equals_eager(small_model):
    from gtr_b200.backbone import GraphedBackbone
    dev = copy.deepcopy(small_model).half().cuda()
    img = torch.rand(1, 3, 256, 320, device="cuda").half()      # 16 x 20 grid: non-square
    with torch.no_grad():
        eager = [t.clone() for t in dev(img)]
    graphed = GraphedBackbone(dev)
    for _ in range(2):
        out = graphed(img)
    torch.cuda.synchronize()
    for a, b in zip(eager, out):
        assert torch.equal(a, b)


def test_rejects_cpu_and_other_head_dims():
    from gtr_b200.backbone import GatedLinearAttention
    with pytest.raises(ValueError):
        GatedLinearAttention(192, 6, expand_k=0.5)              # K = 16 per head
    assert GatedLinearAttention(192, 3, expand_k=0.5).head_k_dim == 32      # the released GTR-S shape
    att = GatedLinearAttention(128, 2)
    with pytest.raises(RuntimeError):
        att(torch.zeros(1, 64, 128))
