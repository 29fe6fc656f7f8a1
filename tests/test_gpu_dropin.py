"""Drop-in hooks on stand-in timm modules (ViT attention, Swin-v1 window attention incl. the
shifted-window mask): patched model == plain-PyTorch model, forward and backward."""
import copy

import pytest
import torch
import torch.nn as nn

import elsa_b200 as E
from tests.standins import SwinWindowAttention, VitAttention

pytestmark = pytest.mark.gpu
DEV = "cuda"


class Block(nn.Module):
    def __init__(self, attn):
        super().__init__()
        self.norm = nn.LayerNorm(attn.qkv.in_features)
        self.attn = attn

    def forward(self, x, **kw):
        return x + self.attn(self.norm(x), **kw)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.float16, 4e-3)])
def test_vit_dropin_inference_and_training(dtype, tol):
    torch.manual_seed(0)
    base = nn.Sequential(Block(VitAttention(192, 3)), Block(VitAttention(192, 3))).to(DEV, dtype)
    inf = copy.deepcopy(base)
    trn = copy.deepcopy(base)
    rep = E.patch_timm_attention(inf)
    assert (rep.vit_attention, rep.swin_window_attention, rep.total) == (2, 0, 2)
    rep = E.patch_timm_attention_train(trn)
    assert isinstance(rep, E.TrainPatchReport) and rep.total == 2
    x = torch.randn(2, 197, 192, device=DEV, dtype=dtype)
    with torch.no_grad():
        ref = base(x)
        assert (inf(x) - ref).abs().max().item() <= tol
    xr = x.clone().requires_grad_(True)
    xt = x.clone().requires_grad_(True)
    base(xr).square().mean().backward()
    trn(xt).square().mean().backward()
    assert (xt.grad - xr.grad).abs().max().item() <= tol
    for (n1, p1), (n2, p2) in zip(base.named_parameters(), trn.named_parameters()):
        assert n1 == n2
        assert (p1.grad - p2.grad).abs().max().item() <= tol * 10, n1
    with pytest.raises(ValueError, match="unmasked"):
        inf[0].attn(x, attn_mask=torch.zeros(197, 197, device=DEV))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.float16, 4e-3)])
@pytest.mark.parametrize("shifted", [False, True])
def test_swin_dropin(dtype, tol, shifted):
    torch.manual_seed(1)
    base = Block(SwinWindowAttention(96, 3, (7, 7))).to(DEV, dtype)
    trn = copy.deepcopy(base)
    inf = copy.deepcopy(base)
    assert E.patch_timm_attention(inf).swin_window_attention == 1
    assert E.patch_timm_attention_train(trn).swin_window_attention == 1
    n_win, images = 4, 3
    x = torch.randn(images * n_win, 49, 96, device=DEV, dtype=dtype)
    kw = {}
    if shifted:
        mask = torch.zeros(n_win, 49, 49, device=DEV, dtype=dtype)
        mask[1, :20, 20:] = -100.0
        mask[1, 20:, :20] = -100.0
        mask[3, :7, 7:] = -100.0
        kw = {"mask": mask}
    with torch.no_grad():
        ref = base(x, **kw)
        assert (inf(x, **kw) - ref).abs().max().item() <= tol
    xr = x.clone().requires_grad_(True)
    xt = x.clone().requires_grad_(True)
    base(xr, **kw).square().mean().backward()
    trn(xt, **kw).square().mean().backward()
    assert (xt.grad - xr.grad).abs().max().item() <= tol
    gb = dict(base.named_parameters())["attn.relative_position_bias_table"].grad
    gt = dict(trn.named_parameters())["attn.relative_position_bias_table"].grad
    assert gt is not None and (gt - gb).abs().max().item() <= tol * 10


def test_swin_noncanonical_scale_and_dropout_rejection():
    torch.manual_seed(2)
    src = SwinWindowAttention(64, 2, (7, 7)).to(DEV)
    src.scale = 0.3
    patched = E.timm_dropin.ElsaTimmSwinWindowAttention(src)
    x = torch.randn(6, 49, 64, device=DEV)
    with torch.no_grad():
        assert (patched(x) - src(x)).abs().max().item() <= 2e-5
    src.attn_drop = nn.Dropout(0.1)
    t = E.timm_dropin_bwd.ElsaTrainTimmSwinWindowAttention(src).train()
    with pytest.raises(ValueError, match="dropout"):
        t(x)
