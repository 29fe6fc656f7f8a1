"""Whole models through the drop-in hooks and the toy encoder pair, on the GPU.

* ViT-Tiny and Swin-T (timm-shaped attention modules, elsa_b200/vision.py): the model patched with
  patch_timm_attention_train against the same, unpatched model -- logits and parameter gradients -- at the
  reference's model-level tolerances (tests/test_attention.py:116-130: 5e-3 in fp32, 8e-2 in fp16).
* make_model_pair / make_train_model_pair: the reference's own model test (tests/test_attention.py:116-130) and
  its training counterpart.
* The forward cells of the reference's spot check (scripts/spot_check.py:39-51): max-abs against PyTorch SDPA below
  1e-5 (fp32) / 5e-3 (fp16) on (8,3,1025,64), (8,3,2305,64), (1,8,4096,64)."""
import copy

import pytest
import torch
import torch.nn.functional as F

import elsa_b200 as E
from elsa_b200 import full_model, vision

pytestmark = pytest.mark.gpu
F32, F16 = torch.float32, torch.float16


def _train_step(model, img, labels):
    model.zero_grad(set_to_none=True)
    logits = model(img)
    F.cross_entropy(logits.float(), labels).backward()
    return logits.detach(), {n: p.grad.detach().clone() for n, p in model.named_parameters() if p.grad is not None}


@pytest.mark.parametrize("kind,img,dtype", [("vit", 224, F32), ("vit", 512, F16), ("swin", 224, F32), ("swin", 224, F16)])
def test_patched_model_matches_unpatched(kind, img, dtype):
    torch.manual_seed(3)
    base = (vision.vit_tiny(img, num_classes=100) if kind == "vit" else vision.swin_tiny(img, num_classes=100))
    base = base.to("cuda", dtype)
    ours = copy.deepcopy(base)
    rep = E.patch_timm_attention_train(ours)
    assert rep.total == 12
    assert sorted(n for n, _ in base.named_parameters()) == sorted(n for n, _ in ours.named_parameters())
    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 3, img, img, generator=g).to("cuda", dtype)
    y = torch.randint(0, 100, (2,), generator=g).cuda()
    lo_b, gr_b = _train_step(base, x, y)
    lo_o, gr_o = _train_step(ours, x, y)
    tol = 5e-3 if dtype == F32 else 8e-2
    torch.testing.assert_close(lo_o.float(), lo_b.float(), atol=tol, rtol=tol)
    assert set(gr_b) == set(gr_o)
    for name in gr_b:
        big = max(1e-3, float(gr_b[name].float().abs().max()))
        err = float((gr_o[name].float() - gr_b[name].float()).abs().max())
        assert err <= tol * big + (1e-6 if dtype == F32 else 2e-3), (name, err, big)


@pytest.mark.parametrize("dtype", [F32, F16])
def test_full_model_pair_matches(dtype):
    torch.manual_seed(6)
    baseline, elsa = full_model.make_model_pair(dim=96, depth=2, heads=3)
    baseline, elsa = baseline.eval().to("cuda", dtype), elsa.eval().to("cuda", dtype)
    x = torch.randn((1, 128, 96), device="cuda", dtype=dtype)
    with torch.no_grad():
        ref, out = baseline(x), elsa(x)
    tol = 5e-3 if dtype is F32 else 8e-2
    torch.testing.assert_close(out, ref, atol=tol, rtol=tol)


@pytest.mark.parametrize("dtype,causal", [(F32, False), (F16, True)])
def test_train_model_pair_gradients_match(dtype, causal):
    torch.manual_seed(7)
    baseline, elsa = full_model.make_train_model_pair(dim=192, depth=2, heads=3, is_causal=causal)
    baseline, elsa = baseline.to("cuda", dtype), elsa.to("cuda", dtype)
    x = torch.randn((2, 600, 192), device="cuda", dtype=dtype)          # 600 tokens: the tensor-core path in fp16
    for m in (baseline, elsa):
        m(x).float().square().mean().backward()
    tol = 5e-3 if dtype is F32 else 8e-2
    for (n, pb), (_, pe) in zip(baseline.named_parameters(), elsa.named_parameters()):
        big = max(1e-4, float(pb.grad.float().abs().max()))
        assert float((pe.grad.float() - pb.grad.float()).abs().max()) <= tol * big + (1e-7 if dtype is F32 else 1e-4), n


@pytest.mark.parametrize("shape,dtype", [((8, 3, 1025, 64), F32), ((8, 3, 2305, 64), F16), ((1, 8, 4096, 64), F32)])
def test_spot_check_forward_cells(shape, dtype):
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(shape, generator=g).to("cuda", dtype) for _ in range(3))
    out = E.twopass_attention(q, k, v)
    ref = F.scaled_dot_product_attention(q.float(), k.float(), v.float(), scale=1.0 / shape[-1] ** 0.5)
    assert (out.float() - ref).abs().max().item() < (5e-3 if dtype is F16 else 1e-5)
