"""Host-side checks of the whole-model workloads: the models build with the published sizes, the drop-in hooks find
every attention module, the toy encoder pair shares weights, and the bucketed gradient exchange averages gradients
between two CPU ranks (gloo) exactly like a plain all_reduce would."""
import os
import socket

import pytest
import torch
import torch.nn as nn

import elsa_b200 as E
from elsa_b200 import full_model, vision


def n_params(m):
    return sum(p.numel() for p in m.parameters())


def test_vit_tiny_and_swin_tiny_shapes_and_patch_counts():
    vit = vision.vit_tiny(img_size=64)           # same architecture, small image: 17 tokens
    assert 5.4e6 < n_params(vision.vit_tiny(img_size=224)) < 5.9e6          # ViT-Tiny has about 5.7 M parameters
    with torch.no_grad():
        assert vit(torch.randn(2, 3, 64, 64)).shape == (2, 1000)
    assert vision.vit_tiny(img_size=1024).pos_embed.shape[1] == 4097
    rep = E.patch_timm_attention_train(vit)
    assert (rep.vit_attention, rep.swin_window_attention, rep.total) == (12, 0, 12)
    swin = vision.swin_tiny(img_size=224)
    assert 27e6 < n_params(swin) < 30e6                                       # Swin-T has about 28 M parameters
    blocks = [m for m in swin.layers if isinstance(m, vision.SwinBlock)]
    assert [b.attn.num_heads for b in blocks] == [3, 3, 6, 6] + [12] * 6 + [24, 24]
    assert [b.shift for b in blocks] == [0, 3, 0, 3, 0, 3, 0, 3, 0, 3, 0, 0]  # 7x7 tokens in stage 4: one window, no shift
    assert blocks[1].attn_mask.shape == (64, 49, 49)
    with torch.no_grad():
        assert swin(torch.randn(1, 3, 224, 224)).shape == (1, 1000)
    rep = E.patch_timm_attention(swin)
    assert (rep.vit_attention, rep.swin_window_attention) == (0, 12)
    with pytest.raises(ValueError, match="no compatible"):
        E.patch_timm_attention(nn.Linear(4, 4))


def test_toy_encoder_pair_shares_weights_and_baseline_runs():
    base, elsa = full_model.make_model_pair(dim=96, depth=2, heads=3)
    tb, te = full_model.make_train_model_pair(dim=96, depth=2, heads=3, is_causal=True)
    for a, b in ((base, elsa), (tb, te)):
        for (na, pa), (nb, pb) in zip(a.state_dict().items(), b.state_dict().items()):
            assert na == nb and torch.equal(pa, pb)
    assert te.blocks[0].attn.trainable and not elsa.blocks[0].attn.trainable
    with torch.no_grad():
        assert base(torch.randn(2, 33, 96)).shape == (2, 33, 96)
    with pytest.raises(ValueError, match="requires CUDA"):
        elsa(torch.randn(1, 8, 96))                     # the operator has no CPU path


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _dp_worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        model = nn.Sequential(nn.Linear(16, 64), nn.GELU(), nn.Linear(64, 64), nn.GELU(), nn.Linear(64, 4),
                              nn.Linear(4, 4))
        model[5].weight.requires_grad_(True)
        sync = vision.BucketedGradientAllReduce(model, bucket_bytes=1024)
        assert len(sync.buckets) >= 3
        for step in range(2):
            x = torch.randn(8, 16, generator=torch.Generator().manual_seed(100 * step + rank))
            model.zero_grad(set_to_none=True)
            loss = model[:5](x).square().mean()      # the last layer gets no gradient: its bucket is flushed by finish()
            loss.backward()
            local = [None if p.grad is None else p.grad.clone() for p in model.parameters()]
            sync.finish()
            worst = 0.0
            for p, g in zip(model.parameters(), local):
                if g is None:
                    assert p.grad is None
                    continue
                dist.all_reduce(g)
                worst = max(worst, (p.grad - g / world).abs().max().item())
            ret[(rank, step)] = worst
    finally:
        dist.destroy_process_group()


def test_bucketed_gradient_exchange_two_cpu_ranks():
    import torch.multiprocessing as mp
    ret = mp.Manager().dict()
    mp.spawn(_dp_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert len(ret) == 4 and all(v <= 1e-6 for v in ret.values()), dict(ret)


def test_layout_helpers_decide_in_place_or_copy():
    """Host logic of the strided entry points: which [B, H, N, D] views the kernels may read in place."""
    from elsa_b200.attention import _bhnd_strides, _empty_like_layout, _i64x
    b, n, h, d = 2, 50, 3, 64
    qkv = torch.zeros(b, n, 3, h, d, dtype=torch.float16)
    q, k, v = qkv.permute(2, 0, 3, 1, 4).unbind(0)
    assert _bhnd_strides(q) == (n * 3 * h * d, d, 3 * h * d) == _bhnd_strides(k) == _bhnd_strides(v)
    assert k.data_ptr() - q.data_ptr() == h * d * 2
    assert _bhnd_strides(torch.zeros(b, h, n, d)) == (h * n * d, n * d, d)
    assert _bhnd_strides(torch.zeros(1, 1, n, d)) == (d * 8, d * 8, d)              # size-1 axes: any valid stride
    assert _bhnd_strides(torch.zeros(b, h, d, n).transpose(2, 3)) is None            # D axis not contiguous
    assert _bhnd_strides(torch.zeros(b, h, n, d + 4, dtype=torch.float16)[..., :d]) is None   # row stride 68: not 16-byte rows
    assert _bhnd_strides(torch.zeros(b, h, n, d + 8, dtype=torch.float16)[..., 4:4 + d]) is None   # first element off a 16-byte boundary
    assert _bhnd_strides(torch.zeros(1, h, n, d).expand(b, h, n, d)) is None         # broadcast batch axis
    out = _empty_like_layout(q, _bhnd_strides(q))
    assert out.shape == q.shape and out.transpose(1, 2).reshape(b, n, h * d).data_ptr() == out.data_ptr()
    assert _empty_like_layout(torch.zeros(b, h, n, d), (h * n * d, n * d, d)).is_contiguous()
    arr = _i64x((1, 2, 3), (4, 5, 6))
    assert list(arr) == [1, 2, 3, 4, 5, 6]


def test_packed_operator_validates_its_arguments():
    from elsa_b200.attention_bwd import twopass_attention_qkvpacked
    with pytest.raises(ValueError, match=r"\[B,N,3,H,D\]"):
        twopass_attention_qkvpacked(torch.zeros(2, 5, 2, 3, 8))
    with pytest.raises(ValueError, match="num_warps"):
        twopass_attention_qkvpacked(torch.zeros(2, 5, 3, 3, 8), bwd_num_warps=3)
    with pytest.raises(ValueError, match="requires CUDA"):
        twopass_attention_qkvpacked(torch.zeros(2, 5, 3, 3, 8))
