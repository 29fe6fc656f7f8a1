"""Randomised sweep over the tensor-core routes (fp16 / bf16 / fp32, head dims 8..64, and 72..128 for the 16-bit types, ragged lengths, causal or not,
contiguous or packed-qkv layouts): forward and gradients against fp64 softmax attention evaluated on the same device.
Seeded, so every run checks the same 36 problems."""
import random

import pytest
import torch

import elsa_b200 as E
from elsa_b200.attention_bwd import twopass_attention_qkvpacked

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cases():
    rng = random.Random(20240607)
    out = []
    for i in range(36):
        dtype = (torch.float16, torch.bfloat16, torch.float32)[i % 3]
        d = rng.choice((8, 16, 24, 32, 40, 48, 56, 64))
        if dtype != torch.float32 and i % 2 == 1:
            d = rng.choice((72, 80, 96, 104, 120, 128))      # the wide-head kernels (16-bit inputs only)
        n = rng.choice((512, 513, 640, 777, 1000, 1024, 1153, 1500, 2049, 2500))
        b, h = rng.choice(((1, 1), (1, 3), (2, 2), (3, 1)))
        out.append((i, dtype, b, h, n, d, rng.random() < 0.5, rng.random() < 0.4))
    return out


def _fp64(q, k, v, causal):
    n, d = q.shape[-2], q.shape[-1]
    s = (q.double() @ k.double().transpose(-1, -2)) / d ** 0.5
    if causal:
        s = s.masked_fill(torch.ones(n, n, device=q.device, dtype=torch.bool).triu(1), float("-inf"))
    return torch.softmax(s, -1) @ v.double()


@pytest.mark.parametrize("case", _cases(), ids=lambda c: f"{c[0]}-{str(c[1])[6:]}-b{c[2]}h{c[3]}n{c[4]}d{c[5]}-{'c' if c[6] else 'f'}{'p' if c[7] else ''}")
def test_random_problem_against_fp64(case):
    i, dtype, b, h, n, d, causal, packed = case
    from elsa_b200 import _lib
    lib = _lib.load()
    assert lib.elsa_uses_tensor_cores(_lib.dtype_code(dtype), d, n, 0, int(causal), 0) == 1
    assert lib.elsa_uses_tensor_cores(_lib.dtype_code(dtype), d, n, 0, int(causal), 1) == 1
    g = torch.Generator().manual_seed(1000 + i)
    qkv = torch.randn(b, n, 3, h, d, generator=g).to(dtype).to(DEV)
    go = torch.randn(b, h, n, d, generator=g).to(dtype).to(DEV)
    qkv.requires_grad_(True)
    if packed:
        out = twopass_attention_qkvpacked(qkv, is_causal=causal)
    else:
        q, k, v = (t.contiguous() for t in qkv.permute(2, 0, 3, 1, 4).unbind(0))
        out = E.twopass_attention_train(q, k, v, is_causal=causal)
    out.backward(go)
    grad = qkv.grad.detach().clone()

    ref_in = qkv.detach().double().requires_grad_(True)
    rq, rk, rv = ref_in.permute(2, 0, 3, 1, 4).unbind(0)
    ref = _fp64(rq, rk, rv, causal)
    ref.backward(go.double())
    out_lim = {torch.float32: 2e-6, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[dtype]
    grad_lim = {torch.float32: 4e-6, torch.float16: 3e-3, torch.bfloat16: 2.4e-2}[dtype]
    assert torch.isfinite(out).all() and torch.isfinite(grad).all()
    assert (out.double() - ref).abs().max().item() <= out_lim * max(1.0, ref.abs().max().item())
    assert (grad.double() - ref_in.grad).abs().max().item() <= grad_lim * max(1.0, ref_in.grad.abs().max().item())
    assert lib.elsa_device_status(0) == 0
