"""Parity at the sizes of the headline workloads, where the CPU oracle is too slow: one whole head checked
against fp64 math attention evaluated on the same GPU (forward and gradients), plus size-independent
properties on the full problem (rows of P sum to one: V = 1 gives out = 1; linearity in V; determinism)."""
import math

import pytest
import torch

import elsa_b200 as E
from tests import _util as U

pytestmark = pytest.mark.gpu
F32, F16, BF16 = torch.float32, torch.float16, torch.bfloat16


def fp64_head(q, k, v, do, causal):
    """fp64 attention + gradients of ONE head on the GPU: q,k,v,do [N, D]."""
    q64, k64, v64 = (t.double().requires_grad_(True) for t in (q, k, v))
    s = (q64 @ k64.T) / math.sqrt(q.shape[-1])
    if causal:
        s = s.masked_fill(~torch.ones_like(s, dtype=torch.bool).tril(), float("-inf"))
    p = torch.softmax(s, dim=-1)
    out = p @ v64
    out.backward(do.double())
    return out.detach(), q64.grad, k64.grad, v64.grad


@pytest.mark.parametrize("dtype,causal,n", [(F16, False, 16384), (BF16, True, 16384), (F16, False, 4097)])
def test_one_head_of_the_headline_shape_vs_fp64(dtype, causal, n):
    b, h, d = 1, 8, 64
    q, k, v, do = (U.seeded((b, h, n, d), dtype, 200 + i).cuda() for i in range(4))
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    out = E.twopass_attention_train(qg, kg, vg, is_causal=causal)
    out.backward(do)
    head = 5
    ro, rq, rk, rv = fp64_head(q[0, head], k[0, head], v[0, head], do[0, head], causal)
    assert U.out_close(out[0, head], ro, dtype) <= 2.0
    lim = {F16: 2e-5, BF16: 2e-5}[dtype]
    for got, ref, nm in ((qg.grad, rq, "dq"), (kg.grad, rk, "dk"), (vg.grad, rv, "dv")):
        g = got[0, head].double()
        # task bound 2e-5 plus two spacings of the 16-bit output format at the gradient's magnitude
        tol = lim + 2 * U.ulp(dtype, float(ref.abs().max()))
        assert (g - ref).abs().max().item() <= tol, nm
    # determinism of the forward; the backward accumulates dQ with floating-point reductions whose order is
    # not fixed, so dQ is compared at one 16-bit spacing and dK, dV bit for bit
    out2 = E.twopass_attention(q, k, v, is_causal=causal)
    assert torch.equal(out2, out.detach())
    q2, k2, v2 = (t.clone().requires_grad_(True) for t in (q, k, v))
    E.twopass_attention_train(q2, k2, v2, is_causal=causal).backward(do)
    assert torch.equal(k2.grad, kg.grad) and torch.equal(v2.grad, vg.grad)
    assert (q2.grad.float() - qg.grad.float()).abs().max().item() <= U.ulp(dtype, float(qg.grad.float().abs().max()))


@pytest.mark.parametrize("dtype,causal,n,h", [(F16, False, 16384, 8), (BF16, True, 16384, 8), (F32, False, 65536, 1),
                                              (F32, False, 1024, 8)])
def test_full_size_properties(dtype, causal, n, h):
    b, d = 1, 64
    q, k = (U.seeded((b, h, n, d), dtype, 210 + i).cuda() for i in range(2))
    ones = torch.ones((b, h, n, d), dtype=dtype, device="cuda")
    out = E.twopass_attention(q, k, ones, is_causal=causal)
    # every row of P sums to one; fp32: z and s are two length-N fp32 sums in different orders, so the bound
    # grows like sqrt(N) from 2e-6 at N = 1024
    tol = {F32: 2e-6 * max(1.0, math.sqrt(n / 1024)), F16: 1e-3, BF16: 8e-3}[dtype]
    assert (out.float() - 1.0).abs().max().item() <= tol
    v1, v2 = (U.seeded((b, h, n, d), dtype, 220 + i).cuda() for i in range(2))
    o1 = E.twopass_attention(q, k, v1, is_causal=causal).float()
    o2 = E.twopass_attention(q, k, v2, is_causal=causal).float()
    o12 = E.twopass_attention(q, k, (v1.float() + v2.float()).to(dtype), is_causal=causal).float()
    lin_tol = {F32: 4e-6 * max(1.0, math.sqrt(n / 1024)), F16: 4e-3, BF16: 3e-2}[dtype]           # v1+v2 is itself rounded to the input dtype
    assert (o12 - (o1 + o2)).abs().max().item() <= lin_tol
    # sampled rows against fp64 on the same device
    rows = torch.tensor([0, 1, 127, 128, n // 2 + 3, n - 1], device="cuda")
    for head in (0, h - 1):
        s = (q[0, head, rows].double() @ k[0, head].double().T) / math.sqrt(d)
        if causal:
            s = s.masked_fill(torch.arange(n, device="cuda")[None, :] > rows[:, None], float("-inf"))
        ref = torch.softmax(s, -1) @ v1[0, head].double()
        got = E.twopass_attention(q, k, v1, is_causal=causal)[0, head, rows]
        assert U.out_close(got, ref, dtype) <= 2.0
