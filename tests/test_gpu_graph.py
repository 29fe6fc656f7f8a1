"""The forward and backward entry points allocate nothing and never synchronise, so a whole training step can be
captured into a CUDA graph and replayed on new data (the reference captures its model the same way,
benchmarks/full_model_graph.py:41-44).  Tensor-core path (fp16, N = 640) and FP32-FMA path with a bias gradient."""
import pytest
import torch

import elsa_b200 as E
from tests import _util as U

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,n,d,causal,use_bias", [(torch.float16, 640, 64, True, False),
                                                       (torch.float32, 49, 32, False, True)])
def test_training_step_replays_from_a_cuda_graph(dtype, n, d, causal, use_bias):
    b, h = 2, 3
    q, k, v, do = (U.seeded((b, h, n, d), dtype, 300 + i).cuda() for i in range(4))
    bias = (U.seeded((1, h, n, n), torch.float32, 310).cuda() * 0.1).requires_grad_(True) if use_bias else None
    sq, sk, sv = (t.clone().requires_grad_(True) for t in (q, k, v))
    sdo = do.clone()

    def step():
        for t in (sq, sk, sv, bias):
            if t is not None:
                t.grad = None
        out = E.twopass_attention_train(sq, sk, sv, bias=bias, is_causal=causal)
        out.backward(sdo)
        return out

    # warm-up on a side stream (first calls set function attributes and build tensor maps), then capture
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out_g = step()
    grads_g = [sq.grad, sk.grad, sv.grad] + ([bias.grad] if use_bias else [])

    # replay on different data written into the captured tensors
    q2, k2, v2, do2 = (U.seeded((b, h, n, d), dtype, 400 + i).cuda() for i in range(4))
    with torch.no_grad():
        sq.copy_(q2); sk.copy_(k2); sv.copy_(v2); sdo.copy_(do2)
    graph.replay()
    torch.cuda.synchronize()
    got = [out_g.clone()] + [g.clone() for g in grads_g]

    eq, ek, ev = (t.clone().requires_grad_(True) for t in (q2, k2, v2))
    ebias = bias.detach().clone().requires_grad_(True) if use_bias else None
    out_e = E.twopass_attention_train(eq, ek, ev, bias=ebias, is_causal=causal)
    out_e.backward(do2)
    want = [out_e.detach(), eq.grad, ek.grad, ev.grad] + ([ebias.grad] if use_bias else [])
    # same kernels on the same data; only the fp32 atomics of the dQ / dbias reductions may reorder
    for name, a, w in zip(("out", "dq", "dk", "dv", "dbias"), got, want):
        tol = 1e-6 if dtype == torch.float32 else 2e-3
        assert (a.float() - w.float()).abs().max().item() <= tol * max(1.0, w.float().abs().max().item()), name
    from elsa_b200 import _lib
    assert _lib.load().elsa_device_status(0) == 0
