"""q, k, v read in place from a packed projection output, `out` and the gradients written in the layout the model
hooks need: no copy kernels on either side of the operator, and the same bits as the contiguous path.

The test counts the library's own launches (elsa_kernel_launches) and checks with torch's profiler that no copy /
elementwise kernel of PyTorch runs between the projection output and the operator's result."""
import pytest
import torch
from torch.profiler import ProfilerActivity, profile

import elsa_b200 as E
from elsa_b200 import _lib
from elsa_b200.attention_bwd import twopass_attention_qkvpacked
from tests import _util as U

pytestmark = pytest.mark.gpu
F16, BF16, F32 = torch.float16, torch.bfloat16, torch.float32


def _cuda_kernel_names(fn):
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        fn()
        torch.cuda.synchronize()
    return [e.key for e in prof.key_averages() if e.device_type == torch.autograd.DeviceType.CUDA]


@pytest.mark.parametrize("dtype,b,h,n,d,causal", [(F16, 2, 3, 4097, 64, False),     # tensor-core kernels, ragged length
                                                  (BF16, 1, 4, 1000, 64, True),
                                                  (F32, 2, 3, 197, 64, False),      # FP32-FMA kernels
                                                  (F16, 4, 3, 49, 32, False)])      # Swin-sized windows
def test_packed_views_are_read_in_place_and_match_the_contiguous_path(dtype, b, h, n, d, causal):
    lib = _lib.load()
    qkv = U.seeded((b, n, 3, h, d), dtype, 60).cuda()
    q, k, v = qkv.permute(2, 0, 3, 1, 4).unbind(0)
    assert not q.is_contiguous()
    ref = E.twopass_attention(q.contiguous(), k.contiguous(), v.contiguous(), is_causal=causal)
    l0 = lib.elsa_kernel_launches()
    names = _cuda_kernel_names(lambda: E.twopass_attention(q, k, v, is_causal=causal))
    out = E.twopass_attention(q, k, v, is_causal=causal)
    # phase 1 + phase 2 per call, profiled call and this one; one launch per call where phase 1 finalises the rows itself
    # (a sequence of at most 64 tokens; a single partition on the 16-bit tensor-core fold)
    import ctypes
    n_parts = ctypes.c_int()
    assert lib.elsa_forward_plan(_lib.dtype_code(dtype), _lib.dtype_code(dtype), b, h, n, d, 0, int(causal), 0, 0, 0, None,
                                 ctypes.byref(n_parts), None) == 0
    one_launch = n <= 64 or (dtype != F32 and n_parts.value == 1 and lib.elsa_uses_tensor_cores_for(_lib.dtype_code(dtype), d, n, 0, int(causal), 0, b, h))
    assert lib.elsa_kernel_launches() - l0 == (2 if one_launch else 4)
    assert not any("copy" in nm.lower() or "elementwise" in nm.lower() for nm in names), names
    assert torch.equal(out, ref)                                     # same kernels, same arithmetic: same bits
    # the result sits in [B, N, H, D] memory: the hooks' transpose + reshape is a view
    merged = out.transpose(1, 2).reshape(b, n, h * d)
    assert merged.data_ptr() == out.data_ptr() and merged.is_contiguous()


@pytest.mark.parametrize("dtype,b,h,n,d,causal,bias", [(F16, 2, 3, 1025, 64, False, False), (BF16, 1, 2, 640, 64, True, False),
                                                       (F32, 1, 3, 130, 64, True, False), (F16, 6, 3, 49, 32, False, True)])
def test_packed_training_step_matches_the_unpacked_operator(dtype, b, h, n, d, causal, bias):
    qkv = U.seeded((b, n, 3, h, d), dtype, 61).cuda()
    do = U.seeded((b, n, h * d), dtype, 62, 0.5).cuda()
    bias_t = (U.seeded((1, h, n, n), F32, 63, 0.05).cuda().requires_grad_(True)) if bias else None
    # reference: contiguous q, k, v through the ordinary autograd operator
    q, k, v = (t.contiguous().requires_grad_(True) for t in qkv.permute(2, 0, 3, 1, 4).unbind(0))
    out_r = E.twopass_attention_train(q, k, v, bias=bias_t, is_causal=causal)
    out_r.transpose(1, 2).reshape(b, n, h * d).backward(do)
    dbias_r = None if bias_t is None else bias_t.grad.clone()
    if bias_t is not None:
        bias_t.grad = None
    # packed: one tensor in, one gradient tensor out
    pk = qkv.clone().requires_grad_(True)
    out_p = twopass_attention_qkvpacked(pk, bias=bias_t, is_causal=causal)
    y = out_p.transpose(1, 2).reshape(b, n, h * d)
    assert y.data_ptr() == out_p.data_ptr()
    names = _cuda_kernel_names(lambda: y.backward(do))
    assert not any("copy" in nm.lower() or "cat" in nm.lower() for nm in names), names
    assert torch.equal(out_p, out_r)
    gq, gk, gv = pk.grad.permute(2, 0, 3, 1, 4).unbind(0)
    if dtype == F32:
        # fp32: the contiguous operator takes the fused backward, the packed one the two-kernel backward
        for got, ref in ((gk, k.grad), (gv, v.grad)):
            assert (got - ref).abs().max().item() <= 2e-6 * max(1.0, float(ref.abs().max()))
    else:
        assert torch.equal(gk, k.grad) and torch.equal(gv, v.grad)
    # dQ of the tensor-core path is accumulated by reductions whose order is not fixed: one output spacing
    # fp32 with a contiguous dq takes the fused backward, whose dQ is summed by reductions in arrival order as well
    big = float(q.grad.float().abs().max())
    tol = 2e-6 * max(1.0, big) if dtype == F32 else (0.0 if n < 512 else U.ulp(dtype, big))
    assert (gq.float() - q.grad.float()).abs().max().item() <= tol
    if bias_t is not None:
        assert torch.allclose(bias_t.grad, dbias_r, rtol=0, atol=2e-6 * max(1.0, float(dbias_r.abs().max())))


def test_layouts_that_cannot_be_read_in_place_are_copied():
    b, h, n, d = 1, 2, 200, 64
    x = U.seeded((b, h, n, d + 8), F16, 64).cuda()
    q = x[..., 4:4 + d]                      # rows start 8 bytes off a 16-byte boundary: copied, still correct
    k = x[..., :d]                           # row stride 72 elements: readable in place
    v = U.seeded((b, h, d, n), F16, 65).cuda().transpose(2, 3)     # D axis not contiguous: copied
    out = E.twopass_attention(q, k, v)
    ref = E.twopass_attention(q.contiguous(), k.contiguous(), v.contiguous())
    assert torch.equal(out, ref)
