"""GPU parity of the backward path against the oracle, the reference fixtures and fp64 autograd.

Tolerances: gradients <= 1e-6 in fp32 (task statement).  For 16-bit inputs the task's 2e-5 was
measured by the reference with dO scaled by 0.1 on long rows; gradients here are O(0.1-1) and are
rounded to the input dtype, so the bound is 2e-5 + 2 output ulps of the largest gradient element
against the oracle (same rounding points), and the reference's own test tolerance against fp64.
"""
import pytest
import torch

import elsa_b200 as E
from oracle import elsa_oracle as O
from tests import _util as U

pytestmark = pytest.mark.gpu
DEV = "cuda"
F32, F16, BF16 = torch.float32, torch.float16, torch.bfloat16


def grad_tol(dtype, ref):
    if dtype == F32:
        return 1e-6 * max(1.0, float(ref.abs().max()))
    return 2e-5 + 2 * U.ulp(dtype, float(ref.float().abs().max()))


@pytest.mark.parametrize("name", ["bwd_f32_n70_d64", "bwd_f32_causal_n70_d64", "bwd_f16_n70_d64",
                                  "bwd_f16_causal_n70_d64", "bwd_swin_f32_n49_d32", "bwd_swin_f16_n49_d32"])
def test_backward_matches_reference_fixture(golden, name):
    g = golden(name)
    q, k, v, out, dout = (g[x].to(DEV) for x in ("q", "k", "v", "out", "dout"))
    bias = g.get("bias")
    causal = bool(g["causal"])
    biasd = None if bias is None else bias.to(DEV)
    dq, dk, dv = E.twopass_attention_backward(q, k, v, out, dout, bias=biasd, is_causal=causal,
                                              row_m=g["row_m"].to(DEV), row_z=g["row_z"].to(DEV))
    for got, nm in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert U.max_abs(got, g[nm]) <= grad_tol(q.dtype, g[nm]), nm
    # without saved state the statistics are recomputed (reference: _row_stats_kernel)
    dq2, dk2, dv2 = E.twopass_attention_backward(q, k, v, out, dout, bias=biasd, is_causal=causal)
    for got, nm in ((dq2, "dq"), (dk2, "dk"), (dv2, "dv")):
        assert U.max_abs(got, g[nm]) <= 4 * grad_tol(q.dtype, g[nm]), nm
    if "dbias" in g:
        from elsa_b200.attention_bwd import _backward_impl
        res = _backward_impl(q, k, v, out, dout, bias=biasd, is_causal=causal, row_m=g["row_m"].to(DEV),
                             row_z=g["row_z"].to(DEV), want_dbias=True)
        tol = (2e-6 if q.dtype == F32 else 2e-3) * max(1.0, float(g["dbias"].abs().max()))
        assert U.max_abs(res[3], g["dbias"]) <= tol


CASES = [
    # (B, H, N, D, dtype, causal, bias_kind)
    (1, 2, 64, 32, F32, False, None),
    (1, 2, 64, 32, F32, True, None),
    (1, 2, 64, 32, F16, False, None),
    (1, 2, 64, 32, F16, True, None),
    (1, 2, 193, 64, F32, False, None),
    (2, 2, 130, 64, F16, True, None),
    (1, 2, 257, 64, BF16, True, None),
    (1, 2, 100, 128, BF16, False, None),
    (1, 2, 75, 48, F32, True, None),
    (8, 3, 49, 32, F16, False, "1hnn"),
    (8, 3, 49, 32, F32, False, "bhnn"),
    (2, 3, 49, 32, F32, False, "b1nn"),
    (2, 3, 60, 32, F32, False, "nn"),
    (2, 3, 60, 32, F16, True, "hnn"),
    (1, 2, 1025, 64, F16, False, None),
    # head dims below 64 on the tensor cores (N >= 512, no bias)
    (1, 2, 640, 32, F16, False, None),
    (1, 2, 777, 32, BF16, True, None),
    (1, 2, 600, 48, F16, True, None),
    (1, 2, 640, 32, F32, False, None),
    (1, 2, 900, 40, F32, True, None),
    # head dims above 64 on the tensor cores (16-bit inputs)
    (1, 2, 640, 128, F16, False, None),
    (1, 2, 777, 96, BF16, True, None),
    (2, 1, 1030, 72, F16, True, None),
    # biased problems on the tensor cores, with the bias gradient (16-bit inputs)
    (2, 2, 640, 64, F16, False, "bhnn"),
    (2, 3, 600, 32, BF16, False, "1hnn"),
    (1, 2, 777, 96, F16, True, "hnn"),
    (2, 2, 520, 128, BF16, False, "b1nn"),
    (1, 2, 1030, 64, F16, True, "nn"),
    (2, 2, 640, 64, F32, False, "bhnn"),
    (1, 3, 900, 40, F32, True, "hnn"),
    (2, 2, 1024, 32, F32, False, "b1nn"),
    # 65 to 511 tokens with at least 4096 rows in total: the tensor-core kernels
    (24, 3, 197, 64, F16, False, None),
    (6, 4, 257, 64, BF16, True, None),
    (12, 3, 197, 32, F32, False, None),
    (12, 3, 150, 64, F16, False, "1hnn"),
    (8, 3, 197, 96, BF16, False, None),
    (10, 3, 160, 40, F32, True, "bhnn"),
    # sequences of at most 64 tokens, 16-bit: two per tensor-core tile (odd batch: the last tile is half empty)
    (5, 3, 49, 32, BF16, False, "1hnn"),
    (3, 2, 64, 64, F16, False, "bhnn"),
    (4, 3, 49, 32, F16, False, "b1nn"),
    (6, 4, 16, 64, BF16, False, "hnn"),
    (2, 2, 7, 24, F16, False, None),
    (1, 1, 1, 8, BF16, False, None),
    (7, 2, 33, 40, F16, False, "nn"),
    (5, 2, 49, 32, F16, True, None),          # causal windows
    (4, 3, 64, 64, BF16, True, "1hnn"),
]


def make_bias(kind, b, h, n, seed):
    if kind is None:
        return None
    shape = {"nn": (n, n), "hnn": (h, n, n), "1hnn": (1, h, n, n), "b1nn": (b, 1, n, n), "bhnn": (b, h, n, n)}[kind]
    return U.seeded(shape, F32, seed, 0.05)


@pytest.mark.parametrize("case", CASES, ids=lambda c: "-".join(str(x).replace("torch.", "") for x in c))
def test_train_vs_oracle_and_fp64(case):
    b, h, n, d, dtype, causal, bias_kind = case
    q = U.seeded((b, h, n, d), dtype, 60, 0.5)
    k = U.seeded((b, h, n, d), dtype, 61, 0.5)
    v = U.seeded((b, h, n, d), dtype, 62)
    dout = U.seeded((b, h, n, d), dtype, 63, 0.25)
    bias = make_bias(bias_kind, b, h, n, 64)

    qd, kd, vd = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    biasd = None if bias is None else bias.to(DEV).requires_grad_(True)
    out = E.twopass_attention_train(qd, kd, vd, bias=biasd, is_causal=causal)
    out.backward(dout.to(DEV))

    o_ref, rm, rz = O.twopass_forward(q, k, v, bias=bias, is_causal=causal, training=True)
    # the oracle's backward starts from the CUDA forward's saved output so that both sides see the same D
    res = O.twopass_backward(q, k, v, out.detach().cpu(), dout, rm, rz, bias=bias, is_causal=causal,
                             want_dbias=bias is not None)
    for got, ref, nm in ((qd.grad, res[0], "dq"), (kd.grad, res[1], "dk"), (vd.grad, res[2], "dv")):
        assert got.dtype == dtype
        assert U.max_abs(got, ref) <= grad_tol(dtype, ref), nm
    if bias is not None:
        ref_db = O.reduce_dbias(res[3], bias, b, h)
        assert biasd.grad.shape == bias.shape
        assert U.max_abs(biasd.grad, ref_db) <= (2e-6 if dtype == F32 else 2e-3) * max(1.0, float(ref_db.abs().max()))

    # absolute truth: fp64 autograd (the reference's tests use fp32 SDPA with atol=rtol 2.5e-3 / 8e-2)
    q64, k64, v64 = (t.double().requires_grad_(True) for t in (q, k, v))
    b64 = None if bias is None else bias.double().requires_grad_(True)
    O.softmax_attention_fp64(q64, k64, v64, bias=b64, is_causal=causal).backward(dout.double())
    lim = {F32: 2e-6, F16: 2e-3, BF16: 1.6e-2}[dtype]
    for got, ref in ((qd.grad, q64.grad), (kd.grad, k64.grad), (vd.grad, v64.grad)):
        assert U.max_abs(got, ref) <= lim * max(1.0, float(ref.abs().max()))
    if bias is not None:
        assert U.max_abs(biasd.grad, b64.grad) <= lim * max(1.0, float(b64.grad.abs().max()))


@pytest.mark.parametrize("b,n,d", [(1, 150, 64), (3, 49, 32), (28, 150, 64), (4, 640, 64)])
def test_backward_is_deterministic_and_masked_rows_are_zero(b, n, d):
    h = 2
    q, k, v, do = (U.seeded((b, h, n, d), F16, 70 + i).to(DEV) for i in range(4))
    bias = torch.zeros(n, n, device=DEV)
    bias[7, :] = float("-inf")
    out, rm, rz = E.twopass_attention_with_state(q, k, v, bias=bias)
    a = E.twopass_attention_backward(q, k, v, out, do, bias=bias, row_m=rm, row_z=rz)
    c = E.twopass_attention_backward(q, k, v, out, do, bias=bias, row_m=rm, row_z=rz)
    for x, y in zip(a, c):
        assert torch.equal(x, y)
        assert torch.isfinite(x).all()
    assert float(a[0][:, :, 7].abs().max()) == 0.0


def test_preprocess_abi():
    from elsa_b200 import _lib
    lib = _lib.load()
    bh, n, d = 3, 77, 48
    out = U.seeded((bh, n, d), BF16, 80).to(DEV)
    dout = U.seeded((bh, n, d), BF16, 81).to(DEV)
    rm = U.seeded((bh, n), F32, 82).to(DEV)
    rz = (U.seeded((bh, n), F32, 83).abs() + 0.1).to(DEV)
    rm[0, 0] = float("-inf"); rz[0, 0] = 0
    rd = torch.empty_like(rm); lse = torch.empty_like(rm)
    rc = lib.elsa_bwd_preprocess(out.data_ptr(), dout.data_ptr(), rm.data_ptr(), rz.data_ptr(), rd.data_ptr(),
                                 lse.data_ptr(), 2, bh, n, d, U.stream())
    assert rc == 0
    ref_d, ref_l = O.bwd_preprocess(out.cpu(), dout.cpu(), rm.cpu(), rz.cpu())
    assert U.max_abs(rd, ref_d) <= 1e-5 and U.max_abs(lse, ref_l) <= 1e-5


@pytest.mark.parametrize("dtype,causal", [(torch.float16, False), (torch.bfloat16, True)])
def test_tensor_core_path_repeats_bit_for_bit(dtype, causal):
    """The tcgen05 kernels hand tiles between warps through mbarriers and reuse TMEM columns and shared-memory stages:
    a missing ordering would show up as run-to-run differences.  out, row state, dK and dV have a fixed summation
    order and must repeat bit for bit; dQ is summed by TMA reduce-adds whose order varies, so it repeats to one spacing of
    the output type only."""
    import elsa_b200 as E
    b, h, n, d = 1, 4, 4096 + 77, 64
    g = torch.Generator().manual_seed(4242)
    q, k, v, do = (torch.randn(b, h, n, d, generator=g).to(dtype).cuda() for _ in range(4))
    ref = None
    for rep in range(12):
        out, rm, rz = E.twopass_attention_with_state(q, k, v, is_causal=causal)[:3]
        dq, dk, dv = E.twopass_attention_backward(q, k, v, out, do, row_m=rm, row_z=rz, is_causal=causal)
        cur = [t.clone() for t in (out, rm, rz, dk, dv, dq)]
        if ref is None:
            ref = cur
            continue
        for name, a, r in zip(("out", "row_m", "row_z", "dk", "dv"), cur[:5], ref[:5]):
            assert torch.equal(a, r), (name, rep)
        scale = ref[5].float().abs().max().item()
        # one spacing of the output type at the largest magnitude: a different fp32 summation order can move a
        # value across a rounding boundary, nothing more
        assert (cur[5].float() - ref[5].float()).abs().max().item() <= scale * (2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7), rep


@pytest.mark.parametrize("n,causal,h", [(512, False, 2), (1000, True, 2), (1153, False, 3), (4097, True, 1)])
def test_fp32_tensor_core_backward_matches_the_fma_backward_and_fp64(n, causal, h):
    """fp32 inputs with head dim 64 and at least 512 tokens take the tensor-core backward (two fp16 planes per
    operand, fresh accumulators per tile pair); ELSA_FLAG_FP32_FMA selects the FP32-FMA kernels.  Both must meet the
    fp32 gradient bound against fp64, and the tensor-core result must repeat bit for bit (no atomics anywhere)."""
    from elsa_b200 import _lib
    from elsa_b200.attention_bwd import _backward_impl
    g = torch.Generator().manual_seed(900 + n)
    q, k, v, do = (torch.randn(1, h, n, 64, generator=g).to(DEV) for _ in range(4))
    out, rm, rz = E.twopass_attention_with_state(q, k, v, is_causal=causal)[:3]
    tc = _backward_impl(q, k, v, out, do, bias=None, is_causal=causal, row_m=rm, row_z=rz, want_dbias=False)[:3]
    tc2 = _backward_impl(q, k, v, out, do, bias=None, is_causal=causal, row_m=rm, row_z=rz, want_dbias=False)[:3]
    fma = _backward_impl(q, k, v, out, do, bias=None, is_causal=causal, row_m=rm, row_z=rz, want_dbias=False,
                         flags=_lib.FLAG_FP32_FMA)[:3]
    q64, k64, v64 = (t.cpu().double().requires_grad_(True) for t in (q, k, v))
    O.softmax_attention_fp64(q64, k64, v64, bias=None, is_causal=causal).backward(do.cpu().double())
    for name, a, a2, b, ref in zip(("dq", "dk", "dv"), tc, tc2, fma, (q64.grad, k64.grad, v64.grad)):
        assert torch.equal(a, a2), name
        bound = 2e-6 * max(1.0, float(ref.abs().max()))
        assert U.max_abs(a, ref) <= bound, (name, "tensor cores")
        # (the FP32-FMA kernels sum a row's thousands of terms in one fp32 chain per thread: twice the bound at N = 4097)
        assert U.max_abs(b, ref) <= 2 * bound, (name, "fma")


def test_fp32_tensor_core_backward_keeps_its_accuracy_on_long_rows():
    """On long rows dS = P (dP - D) is orders of magnitude below any a-priori bound (P ~ 1/N); the fp16-plane kernels
    scale every row of every tile pair by its own largest |dS| so that the second fp16 term stays normal.  With a fixed
    scale dQ and dK were 2.5e-5 (relative) off at N = 65536.  Checked against the FP32-FMA kernels (each is within
    1e-6 of fp64 at the sizes where fp64 fits)."""
    from elsa_b200 import _lib
    from elsa_b200.attention_bwd import _backward_impl
    n = 32768
    g = torch.Generator().manual_seed(77)
    q, k, v, do = (torch.randn(1, 1, n, 64, generator=g).to(DEV) for _ in range(4))
    out, rm, rz = E.twopass_attention_with_state(q, k, v)[:3]
    tc = _backward_impl(q, k, v, out, do, bias=None, is_causal=False, row_m=rm, row_z=rz, want_dbias=False)[:3]
    fma = _backward_impl(q, k, v, out, do, bias=None, is_causal=False, row_m=rm, row_z=rz, want_dbias=False,
                         flags=_lib.FLAG_FP32_FMA)[:3]
    for name, a, b in zip(("dq", "dk", "dv"), tc, fma):
        assert U.max_abs(a, b) <= 1.5e-6 * max(1.0, float(b.abs().max())), name
        # relative to the gradient's own size: the fixed-scale version failed this by a factor of five
        assert U.max_abs(a, b) <= 1e-5 * float(b.abs().max()), name


def test_first_cuda_call_of_a_thread_may_be_the_backward():
    """An autograd worker thread whose first CUDA work is this library's has no driver context bound yet; the
    tensor-map encode of the tensor-core kernels needs one.  Everything is allocated beforehand so that the library
    call is the thread's first CUDA call."""
    import threading
    b, h, n, d = 6, 3, 49, 32
    q, k, v, do = (U.seeded((b, h, n, d), F16, 90 + i).to(DEV) for i in range(4))
    out, rm, rz = E.twopass_attention_with_state(q, k, v)
    ref = E.twopass_attention_backward(q, k, v, out, do, row_m=rm, row_z=rz)
    del ref                                        # (its blocks go back to the caching allocator for the thread's call)
    res = {}

    def work():
        try:
            res["g"] = E.twopass_attention_backward(q, k, v, out, do, row_m=rm, row_z=rz)
        except Exception as exc:  # noqa: BLE001
            res["err"] = exc

    t = threading.Thread(target=work)
    t.start(); t.join()
    assert "err" not in res, res.get("err")
    again = E.twopass_attention_backward(q, k, v, out, do, row_m=rm, row_z=rz)
    for x, y in zip(res["g"], again):
        assert torch.equal(x, y)


@pytest.mark.parametrize("b,h,n,d,dtype,bias_kind", [
    (301, 3, 49, 32, F16, "1hnn"),      # odd batch, a bias shared by the batch (staged once per CTA), dbias by reduction
    (77, 2, 64, 64, BF16, "bhnn"),      # a bias per sequence (staged for every pair), dbias by plain stores
    (150, 4, 49, 32, F16, None),
    (333, 5, 16, 24, BF16, "hnn"),
])
def test_many_windows_per_cta_vs_fp64_and_fma(b, h, n, d, dtype, bias_kind):
    """More pairs of sequences than CTAs: the persistent backward walks several pairs per CTA through its two stages
    of shared memory and its barrier phases.  Checked against fp64 autograd on the GPU and against the FP32-FMA
    kernels of the same library."""
    from elsa_b200 import _lib
    from elsa_b200.attention import _forward_impl
    from elsa_b200.attention_bwd import _backward_impl
    q = U.seeded((b, h, n, d), dtype, 110, 0.5).to(DEV)
    k = U.seeded((b, h, n, d), dtype, 111, 0.5).to(DEV)
    v = U.seeded((b, h, n, d), dtype, 112).to(DEV)
    do = U.seeded((b, h, n, d), dtype, 113, 0.25).to(DEV)
    bias = make_bias(bias_kind, b, h, n, 114)
    bias = None if bias is None else bias.to(DEV)
    res = {}
    for tag, fl in (("tc", 0), ("fma", _lib.FLAG_FORCE_SIMT)):
        o, rm, rz = _forward_impl(q, k, v, bias=bias, is_causal=False, summary_dtype=dtype, part_width=0, q_chunk=0,
                                  want_state=True, flags=fl)[:3]
        g = _backward_impl(q, k, v, o, do, bias=bias, is_causal=False, row_m=rm, row_z=rz, want_dbias=bias is not None,
                           flags=fl)
        res[tag] = (o,) + tuple(g)
    q64, k64, v64 = (t.double().requires_grad_(True) for t in (q, k, v))
    b64 = None if bias is None else bias.double().requires_grad_(True)
    s64 = q64 @ k64.transpose(-1, -2) / d ** 0.5
    if b64 is not None:
        s64 = s64 + b64
    o64 = torch.softmax(s64, dim=-1) @ v64
    o64.backward(do.double())
    refs = [o64.detach(), q64.grad, k64.grad, v64.grad] + ([] if b64 is None else [b64.grad])
    lim = {F16: 2e-3, BF16: 1.6e-2}[dtype]
    for i, ref in enumerate(refs):
        scale = max(1.0, float(ref.abs().max()))
        assert U.max_abs(res["tc"][i].double().cpu(), ref.cpu()) <= lim * scale, i
        # the two kernel families round P and dS at different points: a few output ulps apart
        assert U.max_abs(res["tc"][i].double().cpu(), res["fma"][i].double().cpu()) <= lim * scale, i
