"""Helpers shared by the GPU parity tests: seeded inputs and thin wrappers that call the C ABI
directly on torch tensors (so the tests exercise exactly what a foreign-language binding would)."""
import math

import torch

from elsa_b200 import _lib

DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def seeded(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def stream():
    return torch.cuda.current_stream().cuda_stream


def phase1(q, k, v, *, part_width, bias=None, bias_strides=(0, 0, 0, 0), is_causal=False, summary_dtype=None,
           q_start=0, q_len=None, flags=0):
    """q,k,v: [B,H,N,D] cuda.  Returns (m, z, s) as [P, BH, q_len], [P, BH, q_len, D]."""
    lib = _lib.load()
    b, h, n, d = q.shape
    sdt = summary_dtype or q.dtype
    q_len = n - q_start if q_len is None else q_len
    parts = -(-n // part_width)
    m = torch.full((parts, b * h, q_len), float("nan"), device=q.device)
    z = torch.full_like(m, float("nan"))
    s = torch.full((parts, b * h, q_len, d), float("nan"), device=q.device, dtype=sdt)
    rc = lib.elsa_phase1_fold(q.data_ptr(), k.data_ptr(), v.data_ptr(),
                              None if bias is None else bias.data_ptr(), *bias_strides,
                              m.data_ptr(), z.data_ptr(), s.data_ptr(), DT[q.dtype], DT[sdt], b, h, n, d,
                              q_start, q_len, part_width, parts, int(is_causal), flags, stream())
    _lib.check(rc, "elsa_phase1_fold")
    return m, z, s


def merge_final(m, z, s, out_dtype, n_ctx, q_start=0, store_state=True):
    lib = _lib.load()
    parts, bh, q_len = m.shape
    d = s.shape[-1]
    out = torch.zeros((bh, n_ctx, d), device=m.device, dtype=out_dtype)
    rm = torch.zeros((bh, n_ctx), device=m.device)
    rz = torch.zeros_like(rm)
    rc = lib.elsa_merge_final(m.data_ptr(), z.data_ptr(), s.data_ptr(), out.data_ptr(), rm.data_ptr(), rz.data_ptr(),
                              DT[s.dtype], DT[out_dtype], parts, bh, q_start, q_len, n_ctx, d, int(store_state), stream())
    _lib.check(rc, "elsa_merge_final")
    return out, rm, rz


def finalize(m, z, s, out_dtype, n_ctx, final_part, q_start=0):
    lib = _lib.load()
    parts, bh, q_len = m.shape
    d = s.shape[-1]
    out = torch.zeros((bh, n_ctx, d), device=m.device, dtype=out_dtype)
    rm = torch.zeros((bh, n_ctx), device=m.device)
    rz = torch.zeros_like(rm)
    rc = lib.elsa_finalize(m.data_ptr(), z.data_ptr(), s.data_ptr(), out.data_ptr(), rm.data_ptr(), rz.data_ptr(),
                           DT[s.dtype], DT[out_dtype], final_part, bh, q_start, q_len, n_ctx, d, 1, stream())
    _lib.check(rc, "elsa_finalize")
    return out, rm, rz


def _pair(fn_name, m, z, s, n_out, *extra):
    lib = _lib.load()
    parts, bh, q_len = m.shape
    d = s.shape[-1]
    mo = torch.full((n_out, bh, q_len), float("nan"), device=m.device)
    zo = torch.full_like(mo, float("nan"))
    so = torch.full((n_out, bh, q_len, d), float("nan"), device=m.device, dtype=s.dtype)
    rc = getattr(lib, fn_name)(m.data_ptr(), z.data_ptr(), s.data_ptr(), mo.data_ptr(), zo.data_ptr(), so.data_ptr(),
                               DT[s.dtype], parts, bh, q_len, d, *extra, stream())
    _lib.check(rc, fn_name)
    return mo, zo, so


def scan_step(m, z, s, step):
    return _pair("elsa_scan_step", m, z, s, m.shape[0], step)


def upsweep(m, z, s):
    return _pair("elsa_upsweep_level", m, z, s, (m.shape[0] + 1) // 2)


def prefix_scan(m, z, s):
    return _pair("elsa_prefix_scan", m, z, s, m.shape[0])


def max_abs(a, b):
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    fin = torch.isfinite(b)
    assert torch.equal(torch.isfinite(a), fin), "finite pattern differs"
    if not fin.any():
        return 0.0
    return (a[fin] - b[fin]).abs().max().item()


def ulp(dtype, magnitude=1.0):
    """spacing of `dtype` just below `magnitude`"""
    bits = {torch.float16: 10, torch.bfloat16: 7, torch.float32: 23}[dtype]
    return 2.0 ** (math.floor(math.log2(max(magnitude, 1e-30))) - bits)


def out_close(got, ref, dtype):
    """Forward-output criterion, elementwise: fp32 <= 1e-6; fp16 <= 5e-4 or, where |ref| >= 1 so that
    one fp16 spacing already exceeds 5e-4, one spacing of the reference value; bf16 <= 5e-4 + two bf16
    spacings of the LARGEST reference value: the partition summaries s are stored in bf16 (the reference's
    default summary dtype is the input dtype) and partial sums of opposite sign cancel in the merge, so the
    absolute error of an element follows the size of the partial sums, not the element's own size.
    Returns the worst ratio err/limit (<= 1 passes)."""
    a = got.detach().double().cpu()
    b = ref.detach().double().cpu()
    assert torch.isfinite(a).all() and torch.isfinite(b).all()
    err = (a - b).abs()
    if dtype == torch.float32:
        lim = torch.full_like(err, 1e-6)
    else:
        bits = 10 if dtype == torch.float16 else 7
        spacing = torch.exp2(torch.floor(torch.log2(b.abs().clamp_min(1e-30))) - bits)
        lim = (torch.maximum(torch.full_like(err, 5e-4), spacing) if dtype == torch.float16
               else torch.full_like(err, 5e-4 + 2 * float(spacing.max())))
    return (err / lim).max().item()
