"""Generate the golden fixtures in this directory from the reference's own device code.

Runs ONLY where the reference checkout and Triton are available (the build container):
    python tests/golden/make_golden.py [/path/to/reference]
The reference's `@triton.jit` kernels are executed by Triton's CPU interpreter
(TRITON_INTERPRET=1) on CPU tensors, driven by the same host loops the reference uses
(attention_parallel_scan.py:667-753, 861-955; attention_bwd.py:739-838, 939-970).  The
interpreter cannot execute bf16, and the reference's single CUDA kernel cannot run without a
GPU, so fixtures cover fp32 and fp16 and stop at the phase-1 summaries for the d64 fast path.

Every fixture is one .npz holding the inputs and the reference's outputs.
"""
import math
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/make_golden.py <checkout of ming053l/ELSA>")
REF = sys.argv[1]
sys.path.insert(0, os.path.join(REF, "src"))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402

import elsa_twopass_clean.attention as A  # noqa: E402
import elsa_twopass_clean.attention_bwd as BW  # noqa: E402
import elsa_twopass_clean.attention_parallel_scan as APS  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
LOG2E = 1.4426950408889634


def _np(t):
    return t.detach().cpu().numpy()


def _randn(gen, shape, dtype, scale=1.0):
    return (torch.randn(shape, generator=gen) * scale).to(dtype)


def _unblock(buf, kb, qb, bh, bm, n, d=None):
    """reference summary layout [kb][qb][bh][bm](,d) -> [kb][bh][n](,d)."""
    if d is None:
        t = buf.view(kb, qb, bh, bm).permute(0, 2, 1, 3).reshape(kb, bh, qb * bm)
        return t[:, :, :n].contiguous()
    t = buf.view(kb, qb, bh, bm, d).permute(0, 2, 1, 3, 4).reshape(kb, bh, qb * bm, d)
    return t[:, :, :n].contiguous()


def save(name, **arrays):
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **{k: _np(v) if torch.is_tensor(v) else np.asarray(v) for k, v in arrays.items()})
    print("wrote", name)


def fwd_generic(name, seed, shape, dtype, bm, bn, *, causal=False, bias_shape=None, mask_frac=0.0):
    gen = torch.Generator().manual_seed(seed)
    B, H, N, D = shape
    q, k, v = (_randn(gen, shape, dtype) for _ in range(3))
    sdt = dtype
    bh = B * H
    kb = triton.cdiv(N, bn)
    qb = triton.cdiv(N, bm)
    el = kb * qb * bh * bm
    bufs = [(torch.zeros(el), torch.zeros(el), torch.zeros(el, D, dtype=sdt)) for _ in range(2)]
    bias = None
    if bias_shape is not None:
        bias = torch.randn(bias_shape, generator=gen) * 0.02
        if mask_frac > 0:
            # shifted-window style: additive 0 / -100 mask folded into the bias
            msk = (torch.rand(bias_shape[-2:], generator=gen) < mask_frac).float() * -100.0
            msk.fill_diagonal_(0.0)
            bias = bias + msk
    meta = A._canonical_bias(bias, batch=B, heads=H, seq_len=N, device=q.device)
    bd = A._next_power_of_2(D)
    A._phase1_summary_kernel[(qb, bh, kb)](
        q, k, v, meta.tensor, *bufs[0], 0, H, N, D, kb, qb, bm, bn, bd, 1 / math.sqrt(D), "ieee",
        meta.has_bias, causal, dtype != torch.float16 or sdt == torch.float32,
        meta.stride_b, meta.stride_h, meta.stride_q, meta.stride_k)
    p1 = tuple(t.clone() for t in bufs[0])
    src, dst = bufs
    if causal:
        step = 1
        while step < kb:
            APS._summary_scan_step_kernel[(kb, qb, bh)](*src, *dst, step, qb, bh, D, bm, bd)
            src, dst = dst, src
            step *= 2
        final_kb = kb - 1
    else:
        inb = kb
        while inb > 1:
            ob = triton.cdiv(inb, 2)
            APS._summary_blelloch_upsweep_kernel[(ob, qb, bh)](*src, *dst, inb, qb, bh, D, bm, bd)
            src, dst = dst, src
            inb = ob
        final_kb = 0
    out = torch.empty_like(q)
    rm = torch.empty(bh, N)
    rz = torch.empty(bh, N)
    APS._scan_last_to_out_kernel[(qb, bh)](*src, out, rm, rz, 0, N, D, final_kb, qb, bh, bm, bd, True)
    arrays = dict(q=q, k=k, v=v, out=out, row_m=rm, row_z=rz,
                  p1_m=_unblock(p1[0], kb, qb, bh, bm, N), p1_z=_unblock(p1[1], kb, qb, bh, bm, N),
                  p1_s=_unblock(p1[2], kb, qb, bh, bm, N, D),
                  block_m=bm, block_n=bn, causal=int(causal))
    if causal:
        arrays.update(scan_m=_unblock(src[0], kb, qb, bh, bm, N), scan_z=_unblock(src[1], kb, qb, bh, bm, N),
                      scan_s=_unblock(src[2], kb, qb, bh, bm, N, D))
    if bias is not None:
        arrays["bias"] = bias
    save(name, **arrays)


def fwd_d64(name, seed, shape, dtype, bm, bn):
    """d64 fast phase-1 kernels (tiled when bn > 512 like the reference's own routing)."""
    gen = torch.Generator().manual_seed(seed)
    B, H, N, D = shape
    assert D == 64
    q, k, v = (_randn(gen, shape, dtype) for _ in range(3))
    bh = B * H
    kb = triton.cdiv(N, bn)
    qb = triton.cdiv(N, bm)
    el = kb * qb * bh * bm
    m = torch.zeros(el); z = torch.zeros(el); s = torch.zeros(el, 64, dtype=dtype)
    needs_mask = 1 if (N % bn != 0 or N % bm != 0) else 0
    ls = (1 / 8) * LOG2E
    if bn > 512:
        kern = APS._phase1_d64_tiled_fp32_nomask_kernel if dtype == torch.float32 else APS._phase1_d64_tiled_fp16_nomask_kernel
        kern[(qb, bh, kb)](q, k, v, m, z, s, 0, N, qb, bm, bn, 64, ls, "ieee", needs_mask)
    else:
        kern = APS._phase1_d64_fp32_nomask_kernel if dtype == torch.float32 else APS._phase1_d64_fp16_nomask_kernel
        kern[(qb, bh, kb)](q, k, v, m, z, s, 0, N, qb, bm, bn, ls, "ieee", needs_mask)
    save(name, q=q, k=k, v=v, p1_m=_unblock(m, kb, qb, bh, bm, N), p1_z=_unblock(z, kb, qb, bh, bm, N),
         p1_s=_unblock(s, kb, qb, bh, bm, N, 64), block_m=bm, block_n=bn)


def bwd(name, seed, shape, dtype, *, causal=False, bias_shape=None, dbias=False):
    gen = torch.Generator().manual_seed(seed)
    B, H, N, D = shape
    q = _randn(gen, shape, dtype, 0.5); k = _randn(gen, shape, dtype, 0.5); v = _randn(gen, shape, dtype)
    do = _randn(gen, shape, dtype, 0.25)
    bias = None if bias_shape is None else torch.randn(bias_shape, generator=gen) * 0.02
    meta = A._canonical_bias(bias, batch=B, heads=H, seq_len=N, device=q.device)
    bargs = (meta.stride_b, meta.stride_h, meta.stride_q, meta.stride_k)
    bh = B * H
    bm, bn = (32, 32) if dtype == torch.float32 else (64, 32)
    bd = A._next_power_of_2(D)
    sc = 1 / math.sqrt(D)
    grid = (bh, triton.cdiv(N, bm))
    rm = torch.empty(bh, N); rz = torch.empty(bh, N)
    BW._row_stats_kernel[grid](q, k, meta.tensor, rm, rz, H, N, D, bm, bn, bd, sc, "ieee", meta.has_bias, causal, *bargs)
    # forward output from fp64 math, rounded to the input dtype (what a forward would have saved)
    s = (q.double() @ k.double().transpose(-1, -2)) * sc
    if bias is not None:
        s = s + meta.tensor.double()
    if causal:
        s = s.masked_fill(~torch.ones(N, N, dtype=torch.bool).tril(), float("-inf"))
    out = (torch.softmax(s, -1) @ v.double()).to(dtype)
    rd = torch.empty_like(rm); lse = torch.empty_like(rm)
    BW._bwd_preprocess_kernel[grid](out, do, rm, rz, rd, lse, N, D, bm, bd)
    dq = torch.empty_like(q); dk = torch.empty_like(q); dv = torch.empty_like(q)
    BW._bwd_dq_kernel[grid](q, k, v, meta.tensor, do, lse, rd, dq, H, N, D, bm, bn, bd, sc, "ieee", meta.has_bias, causal, *bargs)
    BW._bwd_dkdv_kernel[(bh, triton.cdiv(N, bn))](q, k, v, meta.tensor, do, lse, rd, dk, dv, H, N, D, bm, bn, bd, sc, "ieee",
                                                   meta.has_bias, causal, *bargs)
    arrays = dict(q=q, k=k, v=v, out=out, dout=do, row_m=rm, row_z=rz, row_d=rd, row_lse=lse, dq=dq, dk=dk, dv=dv,
                  causal=int(causal))
    if bias is not None:
        arrays["bias"] = bias
    if dbias:
        assert bias is not None and bias.dim() == 4 and bias.shape[1] == H
        tb = 16 if N <= 128 else 32
        db = torch.empty_like(meta.tensor, dtype=torch.float32)
        one = bias.shape[0] == 1
        BW._dbias_dense_kernel[(1 if one else B, H, triton.cdiv(N, tb) * triton.cdiv(N, tb))](
            q, k, v, out, do, rm, rz, meta.tensor, db, B, H, N, D, tb, tb, bd, sc, "ieee", one, causal)
        arrays["dbias"] = db
    save(name, **arrays)


if __name__ == "__main__":
    f32, f16 = torch.float32, torch.float16
    fwd_generic("fwd_generic_f32_n96_d64", 101, (1, 2, 96, 64), f32, 32, 32)
    fwd_generic("fwd_generic_f16_n100_d32", 102, (2, 2, 100, 32), f16, 64, 64)
    fwd_generic("fwd_causal_f32_n129_d32", 103, (1, 2, 129, 32), f32, 32, 32, causal=True)
    fwd_generic("fwd_causal_f16_n129_d32", 104, (1, 2, 129, 32), f16, 32, 32, causal=True)
    fwd_generic("fwd_swin_f32_n49_d32", 105, (4, 3, 49, 32), f32, 64, 64, bias_shape=(1, 3, 49, 49))
    fwd_generic("fwd_swin_f16_n49_d32", 106, (4, 3, 49, 32), f16, 64, 64, bias_shape=(1, 3, 49, 49))
    fwd_generic("fwd_swinshift_f16_n49_d32", 107, (4, 3, 49, 32), f16, 64, 64, bias_shape=(4, 3, 49, 49), mask_frac=0.3)
    fwd_generic("fwd_generic_f32_n70_d128", 108, (1, 2, 70, 128), f32, 32, 64)
    fwd_d64("fwd_d64tiled_f32_n200", 111, (1, 2, 200, 64), f32, 32, 128 * 5)
    fwd_d64("fwd_d64tiled_f16_n200", 112, (1, 2, 200, 64), f16, 64, 128 * 5)
    fwd_d64("fwd_d64tiled_f32_n700", 115, (1, 1, 700, 64), f32, 32, 576)
    fwd_d64("fwd_d64_f32_n130", 113, (1, 2, 130, 64), f32, 32, 64)
    fwd_d64("fwd_d64_f16_n130", 114, (1, 2, 130, 64), f16, 64, 64)
    bwd("bwd_f32_n70_d64", 121, (1, 2, 70, 64), f32)
    bwd("bwd_f32_causal_n70_d64", 122, (1, 2, 70, 64), f32, causal=True)
    bwd("bwd_f16_n70_d64", 123, (1, 2, 70, 64), f16)
    bwd("bwd_f16_causal_n70_d64", 124, (1, 2, 70, 64), f16, causal=True)
    bwd("bwd_swin_f32_n49_d32", 125, (4, 3, 49, 32), f32, bias_shape=(1, 3, 49, 49), dbias=True)
    bwd("bwd_swin_f16_n49_d32", 126, (4, 3, 49, 32), f16, bias_shape=(1, 3, 49, 49), dbias=True)
