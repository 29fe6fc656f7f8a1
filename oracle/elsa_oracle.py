"""CPU restatement of ELSA's two-pass monoid attention (TEST INFRASTRUCTURE, not product code).

This module is the parity oracle: a plain PyTorch-on-CPU restatement of the reference
algorithm, with the reference's rounding points, used only by the tests, by the smoke
check and by the CPU-baseline leg of the benchmark.  The product package never imports it.

Reference (paths inside the reference project, `src/elsa_twopass_clean/`):
  * monoid merge ............ attention_parallel_scan.py:55-60, 111-116
  * generic phase 1 ......... attention.py:72-106
  * d64 non-tiled phase 1 ... attention_parallel_scan.py:151-172 (fp16), 203-224 (fp32)
  * d64 tiled fold .......... attention_parallel_scan.py:261-295 (fp16), 334-372 (fp32)
  * Blelloch up-sweep ....... attention_parallel_scan.py:89-120, host loop 911-935
  * Hillis-Steele step ...... attention_parallel_scan.py:36-64, host loop 710-733
  * finaliser ............... attention_parallel_scan.py:402-415
  * CUDA one-shot merge ..... cuda/paper_scan_d64_kernel.cu:39-95
  * routing ................. attention.py:162-236, attention_bwd.py:130-158,
                              attention_parallel_scan.py:418-440, 468-472, 983-1001
  * backward ................ attention_bwd.py:220-224 (D, LSE), 379-407 (dQ), 488-517 (dK,dV),
                              610-618 (dbias), 227-306 (row stats), 627-658 (tiles)

Parity pin: fp32 and fp16 routes are pinned against outputs of the reference's own Triton
kernels executed by the Triton CPU interpreter (fixtures in tests/golden/, generator
tests/golden/make_golden.py).  The bf16 route is the same code with a different rounding
type; the interpreter cannot execute bf16, so for bf16 this oracle is "parity unpinned"
beyond that shared code.

Summary layout used here (and by the CUDA path): m, z are [P, BH, N] and s is [P, BH, N, D]
with P the number of K partitions; the reference interleaves q-blocks differently
(attention.py:102) but every summary value is the same number.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

LOG2E = 1.4426950408889634
NEG_INF = float("-inf")


# --------------------------------------------------------------------------------------
# monoid
# --------------------------------------------------------------------------------------
def monoid_identity(shape, d):
    return (torch.full(shape, NEG_INF), torch.zeros(shape), torch.zeros(*shape, d))


def monoid_merge(a, b):
    """(m,z,s) (+) (m,z,s); attention_parallel_scan.py:55-60."""
    m_a, z_a, s_a = a
    m_b, z_b, s_b = b
    m = torch.maximum(m_a, m_b)
    alpha = torch.where(z_a > 0, torch.exp2(m_a - m), torch.zeros(()))
    beta = torch.where(z_b > 0, torch.exp2(m_b - m), torch.zeros(()))
    z = z_a * alpha + z_b * beta
    s = s_a * alpha[..., None] + s_b * beta[..., None]
    m = torch.where(z > 0, m, torch.full((), NEG_INF))
    return m, z, s


def _cdiv(a, b):
    return -(-a // b)


# --------------------------------------------------------------------------------------
# routing (restated; attention.py:162-236 and attention_bwd.py:130-158)
# --------------------------------------------------------------------------------------
def paper_scan_defaults(dtype, seq_len, head_dim, block_m=None, block_n=None, q_chunk_size=None,
                        training=False):
    if dtype == torch.float32:
        dm = 32
        if head_dim <= 64:
            if seq_len <= 512:
                dn = 256
            elif seq_len < 2048:
                dn = ((seq_len + 63) // 64) * 64
            else:
                dn = 2048
        else:
            dn = 64
        dq = 512 if seq_len >= 4096 else 1024
    elif (not training) and dtype == torch.float16 and head_dim == 64 and seq_len >= 8192:
        dm, dn = 64, 2048
        dq = 4096 if seq_len >= 16384 else 2048
    else:
        dm = 64 if head_dim <= 64 else 32
        dn = 256 if head_dim <= 64 else 64
        dq = 1024 if seq_len >= 4096 else min(seq_len, 1024)
    bm = max(16, int(dm if block_m is None else block_m))
    bn = max(16, int(dn if block_n is None else block_n))
    qc = max(16, int(dq if q_chunk_size is None else q_chunk_size))
    qc = max(bm, (qc // bm) * bm)
    return bm, bn, qc


def can_use_d64_fast(dtype, head_dim, has_bias, block_m, block_n, q_chunk, summary_dtype):
    """attention_parallel_scan.py:418-440."""
    return ((not has_bias) and dtype in (torch.float16, torch.float32) and head_dim == 64
            and block_n % 64 == 0 and q_chunk % block_m == 0 and summary_dtype == dtype)


def canonical_bias(bias, batch, heads, n):
    """attention.py:120-159 -> a [Bb, Hb, N, N] fp32 view that broadcasts over B and H."""
    if bias is None:
        return None
    if bias.shape[-2:] != (n, n):
        raise ValueError("bias last dims must be (N, N)")
    if bias.dim() == 2:
        view = bias.reshape(1, 1, n, n)
    elif bias.dim() == 3:
        if bias.shape[0] not in (1, heads):
            raise ValueError("3D bias must have shape [1,N,N] or [H,N,N]")
        view = bias.reshape(1, bias.shape[0], n, n)
    elif bias.dim() == 4:
        if bias.shape[0] not in (1, batch) or bias.shape[1] not in (1, heads):
            raise ValueError("4D bias must broadcast as [B,H,N,N]")
        view = bias
    else:
        raise ValueError("bias must have shape [N,N], [H,N,N], or [B,H,N,N]")
    return view.float().expand(batch, heads, n, n).reshape(batch * heads, n, n)


# --------------------------------------------------------------------------------------
# phase 1
# --------------------------------------------------------------------------------------
def _tile_summary(scores, valid, v32, p_round_dtype):
    """One score tile -> (m, z, s) exactly as attention.py:90-100: scores are already in the
    log2 domain; invalid entries are forced to -inf; rows with no valid key give (-inf,0,0)."""
    scores = torch.where(valid, scores, torch.full((), NEG_INF))
    row_has = valid.any(dim=-1)
    m_raw = scores.max(dim=-1).values
    m_safe = torch.where(row_has, m_raw, torch.zeros(()))
    p = torch.where(valid, torch.exp2(scores - m_safe[..., None]), torch.zeros(()))
    z = p.sum(dim=-1)
    if p_round_dtype is not None:
        p = p.to(p_round_dtype).float()
    s = p @ v32
    m = torch.where(row_has, m_raw, torch.full((), NEG_INF))
    return m, z, s


def phase1_generic(q, k, v, *, bias=None, is_causal=False, block_n, summary_dtype,
                   q_start=0, q_len=None):
    """Generic phase 1 (attention.py:22-106).  q,k,v: [BH,N,D] in the input dtype; bias:
    [BH,N,N] fp32 or None.  Returns m,z [P,BH,q_len] fp32 and s [P,BH,q_len,D] rounded to
    summary_dtype (kept as fp32 storage of the rounded values)."""
    bh, n, d = q.shape
    q_len = n - q_start if q_len is None else q_len
    scale = 1.0 / math.sqrt(d)
    # attention_parallel_scan.py:701 - P stays fp32 unless fp16 inputs with a non-fp32 summary
    dot_fp32 = (q.dtype != torch.float16) or (summary_dtype == torch.float32)
    p_round = None if dot_fp32 else torch.float16
    q32 = q[:, q_start:q_start + q_len].float()
    k32, v32 = k.float(), v.float()
    parts = _cdiv(n, block_n)
    q_idx = torch.arange(q_start, q_start + q_len)
    ms, zs, ss = [], [], []
    for p in range(parts):
        k0, k1 = p * block_n, min(n, (p + 1) * block_n)
        scores = (q32 @ k32[:, k0:k1].transpose(-1, -2)) * scale
        k_idx = torch.arange(k0, k1)
        valid = torch.ones(q_len, k1 - k0, dtype=torch.bool)
        if is_causal:
            valid = q_idx[:, None] >= k_idx[None, :]
        valid = valid[None].expand(bh, -1, -1)
        if bias is not None:
            scores = scores + bias[:, q_start:q_start + q_len, k0:k1]
        scores = scores * LOG2E
        m, z, s = _tile_summary(scores, valid, v32[:, k0:k1], p_round)
        ms.append(m); zs.append(z); ss.append(s.to(summary_dtype).float())
    return torch.stack(ms), torch.stack(zs), torch.stack(ss)


def phase1_d64(q, k, v, *, block_n, q_start=0, q_len=None, micro=64):
    """d=64 fast phase 1: non-tiled for block_n <= 512 (attention_parallel_scan.py:151-172,
    203-224), tiled register fold over 64-key micro tiles otherwise (:261-295, :334-372).
    Q is pre-multiplied by log2(e)/8 and, for fp16, re-rounded to fp16 (:153-154)."""
    bh, n, d = q.shape
    assert d == 64
    q_len = n - q_start if q_len is None else q_len
    log2_scale = (1.0 / math.sqrt(64)) * LOG2E
    is16 = q.dtype == torch.float16
    if is16:
        # fp16 tensor * python constant is evaluated in fp16 by Triton: the constant itself is
        # rounded to fp16 first (0.18033688 -> 0.18029785), then the product is rounded again.
        ls16 = torch.tensor(log2_scale).to(torch.float16).float()
        qs = (q[:, q_start:q_start + q_len].float() * ls16).to(torch.float16).float()
    else:
        qs = q[:, q_start:q_start + q_len].float() * log2_scale
    k32, v32 = k.float(), v.float()
    p_round = torch.float16 if is16 else None
    tiled = block_n > 512
    parts = _cdiv(n, block_n)
    ms, zs, ss = [], [], []
    for p in range(parts):
        k0 = p * block_n
        if not tiled:
            k1 = min(n, k0 + block_n)
            scores = qs @ k32[:, k0:k1].transpose(-1, -2)
            # keys >= N inside the block are -inf columns; here they are simply absent,
            # which is the same number (exp2(-inf) = 0 contributes nothing).
            m = scores.max(dim=-1).values
            pr = torch.exp2(scores - m[..., None])
            z = pr.sum(dim=-1)
            if p_round is not None:
                pr = pr.to(p_round).float()
            s = pr @ v32[:, k0:k1]
        else:
            m = torch.full((bh, q_len), NEG_INF)
            z = torch.zeros(bh, q_len)
            s = torch.zeros(bh, q_len, 64)
            for mu in range(k0, k0 + block_n, micro):
                m0, m1 = mu, min(n, mu + micro)
                if m0 >= n:
                    # fully out-of-range micro tile: local_m = -inf, p = 0 (:281); the merge
                    # below then leaves the running state unchanged (beta = exp2(-inf - m) = 0)
                    # unless nothing has been seen yet, in which case everything stays 0/-inf.
                    continue
                scores = qs @ k32[:, m0:m1].transpose(-1, -2)
                lm = scores.max(dim=-1).values
                pr = torch.exp2(scores - lm[..., None])
                lz = pr.sum(dim=-1)
                if p_round is not None:
                    pr = pr.to(p_round).float()
                ls = pr @ v32[:, m0:m1]
                m_new = torch.maximum(m, lm)
                alpha = torch.where(z > 0, torch.exp2(m - m_new), torch.zeros(()))
                beta = torch.exp2(lm - m_new)
                z = z * alpha + lz * beta
                s = s * alpha[..., None] + ls * beta[..., None]
                m = m_new
        ms.append(m); zs.append(z); ss.append(s.to(q.dtype).float())
    return torch.stack(ms), torch.stack(zs), torch.stack(ss)


# --------------------------------------------------------------------------------------
# phase 2
# --------------------------------------------------------------------------------------
def final_reduce(m, z, s):
    """One-shot merge over partitions (cuda/paper_scan_d64_kernel.cu:39-95).
    Returns out (fp32, not yet rounded), row_m, row_z."""
    fm = m.max(dim=0).values
    w = torch.where(z > 0, torch.exp2(m - fm), torch.zeros(()))
    fz = (z * w).sum(dim=0)
    fs = (s * w[..., None]).sum(dim=0)
    out = torch.where(fz[..., None] > 0, fs / fz[..., None], torch.zeros(()))
    row_m = torch.where(fz > 0, fm, torch.full((), NEG_INF))
    return out, row_m, fz


def upsweep_level(m, z, s, summary_dtype):
    """One Blelloch up-sweep level (attention_parallel_scan.py:89-120): out[i] =
    in[2i] (+) in[2i+1]; an odd tail merges with the identity.  s is re-rounded to
    summary_dtype at each level because the buffers have that dtype (:866)."""
    n_in = m.shape[0]
    n_out = _cdiv(n_in, 2)
    om, oz, os_ = [], [], []
    for i in range(n_out):
        a = (m[2 * i], z[2 * i], s[2 * i])
        if 2 * i + 1 < n_in:
            b = (m[2 * i + 1], z[2 * i + 1], s[2 * i + 1])
        else:
            b = (torch.full_like(a[0], NEG_INF), torch.zeros_like(a[1]), torch.zeros_like(a[2]))
        mm, zz, sv = monoid_merge(a, b)
        om.append(mm); oz.append(zz); os_.append(sv.to(summary_dtype).float())
    return torch.stack(om), torch.stack(oz), torch.stack(os_)


def upsweep_reduce(m, z, s, summary_dtype):
    """Host loop attention_parallel_scan.py:911-935; returns the root summary."""
    while m.shape[0] > 1:
        m, z, s = upsweep_level(m, z, s, summary_dtype)
    return m[0], z[0], s[0]


def hillis_steele_step(m, z, s, step, summary_dtype):
    """out[k] = in[k-step] (+) in[k] (attention_parallel_scan.py:36-64)."""
    parts = m.shape[0]
    om, oz, os_ = [], [], []
    for kb in range(parts):
        cur = (m[kb], z[kb], s[kb])
        if kb >= step:
            left = (m[kb - step], z[kb - step], s[kb - step])
        else:
            left = (torch.full_like(cur[0], NEG_INF), torch.zeros_like(cur[1]), torch.zeros_like(cur[2]))
        mm, zz, sv = monoid_merge(left, cur)
        om.append(mm); oz.append(zz); os_.append(sv.to(summary_dtype).float())
    return torch.stack(om), torch.stack(oz), torch.stack(os_)


def hillis_steele_scan(m, z, s, summary_dtype):
    """Inclusive prefix scan over partitions (host loop :710-733)."""
    step = 1
    while step < m.shape[0]:
        m, z, s = hillis_steele_step(m, z, s, step, summary_dtype)
        step *= 2
    return m, z, s


def finalize(m, z, s):
    """attention_parallel_scan.py:402-415: out = s / z (0 where z == 0)."""
    out = torch.where(z[..., None] > 0, s / z[..., None], torch.zeros(()))
    return out, m, z


# --------------------------------------------------------------------------------------
# whole forward, routed like the reference
# --------------------------------------------------------------------------------------
def twopass_forward(q, k, v, *, bias=None, is_causal=False, block_m=None, block_n=None,
                    q_chunk_size=None, summary_dtype=None, training=False, return_parts=False):
    """q,k,v: [B,H,N,D] CPU tensors (fp32 / fp16 / bf16).  Returns (out, row_m, row_z) with
    out in the input dtype and the state as fp32 [B*H, N] (row_m in the log2 domain)."""
    b, h, n, d = q.shape
    dtype = q.dtype
    if summary_dtype is None:
        summary_dtype = dtype
    bm, bn, qc = paper_scan_defaults(dtype, n, d, block_m, block_n, q_chunk_size, training=training)
    bh = b * h
    q3, k3, v3 = (t.reshape(bh, n, d).contiguous() for t in (q, k, v))
    bias3 = canonical_bias(bias, b, h, n)
    fast = (not is_causal) and can_use_d64_fast(dtype, d, bias is not None, bm, bn, qc, summary_dtype)
    out = torch.empty(bh, n, d)
    row_m = torch.empty(bh, n)
    row_z = torch.empty(bh, n)
    parts_dbg = []
    for q_start in range(0, n, qc):
        q_len = min(qc, n - q_start)
        if fast:
            m, z, s = phase1_d64(q3, k3, v3, block_n=bn, q_start=q_start, q_len=q_len)
            o, rm, rz = final_reduce(m, z, s)
        else:
            m, z, s = phase1_generic(q3, k3, v3, bias=bias3, is_causal=is_causal, block_n=bn,
                                     summary_dtype=summary_dtype, q_start=q_start, q_len=q_len)
            if is_causal:
                pm, pz, ps = hillis_steele_scan(m, z, s, summary_dtype)
                o, rm, rz = finalize(pm[-1], pz[-1], ps[-1])
            else:
                rm_, rz_, rs_ = upsweep_reduce(m, z, s, summary_dtype)
                o, rm, rz = finalize(rm_, rz_, rs_)
        if return_parts:
            parts_dbg.append((m, z, s))
        out[:, q_start:q_start + q_len] = o
        row_m[:, q_start:q_start + q_len] = rm
        row_z[:, q_start:q_start + q_len] = rz
    res = (out.to(dtype).reshape(b, h, n, d), row_m, row_z)
    if return_parts:
        return res + (parts_dbg,)
    return res


# --------------------------------------------------------------------------------------
# backward (exact recompute from saved row statistics)
# --------------------------------------------------------------------------------------
def bwd_preprocess(out, dout, row_m, row_z):
    """attention_bwd.py:220-224: D = sum_d out*dout; LSE = m + log2(max(z, 1e-30))."""
    d_row = (out.float() * dout.float()).sum(dim=-1)
    lse = row_m + torch.log2(torch.clamp(row_z, min=1.0e-30))
    return d_row, lse


def row_stats(q, k, *, bias=None, is_causal=False):
    """attention_bwd.py:227-306 (recompute (m, z) when the caller saved no state)."""
    bh, n, d = q.shape
    scores = (q.float() @ k.float().transpose(-1, -2)) * (1.0 / math.sqrt(d))
    if bias is not None:
        scores = scores + bias
    scores = scores * LOG2E
    if is_causal:
        idx = torch.arange(n)
        scores = torch.where(idx[:, None] >= idx[None, :], scores, torch.full((), NEG_INF))
    m = scores.max(dim=-1).values
    z = torch.exp2(scores - torch.where(torch.isinf(m), torch.zeros(()), m)[..., None]).sum(dim=-1)
    z = torch.where(torch.isinf(m), torch.zeros(()), z)
    return m, z


def twopass_backward(q, k, v, out, dout, row_m, row_z, *, bias=None, is_causal=False,
                     want_dbias=False, block=1024):
    """Returns dq, dk, dv in the input dtype (+ dbias fp32 [BH,N,N] un-reduced when asked).

    Rounding points (attention_bwd.py): P fp32; dV += P.to(dtype)^T dO (:512); dS =
    (P*(dP-D)).to(dtype) (:404,:514); dQ = scale * dS K (:405-407); dK = scale * dS^T Q (:515-517);
    fp32 accumulators rounded once on store.  dbias = P*(dP-D) in fp32 (:615-618)."""
    b, h, n, d = q.shape
    dtype = q.dtype
    bh = b * h
    scale = 1.0 / math.sqrt(d)
    q3, k3, v3, o3, do3 = (t.reshape(bh, n, d).float() for t in (q, k, v, out, dout))
    bias3 = canonical_bias(bias, b, h, n)
    d_row, lse = bwd_preprocess(o3, do3, row_m, row_z)
    dq = torch.zeros(bh, n, d)
    dk = torch.zeros(bh, n, d)
    dv = torch.zeros(bh, n, d)
    dbias = torch.zeros(bh, n, n) if want_dbias else None
    idx = torch.arange(n)
    for q0 in range(0, n, block):
        q1 = min(n, q0 + block)
        s = q3[:, q0:q1] @ k3.transpose(-1, -2)
        if bias3 is not None:
            s = (s * scale + bias3[:, q0:q1]) * LOG2E
        else:
            s = s * (scale * LOG2E)
        valid = torch.ones(q1 - q0, n, dtype=torch.bool)
        if is_causal:
            valid = idx[q0:q1, None] >= idx[None, :]
        s = torch.where(valid, s, torch.full((), NEG_INF))
        p = torch.where(valid, torch.exp2(s - lse[:, q0:q1, None]), torch.zeros(()))
        dp = do3[:, q0:q1] @ v3.transpose(-1, -2)
        ds32 = p * (dp - d_row[:, q0:q1, None])
        ds = ds32.to(dtype).float()
        dq[:, q0:q1] = (ds @ k3) * scale
        dk += ds.transpose(-1, -2) @ q3[:, q0:q1]
        dv += p.to(dtype).float().transpose(-1, -2) @ do3[:, q0:q1]
        if want_dbias:
            dbias[:, q0:q1] = ds32
    dk = dk * scale
    shp = (b, h, n, d)
    res = (dq.to(dtype).reshape(shp), dk.to(dtype).reshape(shp), dv.to(dtype).reshape(shp))
    if want_dbias:
        return res + (dbias,)
    return res


def reduce_dbias(dbias_full, bias, batch, heads):
    """Sum an un-reduced [BH,N,N] bias gradient down to bias.shape (attention_bwd.py:987-999)."""
    n = dbias_full.shape[-1]
    g = dbias_full.reshape(batch, heads, n, n)
    if bias.dim() == 2:
        return g.sum(dim=(0, 1)).to(bias.dtype)
    if bias.dim() == 3:
        g = g.sum(dim=0)
        if bias.shape[0] == 1:
            g = g.sum(dim=0, keepdim=True)
        return g.to(bias.dtype)
    if bias.shape[0] == 1:
        g = g.sum(dim=0, keepdim=True)
    if bias.shape[1] == 1:
        g = g.sum(dim=1, keepdim=True)
    return g.to(bias.dtype)


# --------------------------------------------------------------------------------------
# absolute truth
# --------------------------------------------------------------------------------------
def softmax_attention_fp64(q, k, v, *, bias=None, is_causal=False):
    """Math softmax attention evaluated in fp64 (the check the reference's tests use is fp32
    SDPA, tests/test_attention.py:16-25; fp64 is stricter)."""
    n, d = q.shape[-2], q.shape[-1]
    s = (q.double() @ k.double().transpose(-1, -2)) / math.sqrt(d)
    if bias is not None:
        s = s + bias.double()
    if is_causal:
        s = s.masked_fill(~torch.ones(n, n, dtype=torch.bool).tril(), NEG_INF)
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    return p @ v.double()
