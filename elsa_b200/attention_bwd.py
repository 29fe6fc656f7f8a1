"""Training side of the two-pass attention: forward that keeps the per-row state, the exact
recompute backward, and the autograd wrapper.

Mirrors src/elsa_twopass_clean/attention_bwd.py of the reference: `twopass_attention_with_state`
(:77-185), `twopass_attention_backward` (:661-839), `_TwopassAttentionAutograd` (:842-905),
`_dense_bias_backward` (:908-1000) and `twopass_attention_train` (:1003-1030).  Differences that are
deliberate: the bias gradient is produced by the same backward launch (no second pass, no
materialised score matrix, any broadcast shape), and rows whose keys are all masked get zero
gradients instead of NaN.
"""
from __future__ import annotations

from typing import Literal, Optional

import torch

from . import _lib
from .attention import (_DeviceScope, _aligned, _bhnd_strides, _cached_bytes, _canonical_bias, _check_qkv, _empty_like_layout, _forward_impl, _i64x,
                        _in_place_or_copy, _resolve_common, _validate_warps)


def twopass_attention_with_state(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    bias: Optional[torch.Tensor] = None,
    is_causal: bool = False,
    block_m: Optional[int] = None,
    block_n: Optional[int] = None,
    q_chunk_size: Optional[int] = None,
    summary_dtype: Optional[torch.dtype] = None,
    phase1_warps: Optional[int] = None,
    phase2_warps: Optional[int] = None,
    phase1_stages: Optional[int] = None,
    phase2_stages: Optional[int] = None,
    input_precision: Literal["auto", "ieee", "tf32", "tf32x3"] = "auto",
    algorithm: Literal["auto", "paper_scan"] = "auto",
    return_contiguous_inputs: bool = False,
    reference_rounding: bool = False,
) -> tuple[torch.Tensor, ...]:
    """Forward that also returns the row statistics the backward needs.

    Returns (out, row_m, row_z) or, with return_contiguous_inputs, (out, row_m, row_z, q_c, k_c, v_c);
    row_m (log2 domain, -inf for a row without admissible keys) and row_z are fp32 [B*H, N]."""
    _check_qkv(q, k, v, "twopass_attention_with_state")
    batch, heads, seq_len, head_dim = map(int, q.shape)
    if seq_len <= 0:
        empty_state = torch.empty((batch * heads, 0), device=q.device, dtype=torch.float32)
        out_empty = torch.empty_like(q)
        if return_contiguous_inputs:
            return out_empty, empty_state, empty_state, q.contiguous(), k.contiguous(), v.contiguous()
        return out_empty, empty_state, empty_state
    if head_dim > 128:
        raise ValueError("head_dim > 128 is not supported by the current kernels")
    summary_dtype, part_width, q_chunk = _resolve_common(
        q, algorithm=algorithm, input_precision=input_precision, summary_dtype=summary_dtype, block_m=block_m,
        block_n=block_n, q_chunk_size=q_chunk_size, phase1_warps=phase1_warps, phase2_warps=phase2_warps,
        phase1_stages=phase1_stages, phase2_stages=phase2_stages)
    out, row_m, row_z, q_c, k_c, v_c = _forward_impl(
        q, k, v, bias=bias, is_causal=is_causal, summary_dtype=summary_dtype, part_width=part_width,
        q_chunk=q_chunk, want_state=True, flags=_lib.FLAG_REF_ROUNDING if reference_rounding else 0)
    if return_contiguous_inputs:
        return out, row_m, row_z, q_c, k_c, v_c
    return out, row_m, row_z


def _row_stats(q_c, k_c, meta, is_causal):
    lib = _lib.load()
    batch, heads, seq_len, head_dim = map(int, q_c.shape)
    dt = _lib.dtype_code(q_c.dtype)
    row_m = torch.empty((batch * heads, seq_len), device=q_c.device, dtype=torch.float32)
    row_z = torch.empty_like(row_m)
    nbytes = lib.elsa_row_stats_workspace_bytes(dt, batch, heads, seq_len, head_dim, int(meta.has_bias),
                                                int(bool(is_causal)))
    if nbytes < 0:
        raise ValueError("elsa_b200: unsupported problem size for row statistics")
    with torch.cuda.device(q_c.device):
        ws = torch.empty((max(int(nbytes), 256),), device=q_c.device, dtype=torch.uint8)
        rc = lib.elsa_row_stats(q_c.data_ptr(), k_c.data_ptr(), *meta.c_args(), row_m.data_ptr(), row_z.data_ptr(),
                                ws.data_ptr(), ws.numel(), dt, batch, heads, seq_len, head_dim,
                                int(bool(is_causal)), _lib.raw_stream(q_c.device))
    _lib.check(rc, "elsa_row_stats")
    return row_m, row_z


def _backward_impl(q, k, v, out, grad_out, *, bias, is_causal, row_m, row_z, want_dbias, flags=0, grads_into=None):
    """dq, dk, dv (and dbias) through the library.  Inputs are read in place where their layout allows it (see
    `_forward_impl`); `grads_into` = (dq, dk, dv) lets the caller supply the gradient tensors, e.g. the three slices
    of one packed [B, N, 3, H, D] buffer."""
    lib = _lib.load()
    batch, heads, seq_len, head_dim = map(int, q.shape)
    strided = head_dim % 8 == 0 and (grads_into is not None or
                                     not all(t.is_contiguous() for t in (q, k, v, out, grad_out)))
    if strided:
        pairs = [_in_place_or_copy(t) for t in (q, k, v, out, grad_out)]
        (q_c, qs), (k_c, ks), (v_c, vs), (out_c, os_), (go_c, gs) = pairs
        strided = any(not t.is_contiguous() for t, _ in pairs) or grads_into is not None
    if not strided:
        q_c, k_c, v_c, out_c, go_c = (_aligned(t) for t in (q, k, v, out, grad_out))
    meta = _canonical_bias(bias, batch=batch, heads=heads, seq_len=seq_len, device=q.device)
    if row_m is None or row_z is None:
        row_m, row_z = _row_stats(_aligned(q_c), _aligned(k_c), meta, is_causal)
    else:
        if tuple(row_m.shape) != (batch * heads, seq_len) or tuple(row_z.shape) != (batch * heads, seq_len):
            raise ValueError("row_m and row_z must have shape [B*H,N]")
        if row_m.dtype != torch.float32 or not row_m.is_contiguous():
            row_m = row_m.to(torch.float32).contiguous()
        if row_z.dtype != torch.float32 or not row_z.is_contiguous():
            row_z = row_z.to(torch.float32).contiguous()
    if grads_into is not None:
        dq, dk, dv = grads_into
        g_strides = [_bhnd_strides(t) for t in (dq, dk, dv)]
        if any(st is None for st in g_strides) or not strided:
            raise ValueError("elsa_b200: the supplied gradient tensors cannot be written in place")
    elif strided:
        dq, dk, dv = (_empty_like_layout(t, st) for t, st in ((q_c, qs), (k_c, ks), (v_c, vs)))
        g_strides = [_bhnd_strides(t) for t in (dq, dk, dv)]
    else:
        dq, dk, dv = torch.empty_like(q_c), torch.empty_like(k_c), torch.empty_like(v_c)
    dbias = None
    dargs = (None, 0, 0, 0, 0)
    if want_dbias:
        if not meta.has_bias:
            raise ValueError("a bias gradient was requested without a bias")
        # same broadcast layout as the bias itself: contributions of broadcast axes are summed
        dbias = torch.zeros_like(meta.tensor)
        dargs = (dbias.data_ptr(), meta.stride_b, meta.stride_h, meta.stride_q, meta.stride_k)
    dt = _lib.dtype_code(q.dtype)
    nbytes = _cached_bytes("elsa_backward_workspace_bytes", dt, batch, heads, seq_len, head_dim, int(meta.has_bias),
                           int(bool(is_causal)), flags)
    if nbytes < 0:
        raise ValueError("elsa_b200: unsupported problem size for the backward")
    with _DeviceScope(q.device):
        ws = torch.empty((max(int(nbytes), 256),), device=q.device, dtype=torch.uint8)
        stream = _lib.raw_stream(q.device)
        if strided:
            rc = lib.elsa_twopass_backward_strided(
                q_c.data_ptr(), k_c.data_ptr(), v_c.data_ptr(), out_c.data_ptr(), go_c.data_ptr(),
                _i64x(qs, ks, vs, os_, gs, *g_strides), row_m.data_ptr(), row_z.data_ptr(), *meta.c_args(),
                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), *dargs, ws.data_ptr(), ws.numel(), dt, batch, heads, seq_len,
                head_dim, int(bool(is_causal)), flags, stream)
        else:
            rc = lib.elsa_twopass_backward(
                q_c.data_ptr(), k_c.data_ptr(), v_c.data_ptr(), out_c.data_ptr(), go_c.data_ptr(),
                row_m.data_ptr(), row_z.data_ptr(), *meta.c_args(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                *dargs, ws.data_ptr(), ws.numel(), dt, batch, heads, seq_len, head_dim, int(bool(is_causal)), flags, stream)
    _lib.check(rc, "elsa_twopass_backward")
    if dbias is not None:
        dbias = dbias.view(bias.shape).to(bias.dtype)
    return dq, dk, dv, dbias


def twopass_attention_backward(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    out: torch.Tensor,
    grad_out: torch.Tensor,
    *,
    bias: Optional[torch.Tensor] = None,
    is_causal: bool = False,
    block_m: Optional[int] = None,
    block_n: Optional[int] = None,
    num_warps: Optional[int] = None,
    num_stages: Optional[int] = None,
    input_precision: Literal["auto", "ieee", "tf32", "tf32x3"] = "auto",
    row_m: Optional[torch.Tensor] = None,
    row_z: Optional[torch.Tensor] = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """dq, dk, dv by exact recompute; the score matrix is never materialised.  A dense bias takes
    part in the softmax when given; its gradient is only produced through `twopass_attention_train`.
    Without (row_m, row_z) the row statistics are recomputed first."""
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k, v must have shape [B,H,N,D]")
    if q.shape != k.shape or q.shape != v.shape or q.shape != out.shape or q.shape != grad_out.shape:
        raise ValueError("q, k, v, out, and grad_out must have identical shapes")
    if q.device.type != "cuda":
        raise ValueError("twopass_attention_backward currently requires CUDA tensors")
    if q.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise ValueError("supported dtypes are fp16, bf16, and fp32")
    if int(q.shape[3]) > 128:
        raise ValueError("head_dim > 128 is not supported by the current kernels")
    if int(q.shape[2]) <= 0:
        return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    if input_precision not in ("auto", "ieee", "tf32", "tf32x3"):
        raise ValueError("input_precision must be 'auto', 'ieee', 'tf32', or 'tf32x3'")
    if num_warps is not None:
        _validate_warps("num_warps", num_warps)
    for val in (block_m, block_n, num_stages):
        if val is not None:
            int(val)
    grad_out = grad_out.to(q.dtype)
    dq, dk, dv, _ = _backward_impl(q, k, v, out.to(q.dtype), grad_out, bias=bias, is_causal=is_causal, row_m=row_m,
                                   row_z=row_z, want_dbias=False)
    return dq, dk, dv


class _TwopassAttentionAutograd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, bias, is_causal, fwd_kwargs, bwd_kwargs):
        out, row_m, row_z, q_s, k_s, v_s = twopass_attention_with_state(
            q, k, v, bias=bias, is_causal=is_causal, return_contiguous_inputs=True, **fwd_kwargs)
        has_bias = bias is not None
        ctx.save_for_backward(q_s, k_s, v_s, out, bias if has_bias else q_s.new_empty(1, dtype=torch.float32),
                              row_m, row_z)
        ctx.has_bias = has_bias
        ctx.bias_requires_grad = bool(has_bias and bias.requires_grad)
        ctx.is_causal = bool(is_causal)
        ctx.bwd_kwargs = dict(bwd_kwargs)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        q, k, v, out, saved_bias, row_m, row_z = ctx.saved_tensors
        bias = saved_bias if ctx.has_bias else None
        if q.numel() == 0:
            return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v), None, None, None, None
        dq, dk, dv, dbias = _backward_impl(q, k, v, out, grad_out.to(q.dtype), bias=bias, is_causal=ctx.is_causal,
                                           row_m=row_m, row_z=row_z, want_dbias=ctx.bias_requires_grad)
        return dq, dk, dv, dbias, None, None, None


# ---- packed projection output: the model hooks' path, kept short on the host ------------------------------------
# Everything that depends only on the problem's shape (stride arrays for the C ABI, workspace sizes, dtype codes) is
# built once per shape; a call then allocates its outputs, takes pointers and goes through ctypes.
_PACKED_PLANS: dict = {}


class _PackedPlan:
    __slots__ = ("dt", "esize", "hd", "qkv_strides", "out_strides", "fwd_ws", "bwd_ws", "bwd_strides")

    def __init__(self, qkv, has_bias, is_causal, summary_dtype, part_width, q_chunk):
        batch, seq_len, _, heads, head_dim = map(int, qkv.shape)
        self.dt = _lib.dtype_code(qkv.dtype)
        self.esize = qkv.element_size()
        self.hd = heads * head_dim
        # (batch, head, row) element strides of the q / k / v views of [B, N, 3, H, D] and of out as [B, N, H, D]
        packed = (seq_len * 3 * self.hd, head_dim, 3 * self.hd)
        plain = (seq_len * self.hd, head_dim, self.hd)
        self.qkv_strides = _i64x(packed)
        self.out_strides = _i64x(plain)
        self.fwd_ws = _cached_bytes("elsa_forward_workspace_bytes", self.dt, _lib.dtype_code(summary_dtype), batch, heads,
                                    seq_len, head_dim, int(has_bias), int(is_causal), part_width, q_chunk, 0)
        self.bwd_ws = _cached_bytes("elsa_backward_workspace_bytes", self.dt, batch, heads, seq_len, head_dim,
                                    int(has_bias), int(is_causal), 0)
        self.bwd_strides = {}                    # keyed by grad_out's strides: q, k, v, out, dout, dq, dk, dv

    def backward_strides(self, gs):
        arr = self.bwd_strides.get(gs)
        if arr is None:
            q = tuple(self.qkv_strides)
            o = tuple(self.out_strides)
            arr = self.bwd_strides[gs] = _i64x(q, q, q, o, gs, q, q, q)
        return arr


def _packed_plan(qkv, has_bias, is_causal, summary_dtype, part_width, q_chunk):
    key = (tuple(qkv.shape), qkv.dtype, has_bias, is_causal, summary_dtype, part_width, q_chunk)
    plan = _PACKED_PLANS.get(key)
    if plan is None:
        plan = _PACKED_PLANS[key] = _PackedPlan(qkv, has_bias, is_causal, summary_dtype, part_width, q_chunk)
    return plan


def _packed_fast_ok(qkv) -> bool:
    """The short path reads q, k, v as three pointers into one contiguous [B, N, 3, H, D] buffer."""
    return (qkv.device.type == "cuda" and qkv.is_contiguous() and int(qkv.shape[-1]) % 8 == 0 and 0 < int(qkv.shape[-1]) <= 128 and int(qkv.shape[1]) > 0
            and qkv.data_ptr() % 16 == 0 and qkv.dtype in (torch.float16, torch.bfloat16, torch.float32))


def _packed_forward_fast(qkv, bias32, is_causal, fwd_kwargs, want_state):
    """The forward on a contiguous packed qkv: (out as [B, N, H, D], state or None, bias meta, plan).  `state` holds
    row_m and row_z in one allocation, the second at a 256-byte boundary like a tensor of its own."""
    batch, seq_len, _, heads, head_dim = map(int, qkv.shape)
    if not fwd_kwargs:                                     # (the ViT hooks' call: nothing to validate or resolve)
        summary_dtype, part_width, q_chunk, kw = qkv.dtype, 0, 0, None
    else:
        kw = dict(fwd_kwargs)
        kw.pop("reference_rounding", None)
        summary_dtype, part_width, q_chunk = _resolve_common(
            qkv, algorithm=kw.pop("algorithm", "auto"), input_precision=kw.pop("input_precision", "auto"),
            summary_dtype=kw.pop("summary_dtype", None), block_m=kw.pop("block_m", None), block_n=kw.pop("block_n", None),
            q_chunk_size=kw.pop("q_chunk_size", None), phase1_warps=kw.pop("phase1_warps", None),
            phase2_warps=kw.pop("phase2_warps", None), phase1_stages=kw.pop("phase1_stages", None),
            phase2_stages=kw.pop("phase2_stages", None))
    if kw:
        raise TypeError(f"unexpected keyword arguments: {sorted(kw)}")
    meta = _canonical_bias(bias32, batch=batch, heads=heads, seq_len=seq_len, device=qkv.device)
    plan = _packed_plan(qkv, meta.has_bias, bool(is_causal), summary_dtype, part_width, q_chunk)
    if plan.fwd_ws < 0 or plan.bwd_ws < 0:
        raise ValueError("elsa_b200: unsupported problem size")
    out = torch.empty((batch, seq_len, heads, head_dim), device=qkv.device, dtype=qkv.dtype)
    state = rm_p = rz_p = None
    if want_state:
        pad = (batch * heads * seq_len + 63) // 64 * 64
        state = torch.empty((2 * pad,), device=qkv.device, dtype=torch.float32)
        rm_p = state.data_ptr()
        rz_p = rm_p + 4 * pad
    base, step = qkv.data_ptr(), plan.hd * plan.esize
    with _DeviceScope(qkv.device):
        ws = torch.empty((max(plan.fwd_ws, 256),), device=qkv.device, dtype=torch.uint8)
        rc = _lib.load().elsa_twopass_forward_strided(
            base, base + step, base + 2 * step, plan.qkv_strides, plan.qkv_strides, plan.qkv_strides,
            *meta.c_args(), out.data_ptr(), plan.out_strides, rm_p, rz_p, ws.data_ptr(), ws.numel(), plan.dt,
            _lib.dtype_code(summary_dtype), batch, heads, seq_len, head_dim, int(bool(is_causal)), part_width, q_chunk,
            0, _lib.raw_stream(qkv.device))
    _lib.check(rc, "elsa_twopass_forward")
    return out, state, meta, plan


class _PackedQkvAttentionAutograd(torch.autograd.Function):
    """Attention on a packed projection output qkv [B, N, 3, H, D] (what `nn.Linear(dim, 3*dim)` produces, viewed):
    q, k, v are read in place, the output is written as [B, N, H, D] memory, and the backward writes dq, dk, dv
    straight into one packed gradient -- no `.contiguous()` copies, no `stack` in autograd."""

    @staticmethod
    def forward(ctx, qkv, bias, is_causal, fwd_kwargs):
        # the kernels read the bias in fp32: convert once, and let the backward reuse the converted tensor
        bias32 = None
        if bias is not None:
            bias32 = bias.detach()
            if bias32.dtype != torch.float32:
                bias32 = bias32.to(torch.float32)
        has_bias = bias is not None
        ctx.has_bias = has_bias
        ctx.bias_requires_grad = bool(has_bias and bias.requires_grad)
        ctx.bias_dtype = bias.dtype if has_bias else None
        ctx.bias_shape = tuple(bias.shape) if has_bias else None
        ctx.is_causal = bool(is_causal)
        ctx.fast = not fwd_kwargs.get("reference_rounding", False) and _packed_fast_ok(qkv)
        if ctx.fast:
            out, state, meta, plan = _packed_forward_fast(qkv, bias32, ctx.is_causal, fwd_kwargs, want_state=True)
            ctx.plan = plan
            if has_bias:
                ctx.save_for_backward(qkv, out, state, meta.tensor)
            else:
                ctx.save_for_backward(qkv, out, state)
            return out.permute(0, 2, 1, 3)
        q, k, v = qkv.permute(2, 0, 3, 1, 4).unbind(0)           # three [B, H, N, D] views
        out, row_m, row_z, q_s, k_s, v_s = twopass_attention_with_state(
            q, k, v, bias=bias32, is_causal=is_causal, return_contiguous_inputs=True, **fwd_kwargs)
        ctx.save_for_backward(qkv, out, bias32 if has_bias else qkv.new_empty(1, dtype=torch.float32), row_m, row_z)
        return out

    @staticmethod
    def _fast_backward(ctx, grad_out):
        saved = ctx.saved_tensors
        qkv, out, state = saved[0], saved[1], saved[2]
        bias32 = saved[3] if ctx.has_bias else None
        plan = ctx.plan
        batch, seq_len, _, heads, head_dim = map(int, qkv.shape)
        if grad_out.dtype != qkv.dtype:
            grad_out = grad_out.to(qkv.dtype)
        gs = _bhnd_strides(grad_out)
        if gs is None:
            grad_out = _aligned(grad_out)
            gs = _bhnd_strides(grad_out)
        dqkv = torch.empty_like(qkv)
        meta = _canonical_bias(bias32, batch=batch, heads=heads, seq_len=seq_len, device=qkv.device)
        dbias = None
        dargs = (None, 0, 0, 0, 0)
        if ctx.bias_requires_grad:
            dbias = torch.zeros_like(meta.tensor)
            dargs = (dbias.data_ptr(), meta.stride_b, meta.stride_h, meta.stride_q, meta.stride_k)
        base, dbase, step = qkv.data_ptr(), dqkv.data_ptr(), plan.hd * plan.esize
        with _DeviceScope(qkv.device):
            ws = torch.empty((max(plan.bwd_ws, 256),), device=qkv.device, dtype=torch.uint8)
            rc = _lib.load().elsa_twopass_backward_strided(
                base, base + step, base + 2 * step, out.data_ptr(), grad_out.data_ptr(), plan.backward_strides(gs),
                state.data_ptr(), state.data_ptr() + 2 * state.numel(), *meta.c_args(),
                dbase, dbase + step, dbase + 2 * step, *dargs, ws.data_ptr(), ws.numel(), plan.dt, batch, heads, seq_len,
                head_dim, int(ctx.is_causal), 0, _lib.raw_stream(qkv.device))
        _lib.check(rc, "elsa_twopass_backward")
        return dqkv, dbias

    @staticmethod
    def backward(ctx, grad_out):
        if ctx.fast:
            dqkv, dbias = _PackedQkvAttentionAutograd._fast_backward(ctx, grad_out)
            if dbias is not None:
                # (the saved fp32 bias has the [B|1, H|1, N, N] form: back to the caller's shape and dtype)
                dbias = dbias.view(ctx.bias_shape)
                if dbias.dtype != ctx.bias_dtype:
                    dbias = dbias.to(ctx.bias_dtype)
            return dqkv, dbias, None, None
        qkv, out, saved_bias, row_m, row_z = ctx.saved_tensors
        bias = saved_bias if ctx.has_bias else None
        q, k, v = qkv.permute(2, 0, 3, 1, 4).unbind(0)
        dqkv = torch.empty_like(qkv, memory_format=torch.contiguous_format)
        grads = dqkv.permute(2, 0, 3, 1, 4).unbind(0)
        if grad_out.dtype != q.dtype:
            grad_out = grad_out.to(q.dtype)
        # (dqkv is freshly allocated and contiguous: its three views are writable in place whenever q's layout is)
        in_place = int(qkv.shape[-1]) % 8 == 0 and _bhnd_strides(q) is not None and _bhnd_strides(grads[0]) is not None
        if in_place:
            _, _, _, dbias = _backward_impl(q, k, v, out, grad_out, bias=bias, is_causal=ctx.is_causal,
                                            row_m=row_m, row_z=row_z, want_dbias=ctx.bias_requires_grad, grads_into=grads)
        else:
            dq, dk, dv, dbias = _backward_impl(q, k, v, out, grad_out, bias=bias, is_causal=ctx.is_causal,
                                               row_m=row_m, row_z=row_z, want_dbias=ctx.bias_requires_grad)
            for dst, src in zip(grads, (dq, dk, dv)):
                dst.copy_(src)
        if dbias is not None and dbias.dtype != ctx.bias_dtype:
            dbias = dbias.to(ctx.bias_dtype)
        return dqkv, dbias, None, None


def twopass_attention_qkvpacked(qkv: torch.Tensor, *, bias: Optional[torch.Tensor] = None, is_causal: bool = False,
                                train: bool = True, **fwd_kwargs) -> torch.Tensor:
    """Attention on a packed qkv [B, N, 3, H, D] (not an entry point of the reference: the form its hooks would need to
    avoid their per-layer copies, src/elsa_twopass_clean/timm_dropin.py:46-55, timm_dropin_bwd.py:68-73).
    Returns out as a [B, H, N, D] view of [B, N, H, D] memory, so `out.transpose(1, 2).reshape(B, N, H*D)` is free.
    train=False skips autograd and the row state."""
    if qkv.dim() != 5 or qkv.shape[2] != 3:
        raise ValueError("qkv must have shape [B,N,3,H,D]")
    # the backward tile hints of twopass_attention_train are validated and advisory, as there
    if fwd_kwargs.get("bwd_input_precision", "auto") not in ("auto", "ieee", "tf32", "tf32x3"):
        raise ValueError("input_precision must be 'auto', 'ieee', 'tf32', or 'tf32x3'")
    if fwd_kwargs.get("bwd_num_warps") is not None:
        _validate_warps("num_warps", fwd_kwargs["bwd_num_warps"])
    fwd_kwargs = {name: val for name, val in fwd_kwargs.items() if not name.startswith("bwd_")}
    if not train:
        if not fwd_kwargs.get("reference_rounding", False) and _packed_fast_ok(qkv):
            bias32 = None
            if bias is not None:
                bias32 = bias.detach()
                if bias32.dtype != torch.float32:
                    bias32 = bias32.to(torch.float32)
            return _packed_forward_fast(qkv, bias32, is_causal, fwd_kwargs, want_state=False)[0].permute(0, 2, 1, 3)
        from .attention import twopass_attention
        q, k, v = qkv.permute(2, 0, 3, 1, 4).unbind(0)
        return twopass_attention(q, k, v, bias=bias, is_causal=is_causal, **fwd_kwargs)
    return _PackedQkvAttentionAutograd.apply(qkv, bias, is_causal, dict(fwd_kwargs))


def twopass_attention_train(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    bias: Optional[torch.Tensor] = None,
    is_causal: bool = False,
    bwd_block_m: Optional[int] = None,
    bwd_block_n: Optional[int] = None,
    bwd_num_warps: Optional[int] = None,
    bwd_num_stages: Optional[int] = None,
    bwd_input_precision: Literal["auto", "ieee", "tf32", "tf32x3"] = "auto",
    **fwd_kwargs,
) -> torch.Tensor:
    """Differentiable `twopass_attention`: two-pass forward with saved (m, z), recompute backward."""
    if bwd_input_precision not in ("auto", "ieee", "tf32", "tf32x3"):
        raise ValueError("input_precision must be 'auto', 'ieee', 'tf32', or 'tf32x3'")
    if bwd_num_warps is not None:
        _validate_warps("num_warps", bwd_num_warps)
    bwd_kwargs = {name: val for name, val in (("block_m", bwd_block_m), ("block_n", bwd_block_n),
                                              ("num_warps", bwd_num_warps), ("num_stages", bwd_num_stages))
                  if val is not None}
    return _TwopassAttentionAutograd.apply(q, k, v, bias, is_causal, dict(fwd_kwargs), bwd_kwargs)
