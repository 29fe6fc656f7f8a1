"""`twopass_attention`: the PyTorch-facing forward of the B200-native two-pass monoid attention.

Mirrors the public contract of the reference's `twopass_attention`
(src/elsa_twopass_clean/attention.py:239-321): same keyword arguments, same validation and error
types.  The work is done by hand-written sm_100a CUDA behind the C ABI in include/elsa_b200.h;
this file only validates, allocates through PyTorch's caching allocator and passes raw pointers.

Tile knobs (`block_m`, `phase*_warps`, `phase*_stages`, `input_precision`) are validated and then
advisory: the kernels have fixed tiles.  `block_n` is the K-partition width and `q_chunk_size` the
number of query rows whose partition summaries are resident at once; both are honoured (rounded up
to the kernel tile) when given and chosen by the library otherwise.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Literal, Optional

import torch

from . import _lib


@dataclass(frozen=True)
class _BiasMeta:
    """fp32 bias seen as [B|1, H|1, N, N] with zero strides on broadcast axes
    (reference: `_BiasMeta` / `_canonical_bias`, attention.py:12-19, 120-159)."""
    tensor: Optional[torch.Tensor]
    stride_b: int
    stride_h: int
    stride_q: int
    stride_k: int
    has_bias: bool

    @property
    def ptr(self):
        return self.tensor.data_ptr() if self.has_bias else None

    def c_args(self):
        return (self.ptr, self.stride_b, self.stride_h, self.stride_q, self.stride_k)


def _validate_warps(name: str, value: int) -> int:
    value = int(value)
    if value not in (1, 2, 4, 8):
        raise ValueError(f"{name} must be one of 1, 2, 4, or 8")
    return value


def _canonical_bias(bias: Optional[torch.Tensor], *, batch: int, heads: int, seq_len: int,
                    device: torch.device) -> _BiasMeta:
    if bias is None:
        return _BiasMeta(None, 0, 0, 0, 0, False)
    if bias.device != device:
        raise ValueError("bias must live on the same device as q/k/v")
    if tuple(bias.shape[-2:]) != (seq_len, seq_len):
        raise ValueError(f"bias last dims must be {(seq_len, seq_len)}, got {tuple(bias.shape)}")
    if bias.dim() == 2:
        lead = (1, 1)
    elif bias.dim() == 3:
        if bias.shape[0] not in (1, heads):
            raise ValueError("3D bias must have shape [1,N,N] or [H,N,N]")
        lead = (1, int(bias.shape[0]))
    elif bias.dim() == 4:
        if bias.shape[0] not in (1, batch) or bias.shape[1] not in (1, heads):
            raise ValueError("4D bias must broadcast as [B,H,N,N]")
        lead = (int(bias.shape[0]), int(bias.shape[1]))
    else:
        raise ValueError("bias must have shape [N,N], [H,N,N], or [B,H,N,N]")
    view = bias.detach()
    if view.dtype != torch.float32:
        view = view.to(torch.float32)
    if not view.is_contiguous():
        view = view.contiguous()
    view = view.view(lead[0], lead[1], seq_len, seq_len)
    return _BiasMeta(view,
                     0 if lead[0] == 1 else int(view.stride(0)),
                     0 if lead[1] == 1 else int(view.stride(1)),
                     int(view.stride(2)), int(view.stride(3)), True)


def _check_qkv(q, k, v, who: str):
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k, v must have shape [B,H,N,D]")
    if q.shape != k.shape or q.shape != v.shape:
        raise ValueError("q, k, v must have identical shapes")
    if q.device.type != "cuda":
        raise ValueError(f"{who} currently requires CUDA tensors")
    if q.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise ValueError("supported dtypes are fp16, bf16, and fp32")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q, k, v must share one dtype")


def _resolve_common(q, *, algorithm, input_precision, summary_dtype, block_m, block_n, q_chunk_size,
                    phase1_warps, phase2_warps, phase1_stages, phase2_stages):
    if algorithm not in ("auto", "paper_scan"):
        raise ValueError("only algorithm='paper_scan' is available in this strict release")
    if input_precision not in ("auto", "ieee", "tf32", "tf32x3"):
        raise ValueError("input_precision must be 'auto', 'ieee', 'tf32', or 'tf32x3'")
    if summary_dtype is None:
        summary_dtype = q.dtype
    if summary_dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise ValueError("summary_dtype must be fp16, bf16, or fp32")
    for name, val in (("phase1_warps", phase1_warps), ("phase2_warps", phase2_warps)):
        if val is not None:
            _validate_warps(name, val)
    for val in (block_m, phase1_stages, phase2_stages):
        if val is not None:
            int(val)
    part_width = 0 if block_n is None else max(16, int(block_n))
    q_chunk = 0 if q_chunk_size is None else max(16, int(q_chunk_size))
    return summary_dtype, part_width, q_chunk


def _aligned(t: torch.Tensor) -> torch.Tensor:
    t = t.contiguous()
    if t.data_ptr() % 16:
        t = t.clone()
    return t


def _bhnd_strides(t: torch.Tensor):
    """(batch, head, row) element strides of a [B, H, N, D] view the kernels can read in place, or None when it has
    to be copied first: the D axis must be contiguous, the other strides multiples of 8 elements (size-1 axes may
    have any stride) and the first element 16-byte aligned."""
    if t.dim() != 4:
        return None
    b, h, n, d = t.shape
    s0, s1, s2, s3 = t.stride()
    if (d > 1 and s3 != 1) or t.data_ptr() % 16:
        return None
    pad = d * 8                                  # any valid value for a size-1 axis
    if b <= 1:
        s0 = pad
    if h <= 1:
        s1 = pad
    if n <= 1:
        s2 = pad
    if (s0 | s1 | s2) % 8 or s0 <= 0 or s1 <= 0 or s2 < d or s2 <= 0:
        return None
    return (s0, s1, s2)


def _in_place_or_copy(t: torch.Tensor):
    """(tensor, strides): the tensor itself with its strides when the kernels can read it in place, else an aligned
    contiguous copy."""
    st = _bhnd_strides(t)
    if st is not None:
        return t, st
    t = _aligned(t)
    return t, _bhnd_strides(t)


def _empty_like_layout(ref: torch.Tensor, like_strides) -> torch.Tensor:
    """An uninitialised [B, H, N, D] tensor whose axis order in memory follows `ref`: when ref is a row-major
    [B, N, H, D] view (what the model hooks produce from a packed projection), so is the result, and a later
    transpose(1, 2).reshape(B, N, H*D) is free; otherwise plain contiguous."""
    b, h, n, d = ref.shape
    if like_strides is not None and h > 1 and n > 1 and like_strides[1] < like_strides[2]:
        return torch.empty((b, n, h, d), device=ref.device, dtype=ref.dtype).permute(0, 2, 1, 3)
    return torch.empty((b, h, n, d), device=ref.device, dtype=ref.dtype)


_WS_CACHE: dict = {}


def _cached_bytes(fn_name: str, *args) -> int:
    """Workspace size queries are pure functions of their arguments: remember them (the per-call ctypes round trip is
    a measurable part of a 49-token window problem)."""
    key = (fn_name,) + args
    val = _WS_CACHE.get(key)
    if val is None:
        val = int(getattr(_lib.load(), fn_name)(*args))
        _WS_CACHE[key] = val
    return val


class _DeviceScope:
    """`torch.cuda.device(dev)` only when dev is not already current (entering the context manager costs several
    microseconds per call)."""

    def __init__(self, dev):
        self._ctx = None if dev.index is None or dev.index == torch.cuda.current_device() else torch.cuda.device(dev)

    def __enter__(self):
        if self._ctx is not None:
            self._ctx.__enter__()

    def __exit__(self, *exc):
        if self._ctx is not None:
            self._ctx.__exit__(*exc)
        return False


def _i64x(*triples):
    import ctypes
    flat = [int(x) for tr in triples for x in tr]
    return (ctypes.c_int64 * len(flat))(*flat)


def _forward_impl(q, k, v, *, bias, is_causal, summary_dtype, part_width, q_chunk, want_state, flags=0):
    """Runs the two passes; returns (out, row_m, row_z, q_c, k_c, v_c).  q, k, v are read in place when their layout
    allows it (any [B, H, N, D] view with a contiguous D axis and 16-byte aligned rows), and `out` follows q's axis
    order in memory; only other layouts are copied first."""
    lib = _lib.load()
    batch, heads, seq_len, head_dim = map(int, q.shape)
    strided = (not (flags & _lib.FLAG_REF_ROUNDING) and head_dim % 8 == 0 and
               not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()))
    if strided:
        (q_c, qs), (k_c, ks), (v_c, vs) = (_in_place_or_copy(t) for t in (q, k, v))
        strided = any(not t.is_contiguous() for t in (q_c, k_c, v_c))
    if not strided:
        q_c, k_c, v_c = _aligned(q), _aligned(k), _aligned(v)
        out = torch.empty_like(q_c)
    else:
        out = _empty_like_layout(q_c, qs)
        os_ = _bhnd_strides(out)
    bh = batch * heads
    row_m = row_z = None
    if want_state:
        row_m = torch.empty((bh, seq_len), device=q.device, dtype=torch.float32)
        row_z = torch.empty_like(row_m)
    meta = _canonical_bias(bias, batch=batch, heads=heads, seq_len=seq_len, device=q.device)
    dt, sdt = _lib.dtype_code(q.dtype), _lib.dtype_code(summary_dtype)
    nbytes = _cached_bytes("elsa_forward_workspace_bytes", dt, sdt, batch, heads, seq_len, head_dim, int(meta.has_bias),
                           int(bool(is_causal)), part_width, q_chunk, flags)
    if nbytes < 0:
        raise ValueError("elsa_b200: unsupported problem size for the forward")
    with _DeviceScope(q.device):
        ws = torch.empty((max(int(nbytes), 256),), device=q.device, dtype=torch.uint8)
        stream = _lib.raw_stream(q.device)
        rm_p = None if row_m is None else row_m.data_ptr()
        rz_p = None if row_z is None else row_z.data_ptr()
        if strided:
            rc = lib.elsa_twopass_forward_strided(
                q_c.data_ptr(), k_c.data_ptr(), v_c.data_ptr(), _i64x(qs), _i64x(ks), _i64x(vs), *meta.c_args(),
                out.data_ptr(), _i64x(os_), rm_p, rz_p, ws.data_ptr(), ws.numel(), dt, sdt, batch, heads, seq_len,
                head_dim, int(bool(is_causal)), part_width, q_chunk, flags, stream)
        else:
            rc = lib.elsa_twopass_forward(
                q_c.data_ptr(), k_c.data_ptr(), v_c.data_ptr(), *meta.c_args(), out.data_ptr(), rm_p, rz_p,
                ws.data_ptr(), ws.numel(), dt, sdt, batch, heads, seq_len, head_dim, int(bool(is_causal)),
                part_width, q_chunk, flags, stream)
    _lib.check(rc, "elsa_twopass_forward")
    return out, row_m, row_z, q_c, k_c, v_c


def twopass_attention(
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
    reference_rounding: bool = False,
) -> torch.Tensor:
    """Exact softmax attention softmax(q k^T / sqrt(D) + bias) v as a two-pass monoid reduction.

    Phase 1 writes one (m, z, s) summary per K partition to global memory; phase 2 merges the
    partition summaries (for causal attention: the last inclusive prefix) and emits s / z.
    q, k, v: [B, H, N, D], one dtype in {fp16, bf16, fp32}, D <= 128, CUDA.  Returns [B, H, N, D].

    `reference_rounding` (not a keyword of the reference) reproduces the rounding points of the reference's fp16
    head-dim-64 kernels (q scaled by log2(e)/8 in fp16, attention_parallel_scan.py:153-154,160) where the reference
    would run them (fp16, D = 64, no bias, not causal); by default the scale is applied exactly, in fp32.
    """
    _check_qkv(q, k, v, "twopass_attention")
    if algorithm not in ("auto", "paper_scan"):
        raise ValueError("only algorithm='paper_scan' is available in this strict release")
    if int(q.shape[2]) <= 0:
        return torch.empty_like(q)
    if int(q.shape[3]) > 128:
        raise ValueError("head_dim > 128 is not supported by the current kernels")
    summary_dtype, part_width, q_chunk = _resolve_common(
        q, algorithm=algorithm, input_precision=input_precision, summary_dtype=summary_dtype, block_m=block_m,
        block_n=block_n, q_chunk_size=q_chunk_size, phase1_warps=phase1_warps, phase2_warps=phase2_warps,
        phase1_stages=phase1_stages, phase2_stages=phase2_stages)
    return _forward_impl(q, k, v, bias=bias, is_causal=is_causal, summary_dtype=summary_dtype,
                         part_width=part_width, q_chunk=q_chunk, want_state=False,
                         flags=_lib.FLAG_REF_ROUNDING if reference_rounding else 0)[0]
