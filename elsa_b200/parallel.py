"""Multi-GPU forms of the two-pass attention (one process per GPU, torch.distributed for plumbing).

The reference is single-GPU; these are the two ways its path shards:

* batch x heads: rows of B*H are independent (the reference's grid axis `pid_bh`,
  src/elsa_twopass_clean/attention.py:51).  `shard_heads` slices q, k, v; no collective is needed.

* sequence (K partitions): the (m, z, s) merge is associative and commutative for the non-causal
  total, and for causal rows a shard that lies in the future contributes the identity, so every GPU
  folds its own K/V rows for ALL query rows and the per-GPU summaries are combined with the same
  operator the single-GPU phase 2 uses (cuda/paper_scan_d64_kernel.cu:39-70):
      M = max over ranks of m            -> all_reduce(MAX)
      w = 2^(m - M) (0 where z == 0)     -> local
      Z, S = sum over ranks of z*w, s*w  -> all_reduce(SUM) of one concatenated [z | s] buffer
      out = S / Z
  `merge_summaries_across_ranks` is that exchange on plain host or device tensors (the form the CPU
  ranks of the gloo tests run).  On GPUs `merge_shards_on_gpu` does the same with two kernels of the library
  around the collectives and a reduce_scatter instead of the all_reduce, so that every rank finalises only
  N / world rows: all_reduce(MAX) of m (4 B per row), elsa_shard_pack (w, z*w, s*w written chunk-per-rank),
  reduce_scatter(SUM), elsa_shard_finalize (S / Z, row state), then an all_gather of the finished rows where
  the caller wants them everywhere.  `sequence_parallel_attention` is the GPU forward built on it.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import _lib
from .attention import _aligned, _check_qkv


def shard_heads(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """[B, H, N, D] -> this rank's contiguous slice of the flattened batch*head axis, as [1, BH/world, N, D]."""
    b, h, n, d = t.shape
    bh = b * h
    if bh % world:
        raise ValueError("batch*heads must be divisible by the number of ranks")
    per = bh // world
    return t.reshape(bh, n, d)[rank * per:(rank + 1) * per].reshape(1, per, n, d)


def merge_summaries_across_ranks(m: torch.Tensor, z: torch.Tensor, s: torch.Tensor, group=None
                                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Combine one (m, z, s) summary per row per rank into the global result.

    m, z: [...]; s: [..., D]; fp32, same shape on every rank.  Returns (out, row_m, row_z) with
    out = S / Z (0 where Z == 0), row_m = M (-inf where Z == 0), row_z = Z -- the state the backward uses."""
    m = m.float()
    big_m = m.clone()
    dist.all_reduce(big_m, op=dist.ReduceOp.MAX, group=group)
    w = torch.where(z > 0, torch.exp2(m - big_m), torch.zeros((), device=m.device))
    buf = torch.cat([(z * w).unsqueeze(-1), s.float() * w.unsqueeze(-1)], dim=-1).contiguous()
    dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group)
    big_z, big_s = buf[..., 0], buf[..., 1:]
    out = torch.where(big_z.unsqueeze(-1) > 0, big_s / big_z.unsqueeze(-1), torch.zeros((), device=m.device))
    row_m = torch.where(big_z > 0, big_m, torch.full((), float("-inf"), device=m.device))
    return out, row_m, big_z


def local_shard_summary(q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor, *, key_offset: int,
                        is_causal: bool = False, part_width: int = 2048
                        ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Phase 1 + local merge of ONE sequence shard on this GPU.

    q: [B, H, N, D] (all query rows); k_shard, v_shard: [B, H, Nk, D] (rows key_offset .. key_offset+Nk-1 of
    the sequence).  Returns fp32 (m, z, s) with one un-normalised summary per query row: [B*H, N], [B*H, N, D].
    The partition summaries are kept in fp32 whatever the input dtype: they are summed across GPUs next."""
    lib = _lib.load()
    if q.dim() != 4 or k_shard.dim() != 4 or k_shard.shape != v_shard.shape:
        raise ValueError("q must be [B,H,N,D] and k_shard, v_shard [B,H,Nk,D]")
    if q.device.type != "cuda":
        raise ValueError("local_shard_summary currently requires CUDA tensors")
    b, h, n, d = map(int, q.shape)
    nk = int(k_shard.shape[2])
    if tuple(k_shard.shape) != (b, h, nk, d) or k_shard.dtype != q.dtype or v_shard.dtype != q.dtype:
        raise ValueError("k_shard / v_shard must match q in batch, heads, head_dim and dtype")
    q_c, k_c, v_c = _aligned(q), _aligned(k_shard), _aligned(v_shard)
    dt = _lib.dtype_code(q.dtype)
    pw = max(128, (int(part_width) + 127) // 128 * 128)
    parts = max(1, -(-nk // pw))
    bh = b * h
    dev = q.device
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        m = torch.empty((bh, n), device=dev, dtype=torch.float32)
        z = torch.empty_like(m)
        s = torch.empty((bh, n, d), device=dev, dtype=torch.float32)
        if nk == 0:                      # an empty shard contributes the identity
            m.fill_(float("-inf")); z.zero_(); s.zero_()
            return m, z, s
        if parts == 1:                   # one partition: its summary IS the shard's summary
            m_p, z_p, s_p = m, z, s
        else:
            m_p = torch.empty((parts, bh, n), device=dev, dtype=torch.float32)
            z_p = torch.empty_like(m_p)
            s_p = torch.empty((parts, bh, n, d), device=dev, dtype=torch.float32)
        ws_bytes = int(lib.elsa_phase1_fold_shard_workspace_bytes(dt, b, h, n, d, nk, 0))
        if ws_bytes < 0:
            raise ValueError("local_shard_summary: unsupported problem")
        ws = torch.empty((max(ws_bytes, 256),), device=dev, dtype=torch.uint8)
        rc = lib.elsa_phase1_fold_shard_ws(q_c.data_ptr(), k_c.data_ptr(), v_c.data_ptr(), m_p.data_ptr(), z_p.data_ptr(),
                                           s_p.data_ptr(), ws.data_ptr(), ws.numel(), dt, _lib.ELSA_F32, b, h, n, d, nk,
                                           int(key_offset), pw, parts, int(bool(is_causal)), 0, stream)
        _lib.check(rc, "elsa_phase1_fold_shard_ws")
        if parts > 1:
            rc = lib.elsa_merge_partial(m_p.data_ptr(), z_p.data_ptr(), s_p.data_ptr(), s.data_ptr(), m.data_ptr(),
                                        z.data_ptr(), _lib.ELSA_F32, parts, bh, n, d, stream)
            _lib.check(rc, "elsa_merge_partial")
    return m, z, s


def merge_shards_on_gpu(m: torch.Tensor, z: torch.Tensor, s: torch.Tensor, out_dtype: torch.dtype, *, group=None,
                        gather: bool = True):
    """Cross-GPU merge of one fp32 (m, z, s) summary per row per rank, with the library's kernels around NCCL.

    m, z: [BH, N]; s: [BH, N, D]; CUDA fp32.  Returns (out, row_m, row_z): with gather, the finished rows of all
    ranks ([BH, N, D] in out_dtype, [BH, N] fp32) on every rank; without, only this rank's rows
    [rank*N/world, (rank+1)*N/world) as ([BH, N/world, D], [BH, N/world], [BH, N/world]).
    When N does not divide by the world size every rank sums and finalises all rows (all_reduce form)."""
    lib = _lib.load()
    bh, n, d = map(int, s.shape)
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    rank = dist.get_rank(group) if world > 1 else 0
    scatter = world > 1 and n % world == 0 and (bh * (n // world) * (d + 1)) % 4 == 0
    w_eff, r_eff = (world, rank) if scatter else (1, 0)
    dev = s.device
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        m_all = m
        if world > 1:
            m_all = m.clone()
            dist.all_reduce(m_all, op=dist.ReduceOp.MAX, group=group)
        chunk = int(lib.elsa_shard_chunk_elems(bh, n, d, w_eff))
        packed = torch.empty((w_eff * chunk,), device=dev, dtype=torch.float32)
        _lib.check(lib.elsa_shard_pack(m.data_ptr(), z.data_ptr(), s.data_ptr(), m_all.data_ptr(), packed.data_ptr(),
                                       bh, n, d, w_eff, stream), "elsa_shard_pack")
        if scatter:
            mine = torch.empty((chunk,), device=dev, dtype=torch.float32)
            dist.reduce_scatter_tensor(mine, packed, op=dist.ReduceOp.SUM, group=group)
        else:
            mine = packed
            if world > 1:
                dist.all_reduce(mine, op=dist.ReduceOp.SUM, group=group)
        nl = n // w_eff
        out = torch.empty((bh, nl, d), device=dev, dtype=out_dtype)
        row_m = torch.empty((bh, nl), device=dev, dtype=torch.float32)
        row_z = torch.empty_like(row_m)
        _lib.check(lib.elsa_shard_finalize(mine.data_ptr(), m_all.data_ptr(), out.data_ptr(), row_m.data_ptr(),
                                           row_z.data_ptr(), _lib.dtype_code(out_dtype), bh, n, d, w_eff, r_eff, stream),
                   "elsa_shard_finalize")
        if not scatter or not gather:
            return out, row_m, row_z
        # the finished rows of every rank: [world, BH, N/world, ...] -> [BH, N, ...]
        g_out = torch.empty((world, bh, nl, d), device=dev, dtype=out_dtype)
        dist.all_gather_into_tensor(g_out, out, group=group)
        state = torch.stack((row_m, row_z))                              # one collective for both vectors
        g_state = torch.empty((world, 2, bh, nl), device=dev, dtype=torch.float32)
        dist.all_gather_into_tensor(g_state, state, group=group)
        out = g_out.permute(1, 0, 2, 3).reshape(bh, n, d)
        g_state = g_state.permute(1, 2, 0, 3).reshape(2, bh, n)
        return out, g_state[0].contiguous(), g_state[1].contiguous()


def sequence_parallel_attention(q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor, *, key_offset: int,
                                is_causal: bool = False, part_width: int = 2048, group=None,
                                return_state: bool = False):
    """Forward of exact attention with K/V sharded along the sequence over the ranks of `group`.

    Every rank passes the full q and its own K/V rows; every rank gets the full output [B, H, N, D] (input dtype)
    and, with return_state, the global (row_m, row_z)."""
    _check_qkv(q, q, q, "sequence_parallel_attention")
    b, h, n, d = map(int, q.shape)
    m, z, s = local_shard_summary(q, k_shard, v_shard, key_offset=key_offset, is_causal=is_causal, part_width=part_width)
    out, row_m, row_z = merge_shards_on_gpu(m, z, s, q.dtype, group=group, gather=True)
    out = out.reshape(b, h, n, d)
    if return_state:
        return out, row_m, row_z
    return out


# ---- backward of the sequence-sharded form -------------------------------------------------------
# dK and dV of a shard need only the global row state (LSE, D) and are complete on the rank that owns the
# K/V rows; dQ is a sum over the shards: every rank computes its contribution in fp32 and the contributions
# are added across ranks before rounding to the input dtype.

def reduce_dq_across_ranks(dq_partial: torch.Tensor, *, scatter: bool = False, group=None) -> torch.Tensor:
    """Sum the per-shard fp32 dQ contributions ([..., N, D], same shape on every rank).

    scatter=False: every rank gets the full sum (all_reduce).  scatter=True: rank r gets rows
    [r*N/W, (r+1)*N/W) of the sum (reduce_scatter along the sequence axis; N must divide by the world size)."""
    if not scatter:
        dist.all_reduce(dq_partial, op=dist.ReduceOp.SUM, group=group)
        return dq_partial
    world = dist.get_world_size(group)
    n = dq_partial.shape[-2]
    if n % world:
        raise ValueError("reduce_scatter of dQ needs the sequence length to be divisible by the number of ranks")
    chunks = [c.contiguous() for c in dq_partial.chunk(world, dim=-2)]
    out = torch.empty_like(chunks[0])
    if dq_partial.device.type == "cuda":
        dist.reduce_scatter(out, chunks, op=dist.ReduceOp.SUM, group=group)
    else:
        # gloo has no reduce_scatter: all_reduce and keep this rank's rows
        dist.all_reduce(dq_partial, op=dist.ReduceOp.SUM, group=group)
        out = dq_partial.chunk(world, dim=-2)[dist.get_rank(group)].contiguous()
    return out


def local_shard_backward(q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor, out: torch.Tensor,
                         dout: torch.Tensor, row_m: torch.Tensor, row_z: torch.Tensor, *, key_offset: int,
                         is_causal: bool = False, flags: int = 0
                         ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Backward of ONE sequence shard on this GPU.

    q, out, dout: [B, H, N, D]; k_shard, v_shard: [B, H, Nk, D]; row_m, row_z: [B*H, N] fp32, the state of the
    merged forward.  Returns (dq_partial fp32 [B, H, N, D], dk_shard, dv_shard [B, H, Nk, D] in the input dtype)."""
    lib = _lib.load()
    if q.dim() != 4 or k_shard.dim() != 4 or k_shard.shape != v_shard.shape or out.shape != q.shape or dout.shape != q.shape:
        raise ValueError("q, out, dout must be [B,H,N,D] and k_shard, v_shard [B,H,Nk,D]")
    if q.device.type != "cuda":
        raise ValueError("local_shard_backward requires CUDA tensors")
    b, h, n, d = map(int, q.shape)
    nk = int(k_shard.shape[2])
    if tuple(k_shard.shape) != (b, h, nk, d) or any(t.dtype != q.dtype for t in (k_shard, v_shard, out, dout)):
        raise ValueError("k_shard / v_shard / out / dout must match q in batch, heads, head_dim and dtype")
    q_c, k_c, v_c, o_c, g_c = (_aligned(t) for t in (q, k_shard, v_shard, out, dout))
    rm = row_m.reshape(b * h, n).float().contiguous()
    rz = row_z.reshape(b * h, n).float().contiguous()
    dt = _lib.dtype_code(q.dtype)
    dev = q.device
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        dq = torch.empty((b, h, n, d), device=dev, dtype=torch.float32)
        dk = torch.empty((b, h, nk, d), device=dev, dtype=q.dtype)
        dv = torch.empty_like(dk)
        ws_bytes = int(lib.elsa_backward_shard_workspace_bytes(dt, b, h, n, d, flags))
        if ws_bytes < 0:
            raise ValueError("local_shard_backward: unsupported problem")
        ws = torch.empty(max(ws_bytes, 256), device=dev, dtype=torch.uint8)
        rc = lib.elsa_twopass_backward_shard(q_c.data_ptr(), k_c.data_ptr() if nk else None, v_c.data_ptr() if nk else None,
                                             o_c.data_ptr(), g_c.data_ptr(), rm.data_ptr(), rz.data_ptr(), dq.data_ptr(),
                                             dk.data_ptr() if nk else None, dv.data_ptr() if nk else None, ws.data_ptr(),
                                             ws_bytes, dt, b, h, n, d, nk, int(key_offset), int(bool(is_causal)),
                                             int(flags), stream)
        _lib.check(rc, "elsa_twopass_backward_shard")
    return dq, dk, dv


def sequence_parallel_attention_backward(q: torch.Tensor, k_shard: torch.Tensor, v_shard: torch.Tensor,
                                         out: torch.Tensor, dout: torch.Tensor, row_m: torch.Tensor,
                                         row_z: torch.Tensor, *, key_offset: int, is_causal: bool = False,
                                         scatter_dq: bool = False, group=None):
    """Backward of `sequence_parallel_attention`: (dq, dk_shard, dv_shard).

    Every rank passes the full q, out, dout, the global (row_m, row_z) returned by the forward with
    return_state=True, and its own K/V rows.  dk_shard / dv_shard are this rank's rows; dq is the full gradient on
    every rank (or, with scatter_dq, this rank's N/world rows), rounded to the input dtype after the fp32 sum."""
    dq_part, dk, dv = local_shard_backward(q, k_shard, v_shard, out, dout, row_m, row_z, key_offset=key_offset,
                                           is_causal=is_causal)
    dq = reduce_dq_across_ranks(dq_part, scatter=scatter_dq, group=group)
    return dq.to(q.dtype), dk, dv
