"""Multi-rank merge of per-GPU summaries, run among CPU ranks (gloo, world size 2 and 3): the exchange
(max -> rescale -> sum) must reproduce single-process attention, including empty (identity) shards,
a rank whose rows are fully masked, and the causal case where a future shard contributes nothing."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import elsa_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, causal, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from elsa_b200.parallel import merge_summaries_across_ranks, shard_heads
        g = torch.Generator().manual_seed(123)
        b, h, n, d = 1, 3, 150, 32
        q, k, v = (torch.randn(b, h, n, d, generator=g) for _ in range(3))
        # uneven shards; with world 3 the last shard is the empty one for early causal rows
        bounds = [0, 40, 150] if world == 2 else [0, 40, 90, 150]
        k0, k1 = bounds[rank], bounds[rank + 1]
        bh = b * h
        q3, k3, v3 = (t.reshape(bh, n, d) for t in (q, k, v))
        # local summary of this shard via the oracle's phase 1 on a key window
        scores = (q3 @ k3[:, k0:k1].transpose(-1, -2)) * (d ** -0.5) * O.LOG2E
        valid = torch.ones(n, k1 - k0, dtype=torch.bool)
        if causal:
            valid = torch.arange(n)[:, None] >= torch.arange(k0, k1)[None, :]
        m, z, s = O._tile_summary(scores, valid[None].expand(bh, -1, -1), v3[:, k0:k1], None)
        out, row_m, row_z = merge_summaries_across_ranks(m, z, s)
        ref = O.softmax_attention_fp64(q, k, v, is_causal=causal).reshape(bh, n, d)
        err = (out.double() - ref).abs().max().item()
        rm_ref, rz_ref = O.row_stats(q3, k3, is_causal=causal)
        lse = row_m + torch.log2(row_z)
        lse_ref = rm_ref + torch.log2(rz_ref)
        err_lse = (lse - lse_ref).abs().max().item()
        # shard_heads: the slices of all ranks tile the batch*head axis
        if bh % world == 0:
            piece = shard_heads(q, rank, world)
            assert piece.shape == (1, bh // world, n, d)
            assert torch.equal(piece[0], q3[rank * (bh // world):(rank + 1) * (bh // world)])
        ret[rank] = (err, err_lse)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("causal", [False, True])
def test_rank_merge_matches_single_process(world, causal):
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, causal, ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank in range(world):
        err, err_lse = ret[rank]
        assert err < 2e-6, (rank, err)
        assert err_lse < 2e-5, (rank, err_lse)


def _identity_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from elsa_b200.parallel import merge_summaries_across_ranks
        rows, d = 7, 4
        if rank == 0:
            m = torch.full((rows,), float("-inf")); z = torch.zeros(rows); s = torch.zeros(rows, d)
        else:
            m = torch.arange(rows, dtype=torch.float32); z = torch.ones(rows) * 2; s = torch.ones(rows, d) * 6
            m[3] = float("-inf"); z[3] = 0; s[3] = 0           # a row that is empty on every rank
        out, row_m, row_z = merge_summaries_across_ranks(m, z, s)
        ok = torch.isfinite(out).all().item() and float(out[3].abs().max()) == 0.0 and row_m[3] == float("-inf")
        ok = ok and torch.allclose(out[[0, 1, 2, 4, 5, 6]], torch.full((6, d), 3.0)) and row_z[3] == 0
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_rank_merge_identity_and_empty_rows():
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_identity_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret[0] and ret[1]


def _bwd_worker(rank, world, port, causal, scatter, ret):
    """Sequence-sharded backward among CPU ranks: each rank forms its shard's (dq_partial, dk, dv) in plain fp64
    torch from the GLOBAL row state, the ranks sum dQ; the result must equal the oracle's full backward."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from elsa_b200.parallel import reduce_dq_across_ranks
        g = torch.Generator().manual_seed(77)
        b, h, n, d = 1, 2, 96, 16
        q, k, v, do = (torch.randn(b, h, n, d, generator=g) for _ in range(4))
        bh = b * h
        q3, k3, v3, g3 = (t.reshape(bh, n, d).double() for t in (q, k, v, do))
        out = O.softmax_attention_fp64(q, k, v, is_causal=causal).reshape(bh, n, d)
        rm, rz = O.row_stats(q3.float(), k3.float(), is_causal=causal)
        lse = (rm + torch.log2(rz)).double()
        drow = (out * g3).sum(-1)
        bounds = [0, 32, 96] if world == 2 else [0, 32, 64, 96]
        k0, k1 = bounds[rank], bounds[rank + 1]
        sc = (q3 @ k3[:, k0:k1].transpose(-1, -2)) * (d ** -0.5) * O.LOG2E
        p = torch.exp2(sc - lse[..., None])
        if causal:
            p = p * (torch.arange(n)[:, None] >= torch.arange(k0, k1)[None, :])
        dp = g3 @ v3[:, k0:k1].transpose(-1, -2)
        ds = p * (dp - drow[..., None])
        dq_part = (ds @ k3[:, k0:k1]) * (d ** -0.5)
        dk = (ds.transpose(-1, -2) @ q3) * (d ** -0.5)
        dv = p.transpose(-1, -2) @ g3
        dq = reduce_dq_across_ranks(dq_part.float().contiguous(), scatter=scatter)
        dq_ref, dk_ref, dv_ref = O.twopass_backward(q, k, v, out.reshape(b, h, n, d).float(), do, rm, rz, is_causal=causal)
        dq_ref = dq_ref.reshape(bh, n, d)
        if scatter:
            dq_ref = dq_ref.chunk(world, dim=-2)[rank]
        e = [(dq.double() - dq_ref.double()).abs().max().item(),
             (dk - dk_ref.reshape(bh, n, d)[:, k0:k1].double()).abs().max().item(),
             (dv - dv_ref.reshape(bh, n, d)[:, k0:k1].double()).abs().max().item()]
        ret[rank] = e
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,scatter", [(2, False), (3, False), (2, True)])
@pytest.mark.parametrize("causal", [False, True])
def test_rank_sum_of_dq_matches_single_process(world, scatter, causal):
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_bwd_worker, args=(world, port, causal, scatter, ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank in range(world):
        assert max(ret[rank]) < 5e-6, (rank, ret[rank])
