"""Sequence-sharded forward and backward on the GPU: per-shard summaries (C ABI elsa_phase1_fold_shard + elsa_merge_partial)
merged with the monoid give the unsharded result.  One-GPU form: shards are folded one after the other on
the same device and merged on the host with the oracle's operator; two-GPU form (skipped on a single-GPU box):
two NCCL ranks through elsa_b200.parallel.sequence_parallel_attention."""
import os
import socket

import pytest
import torch

import elsa_b200 as E
from elsa_b200.parallel import local_shard_backward, local_shard_summary
from oracle import elsa_oracle as O
from tests import _util as U

pytestmark = pytest.mark.gpu
F32, F16, BF16 = torch.float32, torch.float16, torch.bfloat16


@pytest.mark.parametrize("dtype,n,bounds,d", [(F32, 300, [0, 100, 300], 64), (F16, 1500, [0, 640, 1100, 1500], 64),
                                              (BF16, 1024, [0, 512, 1024], 64), (F16, 200, [0, 64, 200], 64),
                                              (F16, 1500, [0, 640, 1100, 1500], 128), (BF16, 1024, [0, 512, 1024], 32),
                                              (F32, 1024, [0, 384, 1024], 32)])
@pytest.mark.parametrize("causal", [False, True])
def test_shards_merge_to_full_attention(dtype, n, bounds, d, causal):
    b, h = 1, 2
    q, k, v = (U.seeded((b, h, n, d), dtype, 90 + i).cuda() for i in range(3))
    state = None
    for k0, k1 in zip(bounds[:-1], bounds[1:]):
        m, z, s = local_shard_summary(q, k[:, :, k0:k1], v[:, :, k0:k1], key_offset=k0, is_causal=causal, part_width=256)
        cur = (m.cpu(), z.cpu(), s.cpu())
        state = cur if state is None else O.monoid_merge(state, cur)
    out, rm, rz = O.finalize(*state)
    full, fm, fz = E.twopass_attention_with_state(q, k, v, is_causal=causal)
    assert U.out_close(out.reshape(b, h, n, d).to(dtype), full, dtype) <= 1.0
    truth = O.softmax_attention_fp64(q.cpu(), k.cpu(), v.cpu(), is_causal=causal)
    assert U.out_close(out.reshape(b, h, n, d), truth, F32 if dtype == F32 else dtype) <= (1.0 if dtype == F32 else 2.0)
    lse = rm + torch.log2(rz)
    lse_full = fm.cpu() + torch.log2(fz.cpu())
    assert (lse - lse_full).abs().max().item() <= (2e-5 if dtype == F32 else 5e-3)


@pytest.mark.parametrize("dtype,n,bounds,d", [(F32, 300, [0, 100, 300], 64),            # FP32-FMA kernels, ragged shards
                                              (F16, 1500, [0, 640, 1100, 1500], 64),    # tcgen05 kernel, offsets off the 128 grid
                                              (BF16, 1024, [0, 512, 1024], 64),
                                              (F16, 640, [0, 0, 640], 64),              # an empty shard
                                              (F16, 200, [0, 64, 200], 64),             # 16-bit below the tensor-core size
                                              (F32, 1024, [0, 384, 1024], 64),          # fp32 on the tensor cores, ragged shards
                                              (F16, 1500, [0, 640, 1100, 1500], 128),   # wide-head kernels
                                              (BF16, 1024, [0, 512, 1024], 96)])
@pytest.mark.parametrize("causal", [False, True])
def test_shard_backward_sums_to_full_backward(dtype, n, bounds, d, causal):
    """C ABI elsa_twopass_backward_shard per K/V shard (all on one device): the fp32 dQ contributions add up to the
    unsharded dQ, and the shards' dK / dV are the corresponding rows of the unsharded dK / dV."""
    b, h = 1, 2
    q, k, v, do = (U.seeded((b, h, n, d), dtype, 190 + i).cuda() for i in range(4))
    out, rm, rz = E.twopass_attention_with_state(q, k, v, is_causal=causal)[:3]
    dq_f, dk_f, dv_f = E.twopass_attention_backward(q, k, v, out, do, row_m=rm, row_z=rz, is_causal=causal)[:3]
    dq_sum = torch.zeros(b, h, n, d, device="cuda", dtype=torch.float32)
    dk_parts, dv_parts = [], []
    for k0, k1 in zip(bounds[:-1], bounds[1:]):
        dq_p, dk_p, dv_p = local_shard_backward(q, k[:, :, k0:k1], v[:, :, k0:k1], out, do, rm, rz, key_offset=k0,
                                                is_causal=causal)
        assert dq_p.dtype == torch.float32 and dk_p.shape == (b, h, k1 - k0, d)
        dq_sum += dq_p
        dk_parts.append(dk_p); dv_parts.append(dv_p)
    dk_s, dv_s = torch.cat(dk_parts, dim=2), torch.cat(dv_parts, dim=2)
    # the sharded run differs from the unsharded one only in the order of fp32 additions of dQ
    tol = 2e-6 if dtype == F32 else None
    for name, a, ref in (("dq", dq_sum, dq_f), ("dk", dk_s, dk_f), ("dv", dv_s, dv_f)):
        if dtype == F32:
            assert (a.float() - ref.float()).abs().max().item() <= tol * max(1.0, ref.float().abs().max().item()), name
        else:
            assert U.out_close(a.to(dtype), ref, dtype) <= 2.0, name


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _nccl_worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from elsa_b200.parallel import sequence_parallel_attention, sequence_parallel_attention_backward
        # (dtype, N): N divisible by the world size takes the reduce_scatter form, N = 1025 the all_reduce form
        for dtype, n in ((F16, 2048), (F32, 1025)):
            b, h, d = 1, 4, 64
            q, k, v = (U.seeded((b, h, n, d), dtype, 95 + i).cuda() for i in range(3))
            per = -(-n // world)
            lo, hi = rank * per, min(n, (rank + 1) * per)
            for causal in (False, True):
                out = sequence_parallel_attention(q, k[:, :, lo:hi], v[:, :, lo:hi], key_offset=lo, is_causal=causal)
                full = E.twopass_attention(q, k, v, is_causal=causal)
                ret[(rank, str(dtype), causal)] = U.out_close(out, full, dtype)
                # backward: global state from the sharded forward, dQ summed over the ranks
                do = U.seeded((b, h, n, d), dtype, 99).cuda()
                out_s, rm, rz = sequence_parallel_attention(q, k[:, :, lo:hi], v[:, :, lo:hi], key_offset=lo,
                                                            is_causal=causal, return_state=True)
                dq, dk, dv = sequence_parallel_attention_backward(q, k[:, :, lo:hi], v[:, :, lo:hi], out_s, do, rm, rz,
                                                                  key_offset=lo, is_causal=causal)
                fo, fm, fz = E.twopass_attention_with_state(q, k, v, is_causal=causal)[:3]
                dq_f, dk_f, dv_f = E.twopass_attention_backward(q, k, v, fo, do, row_m=fm, row_z=fz, is_causal=causal)[:3]
                if dtype == F32:
                    big = max(1.0, float(dq_f.abs().max()), float(dk_f.abs().max()), float(dv_f.abs().max()))
                    err = max((dq - dq_f).abs().max().item(), (dk - dk_f[:, :, lo:hi]).abs().max().item(),
                              (dv - dv_f[:, :, lo:hi]).abs().max().item()) / (2e-6 * big)
                else:
                    err = max(U.out_close(dq, dq_f, dtype), U.out_close(dk, dk_f[:, :, lo:hi], dtype),
                              U.out_close(dv, dv_f[:, :, lo:hi], dtype))
                ret[(rank, str(dtype), causal, "bwd")] = err
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sequence_parallel_two_gpus():
    import torch.multiprocessing as mp
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_nccl_worker, args=(2, port, ret), nprocs=2, join=True)
    got = {" ".join(map(str, key)): val for key, val in dict(ret).items()}
    report = os.environ.get("ELSA_PARALLEL_REPORT")
    if report:                                   # worst error / limit per (rank, dtype, causal[, bwd])
        import json
        with open(report, "w") as fh:
            json.dump(got, fh, indent=1, sort_keys=True)
    assert len(got) == 16 and all(v <= 2.0 for v in got.values()), got


@pytest.mark.parametrize("world,n,dtype", [(4, 1024, F32), (2, 640, F16), (8, 2048, BF16), (1, 300, F32)])
def test_pack_reduce_finalize_kernels_emulated_ranks(world, n, dtype):
    """elsa_shard_pack / elsa_shard_finalize with the collectives emulated on one device: the shards' summaries are
    packed per emulated rank, the packed buffers are added (what reduce_scatter does), each chunk is finalised, and the
    rows are put back together; the result must be the oracle's merge of the same summaries."""
    from elsa_b200 import _lib
    lib = _lib.load()
    b, h, d = 1, 3, 64
    bh = b * h
    q, k, v = (U.seeded((b, h, n, d), dtype, 70 + i).cuda() for i in range(3))
    shards = max(world, 2)
    per = -(-n // shards)
    summ = [local_shard_summary(q, k[:, :, i * per:min(n, (i + 1) * per)], v[:, :, i * per:min(n, (i + 1) * per)],
                                key_offset=i * per, is_causal=True, part_width=128) for i in range(shards)]
    m_all = torch.stack([x[0] for x in summ]).max(0).values.contiguous()
    chunk = lib.elsa_shard_chunk_elems(bh, n, d, world)
    assert chunk == bh * (n // world) * (d + 1)
    total = torch.zeros(world * chunk, device="cuda")
    for m, z, s in summ:
        packed = torch.full((world * chunk,), float("nan"), device="cuda")
        rc = lib.elsa_shard_pack(m.data_ptr(), z.data_ptr(), s.data_ptr(), m_all.data_ptr(), packed.data_ptr(), bh, n, d,
                                 world, U.stream())
        assert rc == 0
        total += packed
    nl = n // world
    outs, rms, rzs = [], [], []
    for r in range(world):
        out = torch.full((bh, nl, d), float("nan"), device="cuda", dtype=dtype)
        rm = torch.full((bh, nl), float("nan"), device="cuda")
        rz = torch.full_like(rm, float("nan"))
        rc = lib.elsa_shard_finalize(total[r * chunk:(r + 1) * chunk].data_ptr(), m_all.data_ptr(), out.data_ptr(),
                                     rm.data_ptr(), rz.data_ptr(), U.DT[dtype], bh, n, d, world, r, U.stream())
        assert rc == 0
        outs.append(out); rms.append(rm); rzs.append(rz)
    out = torch.cat(outs, dim=1).cpu()
    state = None
    for m, z, s in summ:
        cur = (m.cpu(), z.cpu(), s.cpu())
        state = cur if state is None else O.monoid_merge(state, cur)
    ref_out, ref_m, ref_z = O.finalize(*state)
    assert U.out_close(out, ref_out.to(dtype), dtype) <= 1.0
    lse = torch.cat(rms, dim=1).cpu() + torch.log2(torch.cat(rzs, dim=1).cpu())
    assert (lse - (ref_m + torch.log2(ref_z))).abs().max().item() <= 2e-5
    # argument checks: N must divide by the world size
    assert lib.elsa_shard_chunk_elems(bh, 7, d, 2) == -1
