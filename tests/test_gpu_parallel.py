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


@pytest.mark.parametrize("dtype,n,bounds", [(F32, 300, [0, 100, 300]), (F16, 1500, [0, 640, 1100, 1500]),
                                            (BF16, 1024, [0, 512, 1024]), (F16, 200, [0, 64, 200])])
@pytest.mark.parametrize("causal", [False, True])
def test_shards_merge_to_full_attention(dtype, n, bounds, causal):
    b, h, d = 1, 2, 64
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


@pytest.mark.parametrize("dtype,n,bounds", [(F32, 300, [0, 100, 300]),            # FP32-FMA kernels, ragged shards
                                            (F16, 1500, [0, 640, 1100, 1500]),    # tcgen05 kernel, offsets off the 128 grid
                                            (BF16, 1024, [0, 512, 1024]),
                                            (F16, 640, [0, 0, 640]),              # an empty shard
                                            (F16, 200, [0, 64, 200])])            # 16-bit below the tensor-core size
@pytest.mark.parametrize("causal", [False, True])
def test_shard_backward_sums_to_full_backward(dtype, n, bounds, causal):
    """C ABI elsa_twopass_backward_shard per K/V shard (all on one device): the fp32 dQ contributions add up to the
    unsharded dQ, and the shards' dK / dV are the corresponding rows of the unsharded dK / dV."""
    b, h, d = 1, 2, 64
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
        b, h, n, d = 1, 4, 2048, 64
        q, k, v = (U.seeded((b, h, n, d), F16, 95 + i).cuda() for i in range(3))
        per = n // world
        for causal in (False, True):
            out = sequence_parallel_attention(q, k[:, :, rank * per:(rank + 1) * per], v[:, :, rank * per:(rank + 1) * per],
                                              key_offset=rank * per, is_causal=causal)
            full = E.twopass_attention(q, k, v, is_causal=causal)
            ret[(rank, causal)] = U.out_close(out, full, F16)
            # backward: global state from the sharded forward, dQ summed over the ranks
            do = U.seeded((b, h, n, d), F16, 99).cuda()
            out_s, rm, rz = sequence_parallel_attention(q, k[:, :, rank * per:(rank + 1) * per],
                                                        v[:, :, rank * per:(rank + 1) * per], key_offset=rank * per,
                                                        is_causal=causal, return_state=True)
            dq, dk, dv = sequence_parallel_attention_backward(q, k[:, :, rank * per:(rank + 1) * per],
                                                              v[:, :, rank * per:(rank + 1) * per], out_s, do, rm, rz,
                                                              key_offset=rank * per, is_causal=causal)
            fo, fm, fz = E.twopass_attention_with_state(q, k, v, is_causal=causal)[:3]
            dq_f, dk_f, dv_f = E.twopass_attention_backward(q, k, v, fo, do, row_m=fm, row_z=fz, is_causal=causal)[:3]
            ret[(rank, causal, "bwd")] = max(U.out_close(dq, dq_f, F16),
                                             U.out_close(dk, dk_f[:, :, rank * per:(rank + 1) * per], F16),
                                             U.out_close(dv, dv_f[:, :, rank * per:(rank + 1) * per], F16))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sequence_parallel_two_gpus():
    import torch.multiprocessing as mp
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_nccl_worker, args=(2, port, ret), nprocs=2, join=True)
    assert len(ret) == 8 and all(v <= 2.0 for v in ret.values()), dict(ret)
