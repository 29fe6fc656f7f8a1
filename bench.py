"""Headline benchmark: ELSA two-pass attention forward + backward, fp16, B=1 H=8 N=16384 d=64.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload headline|...]

One "step" = one forward + backward of the attention operator on one batch of synthetic Q, K, V, dO.
Multi-GPU (torchrun, one rank per GPU): every rank runs its own batch element (batch x heads shards
with no data-path collective), so scaling is "weak" and `value` is the whole-job TFLOP/s; the line also
carries `seq_sharded`, the sequence-sharded long fp32 case (K/V split over the ranks, summaries merged
over NCCL), which is the multi-GPU path that has a real exchange step.

Prints ONE JSON line (rank 0).  `value` is kernel throughput with inputs resident in HBM, timed over a region
of at least two seconds (the --steps block repeated back to back, `timed_steps` in all) so that it is a sustained
figure under the power cap; `e2e` is the same metric through the public PyTorch API with pinned HOST buffers
(H2D of q,k,v,dO and D2H of out,dq,dk,dv inside the timed region).  `--impl reference` times the CPU restatement of
the reference's algorithm (the reference itself has no CPU path and its device code is Triton) on the host cores,
on a bounded sample of the same workload; `reference_gpu` in the default line is the unmodified reference (its
Triton kernels compiled for this GPU) timed on the same tensors with the same events.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "ELSA attn fwd+bwd TFLOP/s (% of B200 peak), d=64 N=16K; scaling at 1/2/4/8 GPU"
WORKLOADS = {
    # name: (B, H, N, D, dtype, causal)          the headline is the configuration the metric is quoted on; the
    # others are the remaining benchmark configurations of the reference path
    "headline": (1, 8, 16384, 64, "float16", False),
    "causal_bf16": (1, 8, 16384, 64, "bfloat16", True),          # causal prefix path, bf16
    "fp32_1k": (1, 8, 1024, 64, "float32", False),                # the reference's CPU-runnable case
    "fp32_64k": (1, 8, 65536, 64, "float32", False),              # long non-causal fp32 (one GPU, unsharded)
    "vit_4097": (8, 3, 4097, 64, "float16", False),               # ViT-Tiny attention at 1024x1024 input, NEEDS_MASK
    "swin_s1": (512, 3, 49, 32, "float16", False, "bias"),        # Swin-T stage-1 windows with relative-position bias
    "swin_s4": (8, 24, 49, 32, "float16", False, "bias"),
    "fp32_4k": (1, 8, 4096, 64, "float32", False),
    "small": (1, 8, 2048, 64, "float16", False),
    "prof4k": (1, 8, 4096, 64, "float16", False),      # ncu capture size: same kernels, a few hundred MB on the device
    "d128_8k": (1, 8, 8192, 128, "float16", False),    # head dim 128: the wide-head tensor-core kernels
    "bias_4k": (1, 8, 4096, 64, "float16", False, "bias"),   # a long biased problem: the same kernels with bias / dbias
}
MIN_REGION_S = 2.0        # the timed region of the headline number lasts at least this long


def flops(b, h, n, d, causal):
    pairs = n * (n + 1) // 2 if causal else n * n
    fwd = 4 * b * h * pairs * d
    return fwd, int(2.5 * fwd)


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel (the tcgen05 backward), from one
# ncu capture of this file's own command line at that workload
FP32_TC_MMAS = 3.0   # 16-bit products per fp32 product: x = h0 + h1 in fp16, a*b = h0 h0 + h0 h1 + h1 h0
FP32_TC_PEAK_NOTE = ("measured bf16 dense (sustained) / 3: an fp32 product on the tensor cores is three fp16 products "
                     "(two fp16 planes per operand); the backward also runs seven contractions per tile pair for the "
                     "five counted, so its ceiling in these units is 5/7 of this figure")
NCU_TRAFFIC_BYTES = {"headline": 101780992 + 19949824,
                     "swin_s1": 24829952}     # win_tc_bwd_kernel: dram read + write (the 14.5 MB written stay in L2)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "tflops": p["bf16_tflops"], "tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs."""
    Q = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", os.environ.get("ELSA_BENCH_SAMPLE_MS", "100"), "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")][1:]))

    def mark(self):
        """host time stamp; samples between two marks are the ones taken under load"""
        return time.time()

    def summary(self, t0=None, t1=None):
        rows = [r for (ts, r) in self.rows if (t0 is None or ts >= t0) and (t1 is None or ts <= t1)]
        if not rows:
            rows = [r for (_, r) in self.rows]
        sm = sorted(float(r[1]) for r in rows if len(r) > 8 and r[1].replace(".", "").isdigit())
        mx = [float(r[2]) for r in rows if len(r) > 8 and r[2].replace(".", "").isdigit()]
        pw = sorted(float(r[3]) for r in rows if len(r) > 8 and r[3].replace(".", "").isdigit())
        reasons = set()
        for r in rows:
            if len(r) > 8:
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w": pw[len(pw) // 2] if pw else None, "reasons": sorted(reasons), "samples": len(sm)}

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()


def cpu_sample(b, h, n, d, dtype, causal, rows, threads):
    """One bounded CPU step of the oracle: 1 head, `rows` query rows against all N keys, fwd + bwd."""
    from oracle import elsa_oracle as O
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(1234)
    q, k, v, do = (torch.randn(1, 1, n, d, generator=g).to(dtype) for _ in range(4))
    rows = min(rows, n)
    bh, scale = 1, 1.0 / (d ** 0.5)
    t0 = time.perf_counter()
    m, z, s = O.phase1_generic(q[0], k[0], v[0], is_causal=causal, block_n=2048, summary_dtype=dtype, q_start=0, q_len=rows)
    out, rm, rz = O.final_reduce(m, z, s)
    out = out.to(dtype)
    # backward for the same rows: dQ for those rows, and their contribution to dK, dV
    q3, k3, v3, do3 = q[0, :, :rows].float(), k[0].float(), v[0].float(), do[0, :, :rows].float()
    d_row, lse = O.bwd_preprocess(out, do3, rm, rz)
    sc = (q3 @ k3.transpose(-1, -2)) * (scale * O.LOG2E)
    if causal:
        idx = torch.arange(n)
        sc = torch.where(idx[:rows, None] >= idx[None, :], sc, torch.full((), float("-inf")))
    p = torch.exp2(sc - lse[..., None])
    dp = do3 @ v3.transpose(-1, -2)
    ds = (p * (dp - d_row[..., None])).to(dtype).float()
    dq = (ds @ k3) * scale
    dk = (ds.transpose(-1, -2) @ q3) * scale
    dv = p.to(dtype).float().transpose(-1, -2) @ do3
    dt = time.perf_counter() - t0
    pairs = (rows * (rows + 1) // 2 + 0) if (causal and rows == n) else rows * n
    if causal and rows < n:
        pairs = rows * (rows + 1) // 2
    return 14 * bh * pairs * d, dt, float(dq.abs().sum() + dk.abs().sum() + dv.abs().sum())


def run_reference(args, wl):
    b, h, n, d, dt_name, causal = wl[:6]
    dtype = getattr(torch, dt_name)
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rows = 1024
    for _ in range(max(args.warmup, 1)):
        cpu_sample(b, h, n, d, dtype, causal, rows, threads)
    tot_f, tot_t = 0, 0.0
    for _ in range(args.steps):
        f, t, _ = cpu_sample(b, h, n, d, dtype, causal, rows, threads)
        tot_f += f
        tot_t += t
    val = tot_f / tot_t / 1e12
    sample = f"per step: 1 of {b*h} heads, first {rows} of {n} query rows against all keys, fwd+bwd"
    line = {"metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": tot_t / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 arithmetic on " + dt_name + " inputs", "data": "synthetic", "impl": "reference",
            "config": {"workload": args.workload, "shape": [b, h, n, d], "causal": causal},
            "note": "CPU restatement of the reference's algorithm on the host cores (the reference has no CPU path); "
                    "the reference's own GPU code on this GPU is the `reference_gpu` object of the default line",
            "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------
# pieces of the default line
# ---------------------------------------------------------------------------------------------------------
def ev_pair():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def timed(fn, n):
    """mean milliseconds of n back-to-back calls of fn(i), CUDA events on the current stream"""
    e0, e1 = ev_pair()
    e0.record()
    for i in range(n):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n


class Workload:
    """Device-resident rotating input sets of one workload and its fwd+bwd step through the library."""

    def __init__(self, name, dev, rank=0, rot_bytes=260_000_000):
        import elsa_b200 as E
        from elsa_b200.attention_bwd import _backward_impl
        self.E, self._bwd = E, _backward_impl
        wl = WORKLOADS[name]
        self.name = name
        self.b, self.h, self.n, self.d, dt_name, self.causal = wl[:6]
        self.use_bias = len(wl) > 6
        self.dtype = getattr(torch, dt_name)
        self.dt_name = dt_name
        b, h, n, d = self.b, self.h, self.n, self.d
        self.set_bytes = 4 * b * h * n * d * torch.empty((), dtype=self.dtype).element_size()
        # enough input sets to exceed the 126 MB L2 (at most 32), so that a step never finds its operands there
        self.rot = int(min(32, max(3, -(-rot_bytes // self.set_bytes)))) if self.set_bytes < 400_000_000 else 2
        g = torch.Generator().manual_seed(1234 + rank)
        self.host = [[torch.randn(b, h, n, d, generator=g).to(self.dtype).pin_memory() for _ in range(4)] for _ in range(self.rot)]
        self.sets = [[t.to(dev) for t in s] for s in self.host]
        self.bias = (torch.randn(1, h, n, n, generator=g) * 0.02).to(dev) if self.use_bias else None
        self.fwd_f, self.bwd_f = flops(b, h, n, d, self.causal)

    def step(self, i, ev=None):
        q, k, v, do = self.sets[i % self.rot]
        if ev:
            ev[0].record()
        out, rm, rz, qc, kc, vc = self.E.attention._forward_impl(q, k, v, bias=self.bias, is_causal=self.causal,
                                                                 summary_dtype=self.dtype, part_width=0, q_chunk=0, want_state=True)
        if ev:
            ev[1].record()
        res = self._bwd(qc, kc, vc, out, do, bias=self.bias, is_causal=self.causal, row_m=rm, row_z=rz, want_dbias=self.use_bias)
        if ev:
            ev[2].record()
        return out, res

    def split(self, steps):
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
        for i in range(steps):
            self.step(i, evs[i])
        torch.cuda.synchronize()
        return (sum(e[0].elapsed_time(e[1]) for e in evs) / steps, sum(e[1].elapsed_time(e[2]) for e in evs) / steps)


def measure_fma_peak(lib, dev):
    """FP32-FMA rate of this GPU from the library's register-resident FMA chain, about half a second per form."""
    sink = torch.zeros(4, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    blocks = 148 * 8
    best = {}
    for packed in (0, 1):
        iters = 20000
        lib.elsa_debug_fma_rate(sink.data_ptr(), blocks, iters, packed, stream)
        torch.cuda.synchronize()
        ms = timed(lambda i: lib.elsa_debug_fma_rate(sink.data_ptr(), blocks, iters, packed, stream), 2)
        iters = int(iters * 250.0 / max(ms, 1e-3))           # about 0.25 s per launch
        ms = timed(lambda i: lib.elsa_debug_fma_rate(sink.data_ptr(), blocks, iters, packed, stream), 2)
        best["packed_f32x2" if packed else "scalar"] = blocks * 256 * iters * 32 / (ms * 1e-3) / 1e12
    return {"tflops": max(best.values()), "forms": best, "how": "register-resident FMA chains, 148*8 CTAs x 256 threads, ~0.25 s per launch, CUDA events"}


def window_bytes(b, h, n, d, esize):
    """Algorithmic HBM bytes of the one-launch kernels for sequences of at most 64 tokens: the forward reads q, k, v and
    writes out and the row state; the backward reads q, k, v, out, dout and the row state and writes dq, dk, dv."""
    rows = b * h * n
    return rows * (4 * d * esize + 8), rows * (8 * d * esize + 8)


def measure_phase2(lib, dev, hbm_gbs):
    """Achieved HBM GB/s of the streaming passes (phase-2 merge / scan, backward pre- and post-pass) through the C ABI,
    at the headline plan (fp16, 2 partitions, 131072 rows; buffers rotated so that nothing is L2-resident) and at the
    long fp32 case's 32 partitions (one query chunk of its plan: 15872 rows x 8 heads x 32 partitions, 1.07 GB of summaries)."""
    from elsa_b200 import _lib
    stream = torch.cuda.current_stream().cuda_stream
    out = {}

    def run(tag, fn, nbytes, reps):
        fn(0)
        torch.cuda.synchronize()
        ms = timed(fn, reps)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[tag] = {"ms": ms, "bytes": nbytes, "gbs": gbs, "frac": gbs / hbm_gbs}

    for tag, dtype, parts, bh, rows_q, nset in (("headline_plan_f16_P2", torch.float16, 2, 8, 16384, 6),
                                                 ("long_fp32_P32_chunk", torch.float32, 32, 8, 15872, 1)):
        d = 64
        es = torch.empty((), dtype=dtype).element_size()
        sdt = _lib.dtype_code(dtype)
        rows = bh * rows_q
        sets = []
        for _ in range(nset):
            m = torch.randn(parts, rows, device=dev)
            z = torch.rand(parts, rows, device=dev) + 0.5
            s = torch.randn(parts, rows, d, device=dev).to(dtype)
            sets.append((m, z, s, torch.empty_like(m), torch.empty_like(z), torch.empty_like(s),
                         torch.empty(rows, d, device=dev, dtype=dtype), torch.empty(rows, device=dev), torch.empty(rows, device=dev)))
        sum_bytes = parts * rows * (d * es + 8)
        out_bytes = rows * (d * es + 8)

        def merge(i):
            m, z, s, _, _, _, o, rm, rz = sets[i % nset]
            lib.elsa_merge_final(m.data_ptr(), z.data_ptr(), s.data_ptr(), o.data_ptr(), rm.data_ptr(), rz.data_ptr(), sdt, sdt,
                                 parts, bh, 0, rows_q, rows_q, d, 1, stream)

        def scan(i):
            m, z, s, mo, zo, so = sets[i % nset][:6]
            lib.elsa_prefix_scan(m.data_ptr(), z.data_ptr(), s.data_ptr(), mo.data_ptr(), zo.data_ptr(), so.data_ptr(), sdt,
                                 parts, bh, rows_q, d, stream)

        def step1(i):
            m, z, s, mo, zo, so = sets[i % nset][:6]
            lib.elsa_scan_step(m.data_ptr(), z.data_ptr(), s.data_ptr(), mo.data_ptr(), zo.data_ptr(), so.data_ptr(), sdt,
                               parts, bh, rows_q, d, 1, stream)

        def up(i):
            m, z, s, mo, zo, so = sets[i % nset][:6]
            lib.elsa_upsweep_level(m.data_ptr(), z.data_ptr(), s.data_ptr(), mo.data_ptr(), zo.data_ptr(), so.data_ptr(), sdt,
                                   parts, bh, rows_q, d, stream)

        reps = 12 if nset > 1 else 4
        run(f"{tag}.merge_final", merge, sum_bytes + out_bytes, reps)
        run(f"{tag}.prefix_scan", scan, 2 * sum_bytes, reps)
        run(f"{tag}.scan_step", step1, 3 * sum_bytes - (d * es + 8) * rows, reps)     # partition 0 has no left neighbour
        run(f"{tag}.upsweep_level", up, sum_bytes + (parts + 1) // 2 * rows * (d * es + 8), reps)
        del sets
    # backward pre-pass at the headline shape: D and LSE from out, dO and the row state
    bh, n, d = 8, 16384, 64
    sets = [(torch.randn(bh, n, d, device=dev).half(), torch.randn(bh, n, d, device=dev).half(), torch.randn(bh, n, device=dev),
             torch.rand(bh, n, device=dev) + 0.5, torch.empty(bh, n, device=dev), torch.empty(bh, n, device=dev)) for _ in range(6)]

    def pre(i):
        o, g, rm, rz, rd, rl = sets[i % 6]
        lib.elsa_bwd_preprocess(o.data_ptr(), g.data_ptr(), rm.data_ptr(), rz.data_ptr(), rd.data_ptr(), rl.data_ptr(), 1, bh, n, d, stream)

    run("headline_f16.bwd_preprocess", pre, 2 * bh * n * d * 2 + 4 * bh * n * 4, 12)
    return out


def measure_reference_gpu(wl: Workload, steps):
    """The unmodified reference on this GPU, same tensors, same events: ms per forward + backward step."""
    try:
        from baseline import reference as R
    except Exception as exc:  # noqa: BLE001
        return {"unavailable": f"baseline/reference.py does not import: {exc}"[:200]}
    ok, why = R.available()
    if not ok:
        return {"unavailable": why}
    try:
        ref = R.load()

        def rstep(i):
            q, k, v, do = wl.sets[i % wl.rot]
            qg, kg, vg = (t.detach().requires_grad_(True) for t in (q, k, v))
            ref.twopass_attention_train(qg, kg, vg, bias=wl.bias, is_causal=wl.causal).backward(do)

        def rfwd(i):
            q, k, v, _ = wl.sets[i % wl.rot]
            ref.twopass_attention(q, k, v, bias=wl.bias, is_causal=wl.causal)

        t0 = time.time()
        for i in range(2):          # includes the Triton JIT of every kernel variant
            rstep(i)
            rfwd(i)
        torch.cuda.synchronize()
        jit_s = time.time() - t0
        ms = timed(rstep, steps)
        fms = timed(rfwd, steps)
        tf = (wl.fwd_f + wl.bwd_f) / (ms * 1e-3) / 1e12
        return {"impl": "elsa_twopass_clean (Triton JIT for this GPU + its CUDA phase-2 reduce), twopass_attention_train fwd+bwd",
                "ms_per_step": ms, "value": tf, "unit": "TFLOP/s", "steps": steps, "forward_only_ms": fms,
                "forward_only_value": wl.fwd_f / (fms * 1e-3) / 1e12, "warmup_incl_jit_s": jit_s}
    except Exception as exc:  # noqa: BLE001 - the reference arm must not take the bench line down
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}


def measure_seq_sharded(dev, rank, world, dist, steps=2):
    """The long fp32 case (B=1 H=8 N=65536 d=64, non-causal, 2048-wide partitions) with K/V sharded along the sequence
    over the ranks: forward = local fold + cross-GPU merge, backward = local dK/dV + reduce_scatter of dQ.  With one
    rank the same problem runs unsharded through the ordinary operator."""
    from elsa_b200 import parallel as P
    import elsa_b200 as E
    from elsa_b200.attention_bwd import _backward_impl
    b, h, n, d = WORKLOADS["fp32_64k"][:4]
    g = torch.Generator().manual_seed(4321)
    q, k, v, do = (torch.randn(b, h, n, d, generator=g).to(dev) for _ in range(4))
    fwd_f, bwd_f = flops(b, h, n, d, False)
    per = n // world
    lo, hi = rank * per, (rank + 1) * per
    ks, vs = k[:, :, lo:hi].contiguous(), v[:, :, lo:hi].contiguous()
    marks = {}

    def step(i, split=False):
        if world == 1:
            out, rm, rz, qc, kc, vc = E.attention._forward_impl(q, k, v, bias=None, is_causal=False, summary_dtype=torch.float32,
                                                                part_width=2048, q_chunk=0, want_state=True)
            _backward_impl(qc, kc, vc, out, do, bias=None, is_causal=False, row_m=rm, row_z=rz, want_dbias=False)
            return
        e = [torch.cuda.Event(enable_timing=True) for _ in range(5)] if split else None
        if split:
            e[0].record()
        m, z, s = P.local_shard_summary(q, ks, vs, key_offset=lo, is_causal=False, part_width=2048)
        if split:
            e[1].record()
        out, rm, rz = P.merge_shards_on_gpu(m, z, s, q.dtype, gather=True)
        out = out.reshape(b, h, n, d)
        if split:
            e[2].record()
        dq_p, dk, dv = P.local_shard_backward(q, ks, vs, out, do, rm, rz, key_offset=lo, is_causal=False)
        if split:
            e[3].record()
        P.reduce_dq_across_ranks(dq_p, scatter=True)
        if split:
            e[4].record()
            torch.cuda.synchronize()
            for name, a, c in (("fold_ms", 0, 1), ("merge_exchange_ms", 1, 2), ("backward_ms", 2, 3), ("dq_exchange_ms", 3, 4)):
                marks[name] = e[a].elapsed_time(e[c])

    step(0)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    ms = timed(step, steps)
    step(0, split=True)
    if dist is not None:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    res = {"workload": "fp32 B=1 H=8 N=65536 d=64 non-causal fwd+bwd, K/V sharded along the sequence, 2048-wide partitions",
           "n_gpus": world, "ms_per_step": ms, "value": (fwd_f + bwd_f) / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
           "scaling": "strong", "steps": steps,
           "collectives": "none (one rank: unsharded operator)" if world == 1 else
           "all_reduce(MAX) m 2 MB; reduce_scatter(SUM) [s|z] 136 MB fp32 per rank; all_gather out + state; reduce_scatter(SUM) dQ 134 MB fp32 per rank"}
    if marks:
        res["split_rank0_ms"] = marks
    return res


def measure_models(dev, rank, world, dist, steps=5):
    """Whole-model training steps through the drop-in hooks, data-parallel over the ranks: ViT-Tiny at 1024 x 1024
    (4097 tokens per image) and Swin-T at 224 x 224, batch 8 per GPU, and ViT-Tiny at 224 x 224 (197 tokens per image),
    batch 64 per GPU; fp16 weights and activations, random pixels and
    labels; a step = forward + cross-entropy + backward + the bucketed all-reduce of the parameter gradients (overlapped
    with the backward).  With one rank the same, unpatched model (PyTorch SDPA / plain window attention) is timed too."""
    import copy
    import torch.nn.functional as F
    import elsa_b200 as E
    from elsa_b200 import vision
    res = {}
    for name, build, img, bsz in (("vit_tiny_1024", lambda: vision.vit_tiny(1024), 1024, 8),
                                  ("swin_tiny_224", lambda: vision.swin_tiny(224), 224, 8),
                                  ("vit_tiny_224", lambda: vision.vit_tiny(224), 224, 64)):
        try:
            torch.manual_seed(17)
            base = build().to(dev, torch.float16)
            ours = copy.deepcopy(base)
            rep = E.patch_timm_attention_train(ours)
            g = torch.Generator().manual_seed(99 + rank)
            x = torch.randn(bsz, 3, img, img, generator=g).to(dev, torch.float16)
            y = torch.randint(0, 1000, (bsz,), generator=g).to(dev)
            sync = vision.BucketedGradientAllReduce(ours)

            def train(model, exchange):
                def one(i):
                    model.zero_grad(set_to_none=True)
                    F.cross_entropy(model(x).float(), y).backward()
                    if exchange:
                        sync.finish()
                return one

            entry = {"batch_per_gpu": bsz, "n_gpus": world, "attention_modules_patched": rep.total,
                     "grad_exchange": "none (one rank)" if world == 1 else f"{len(sync.buckets)} buckets, async all_reduce(SUM) per bucket, overlapped with backward"}
            for tag, model, exch in (("elsa_b200", ours, True),) + ((("unpatched", base, False),) if world == 1 else ()):
                f = train(model, exch)
                for i in range(2):
                    f(i)
                torch.cuda.synchronize()
                if dist is not None:
                    dist.barrier()
                ms = timed(f, steps)
                if dist is not None:
                    t = torch.tensor([ms], device=dev)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    ms = float(t.item())
                entry[tag] = {"ms_per_step": ms, "images_per_s": world * bsz / (ms * 1e-3)}
                if world == 1:
                    # the same step replayed from a CUDA graph: what the GPU needs once the host's per-op overhead
                    # (which bounds both models at this batch size) is out of the picture
                    try:
                        model.zero_grad(set_to_none=True)
                        cg = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(cg):
                            F.cross_entropy(model(x).float(), y).backward()
                        for i in range(3):
                            cg.replay()
                        torch.cuda.synchronize()
                        entry[tag]["graph_replay_ms_per_step"] = timed(lambda i: cg.replay(), 10)
                        del cg
                    except Exception as exc:  # noqa: BLE001
                        entry[tag]["graph_replay_ms_per_step"] = None
                        entry[tag]["graph_note"] = f"{type(exc).__name__}: {exc}"[:160]
            if "unpatched" in entry:
                entry["lat_ratio_vs_unpatched"] = entry["elsa_b200"]["ms_per_step"] / entry["unpatched"]["ms_per_step"]
                ga, gb = entry["elsa_b200"].get("graph_replay_ms_per_step"), entry["unpatched"].get("graph_replay_ms_per_step")
                if ga and gb:
                    entry["graph_replay_ratio_vs_unpatched"] = ga / gb
            sync.remove()
            res[name] = entry
            del base, ours, x
        except Exception as exc:  # noqa: BLE001
            res[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="headline", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the side measurements (other configurations, phase-2 bandwidth, FMA peak, reference on the GPU, sequence-sharded case)")
    ap.add_argument("--min-region-s", type=float, default=MIN_REGION_S)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    wl_def = WORKLOADS[args.workload]
    if args.impl == "reference":
        return run_reference(args, wl_def)

    import elsa_b200 as E
    from elsa_b200 import _lib
    lib = _lib.load()   # raises if the CUDA library is missing: there is no fallback

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        import datetime
        # a rank that fails inside a side measurement must not leave the others waiting for ten minutes (the default)
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=240))

    # synthetic inputs: iid N(0,1), CPU generator seeded per rank
    wl = Workload(args.workload, dev, rank)
    b, h, n, d, dtype, causal, dt_name = wl.b, wl.h, wl.n, wl.d, wl.dtype, wl.causal, wl.dt_name
    ROT, set_bytes, fwd_f, bwd_f, step = wl.rot, wl.set_bytes, wl.fwd_f, wl.bwd_f, wl.step

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for i in range(args.warmup):
        step(i)
    barrier()
    # an untimed block of the same steps gives the step time from which the number of repetitions follows: the timed
    # region is the --steps block repeated `reps` times back to back so that it lasts >= min-region-s (a sustained
    # figure under the power cap, to be set against the sustained peak); all ranks use the same count
    est_ms = max_over_ranks(timed(step, args.steps))
    reps = max(1, min(2000, math.ceil(args.min_region_s * 1e3 / max(est_ms * args.steps, 1e-3))))
    n_timed = reps * args.steps
    l0 = lib.elsa_kernel_launches()
    barrier()
    mark0 = sampler.mark()
    t_start, t_end = ev_pair()
    t_start.record()
    for i in range(n_timed):
        step(i)
    t_end.record()
    barrier()
    mark1 = sampler.mark()
    launches = lib.elsa_kernel_launches() - l0
    total_ms = max_over_ranks(t_start.elapsed_time(t_end))
    clocks = sampler.summary(mark0 + 0.3, mark1) if rank == 0 else None
    ms_per_step = total_ms / n_timed
    value = world * (fwd_f + bwd_f) / (ms_per_step * 1e-3) / 1e12
    # the forward / backward split (and with it the dominant kernel's duration for the roofline) comes from a second
    # pass over the same steps with events between the two calls: timing events drain the GPU before they take
    # their time stamp, which costs the timed region above about 1.5 % when they sit inside it
    fwd_ms, bwd_ms = wl.split(args.steps)
    # scale the split to the sustained step time (the split pass itself is short)
    k_split = ms_per_step / max(fwd_ms + bwd_ms, 1e-9)

    # The burst figure: MEASURED_PEAKS.json's burst TFLOP/s is the best of 10 cuBLAS calls on a rested GPU, the timed
    # region above runs under a settled power cap.  The same protocol for one step of this path (best of 10 single
    # steps, 50 ms of idle before each, rotating input sets) pairs with that denominator; the sustained value above
    # pairs with the sustained one.
    burst_ms = None
    for i in range(10):
        torch.cuda.synchronize()
        time.sleep(0.05)
        b0, b1 = ev_pair()
        b0.record()
        step(i)
        b1.record()
        torch.cuda.synchronize()
        t = b0.elapsed_time(b1)
        burst_ms = t if burst_ms is None else min(burst_ms, t)
    burst_ms = max_over_ranks(burst_ms)

    # the same step replayed from a CUDA graph (the entry points allocate nothing and never synchronise): what is
    # left when launch gaps and host work are taken out; reported beside the eager number, never instead of it
    graph_line = None
    try:
        gs = torch.cuda.Stream()
        gs.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(gs):
            step(0)
        torch.cuda.current_stream().wait_stream(gs)
        graphs = []
        for r in range(ROT):                     # one graph per input set: the replays rotate like the eager steps
            cg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cg):
                step(r)
            graphs.append(cg)
        for cg in graphs:
            cg.replay()
        barrier()
        g_n = max(args.steps, min(n_timed, int(1000.0 / max(ms_per_step, 1e-3))))     # about one second of replays
        g_ms = max_over_ranks(timed(lambda i: graphs[i % ROT].replay(), g_n))
        graph_line = {"ms_per_step": g_ms, "value": world * (fwd_f + bwd_f) / (g_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                      "steps": g_n, "note": f"{ROT} graphs, one per input set, replayed in rotation"}
        del graphs
    except Exception as exc:  # noqa: BLE001 - a capture failure must not take the bench line down
        graph_line = {"error": str(exc)[:200]}

    # end to end through the public API with host buffers (pinned), copies inside the timed region
    e2e = None
    if not args.no_e2e:
        host, bias = wl.host, wl.bias
        # Double-buffered pipeline over three streams: H2D of step i+1 and D2H of step i-1 overlap the kernels of
        # step i (PCIe is full duplex); every step still moves its own inputs in and its own results out.
        outs_host = [[torch.empty(b, h, n, d, dtype=dtype).pin_memory() for _ in range(4)] for _ in range(2)]
        dev_in = [[torch.empty(b, h, n, d, dtype=dtype, device=dev) for _ in range(4)] for _ in range(2)]
        s_in, s_out, s_cmp = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_cmp = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]
        keep = [None, None]

        def e2e_step(i):
            slot = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_cmp[slot])          # the kernels that read this slot two steps ago are done
                for dst, src in zip(dev_in[slot], host[i % ROT]):
                    dst.copy_(src, non_blocking=True)
                ev_in[slot].record(s_in)
            s_cmp.wait_event(ev_in[slot])
            s_cmp.wait_event(ev_out[slot])             # results of two steps ago have left the device
            q, k, v = (t.detach().requires_grad_(True) for t in dev_in[slot][:3])
            out = E.twopass_attention_train(q, k, v, bias=bias, is_causal=causal)
            out.backward(dev_in[slot][3])
            ev_cmp[slot].record(s_cmp)
            keep[slot] = (out.detach(), q.grad, k.grad, v.grad)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[slot])
                for dst, src in zip(outs_host[slot], keep[slot]):
                    dst.copy_(src, non_blocking=True)
                ev_out[slot].record(s_out)

        for i in range(2):
            e2e_step(i)
        barrier()
        k_e2e = max(4, min(args.steps, 10))
        # the host link is shared with the other tenants of the machine: the faster of two repetitions is reported
        e_ms = None
        for _rep in range(2):
            t0, t1 = ev_pair()
            t0.record()
            for i in range(k_e2e):
                e2e_step(i)
            s_cmp.wait_stream(s_out)
            s_cmp.wait_stream(s_in)
            t1.record()
            barrier()
            e_ms = t0.elapsed_time(t1) if e_ms is None else min(e_ms, t0.elapsed_time(t1))
        e_ms = max_over_ranks(e_ms)
        nbytes = b * h * n * d * torch.empty((), dtype=dtype).element_size() * 4
        e2e = {"value": world * (fwd_f + bwd_f) / (e_ms / k_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes, "steps": k_e2e,
               "note": "three-stream pipeline (copy in, compute, copy out); bounded by the host link: every rank moves "
                       f"{2 * nbytes / 1e6:.0f} MB per step over its own PCIe link and the ranks share host DRAM"}
        del outs_host, dev_in, keep

    # ---- side measurements -------------------------------------------------------------------------------
    pk = peaks()
    extras = {}
    if not args.no_extras:
        seq = None
        try:
            del wl.host
            seq = measure_seq_sharded(dev, rank, world, dist)
        except Exception as exc:  # noqa: BLE001
            seq = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        extras["seq_sharded"] = seq
        try:
            extras["models"] = measure_models(dev, rank, world, dist)
        except Exception as exc:  # noqa: BLE001
            extras["models"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        if rank == 0 and world == 1:
            try:
                extras["fp32_fma_peak"] = measure_fma_peak(lib, dev)
            except Exception as exc:  # noqa: BLE001
                extras["fp32_fma_peak"] = {"error": str(exc)[:200]}
            try:
                extras["phase2"] = measure_phase2(lib, dev, pk["hbm_gbs"])
            except Exception as exc:  # noqa: BLE001
                extras["phase2"] = {"error": str(exc)[:200]}
            fma = extras["fp32_fma_peak"].get("tflops")
            others = {}
            for name in ("causal_bf16", "fp32_1k", "vit_4097", "swin_s1", "swin_s4", "d128_8k", "bias_4k"):
                try:
                    w2 = Workload(name, dev)
                    for i in range(3):
                        w2.step(i)
                    torch.cuda.synchronize()
                    k2 = max(5, min(200, int(300.0 / max(timed(w2.step, 3), 1e-3))))       # about 0.3 s
                    ms2 = timed(w2.step, k2)
                    tc = bool(lib.elsa_uses_tensor_cores_for(_lib.dtype_code(w2.dtype), w2.d, w2.n, int(w2.use_bias), int(w2.causal), 1, w2.b, w2.h))
                    tf = (w2.fwd_f + w2.bwd_f) / (ms2 * 1e-3) / 1e12
                    split3 = tc and w2.dtype == torch.float32
                    peak = (pk["tflops_sustained"] / (FP32_TC_MMAS if split3 else 1.0)) if tc else fma
                    others[name] = {"shape": [w2.b, w2.h, w2.n, w2.d], "dtype": w2.dt_name, "causal": w2.causal, "bias": w2.use_bias,
                                    "ms_per_step": ms2, "value": tf, "unit": "TFLOP/s", "steps": k2,
                                    "bound": "tensor" if tc else "fp32-fma",
                                    "peak": peak, "frac": (tf / peak) if peak else None,
                                    "peak_source": (FP32_TC_PEAK_NOTE if split3 else "measured bf16 dense, sustained") if tc else "FMA chain measured in this run"}
                    if tc and w2.n <= 64:
                        # the window kernels move a few KB per sequence and use a few percent of the tensor pipe
                        fb, bb = window_bytes(w2.b, w2.h, w2.n, w2.d, 2)
                        gbs = (fb + bb) / (ms2 * 1e-3) / 1e9
                        others[name].update({"bound": "hbm", "achieved_gbs": gbs, "peak": pk["hbm_gbs"], "frac": gbs / pk["hbm_gbs"],
                                             "peak_source": "measured copy bandwidth; algorithmic bytes of forward + backward over the step time"})
                    del w2
                except Exception as exc:  # noqa: BLE001
                    others[name] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
            if seq and "value" in seq:
                p64 = pk["tflops_sustained"] / FP32_TC_MMAS
                others["fp32_64k"] = {"shape": list(WORKLOADS["fp32_64k"][:4]), "dtype": "float32", "ms_per_step": seq["ms_per_step"],
                                      "value": seq["value"], "unit": "TFLOP/s", "bound": "tensor", "peak": p64, "frac": seq["value"] / p64,
                                      "peak_source": FP32_TC_PEAK_NOTE}
            extras["other_configs"] = others
            extras["reference_gpu"] = measure_reference_gpu(wl, max(3, min(args.steps, 10)))

    if rank == 0:
        sampler.stop()
        uses_tc = bool(lib.elsa_uses_tensor_cores_for(_lib.dtype_code(dtype), d, n, int(wl.use_bias), int(causal), 1, b, h))
        bwd_sus = bwd_ms * k_split
        fwd_sus = fwd_ms * k_split
        achieved = bwd_f / (bwd_sus * 1e-3) / 1e12
        split3 = uses_tc and dtype == torch.float32
        if split3:
            peak, peak_src, bound = (pk["tflops_sustained"] or pk["tflops"]) / FP32_TC_MMAS, FP32_TC_PEAK_NOTE, "tensor"
        elif uses_tc:
            peak, peak_src = pk["tflops_sustained"] or pk["tflops"], pk["source"] + " bf16 dense, sustained (seconds-long loop under the power cap: the timed region is one too)"
            bound = "tensor"
        else:
            fma = (extras.get("fp32_fma_peak") or {}).get("tflops")
            peak, peak_src, bound = fma, "FP32-FMA chain measured in this run", "fp32-fma"
        roofline = {"kernel": "backward (dQ, dK, dV recompute)" + ((" tcgen05, fp32 as three bf16 planes" if split3 else " tcgen05") if uses_tc else " fp32-fma"),
                    "bound": bound, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": (achieved / peak) if peak else None, "peak_source": peak_src,
                    "peak_burst": (pk["tflops"] / (FP32_TC_MMAS if split3 else 1.0)) if uses_tc else None,
                    "frac_of_burst": (achieved / (pk["tflops"] / (FP32_TC_MMAS if split3 else 1.0))) if uses_tc else None,
                    "traffic": NCU_TRAFFIC_BYTES.get(args.workload), "traffic_unit": "bytes per launch (ncu dram read+write)",
                    "ms_per_launch": bwd_sus,
                    "forward": {"achieved": fwd_f / (fwd_sus * 1e-3) / 1e12, "ms": fwd_sus,
                                "frac": (fwd_f / (fwd_sus * 1e-3) / 1e12 / peak) if peak else None},
                    "split_note": "forward / backward shares from a separate event-instrumented pass, scaled to the sustained step time"}
        if uses_tc and n <= 64:
            # window kernels: a few KB per sequence, a few percent of the tensor pipe: the bound is HBM (and latency)
            fb, bb = window_bytes(b, h, n, d, 2)
            roofline.update({"kernel": "win_tc_bwd_kernel (dQ, dK, dV, dbias of sequences of at most 64 tokens, one launch)",
                             "bound": "hbm", "achieved": bb / (bwd_sus * 1e-3) / 1e9, "peak": pk["hbm_gbs"], "unit": "GB/s",
                             "peak_source": pk["source"] + " copy bandwidth", "peak_burst": None, "frac_of_burst": None})
            roofline["frac"] = roofline["achieved"] / roofline["peak"]
            roofline["forward"] = {"achieved": fb / (fwd_sus * 1e-3) / 1e9, "ms": fwd_sus, "frac": fb / (fwd_sus * 1e-3) / 1e9 / pk["hbm_gbs"]}
        if "phase2" in extras:
            roofline["phase2"] = extras.pop("phase2")
        cpu = None
        if not args.no_cpu_baseline and world == 1:
            threads = os.cpu_count() or 1
            rows, tot_f, tot_t = 1024, 0, 0.0
            cpu_sample(b, h, n, d, dtype, causal, 256, threads)
            t_lim = time.perf_counter() + 20.0
            while time.perf_counter() < t_lim and tot_t < 12.0:
                f, t, _ = cpu_sample(b, h, n, d, dtype, causal, rows, threads)
                tot_f += f; tot_t += t
            cpu = {"value": tot_f / tot_t / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                   "sample": f"1 of {b*h} heads, first {rows} of {n} query rows against all keys, fwd+bwd, repeated for {tot_t:.1f} s"}
        line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f16" if dtype == torch.float16 else dt_name, "data": "synthetic",
                "timed_steps": n_timed, "timed_region_s": total_ms * 1e-3,
                "config": {"workload": args.workload, "shape_per_gpu": [b, h, n, d], "causal": causal, "global_batch": b * world,
                           "sharding": "batch x heads, no collective (replica scaling; the path with an exchange step is `seq_sharded`)",
                           "l2": f"{ROT} rotating input sets, {ROT * set_bytes / 1e6:.0f} MB in total against 126 MB of L2" + (": a step never finds its operands in L2" if ROT * set_bytes > 1.5 * 126e6 else ": smaller than L2, operands may be L2-resident"),
                           "timed_region": f"the --steps block repeated {reps}x back to back between one pair of events (>= {args.min_region_s} s)",
                           "tensor_cores": uses_tc},
                "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "graph_replay": graph_line,
                "burst": {"ms_per_step": burst_ms, "value": world * (fwd_f + bwd_f) / (burst_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                          "protocol": "best of 10 single steps, 50 ms idle before each (the protocol of the burst peak)",
                          "pct_of_burst_peak": 100.0 * (fwd_f + bwd_f) / (burst_ms * 1e-3) / 1e12 / pk["tflops"]},
                "gpu_launches": int(launches), "clocks": clocks,
                "pct_of_sustained_peak": 100.0 * value / world / pk["tflops_sustained"] if pk["tflops_sustained"] else None,
                "pct_of_burst_peak": 100.0 * value / world / pk["tflops"]}
        line.update(extras)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
