"""The CPU oracle against outputs of the reference's own kernels (tests/golden/*.npz).

Tolerances: the fixtures were produced by the reference kernels with the same rounding points
the oracle restates, so differences are fp32 summation order only: 2e-6 relative on fp32 values;
for fp16 routes one fp16 ulp of the value (a p or s that sits on a rounding boundary can flip).
"""
import math

import pytest
import torch

from oracle import elsa_oracle as O


def _close(a, b, dtype, what, scale=1.0):
    a = a.float(); b = b.float()
    fin = torch.isfinite(b)
    assert torch.equal(torch.isfinite(a), fin), what
    if dtype == torch.float32:
        tol = 3e-6 * scale
    else:
        tol = 1.2e-3 * scale
    err = ((a[fin] - b[fin]).abs() / (1.0 + b[fin].abs())).max().item() if fin.any() else 0.0
    assert err <= tol, f"{what}: rel err {err} > {tol}"


FWD_GENERIC = ["fwd_generic_f32_n96_d64", "fwd_generic_f16_n100_d32", "fwd_causal_f32_n129_d32",
               "fwd_causal_f16_n129_d32", "fwd_swin_f32_n49_d32", "fwd_swin_f16_n49_d32",
               "fwd_swinshift_f16_n49_d32", "fwd_generic_f32_n70_d128"]


@pytest.mark.parametrize("name", FWD_GENERIC)
def test_forward_generic_route(golden, name):
    g = golden(name)
    q, k, v = g["q"], g["k"], g["v"]
    b, h, n, d = q.shape
    bias = g.get("bias")
    causal = bool(g["causal"])
    out, rm, rz, parts = O.twopass_forward(q, k, v, bias=bias, is_causal=causal, block_m=g["block_m"],
                                           block_n=g["block_n"], q_chunk_size=4096, return_parts=True)
    m, z, s = parts[0]
    _close(m, g["p1_m"], q.dtype, "phase1 m")
    _close(z, g["p1_z"], q.dtype, "phase1 z")
    _close(s, g["p1_s"], q.dtype, "phase1 s")
    _close(out, g["out"], q.dtype, "out")
    _close(rm, g["row_m"], q.dtype, "row_m")
    _close(rz, g["row_z"], q.dtype, "row_z")
    if causal:
        pm, pz, ps = O.hillis_steele_scan(g["p1_m"], g["p1_z"], g["p1_s"].float(), q.dtype)
        _close(pm, g["scan_m"], q.dtype, "scan m")
        _close(pz, g["scan_z"], q.dtype, "scan z")
        _close(ps, g["scan_s"], q.dtype, "scan s")
    ref = O.softmax_attention_fp64(q, k, v, bias=bias, is_causal=causal)
    lim = 2e-6 if q.dtype == torch.float32 else 2e-3
    assert (out.double() - ref).abs().max().item() < lim


@pytest.mark.parametrize("name", ["fwd_d64tiled_f32_n200", "fwd_d64tiled_f16_n200", "fwd_d64tiled_f32_n700",
                                  "fwd_d64_f32_n130", "fwd_d64_f16_n130"])
def test_forward_d64_phase1(golden, name):
    g = golden(name)
    q, k, v = g["q"], g["k"], g["v"]
    b, h, n, d = q.shape
    r = lambda t: t.reshape(b * h, n, d)
    m, z, s = O.phase1_d64(r(q), r(k), r(v), block_n=g["block_n"])
    _close(m, g["p1_m"], q.dtype, "phase1 m")
    _close(z, g["p1_z"], q.dtype, "phase1 z")
    _close(s, g["p1_s"], q.dtype, "phase1 s")
    out, rm, rz = O.final_reduce(m, z, s)
    ref = O.softmax_attention_fp64(q, k, v).reshape(b * h, n, d)
    lim = 2e-6 if q.dtype == torch.float32 else 2e-3
    assert (out.double() - ref).abs().max().item() < lim


@pytest.mark.parametrize("name", ["bwd_f32_n70_d64", "bwd_f32_causal_n70_d64", "bwd_f16_n70_d64",
                                  "bwd_f16_causal_n70_d64", "bwd_swin_f32_n49_d32", "bwd_swin_f16_n49_d32"])
def test_backward(golden, name):
    g = golden(name)
    q, k, v, out, dout = g["q"], g["k"], g["v"], g["out"], g["dout"]
    b, h, n, d = q.shape
    bias = g.get("bias")
    causal = bool(g["causal"])
    r = lambda t: t.reshape(b * h, n, d)
    bias3 = O.canonical_bias(bias, b, h, n)
    m, z = O.row_stats(r(q), r(k), bias=bias3, is_causal=causal)
    _close(m, g["row_m"], torch.float32, "row_m", 2.0)
    _close(z, g["row_z"], torch.float32, "row_z", 2.0)
    d_row, lse = O.bwd_preprocess(r(out), r(dout), g["row_m"], g["row_z"])
    _close(d_row, g["row_d"], torch.float32, "D")
    _close(lse, g["row_lse"], torch.float32, "LSE")
    res = O.twopass_backward(q, k, v, out, dout, g["row_m"], g["row_z"], bias=bias, is_causal=causal,
                             want_dbias="dbias" in g)
    for nm, val in zip(("dq", "dk", "dv"), res[:3]):
        _close(val, g[nm], q.dtype, nm)
    if "dbias" in g:
        db = O.reduce_dbias(res[3], g["bias"], b, h)
        _close(db, g["dbias"], torch.float32, "dbias", 2.0 if q.dtype == torch.float32 else 400.0)


def test_monoid_algebra():
    gen = torch.Generator().manual_seed(7)
    def rnd():
        m = torch.randn(5, 9, generator=gen) * 4
        z = torch.rand(5, 9, generator=gen) + 0.1
        s = torch.randn(5, 9, 8, generator=gen)
        dead = torch.rand(5, 9, generator=gen) < 0.2
        m = torch.where(dead, torch.full((), float("-inf")), m)
        z = torch.where(dead, torch.zeros(()), z)
        s = torch.where(dead[..., None], torch.zeros(()), s)
        return m, z, s
    a, b, c = rnd(), rnd(), rnd()
    ident = O.monoid_identity((5, 9), 8)
    for x, y in zip(O.monoid_merge(a, ident), a):
        assert torch.allclose(x, y, equal_nan=False)
    for x, y in zip(O.monoid_merge(ident, a), a):
        assert torch.allclose(x, y)
    l = O.monoid_merge(O.monoid_merge(a, b), c)
    r = O.monoid_merge(a, O.monoid_merge(b, c))
    # compare as normalised outputs (the representation (m,z,s) is unique up to rounding)
    for x, y in zip(l, r):
        fin = torch.isfinite(x)
        assert torch.equal(fin, torch.isfinite(y))
        assert torch.allclose(x[fin], y[fin], rtol=1e-5, atol=1e-6)
    ab, ba = O.monoid_merge(a, b), O.monoid_merge(b, a)
    for x, y in zip(ab, ba):
        fin = torch.isfinite(x)
        assert torch.allclose(x[fin], y[fin], rtol=1e-6, atol=1e-7)


def test_routing_table():
    f32, f16, bf16 = torch.float32, torch.float16, torch.bfloat16
    assert O.paper_scan_defaults(f32, 1024, 64) == (32, 1024, 1024)
    assert O.paper_scan_defaults(f16, 16384, 64) == (64, 2048, 4096)
    assert O.paper_scan_defaults(f16, 16384, 64, training=True) == (64, 256, 1024)
    assert O.paper_scan_defaults(f32, 65536, 64) == (32, 2048, 512)
    assert O.paper_scan_defaults(bf16, 16384, 64) == (64, 256, 1024)
    assert O.paper_scan_defaults(f16, 4097, 64, training=True) == (64, 256, 1024)
    assert O.paper_scan_defaults(f16, 49, 32, 64, 64, 49) == (64, 64, 64)
