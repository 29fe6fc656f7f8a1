"""The allocation-free forward entry point (elsa_twopass_forward_static) against the regular one.

Some users of the library cannot give it a workspace: a foreign-language host with a bare FFI binding and no
device allocator of its own, or a server whose device memory is handed out once at start-up.  For them the
library keeps the partition summaries in a built-in 64 MiB device array.  This test calls that entry point
through the C ABI exactly as such a host would (raw pointers, no workspace), twice in a row with different
inputs because the array is shared between calls, and requires the same bits as the regular entry point,
which takes a caller-allocated workspace.  It also checks a problem that needs several query chunks and that an
oversized problem is refused.

The file name makes pytest collect it last, so a run that stops at the first failure has already run every
other test.
"""
import pytest
import torch

from elsa_b200 import _lib
from elsa_b200.attention import _forward_impl
from tests import _util as U

pytestmark = pytest.mark.gpu


def _static_forward(lib, q, k, v, causal, want_state=True):
    b, h, n, d = q.shape
    out = torch.full_like(q, float("nan"))
    rm = torch.full((b * h, n), float("nan"), device=q.device)
    rz = torch.full_like(rm, float("nan"))
    rc = lib.elsa_twopass_forward_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                         rm.data_ptr() if want_state else None, rz.data_ptr() if want_state else None,
                                         U.DT[q.dtype], b, h, n, d, int(causal), U.stream())
    return rc, out, rm, rz


@pytest.mark.parametrize("dtype,n,causal", [(torch.float16, 2048, False), (torch.float32, 700, True),
                                            (torch.bfloat16, 1030, True)])
def test_static_scratch_forward_matches_workspace_forward(dtype, n, causal):
    lib = _lib.load()
    assert lib.elsa_static_scratch_bytes() == 64 << 20
    for call in range(2):                      # two calls in a row share the built-in array
        q, k, v = (U.seeded((1, 4, n, 64), dtype, 300 + 10 * call + i).cuda() for i in range(3))
        # fp32: the allocation-free entry point stays on the FP32-FMA kernel (the planes of the tensor-core route
        # would not fit the built-in array), so the workspace forward is held to the same kernel
        ref = _forward_impl(q, k, v, bias=None, is_causal=causal, summary_dtype=dtype, part_width=0, q_chunk=0,
                            want_state=True, flags=_lib.FLAG_FP32_FMA if dtype == torch.float32 else 0)
        rc, out, rm, rz = _static_forward(lib, q, k, v, causal)
        assert rc == 0, lib.elsa_strerror(rc)
        torch.cuda.synchronize()
        # same kernels, same plan, same arithmetic: identical bits (tolerance 0)
        assert torch.equal(out, ref[0])
        assert torch.equal(rm, ref[1]) and torch.equal(rz, ref[2])
    assert lib.elsa_device_status(0) == 0


def test_static_scratch_chunks_the_queries_when_the_summaries_exceed_the_array():
    """fp16, 32 heads, 16384 tokens: the summaries of all query rows (68 MiB) exceed the 64 MiB array, so the entry
    point walks the query axis in chunks through the same array; same bits as the workspace forward."""
    lib = _lib.load()
    b, h, n, d = 1, 32, 16384, 64
    assert lib.elsa_forward_workspace_bytes(1, 1, b, h, n, d, 0, 0, 0, 0, 0) > lib.elsa_static_scratch_bytes()
    q, k, v = (U.seeded((b, h, n, d), torch.float16, 330 + i).cuda() for i in range(3))
    ref = _forward_impl(q, k, v, bias=None, is_causal=False, summary_dtype=torch.float16, part_width=0, q_chunk=0,
                        want_state=True)
    rc, out, rm, rz = _static_forward(lib, q, k, v, False)
    assert rc == 0, lib.elsa_strerror(rc)
    torch.cuda.synchronize()
    assert torch.equal(out, ref[0]) and torch.equal(rm, ref[1]) and torch.equal(rz, ref[2])


def test_static_scratch_rejects_oversized_problem():
    lib = _lib.load()
    # 4096 (batch*head) rows: the summaries of even one 256-row query tile exceed 64 MiB: refused before any launch
    b, h, n, d = 256, 16, 4096, 64
    before = lib.elsa_kernel_launches()
    x = torch.zeros(16, device="cuda", dtype=torch.float16)   # never dereferenced: the size check comes first
    rc = lib.elsa_twopass_forward_static(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), None, None, 1, b, h, n,
                                         d, 0, U.stream())
    assert rc == 4 and b"workspace" in lib.elsa_strerror(rc)
    assert lib.elsa_kernel_launches() == before
