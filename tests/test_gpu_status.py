"""The bounded device-side waits report through a status word; this test makes one wait run out in the allowed
form (a barrier that nothing arrives at, 1 ms limit: the kernel records the status and returns, nothing faults)
and checks the whole reporting path: the word, the error code of the next tensor-core call, the Python exception,
and that the context and the library keep working once the word is cleared."""
import pytest
import torch

import elsa_b200 as E
from elsa_b200 import _lib
from tests import _util as U

pytestmark = pytest.mark.gpu


def test_timed_out_wait_is_reported_and_cleared():
    lib = _lib.load()
    q, k, v = (U.seeded((1, 2, 640, 64), torch.float16, 400 + i).cuda() for i in range(3))
    ref = E.twopass_attention(q, k, v)            # also sets the status word up outside of everything else
    torch.cuda.synchronize()
    assert lib.elsa_device_status(1) == 0
    try:
        assert lib.elsa_debug_wait_timeout(1_000_000, U.stream()) == 0        # 1 ms
        torch.cuda.synchronize()
        assert lib.elsa_device_status(0) == (1 << 8) | 99
        # a tensor-core call now refuses to launch and the Python mirror raises
        before = lib.elsa_kernel_launches()
        with pytest.raises(RuntimeError, match="wait gave up"):
            E.twopass_attention(q, k, v)
        assert lib.elsa_kernel_launches() == before
        qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
        with pytest.raises(RuntimeError, match="wait gave up"):
            E.twopass_attention_train(qg, kg, vg)
        # fp32 of this length also runs phase 1 on the tensor cores: refused as well
        with pytest.raises(RuntimeError, match="wait gave up"):
            E.twopass_attention(q.float(), k.float(), v.float())
        # the FP32-FMA kernels (here: a sequence below the tensor-core threshold) have no device-side waits and keep running
        out32 = E.twopass_attention(q[:, :, :200].float(), k[:, :, :200].float(), v[:, :, :200].float())
        assert torch.isfinite(out32).all()
    finally:
        assert lib.elsa_device_status(1) in (0, (1 << 8) | 99)       # read and clear
    assert lib.elsa_device_status(0) == 0
    again = E.twopass_attention(q, k, v)
    torch.cuda.synchronize()
    assert torch.equal(again, ref)
    assert lib.elsa_debug_wait_timeout(0, U.stream()) == 1 and lib.elsa_debug_wait_timeout(2_000_000_000, U.stream()) == 1
