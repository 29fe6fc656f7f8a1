"""CPU-only checks of the drop-in boundary: the library builds, loads without a GPU, exports every
function the header declares, and the Python mirror keeps the reference's argument checking."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from elsa_b200 import _lib, build
    build.build()
    return _lib.load()


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "elsa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(elsa_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = _declared_functions()
    assert len(names) >= 18
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/elsa_b200.h but not exported"


def test_binding_covers_header(lib):
    from elsa_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared_functions()


def test_version_and_strerror(lib):
    assert lib.elsa_abi_version() == 2
    assert lib.elsa_strerror(0) == b"ok"
    assert b"workspace" in lib.elsa_strerror(4)
    assert b"unknown" in lib.elsa_strerror(99)


def test_argument_validation_without_gpu(lib):
    # null pointers / bad sizes are rejected before any CUDA call is made
    rc = lib.elsa_merge_final(None, None, None, None, None, None, 0, 0, 1, 1, 0, 1, 1, 64, 0, None)
    assert rc == 1
    rc = lib.elsa_phase1_fold(None, None, None, None, 0, 0, 0, 0, None, None, None, 0, 0, 1, 1, 8, 64, 0, 8, 64, 1, 0, 0, None)
    assert rc == 1
    assert lib.elsa_forward_workspace_bytes(0, 0, 1, 1, 8, 256, 0, 0, 0, 0, 0) == -1   # head_dim > 128
    assert lib.elsa_forward_workspace_bytes(7, 0, 1, 1, 8, 64, 0, 0, 0, 0, 0) == -1    # bad dtype
    assert lib.elsa_forward_workspace_bytes(0, 0, 1, 1, 0, 64, 0, 0, 0, 0, 0) == 0     # empty sequence


def test_forward_plan(lib):
    pw, parts, qc = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    rc = lib.elsa_forward_plan(0, 0, 1, 8, 65536, 64, 0, 0, 2048, 0, 0, ctypes.byref(pw), ctypes.byref(parts), ctypes.byref(qc))
    assert rc == 0 and pw.value == 2048 and parts.value == 32
    need = lib.elsa_forward_workspace_bytes(0, 0, 1, 8, 65536, 64, 0, 0, 2048, 0, 0)
    rows = parts.value * 8 * qc.value
    assert need >= rows * (64 * 4 + 8) and need <= rows * (64 * 4 + 8) + 4096
    # the library's own choice: no more partitions than needed to fill the machine
    rc = lib.elsa_forward_plan(1, 1, 1, 8, 16384, 64, 0, 0, 0, 0, 0, ctypes.byref(pw), ctypes.byref(parts), ctypes.byref(qc))
    assert rc == 0 and parts.value * pw.value >= 16384 and parts.value <= 8


def test_python_api_errors():
    import elsa_b200 as E
    q = torch.randn(1, 2, 8, 4)
    with pytest.raises(ValueError, match="CUDA"):
        E.twopass_attention(q, q, q)
    with pytest.raises(ValueError, match="shape"):
        E.twopass_attention(q[0], q[0], q[0])
    with pytest.raises(ValueError, match="identical"):
        E.twopass_attention(q, q[:, :1], q)
    with pytest.raises(ValueError, match="CUDA"):
        E.twopass_attention_backward(q, q, q, q, q)
    assert set(E.__all__) >= {"twopass_attention", "twopass_attention_with_state", "twopass_attention_backward",
                              "twopass_attention_train", "patch_timm_attention", "patch_timm_attention_train",
                              "PatchReport", "TrainPatchReport"}


def test_product_never_imports_oracle():
    pkg = os.path.join(ROOT, "elsa_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, f"{f} mentions the oracle"


def test_patch_report_and_detectors():
    import torch.nn as nn
    from elsa_b200.timm_dropin import PatchReport, _is_swin_v1_window_attention, _is_vit_attention, patch_timm_attention
    assert PatchReport(2, 3).total == 5
    with pytest.raises(ValueError, match="no compatible"):
        patch_timm_attention(nn.Sequential(nn.Linear(4, 4)))
    from tests.standins import SwinWindowAttention, VitAttention
    assert _is_vit_attention(VitAttention(32, 2)) and not _is_swin_v1_window_attention(VitAttention(32, 2))
    sw = SwinWindowAttention(32, 2, (7, 7))
    assert _is_swin_v1_window_attention(sw) and not _is_vit_attention(sw)
    sw.logit_scale = nn.Parameter(torch.zeros(1))
    assert not _is_swin_v1_window_attention(sw)
    model = nn.Sequential(VitAttention(32, 2), nn.Sequential(SwinWindowAttention(32, 2, (7, 7))))
    names_before = sorted(n for n, _ in model.named_parameters())
    rep = patch_timm_attention(model)
    assert (rep.vit_attention, rep.swin_window_attention, rep.total) == (1, 1, 2)
    assert sorted(n for n, _ in model.named_parameters()) == names_before


def test_packed_plan_strides_match_the_views():
    """The packed-qkv path hands the C ABI strides computed from the shape alone: they must be the strides of the q / k / v
    views of a contiguous [B, N, 3, H, D] tensor and of the [B, H, N, D] view of the [B, N, H, D] output."""
    from elsa_b200.attention import _bhnd_strides
    from elsa_b200.attention_bwd import _PackedPlan
    b, n, h, d = 3, 49, 4, 32
    qkv = torch.zeros(b, n, 3, h, d, dtype=torch.float16)
    plan = _PackedPlan(qkv, False, False, torch.float16, 0, 0)
    q, k, v = qkv.permute(2, 0, 3, 1, 4).unbind(0)
    for t in (q, k, v):
        assert tuple(plan.qkv_strides) == _bhnd_strides(t)
    out = torch.zeros(b, n, h, d, dtype=torch.float16).permute(0, 2, 1, 3)
    assert tuple(plan.out_strides) == _bhnd_strides(out)
    assert plan.hd * plan.esize == (k.data_ptr() - q.data_ptr()) == (v.data_ptr() - k.data_ptr())
    gs = _bhnd_strides(out)
    arr = tuple(plan.backward_strides(gs))
    assert arr[:9] == tuple(plan.qkv_strides) * 3 and arr[9:12] == tuple(plan.out_strides) and arr[12:15] == gs
    assert arr[15:] == tuple(plan.qkv_strides) * 3 and plan.fwd_ws >= 0 and plan.bwd_ws >= 0
