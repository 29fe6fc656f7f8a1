"""ctypes binding of libelsa_b200.so (the C ABI declared in include/elsa_b200.h).

The library is built ahead of time by `python -m elsa_b200.build` (or `__graft_entry__.build()`)
and lives next to this file.  There is no fallback: if it is missing, every operator raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_uint, c_uint64, c_void_p, POINTER

_HERE = os.path.dirname(os.path.abspath(__file__))
# ELSA_B200_LIB points the loader at another build of the same library (a tuning build, an installed copy)
LIB_PATH = os.environ.get("ELSA_B200_LIB") or os.path.join(_HERE, "libelsa_b200.so")

ELSA_F32, ELSA_F16, ELSA_BF16 = 0, 1, 2
FLAG_FORCE_SIMT, FLAG_SCAN_STEPS, FLAG_TREE_MERGE, FLAG_REF_ROUNDING, FLAG_FP32_FMA = 1, 2, 4, 8, 16

_P = c_void_p
_BIAS = [_P, c_int64, c_int64, c_int64, c_int64]

# name -> (restype, argtypes); must list every function include/elsa_b200.h declares
SIGNATURES = {
    "elsa_abi_version": (c_int, []),
    "elsa_strerror": (c_char_p, [c_int]),
    "elsa_last_cuda_error": (c_int, []),
    "elsa_kernel_launches": (c_int64, []),
    "elsa_device_status": (c_int, [c_int]),
    "elsa_debug_wait_timeout": (c_int, [c_uint64, _P]),
    "elsa_debug_fma_rate": (c_int, [_P, c_int, c_int64, c_int, _P]),
    "elsa_uses_tensor_cores": (c_int, [c_int] * 6),
    "elsa_uses_tensor_cores_for": (c_int, [c_int] * 8),
    "elsa_phase1_fold": (c_int, [_P, _P, _P, *_BIAS, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_int, c_int, c_int, c_uint, _P]),
    "elsa_phase1_fold_shard": (c_int, [_P, _P, _P, _P, _P, _P] + [c_int] * 11 + [c_uint, _P]),
    "elsa_phase1_fold_shard_workspace_bytes": (c_int64, [c_int] * 6 + [c_uint]),
    "elsa_phase1_fold_shard_ws": (c_int, [_P] * 7 + [c_int64] + [c_int] * 11 + [c_uint, _P]),
    "elsa_merge_partial": (c_int, [_P] * 6 + [c_int] * 5 + [_P]),
    "elsa_shard_chunk_elems": (c_int64, [c_int] * 4),
    "elsa_shard_pack": (c_int, [_P] * 5 + [c_int] * 4 + [_P]),
    "elsa_shard_finalize": (c_int, [_P] * 5 + [c_int] * 6 + [_P]),
    "elsa_merge_final": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P]),
    "elsa_scan_step": (c_int, [_P] * 6 + [c_int] * 6 + [_P]),
    "elsa_upsweep_level": (c_int, [_P] * 6 + [c_int] * 5 + [_P]),
    "elsa_prefix_scan": (c_int, [_P] * 6 + [c_int] * 5 + [_P]),
    "elsa_finalize": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P]),
    "elsa_forward_workspace_bytes": (c_int64, [c_int] * 10 + [c_uint]),
    "elsa_forward_plan": (c_int, [c_int] * 10 + [c_uint, POINTER(c_int), POINTER(c_int), POINTER(c_int)]),
    "elsa_twopass_forward": (c_int, [_P, _P, _P, *_BIAS, _P, _P, _P, _P, c_int64, c_int, c_int, c_int, c_int, c_int,
                                     c_int, c_int, c_int, c_int, c_uint, _P]),
    "elsa_twopass_forward_strided": (c_int, [_P, _P, _P, _P, _P, _P, *_BIAS, _P, _P, _P, _P, _P, c_int64, c_int, c_int, c_int,
                                             c_int, c_int, c_int, c_int, c_int, c_int, c_uint, _P]),
    "elsa_twopass_backward_strided": (c_int, [_P] * 6 + [_P, _P] + _BIAS + [_P, _P, _P] + _BIAS + [_P, c_int64] + [c_int] * 6 + [c_uint, _P]),
    "elsa_static_scratch_bytes": (c_int64, []),
    "elsa_twopass_forward_static": (c_int, [_P] * 6 + [c_int] * 6 + [_P]),
    "elsa_bwd_preprocess": (c_int, [_P] * 6 + [c_int] * 4 + [_P]),
    "elsa_row_stats_workspace_bytes": (c_int64, [c_int] * 7),
    "elsa_row_stats": (c_int, [_P, _P, *_BIAS, _P, _P, _P, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, _P]),
    "elsa_backward_workspace_bytes": (c_int64, [c_int] * 7 + [c_uint]),
    "elsa_twopass_backward": (c_int, [_P] * 7 + _BIAS + [_P, _P, _P] + _BIAS + [_P, c_int64] + [c_int] * 6 + [c_uint, _P]),
    "elsa_backward_shard_workspace_bytes": (c_int64, [c_int] * 5 + [c_uint]),
    "elsa_twopass_backward_shard": (c_int, [_P] * 11 + [c_int64] + [c_int] * 8 + [c_uint, _P]),
}

_lib = None


def load():
    """Return the loaded library; raises RuntimeError when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m elsa_b200.build` "
                "(elsa_b200 has no CPU or PyTorch fallback)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    if status == 0:
        return
    lib = load()
    msg = lib.elsa_strerror(status).decode()
    if status == 3:
        msg += f" [cudaError {lib.elsa_last_cuda_error()}]"
    if status in (1, 2):
        raise ValueError(f"{what}: {msg}")
    raise RuntimeError(f"{what}: {msg}")


def dtype_code(dtype) -> int:
    import torch
    if dtype == torch.float32:
        return ELSA_F32
    if dtype == torch.float16:
        return ELSA_F16
    if dtype == torch.bfloat16:
        return ELSA_BF16
    raise ValueError("supported dtypes are fp16, bf16, and fp32")


def raw_stream(device) -> int:
    """cudaStream_t of torch's current stream on `device` as an integer (the private raw getter when this torch has
    it: an order of magnitude cheaper than building a Stream object per call)."""
    import torch
    getter = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if getter is not None:
        idx = device.index
        return int(getter(torch.cuda.current_device() if idx is None else idx))
    return int(torch.cuda.current_stream(device).cuda_stream)
