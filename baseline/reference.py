"""Access to the UNMODIFIED reference (ming053l/ELSA) installed by baseline/install_ref.sh under
baseline/_ref/ (git-ignored).  Used only by the GPU parity test against the reference and by the
`reference_gpu` leg of bench.py; the product never imports this.

The reference package is imported as it is.  Its single CUDA extension (phase-2 reduce,
src/elsa_twopass_clean/cuda/paper_scan_d64_kernel.cu) is normally JIT-built on first use by
src/elsa_twopass_clean/paper_scan_d64_cuda.py:11-34, which takes minutes of nvcc; install_ref.sh runs
that same loader once ahead of time, and `load()` here hands the resulting module to the loader's cache
slot so a GPU process does not compile again.  If the prebuilt module is absent or does not import,
the reference's own JIT path is left in place.
"""
from __future__ import annotations

import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")
REF_SRC = os.path.join(REF_ROOT, "src")
EXT_SO = os.path.join(REF_ROOT, "build", "paper_scan_d64_ext", "elsa_paper_scan_d64_ext.so")

_cached = None


def available() -> tuple[bool, str]:
    """(True, "") when the reference can be imported here, else (False, one-line reason)."""
    if not os.path.isdir(os.path.join(REF_SRC, "elsa_twopass_clean")):
        return False, "baseline/_ref is not installed (run baseline/install_ref.sh where the reference checkout exists)"
    try:
        import triton  # noqa: F401
    except Exception as exc:  # noqa: BLE001
        return False, f"triton does not import: {exc}"
    return True, ""


def load():
    """Import and return the reference package `elsa_twopass_clean` (raises RuntimeError with the reason if it cannot)."""
    global _cached
    if _cached is not None:
        return _cached
    ok, why = available()
    if not ok:
        raise RuntimeError(why)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")   # the loader's default (8.6) has no sm_100 image
    if REF_SRC not in sys.path:
        sys.path.insert(0, REF_SRC)
    import elsa_twopass_clean as ref
    from elsa_twopass_clean import paper_scan_d64_cuda as loader
    if os.path.exists(EXT_SO):
        try:
            import torch  # noqa: F401  (the extension links against libtorch)
            spec = importlib.util.spec_from_file_location("elsa_paper_scan_d64_ext", EXT_SO)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            loader._paper_scan_d64_extension = lambda: mod
        except Exception:  # noqa: BLE001 - fall back to the reference's own JIT build
            pass
    _cached = ref
    return ref
