#!/usr/bin/env bash
# Installs the UNMODIFIED reference (ming053l/ELSA) under baseline/_ref/ (git-ignored) so that the GPU
# tests and bench.py can run it next to elsa_b200 on the same B200:
#   baseline/_ref/src/elsa_twopass_clean/   the reference package, byte for byte
#   baseline/_ref/build/paper_scan_d64_ext/ its one CUDA extension, compiled ahead of time by the
#                                           reference's own loader (torch cpp_extension, sm_100)
# The reference's loader JIT-builds that extension on first use (about 3.5 minutes of nvcc because of the
# torch headers); building it here once keeps that out of every GPU run.  Usage:
#   baseline/install_ref.sh <path-to-reference-checkout>     (or ELSA_REFERENCE_SRC in the environment)
set -euo pipefail
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
src="${1:-${ELSA_REFERENCE_SRC:-}}"
if [ -z "$src" ] || [ ! -d "$src/src/elsa_twopass_clean" ]; then
  echo "usage: baseline/install_ref.sh <path-to-reference-checkout>" >&2
  exit 2
fi
dst="$here/_ref"
mkdir -p "$dst/src"
rm -rf "$dst/src/elsa_twopass_clean"
cp -r "$src/src/elsa_twopass_clean" "$dst/src/elsa_twopass_clean"
find "$dst/src" -name __pycache__ -type d -prune -exec rm -rf {} +
cd "$dst"
TORCH_CUDA_ARCH_LIST=10.0 MAX_JOBS=2 PYTHONPATH="$dst/src" python - <<'PY'
import time
t = time.time()
from elsa_twopass_clean.paper_scan_d64_cuda import _paper_scan_d64_extension
mod = _paper_scan_d64_extension()
print("built", mod.__file__, f"{time.time() - t:.0f}s")
PY
