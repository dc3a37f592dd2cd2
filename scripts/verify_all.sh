#!/usr/bin/env bash
# CPU checks, then (when a GPU is present) the GPU parity tests and the smoke run.
set -euo pipefail
cd "$(dirname "$0")/.."
PY="${PY:-python}"
"$PY" -m pytest tests -x -q -m "not gpu"
if "$PY" -c "import torch,sys; sys.exit(0 if torch.cuda.is_available() else 1)"; then
  "$PY" -m pytest tests -x -q -m gpu
  "$PY" -c "import __graft_entry__ as g; g.smoke()"
fi
