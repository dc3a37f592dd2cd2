#!/usr/bin/env bash
# Build the sm_100a library in-tree (nvcc cross-compiles: no GPU needed) and the C oracle used by the tests.
set -euo pipefail
cd "$(dirname "$0")/.."
PY="${PY:-python}"
"$PY" -m gdn_qsa_sm80_b200.build "$@"
make -C oracle
