#!/usr/bin/env bash
# Format and lint the Python sources (ruff reads its settings from pyproject.toml).
set -euo pipefail
cd "$(dirname "$0")/.."
if ! command -v ruff >/dev/null 2>&1; then
  echo "ruff is not installed; install it (pip install ruff) and run again" >&2
  exit 1
fi
ruff format awex_b200 tests baseline bench.py
ruff check --fix awex_b200 tests baseline bench.py
