"""Offline analysis of debug-mode artefacts: metadata dumps, transfer-plan dumps
and weight comparisons between two sources of named tensors (the reference keeps
such scripts under `awex/tests/experimental/`).  Every module is importable and
runnable: ``python -m awex_b200.debug.<module> --help``."""
