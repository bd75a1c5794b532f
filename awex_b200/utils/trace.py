"""Phase markers: one context manager gives a phase an NVTX range (visible in
Nsight Systems timelines, free when no profiler is attached), a wall-clock
duration in the log, and, with ``AWEX_MEM_DEBUG=1``, device-memory snapshots
before and after (`awex/util/gpu.py:57-78`, `awex/writer/nccl_writer.py:223-255`
in the reference log the same snapshots by hand around each phase)."""

from __future__ import annotations

import os
import time
from contextlib import contextmanager

import torch

from awex_b200 import logging

logger = logging.getLogger(__name__)


_nvtx_broken = False


def _push(name: str) -> bool:
    """Open an NVTX range; False (and never again tried) when this torch build
    cannot."""
    global _nvtx_broken
    if _nvtx_broken or not torch.cuda.is_available():
        return False
    try:
        torch.cuda.nvtx.range_push(name)
        return True
    except Exception:
        _nvtx_broken = True
        return False


def _pop() -> None:
    global _nvtx_broken
    try:
        torch.cuda.nvtx.range_pop()
    except Exception:
        _nvtx_broken = True


@contextmanager
def phase(name: str, log: bool = False):
    mem_debug = os.environ.get("AWEX_MEM_DEBUG", "0") == "1"
    if mem_debug:
        from awex_b200.utils.gpu import memory_snapshot

        logger.info(f"[mem] before {name}: {memory_snapshot(name)}")
    pushed = _push(f"awex:{name}")
    started = time.time()
    try:
        yield
    finally:
        if pushed:
            _pop()
        if log:
            logger.info(f"{name} took {time.time() - started:.4f}s")
        if mem_debug:
            from awex_b200.utils.gpu import memory_snapshot

            logger.info(f"[mem] after {name}: {memory_snapshot(name)}")
