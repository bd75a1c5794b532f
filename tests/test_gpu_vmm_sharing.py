"""Sharing of virtual-memory allocations between processes on a real GPU: the
stand-alone check of `tests/vmm_sharing_it.py` (allocations made with
``cuMemCreate``, exported as file descriptors, mapped and filled by a second
process, read back by the owner), on one GPU and, where there are two, with the
importing process on the peer GPU."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(extra):
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "vmm_sharing_it.py"), *extra], capture_output=True, text=True,
                          timeout=300, cwd=ROOT)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    assert "[vmm] OK" in proc.stdout


def test_a_second_process_maps_and_fills_exported_allocations_on_the_same_gpu():
    _run(["--chunks", "3"])


def test_a_second_process_on_the_peer_gpu_maps_and_fills_them():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run(["--peer", "1", "--chunks", "2"])
