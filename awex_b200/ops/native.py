"""Build and load the CUDA library.

All device code lives in ``awex_b200/ops/csrc`` and is compiled for sm_100a
only, into one shared library inside the package
(``awex_b200/ops/_native/libawex_b200.so``).  The library exports plain C
entry points; Python calls them through ``ctypes`` with raw device addresses
and the current CUDA stream, so no tensor type crosses the boundary.

On a machine with a GPU a missing or unloadable library is an error; nothing in
this package falls back to eager PyTorch for an op that has a kernel here.
"""

from __future__ import annotations

import ctypes
import os
import shutil
import subprocess
import threading
from typing import List, Optional

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "_native")
LIB_PATH = os.path.join(OUT_DIR, "libawex_b200.so")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]

_lib: Optional[ctypes.CDLL] = None
_lock = threading.Lock()


def sources() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = sources() + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every ``.cu`` file into the in-tree shared library."""
    if not force and not is_stale():
        return LIB_PATH
    os.makedirs(OUT_DIR, exist_ok=True)
    objects = []
    for src in sources():
        obj = os.path.join(OUT_DIR, os.path.basename(src)[:-3] + ".o")
        cmd = [_nvcc(), *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-I", CSRC, "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{proc.stdout}\n{proc.stderr}")
        if verbose:
            print(proc.stderr)
        objects.append(obj)
    tmp = LIB_PATH + ".tmp"
    proc = subprocess.run([_nvcc(), *ARCH_FLAGS, "-shared", "-o", tmp, *objects], capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


def _declare(lib: ctypes.CDLL) -> None:
    u32, u64, i32, vp = ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int, ctypes.c_void_p
    sig = {
        "awex_xfer_desc_size": ([], i32),
        "awex_xfer_smem_bytes": ([], i32),
        "awex_xfer_stage_bytes": ([], i32),
        "awex_launch_fused_transfer": ([vp, u32, u64, u64, u64, vp, vp, u32, vp, u32, vp, vp, i32, vp, vp, u32, u32, vp], i32),
        "awex_launch_wait_flags": ([vp, vp, u32, u64, u64, vp, vp], i32),
        "awex_launch_post_flags": ([vp, u32, u64, vp], i32),
        "awex_sum_desc_size": ([], i32),
        "awex_sum_chunk_words": ([], i32),
        "awex_launch_checksum": ([vp, u32, u64, vp, vp, i32, vp], i32),
        "awex_address_range": ([u64, ctypes.POINTER(u64), ctypes.POINTER(u64)], i32),
        "awex_ipc_handle_bytes": ([], i32),
        "awex_ipc_export": ([u64, ctypes.c_char_p], i32),
        "awex_ipc_open": ([ctypes.c_char_p, ctypes.POINTER(u64)], i32),
        "awex_ipc_close": ([u64], i32),
        "awex_enable_peer_access": ([i32, i32], i32),
        "awex_cuda_error_string": ([i32], ctypes.c_char_p),
    }
    for name, (argtypes, restype) in sig.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = argtypes, restype
    optional = {
        "awex_encode_tensor_map_2d": ([vp, i32, u64, u64, u64, u64, u32, u32], i32),
        "awex_launch_fp8_block_quant": ([vp, vp, vp, u64, u64, i64_t(), i64_t(), i64_t(), i32, i32, vp, vp], i32),
        "awex_launch_fp8_block_dequant": ([vp, vp, vp, u64, u64, i64_t(), i64_t(), i64_t(), i32, vp], i32),
        "awex_launch_fp8_scale_table": ([vp, vp, u32, i32, vp], i32),
        "awex_launch_fp8_quotient_check": ([i32, vp, vp], i32),
        "awex_col_normalize_scratch_floats": ([u64, u64], u64),
        "awex_launch_col_l2_normalize": ([vp, vp, vp, u64, u64, i64_t(), i64_t(), i32, ctypes.c_float, vp], i32),
        "awex_vmm_available": ([], i32),
        "awex_vmm_export_fd": ([u64, ctypes.POINTER(i32)], i32),
        "awex_vmm_reserve": ([u64, u64, ctypes.POINTER(u64)], i32),
        "awex_vmm_map_fd": ([u64, u64, u64, i32, i32], i32),
        "awex_vmm_unmap": ([u64, u64, u64], i32),
        "awex_vmm_release_range": ([u64, u64], i32),
        "awex_driver_error_string": ([i32], ctypes.c_char_p),
    }
    for name, (argtypes, restype) in optional.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = argtypes, restype


def i64_t():
    return ctypes.c_int64


def load() -> ctypes.CDLL:
    """The loaded library; builds it first when sources are newer (needs nvcc)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if is_stale():  # missing, or older than a source or header
                build()
            lib = ctypes.CDLL(LIB_PATH)
            _declare(lib)
            _lib = lib
    return _lib


def is_available() -> bool:
    import torch

    return torch.cuda.is_available()


def check(code: int, what: str) -> None:
    if code < 0 or code >= 1000:
        raise RuntimeError(f"{what} failed with code {code} (driver entry point missing, bad argument or tensor-map encode error)")
    if code != 0:
        msg = load().awex_cuda_error_string(code)
        raise RuntimeError(f"{what} failed: CUDA error {code} ({msg.decode() if msg else '?'})")


def current_stream_ptr() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream
