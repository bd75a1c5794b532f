"""Device helpers.

The data plane of this framework is CUDA on B200 only; "cpu" exists so the
control plane, planner and converters can be exercised without a GPU
(``AWEX_DEVICE_TYPE=cpu`` forces it).  The reference additionally dispatches
to Ascend NPUs (`awex/util/device.py:53-206`); that path is intentionally
not reproduced.
"""

from __future__ import annotations

import os
from contextlib import contextmanager

import torch


def get_device_type() -> str:
    forced = os.environ.get("AWEX_DEVICE_TYPE", "").strip().lower()
    if forced:
        if forced not in ("cuda", "cpu"):
            raise ValueError(f"AWEX_DEVICE_TYPE={forced!r} is not supported; use 'cuda' or 'cpu'")
        return forced
    return "cuda" if torch.cuda.is_available() else "cpu"


def is_cuda_available() -> bool:
    return torch.cuda.is_available()


def device_count() -> int:
    return torch.cuda.device_count() if get_device_type() == "cuda" else 0


def current_device() -> int:
    return torch.cuda.current_device() if get_device_type() == "cuda" else 0


def set_device(device_id: int) -> None:
    if get_device_type() == "cuda":
        torch.cuda.set_device(device_id)


def synchronize(device_id: int | None = None) -> None:
    if get_device_type() == "cuda":
        torch.cuda.synchronize(device=device_id)


def get_device_name(device_id: int | None = None) -> str:
    if get_device_type() == "cuda":
        return torch.cuda.get_device_name(current_device() if device_id is None else device_id)
    return "cpu"


def get_torch_device(device_id: int | None = None) -> torch.device:
    if get_device_type() == "cuda":
        return torch.device("cuda", current_device() if device_id is None else device_id)
    return torch.device("cpu")


def get_device_properties(device_id: int | None = None):
    if get_device_type() != "cuda":
        raise RuntimeError("Device properties are only available for CUDA devices.")
    return torch.cuda.get_device_properties(current_device() if device_id is None else device_id)


def empty_cache() -> None:
    if get_device_type() == "cuda":
        torch.cuda.empty_cache()


def memory_stats() -> dict:
    if get_device_type() != "cuda":
        return {"allocated": 0, "reserved": 0, "free": 0, "total": 0}
    free, total = torch.cuda.mem_get_info()
    return {
        "allocated": torch.cuda.memory_allocated(),
        "reserved": torch.cuda.memory_reserved(),
        "free": free,
        "total": total,
    }


def current_stream():
    return torch.cuda.current_stream() if get_device_type() == "cuda" else None


def get_stream_class():
    """``torch.cuda.Stream`` on CUDA, ``None`` on the CPU (`awex/util/device.py:169-176`)."""
    return torch.cuda.Stream if get_device_type() == "cuda" else None


def create_stream(device_id: int | None = None):
    cls = get_stream_class()
    if cls is None:
        return None
    return cls() if device_id is None else cls(device=device_id)


def is_npu_available() -> bool:
    """Always false: Ascend devices are not supported."""
    return False


@contextmanager
def stream_context(stream):
    if stream is None or get_device_type() != "cuda":
        yield
    else:
        with torch.cuda.stream(stream):
            yield


def visible_devices_env_names() -> list:
    return ["CUDA_VISIBLE_DEVICES"]


def visible_devices_env_value() -> str:
    return os.environ.get("CUDA_VISIBLE_DEVICES", "")


def get_dist_backend() -> str:
    return "nccl" if get_device_type() == "cuda" else "gloo"
