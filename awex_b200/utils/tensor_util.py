"""Tensor helpers: NaN scans, detailed diffs, dtype-packed buffers and IPC
serialisation.

Packing by dtype and pickled CUDA-IPC tensors are how the reference hands
training weights to a co-resident inference process every step
(`awex/util/tensor_util.py:159-390`).  The fused transfer path here needs
neither (it publishes addresses of the existing allocations once); the
functions are kept for the CPU IPC backend, for tools and for API parity.
"""

from __future__ import annotations

import io
import pickle
from typing import Dict, Iterable, List, Sequence, Tuple, Union

import torch

from awex_b200 import logging

logger = logging.getLogger(__name__)


# ---- diagnostics ---------------------------------------------------------------------------------
def check_and_log_nan_values(tensor, tensor_name, stage_info: str = "", max_indices: int = 20) -> bool:
    """True when ``tensor`` contains NaN; logs how many and where.  A dict of
    tensors is scanned entry by entry."""
    if isinstance(tensor, dict):
        return any([check_and_log_nan_values(t, f"{tensor_name}:{k}", stage_info, max_indices) for k, t in tensor.items()])
    if not torch.is_tensor(tensor) or not tensor.is_floating_point():
        return False
    probe = tensor.float() if tensor.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else tensor
    mask = torch.isnan(probe)
    count = int(mask.sum())
    if count == 0:
        return False
    where = mask.nonzero()[:max_indices].tolist()
    logger.error(
        f"NaN values in {tensor_name} {stage_info}: {count} of {tensor.numel()} elements "
        f"({100.0 * count / max(tensor.numel(), 1):.4f}%), shape {tuple(tensor.shape)}, first indices {where}"
    )
    return True


def compare_and_log_tensor_differences(tensor1, tensor2, tensor_name, atol: float = 1e-8, rtol: float = 1e-5,
                                       max_differences: int = 20, exact_match: bool = False) -> bool:
    """True when the tensors agree (bitwise with ``exact_match``); otherwise
    logs max/mean absolute and relative differences and the first differing
    positions."""
    if tensor1.shape != tensor2.shape:
        logger.error(f"Shape mismatch for {tensor_name}: {tuple(tensor1.shape)} vs {tuple(tensor2.shape)}")
        return False
    if tensor1.dtype != tensor2.dtype:
        logger.error(f"Dtype mismatch for {tensor_name}: {tensor1.dtype} vs {tensor2.dtype}")
        return False
    a, b = tensor1.detach(), tensor2.detach().to(tensor1.device)
    if exact_match:
        same = torch.equal(a.contiguous().view(torch.uint8), b.contiguous().view(torch.uint8)) if a.numel() else True
        if same:
            return True
        differs = a.float() != b.float()
    else:
        differs = ~torch.isclose(a.float(), b.float(), atol=atol, rtol=rtol, equal_nan=True)
        if not bool(differs.any()):
            return True
    af, bf = a.float(), b.float()
    diff = (af - bf).abs()
    rel = diff / bf.abs().clamp_min(1e-12)
    n_bad = int(differs.sum())
    logger.error(
        f"Tensor {tensor_name} differs in {n_bad} of {a.numel()} elements: max abs {float(diff.max()):.6g}, "
        f"mean abs {float(diff.mean()):.6g}, max rel {float(rel.max()):.6g}, mean rel {float(rel.mean()):.6g}"
    )
    for idx in differs.nonzero()[:max_differences].tolist():
        key = tuple(idx)
        logger.error(f"  {tensor_name}{list(key)}: {float(af[key]):.8g} vs {float(bf[key]):.8g}")
    return False


def release_tensors(tensors: Union[Iterable[torch.Tensor], torch.Tensor]) -> None:
    """Drop the storage of tensors whose objects may still be referenced."""
    for t in [tensors] if torch.is_tensor(tensors) else list(tensors):
        t.data = torch.empty(0, dtype=t.dtype, device=t.device)


# ---- packing by dtype --------------------------------------------------------------------------------
def validate_tensor_for_ipc(tensor: torch.Tensor) -> bool:
    if not torch.is_tensor(tensor):
        raise ValueError(f"expected a tensor, got {type(tensor)}")
    if tensor.is_sparse or tensor.layout != torch.strided:
        raise ValueError("only dense strided tensors can be shared")
    return True


@torch.no_grad()
def group_tensors_by_shape_and_dtype(tensors: List[torch.Tensor], max_tensor_size: int = 5 * 1024**3, **_kw
                                     ) -> Tuple[List[torch.Tensor], List[Dict]]:
    """Pack ``tensors`` into flat per-dtype buffers of at most
    ``max_tensor_size`` bytes (a larger tensor gets a buffer of its own).
    Returns ``(buffers, metadata)``; metadata entries carry ``original_index``,
    ``group_index``, ``offset`` and ``size`` in elements, ``shape`` and
    ``dtype``."""
    if not tensors:
        return [], []
    buckets: Dict[Tuple[torch.dtype, torch.device], List[int]] = {}
    for i, t in enumerate(tensors):
        validate_tensor_for_ipc(t)
        buckets.setdefault((t.dtype, t.device), []).append(i)
    groups: List[torch.Tensor] = []
    metadata: List[Dict] = []
    for (dtype, device), indices in buckets.items():
        pending: List[int] = []
        pending_bytes = 0

        def flush():
            nonlocal pending, pending_bytes
            if not pending:
                return
            total = sum(tensors[i].numel() for i in pending)
            buf = torch.empty(total, dtype=dtype, device=device)
            pos = 0
            for i in pending:
                n = tensors[i].numel()
                buf[pos : pos + n].copy_(tensors[i].reshape(-1))
                metadata.append({"original_index": i, "group_index": len(groups), "offset": pos, "size": n,
                                 "shape": tuple(tensors[i].shape), "dtype": dtype})
                pos += n
            groups.append(buf)
            pending, pending_bytes = [], 0

        for i in indices:
            nbytes = tensors[i].numel() * tensors[i].element_size()
            if pending and pending_bytes + nbytes > max_tensor_size:
                flush()
            pending.append(i)
            pending_bytes += nbytes
        flush()
    return groups, metadata


@torch.no_grad()
def reconstruct_tensors_from_groups(tensor_groups: List[torch.Tensor], metadata: List[Dict]) -> List[torch.Tensor]:
    """Views into the packed buffers, in the original order."""
    if not metadata:
        return []
    out: List = [None] * (max(m["original_index"] for m in metadata) + 1)
    for m in metadata:
        if not 0 <= m["group_index"] < len(tensor_groups):
            raise ValueError(f"metadata refers to group {m['group_index']} but only {len(tensor_groups)} groups were given")
        buf = tensor_groups[m["group_index"]]
        if m["offset"] + m["size"] > buf.numel():
            raise ValueError("metadata entry exceeds its group buffer")
        out[m["original_index"]] = buf[m["offset"] : m["offset"] + m["size"]].view(m["shape"])
    if any(t is None for t in out):
        raise ValueError("metadata does not cover every original index")
    return out


# ---- serialisation -------------------------------------------------------------------------------------
def ipc_serialize(value) -> bytes:
    """Pickle with torch's multiprocessing reductions: CPU tensors travel through
    shared memory, CUDA tensors as IPC handles."""
    from multiprocessing.reduction import ForkingPickler

    import torch.multiprocessing  # noqa: F401  (registers the reductions)

    buf = io.BytesIO()
    ForkingPickler(buf).dump(value)
    return buf.getvalue()


def ipc_deserialize(data: bytes):
    return pickle.loads(data)


cuda_ipc_serialize = ipc_serialize
cuda_ipc_deserialize = ipc_deserialize

# Position of the device index among the arguments torch's reduction of a CUDA
# tensor hands to ``rebuild_cuda_tensor``.
_REBUILD_DEVICE_ARG = 6


def device_to_uuid(index: int) -> str:
    return str(torch.cuda.get_device_properties(index).uuid)


def device_from_uuid(device: Union[int, str]) -> int:
    """The local index of the GPU with this UUID (an index passes through)."""
    if isinstance(device, int):
        return device
    for index in range(torch.cuda.device_count()):
        if device_to_uuid(index) == device:
            return index
    raise RuntimeError(f"no visible GPU has UUID {device}: the process that pickled the tensor sees a GPU this one does not")


def monkey_patch_torch_compile() -> None:
    """Nothing to do: the reference marks two higher-order ops as cacheable for
    ``torch.compile`` on PyTorch older than 2.8 (`awex/util/tensor_util.py:109-116`);
    this package requires a newer PyTorch, where they are."""


def monkey_patch_torch_reductions() -> None:
    """Make pickled CUDA-IPC tensors name their GPU by UUID instead of by index,
    so that two processes whose ``CUDA_VISIBLE_DEVICES`` differ open a handle on
    the right device (`awex/util/tensor_util.py:35-106` in the reference; the
    address books of the fused path carry the UUID themselves).  Idempotent."""
    from torch.multiprocessing import reductions

    if hasattr(reductions, "_awex_reduce_tensor"):
        return
    reductions._awex_reduce_tensor = reductions.reduce_tensor
    reductions._awex_rebuild_cuda_tensor = reductions.rebuild_cuda_tensor

    def rebuild_by_uuid(*args):
        args = list(args)
        args[_REBUILD_DEVICE_ARG] = device_from_uuid(args[_REBUILD_DEVICE_ARG])
        return reductions._awex_rebuild_cuda_tensor(*args)

    def reduce_by_uuid(*args, **kwargs):
        rebuild, rebuild_args = reductions._awex_reduce_tensor(*args, **kwargs)
        # torch's reducer names the module's current ``rebuild_cuda_tensor``, which is the patched one from here on
        if rebuild is rebuild_by_uuid or rebuild is reductions._awex_rebuild_cuda_tensor:
            rebuild_args = list(rebuild_args)
            rebuild_args[_REBUILD_DEVICE_ARG] = device_to_uuid(rebuild_args[_REBUILD_DEVICE_ARG])
            return rebuild_by_uuid, tuple(rebuild_args)
        return rebuild, rebuild_args

    reductions.reduce_tensor = reduce_by_uuid
    reductions.rebuild_cuda_tensor = rebuild_by_uuid
    reductions.init_reductions()  # register the patched reducer for tensors and parameters


def reconstruct_ipc_weights(payload: bytes) -> Dict[str, torch.Tensor]:
    """Inverse of ``ipc_serialize((groups, metadata, names))``: name -> view."""
    groups, metadata, names = ipc_deserialize(payload)
    tensors = reconstruct_tensors_from_groups(groups, metadata)
    return dict(zip(names, tensors))
