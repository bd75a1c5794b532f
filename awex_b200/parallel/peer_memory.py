"""Publish device tensors to other processes and map theirs.

An :class:`AddressBook` is plain data describing where named tensors (views of
live inference parameters, flag pads) live: for each tensor the allocation
("segment") that contains it, its byte offset inside the segment, shape,
strides and dtype; for each segment a CUDA IPC handle.  The exporting process
publishes the book through the MetaServer; an importing process opens every
segment once (`cudaIpcOpenMemHandle` with lazy peer access, so the mapping
works for the same GPU and for NVLink peers alike) and turns entries into
:class:`TensorAddr` values it can write through.

Processes recognise their own books by (host, pid) and use the raw addresses,
because a process cannot open its own IPC handles.

The reference pickles IPC tensors through the MetaServer on every update
(`awex/util/tensor_util.py:35-183`, `awex/writer/nccl_writer.py:372-400`); a
book is exchanged once and re-published only when a base address moves
(:meth:`PeerMemoryExporter.changed`).
"""

from __future__ import annotations

import ctypes
import os
import socket
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from awex_b200 import logging
from awex_b200.transfer.descriptors import TensorAddr

logger = logging.getLogger(__name__)


def process_identity() -> Tuple[str, int]:
    return socket.gethostname(), os.getpid()


@dataclass
class AddressBook:
    owner: Tuple[str, int]  # (host, pid) of the exporting process
    device_index: int
    device_uuid: str
    epoch: int
    # segment -> (ipc handle bytes, base address in the owner, size)
    segments: List[Tuple[bytes, int, int]] = field(default_factory=list)
    # name -> (segment index, byte offset of element 0, shape, strides, dtype name)
    tensors: Dict[str, Tuple[int, int, Tuple[int, ...], Tuple[int, ...], str]] = field(default_factory=dict)
    # segment index -> (chunk sizes, descriptor server address, token) for segments of virtual-memory-managed
    # allocations, which have no IPC handle (see parallel/vmm_memory.py)
    vmm: Dict[int, Tuple[List[int], str, int]] = field(default_factory=dict)
    # the owner may move or re-map these tensors between updates: senders then wait on the host, before
    # every update, for the epoch of the book that is valid for it
    may_move: bool = False


def _device_uuid(index: int) -> str:
    try:
        return str(torch.cuda.get_device_properties(index).uuid)
    except Exception:
        return f"cuda:{index}"


class PeerMemoryExporter:
    def __init__(self, device_index: Optional[int] = None):
        from awex_b200.ops import native

        self.lib = native.load()
        self.device_index = torch.cuda.current_device() if device_index is None else device_index
        self.epoch = 0
        self._last_bases: Dict[str, int] = {}
        self._vmm = None  # created on the first allocation that CUDA IPC refuses
        self._vmm_pending: Dict[int, Tuple[List[int], str, int]] = {}

    def _export_vmm(self, book: AddressBook, name: str, lo: int, hi: int, ipc_code: int) -> Tuple[int, int]:
        """Export the allocations under ``[lo, hi)`` as file descriptors.  Returns
        (base, size) of the range they cover, which becomes a segment of its own."""
        from awex_b200.parallel.vmm_memory import VmmExporter

        if self._vmm is None:
            self._vmm = VmmExporter(self.lib)
        try:
            seg = self._vmm.export_range(lo, hi)
        except RuntimeError as exc:
            raise RuntimeError(
                f"the allocation of {name} can be exported neither as a CUDA IPC handle (cudaIpcGetMemHandle: CUDA error {ipc_code}) "
                f"nor as file descriptors of virtual-memory allocations ({exc})"
            ) from exc
        self._vmm_pending[seg.base] = (list(seg.chunk_sizes), seg.server, seg.token)
        return seg.base, seg.size

    def _segment_of(self, ptr: int) -> Tuple[int, int]:
        base, size = ctypes.c_uint64(0), ctypes.c_uint64(0)
        code = self.lib.awex_address_range(ptr, ctypes.byref(base), ctypes.byref(size))
        if code != 0:
            raise RuntimeError(f"cuMemGetAddressRange failed for {ptr:#x} (code {code})")
        return base.value, size.value

    def export(self, named: Iterable[Tuple[str, torch.Tensor]], with_handles: bool = True) -> AddressBook:
        """Describe ``named`` tensors.  ``with_handles=False`` skips IPC export
        (books that only this process will read)."""
        self.epoch += 1
        book = AddressBook(process_identity(), self.device_index, _device_uuid(self.device_index), self.epoch)
        seg_index: Dict[int, int] = {}
        hbytes = self.lib.awex_ipc_handle_bytes()
        for name, t in named:
            if not t.is_cuda:
                raise ValueError(f"{name}: only CUDA tensors can be published")
            if t.numel() == 0:
                continue
            lo, _hi = TensorAddr.of(t).byte_span()
            base, size = self._segment_of(lo)
            idx = seg_index.get(base)
            vmm_only = False
            if idx is not None and idx in book.vmm and _hi > base + book.segments[idx][2]:
                # an earlier tensor's export of this range of allocations ends before this tensor does
                idx, vmm_only = None, True
            if idx is None:
                handle = b""
                if with_handles:
                    code = -1
                    if not vmm_only:
                        buf = ctypes.create_string_buffer(hbytes)
                        code = self.lib.awex_ipc_export(base, buf)
                    if code != 0:
                        # not a cudaMalloc allocation: try the virtual-memory route over the whole tensor
                        base, size = self._export_vmm(book, name, lo, _hi, code)
                    else:
                        handle = buf.raw
                idx = len(book.segments)
                book.segments.append((handle, base, size))
                seg_index[base] = idx  # later tensors of the same allocation reuse the newest export
                if base in self._vmm_pending:
                    book.vmm[idx] = self._vmm_pending.pop(base)
            book.tensors[name] = (idx, t.data_ptr() - base, tuple(t.shape), tuple(t.stride()), str(t.dtype).replace("torch.", ""))
            self._last_bases[name] = t.data_ptr()
        return book

    def changed(self, named: Iterable[Tuple[str, torch.Tensor]]) -> bool:
        """True when any tensor moved since the last export (engines that
        re-map weights after a sleep/wake cycle): the book must be re-published."""
        return any(self._last_bases.get(n) != t.data_ptr() for n, t in named if t.numel())


class PeerMemoryImporter:
    def __init__(self):
        from awex_b200.ops import native

        self.lib = native.load()
        self._open: Dict[bytes, int] = {}
        self._me = process_identity()

    def resolve(self, book: AddressBook) -> Dict[str, TensorAddr]:
        bases: List[int] = []
        for index, (handle, owner_base, _size) in enumerate(book.segments):
            if tuple(book.owner) == self._me:
                self._own_process_access(book.device_index)
                bases.append(owner_base)
                continue
            if index in getattr(book, "vmm", {}):
                bases.append(self._map_vmm(owner_base, *book.vmm[index]))
                continue
            if not handle:
                raise RuntimeError("address book of another process carries no IPC handles")
            mapped = self._open.get(handle)
            if mapped is None:
                out = ctypes.c_uint64(0)
                code = self.lib.awex_ipc_open(handle, ctypes.byref(out))
                if code != 0:
                    msg = self.lib.awex_cuda_error_string(code)
                    hint = ""
                    if tuple(book.owner)[0] != self._me[0]:
                        hint = (f"; the memory belongs to a process on host {tuple(book.owner)[0]!r}, this is {self._me[0]!r}: peer stores "
                                "work inside one machine, set data_plane='messages' (or AWEX_DATA_PLANE=messages) on the inference side")
                    raise RuntimeError(f"cudaIpcOpenMemHandle failed (CUDA error {code}: {msg.decode() if msg else '?'}){hint}")
                mapped = self._open[handle] = out.value
            bases.append(mapped)
        out_addrs: Dict[str, TensorAddr] = {}
        for name, (seg, offset, shape, strides, dtype) in book.tensors.items():
            out_addrs[name] = TensorAddr(bases[seg] + offset, tuple(shape), tuple(strides), getattr(torch, dtype))
        return out_addrs

    def _own_process_access(self, device_index: int) -> None:
        """Memory that this very process holds on another GPU is reached through its
        plain addresses, which needs peer access between the two devices; without
        it a kernel that writes there faults.  Refuse instead."""
        current = torch.cuda.current_device()
        enabled = self.__dict__.setdefault("_peers", set())
        if device_index == current or device_index in enabled:
            return
        code = self.lib.awex_enable_peer_access(current, device_index)
        if code != 0:
            raise RuntimeError(
                f"device {current} cannot be given access to memory of device {device_index} of this process "
                f"({'no peer path between them' if code == -2 else f'CUDA error {code}'})"
            )
        enabled.add(device_index)

    def _map_vmm(self, owner_base: int, chunk_sizes, server: str, token: int) -> int:
        import torch as _torch

        from awex_b200.parallel.vmm_memory import VmmImporter, VmmSegment

        if getattr(self, "_vmm", None) is None:
            self._vmm = VmmImporter(_torch.cuda.current_device(), self.lib)
        return self._vmm.map(VmmSegment(owner_base, list(chunk_sizes), server, token))

    def close_all(self) -> None:
        """Unmap everything (must happen before the owner frees or re-maps the
        memory)."""
        if getattr(self, "_vmm", None) is not None:
            self._vmm.close_all()
        for handle, mapped in list(self._open.items()):
            code = self.lib.awex_ipc_close(mapped)
            if code != 0:
                logger.warning(f"cudaIpcCloseMemHandle returned {code}")
            del self._open[handle]
