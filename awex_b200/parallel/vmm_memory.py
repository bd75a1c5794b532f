"""Sharing device memory that CUDA IPC handles cannot describe.

Memory created with the virtual-memory-management API (PyTorch expandable
segments, sleep-mode / memory-saver allocators of inference engines) is a range
of addresses onto which several physical allocations are mapped.  The owner
exports every allocation under a tensor as a file descriptor
(:class:`VmmExporter`); descriptors cross process boundaries over a unix domain
socket (:class:`FdServer` / :func:`fetch_fds`), announced through the address
book; the importer reserves an address range of the same size and maps the
allocations into it (:class:`VmmImporter`), after which the range is used like
a CUDA-IPC mapping.  The native half is ``ops/csrc/vmm_memory.cu``.

The reference documents such memory as unsupported (`docs/README.md:91` there).

An importer's mapping holds a reference to the physical allocations.  An
allocator that releases them (an engine going to sleep) does not get the memory
back until importers unmap (:meth:`VmmImporter.close_all`), and one that
creates new allocations at the old addresses on wake-up must be exported again:
the addresses are the same but the memory behind them is not, which a pointer
comparison cannot see.

Limits: one descriptor per physical allocation and per export (process file
descriptor limits apply: a 60 GB shard in 20 MiB allocations needs about 3000);
the allocations must have been created with POSIX file descriptors as a
requested handle type, which the driver checks on export.
"""

from __future__ import annotations

import ctypes
import os
import socket
import struct
import threading
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from awex_b200 import logging

logger = logging.getLogger(__name__)

_TOKEN = struct.Struct("!Q")
_MAX_FDS_PER_MESSAGE = 200  # SCM_RIGHTS carries a bounded number of descriptors per message


class FdServer:
    """Hands registered file descriptors to processes that present the right
    token, over an abstract-namespace unix socket (no file to clean up; only
    processes of this machine and network namespace can connect).  Tokens are
    random 63-bit numbers that travel through the MetaServer with the address
    book, so the descriptors are as private as the MetaServer is.  One server per
    exporting process; runs a daemon thread."""

    def __init__(self, name: Optional[str] = None):
        self.address = "\0" + (name or f"awex-vmm-{os.getpid()}-{id(self):x}")
        self._sets: Dict[int, List[int]] = {}
        self._lock = threading.Lock()
        self._sock = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        self._sock.bind(self.address)
        self._sock.listen(64)
        self._closing = False
        self._thread = threading.Thread(target=self._serve, name="awex-fd-server", daemon=True)
        self._thread.start()

    def register(self, fds: Sequence[int]) -> int:
        """Keep ``fds`` (they stay open and owned by this server) and return the
        token that lets another process fetch copies of them."""
        import secrets

        with self._lock:
            token = secrets.randbits(63)  # unguessable: whoever presents it receives the memory behind the descriptors
            while token in self._sets:
                token = secrets.randbits(63)
            self._sets[token] = list(fds)
        return token

    def _serve(self) -> None:
        while not self._closing:
            try:
                conn, _ = self._sock.accept()
            except OSError:
                return
            with conn:
                if self._closing:
                    return
                try:
                    conn.settimeout(10.0)
                    raw = conn.recv(_TOKEN.size, socket.MSG_WAITALL)
                    if len(raw) != _TOKEN.size:
                        continue
                    with self._lock:
                        fds = list(self._sets.get(_TOKEN.unpack(raw)[0], ()))
                    conn.sendall(struct.pack("!I", len(fds)))
                    for i in range(0, len(fds), _MAX_FDS_PER_MESSAGE):
                        socket.send_fds(conn, [b"F"], fds[i : i + _MAX_FDS_PER_MESSAGE])
                except OSError as exc:
                    logger.warning(f"descriptor hand-over failed: {exc!r}")

    def close(self) -> None:
        """Stop serving and close every registered descriptor."""
        self._closing = True
        for step in (lambda: self._sock.shutdown(socket.SHUT_RDWR), self._sock.close):  # shutdown wakes a blocked accept()
            try:
                step()
            except OSError:
                pass
        self._thread.join(timeout=5)
        with self._lock:
            for fds in self._sets.values():
                for fd in fds:
                    try:
                        os.close(fd)
                    except OSError:
                        pass
            self._sets.clear()


def fetch_fds(address: str, token: int, timeout_s: float = 30.0) -> List[int]:
    """Copies (valid in this process) of the descriptors registered under
    ``token`` at the :class:`FdServer` listening on ``address``.  The caller
    closes them.  An unknown token yields an empty list."""
    with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as conn:
        conn.settimeout(timeout_s)
        conn.connect(address)
        conn.sendall(_TOKEN.pack(token))
        raw = conn.recv(4, socket.MSG_WAITALL)
        if len(raw) != 4:
            raise ConnectionError("the descriptor server closed the connection")
        (count,) = struct.unpack("!I", raw)
        fds: List[int] = []
        while len(fds) < count:
            _msg, got, _flags, _addr = socket.recv_fds(conn, 1, min(_MAX_FDS_PER_MESSAGE, count - len(fds)))
            if not got:
                raise ConnectionError(f"expected {count} descriptors, received {len(fds)}")
            fds.extend(got)
        return fds


# ---- device side ---------------------------------------------------------------------------------------
@dataclass
class VmmSegment:
    """What an importer needs to rebuild a range of the owner's addresses:
    the owner's base address, the sizes of the physical allocations mapped there
    back to back, and where to fetch their descriptors."""

    base: int
    chunk_sizes: List[int] = field(default_factory=list)
    server: str = ""
    token: int = 0

    @property
    def size(self) -> int:
        return sum(self.chunk_sizes)


def driver_error(lib, code: int) -> str:
    if code == -1:
        return "the CUDA driver's virtual-memory entry points could not be resolved"
    text = lib.awex_driver_error_string(code)
    return f"driver error {code}: {text.decode() if text else '?'}"


class VmmExporter:
    """Exports the physical allocations under address ranges of this process."""

    def __init__(self, lib=None, server: Optional[FdServer] = None):
        if lib is None:
            from awex_b200.ops import native

            lib = native.load()
        self.lib = lib
        self._server = server
        self._own_server = server is None

    @property
    def server(self) -> FdServer:
        if self._server is None:
            self._server = FdServer()
        return self._server

    def chunks_of(self, lo: int, hi: int) -> List[Tuple[int, int]]:
        """(base, size) of every mapped allocation that intersects ``[lo, hi)``, in address order."""
        out: List[Tuple[int, int]] = []
        at = lo
        while at < hi:
            base, size = ctypes.c_uint64(0), ctypes.c_uint64(0)
            code = self.lib.awex_address_range(at, ctypes.byref(base), ctypes.byref(size))
            if code != 0 or size.value == 0:
                raise RuntimeError(f"no mapped allocation at {at:#x} (code {code})")
            out.append((base.value, size.value))
            at = base.value + size.value
        return out

    def export_range(self, lo: int, hi: int) -> VmmSegment:
        """Export everything mapped under ``[lo, hi)``.  Raises RuntimeError with
        the driver's reason when an allocation cannot be exported."""
        if not hasattr(self.lib, "awex_vmm_export_fd"):
            raise RuntimeError("this build of the native library has no virtual-memory export")
        chunks = self.chunks_of(lo, hi)
        fds: List[int] = []
        try:
            for base, _size in chunks:
                fd = ctypes.c_int(-1)
                code = self.lib.awex_vmm_export_fd(base, ctypes.byref(fd))
                if code != 0:
                    raise RuntimeError(f"cuMemExportToShareableHandle failed for the allocation at {base:#x}: {driver_error(self.lib, code)}")
                fds.append(fd.value)
        except Exception:
            for fd in fds:
                os.close(fd)
            raise
        token = self.server.register(fds)
        return VmmSegment(chunks[0][0], [s for _b, s in chunks], self.server.address, token)

    def close(self) -> None:
        if self._server is not None and self._own_server:
            self._server.close()
            self._server = None


class VmmImporter:
    """Maps segments exported by other processes into this process for one device."""

    def __init__(self, device_index: int, lib=None):
        if lib is None:
            from awex_b200.ops import native

            lib = native.load()
        self.lib, self.device_index = lib, device_index
        # owner key -> (address here, segment)
        self._mapped: Dict[Tuple[str, int], Tuple[int, VmmSegment]] = {}

    def map(self, seg: VmmSegment, fetch=fetch_fds) -> int:
        """Address in this process at which ``seg.base`` of the owner appears."""
        key = (seg.server, seg.token)
        if key in self._mapped:
            return self._mapped[key][0]
        fds = fetch(seg.server, seg.token)
        try:
            if len(fds) != len(seg.chunk_sizes):
                raise RuntimeError(f"expected {len(seg.chunk_sizes)} descriptors from the owner, received {len(fds)}")
            va = ctypes.c_uint64(0)
            code = self.lib.awex_vmm_reserve(seg.size, 0, ctypes.byref(va))
            if code != 0:
                raise RuntimeError(f"cuMemAddressReserve of {seg.size} bytes failed: {driver_error(self.lib, code)}")
            offset, done = 0, []
            for fd, size in zip(fds, seg.chunk_sizes):
                code = self.lib.awex_vmm_map_fd(va.value, offset, size, fd, self.device_index)
                if code != 0:
                    for o, s in done:
                        self.lib.awex_vmm_unmap(va.value, o, s)
                    self.lib.awex_vmm_release_range(va.value, seg.size)
                    raise RuntimeError(f"mapping an imported allocation of {size} bytes failed: {driver_error(self.lib, code)}")
                done.append((offset, size))
                offset += size
        finally:
            for fd in fds:  # mappings keep the memory alive; the descriptors are not needed any more
                try:
                    os.close(fd)
                except OSError:
                    pass
        self._mapped[key] = (va.value, seg)
        return va.value

    def close_all(self) -> None:
        """Unmap everything (before the owner frees or re-maps the memory)."""
        for key, (va, seg) in list(self._mapped.items()):
            offset = 0
            for size in seg.chunk_sizes:
                code = self.lib.awex_vmm_unmap(va, offset, size)
                if code != 0:
                    logger.warning(f"cuMemUnmap returned {code}")
                offset += size
            self.lib.awex_vmm_release_range(va, seg.size)
            del self._mapped[key]
