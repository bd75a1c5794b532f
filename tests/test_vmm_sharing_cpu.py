"""Host half of sharing virtual-memory-managed device allocations: descriptors
travel between real processes over a unix socket, and the exporter / importer
drive the native calls in the right order (checked against a fake of the
library; the driver calls themselves need a GPU)."""

import os

import pytest
import torch.multiprocessing as mp

from awex_b200.parallel.vmm_memory import FdServer, VmmExporter, VmmImporter, VmmSegment, fetch_fds


def _child_reads(address, token, q):
    try:
        fds = fetch_fds(address, token, timeout_s=20)
        texts = []
        for fd in fds:
            os.lseek(fd, 0, os.SEEK_SET)
            texts.append(os.read(fd, 64).decode())
            os.close(fd)
        q.put(texts)
    except BaseException as exc:
        q.put(repr(exc))
        raise


@pytest.mark.timeout(120)
def test_descriptors_reach_another_process_in_order(tmp_path):
    files = []
    for i in range(450):  # more than one SCM_RIGHTS message carries
        fd = os.open(tmp_path / f"f{i}", os.O_RDWR | os.O_CREAT)
        os.write(fd, f"allocation {i}".encode())
        files.append(fd)
    server = FdServer()
    try:
        token = server.register(files)
        other = server.register(files[:2])
        assert token != other
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        p = ctx.Process(target=_child_reads, args=(server.address, token, q))
        p.start()
        got = q.get(timeout=90)
        p.join(timeout=30)
        assert got == [f"allocation {i}" for i in range(450)]
        assert fetch_fds(server.address, 12345) == []  # a token nobody registered opens nothing
        mine = fetch_fds(server.address, other)
        assert len(mine) == 2 and all(fd not in files for fd in mine)  # copies, not the server's own numbers
        for fd in mine:
            os.close(fd)
    finally:
        server.close()
    with pytest.raises(OSError):
        os.fstat(files[0])  # the server owned the registered descriptors and closed them
    with pytest.raises(OSError):
        fetch_fds(server.address, token, timeout_s=2)


class FakeLib:
    """Address space with three allocations mapped back to back; records every call."""

    def __init__(self, fail_export_at=None, fail_map_at=None):
        self.chunks = [(0x1000, 0x400), (0x1400, 0x400), (0x1800, 0x800)]
        self.calls, self.fail_export_at, self.fail_map_at = [], fail_export_at, fail_map_at
        self.pipes = []

    def awex_address_range(self, ptr, base, size):
        for b, s in self.chunks:
            if b <= ptr < b + s:
                base._obj.value, size._obj.value = b, s
                return 0
        return 1

    def awex_vmm_export_fd(self, base, fd_out):
        if base == self.fail_export_at:
            return 801
        r, w = os.pipe()
        os.close(w)
        self.pipes.append(r)
        fd_out._obj.value = r
        self.calls.append(("export", base))
        return 0

    def awex_vmm_reserve(self, total, alignment, va_out):
        va_out._obj.value = 0x9000
        self.calls.append(("reserve", total))
        return 0

    def awex_vmm_map_fd(self, va, offset, size, fd, device):
        os.fstat(fd)  # must still be open while it is mapped
        if offset == self.fail_map_at:
            return 2
        self.calls.append(("map", va, offset, size, device))
        return 0

    def awex_vmm_unmap(self, va, offset, size):
        self.calls.append(("unmap", va, offset, size))
        return 0

    def awex_vmm_release_range(self, va, total):
        self.calls.append(("free", va, total))
        return 0

    def awex_driver_error_string(self, code):
        return {801: b"operation not supported", 2: b"out of memory"}.get(code, b"?")


def test_exporter_walks_the_allocations_under_a_range_and_importer_rebuilds_it():
    lib = FakeLib()
    exporter = VmmExporter(lib)
    try:
        assert exporter.chunks_of(0x1200, 0x1900) == lib.chunks  # a tensor that starts inside the first and ends inside the last
        assert exporter.chunks_of(0x1400, 0x1800) == [lib.chunks[1]]
        seg = exporter.export_range(0x1200, 0x1900)
        assert seg.base == 0x1000 and seg.chunk_sizes == [0x400, 0x400, 0x800] and seg.size == 0x1000
        importer = VmmImporter(device_index=3, lib=lib)
        va = importer.map(seg)
        assert va == 0x9000 and importer.map(seg) == va  # mapped once, then remembered
        maps = [c for c in lib.calls if c[0] == "map"]
        assert maps == [("map", 0x9000, 0, 0x400, 3), ("map", 0x9000, 0x400, 0x400, 3), ("map", 0x9000, 0x800, 0x800, 3)]
        importer.close_all()
        assert [c for c in lib.calls if c[0] in ("unmap", "free")] == [
            ("unmap", 0x9000, 0, 0x400), ("unmap", 0x9000, 0x400, 0x400), ("unmap", 0x9000, 0x800, 0x800), ("free", 0x9000, 0x1000)]
        with pytest.raises(RuntimeError, match="no mapped allocation"):
            exporter.chunks_of(0x1000, 0x3000)  # runs off the end of what is mapped
    finally:
        exporter.close()


def test_failed_exports_and_maps_clean_up_after_themselves():
    lib = FakeLib(fail_export_at=0x1400)
    exporter = VmmExporter(lib)
    try:
        with pytest.raises(RuntimeError, match="operation not supported"):
            exporter.export_range(0x1000, 0x2000)
        with pytest.raises(OSError):
            os.fstat(lib.pipes[0])  # the descriptor exported before the failure was closed again
    finally:
        exporter.close()
    lib = FakeLib(fail_map_at=0x400)
    exporter = VmmExporter(lib)
    try:
        seg = exporter.export_range(0x1000, 0x2000)
        importer = VmmImporter(device_index=0, lib=lib)
        with pytest.raises(RuntimeError, match="out of memory"):
            importer.map(seg)
        assert ("unmap", 0x9000, 0, 0x400) in lib.calls and ("free", 0x9000, 0x1000) in lib.calls  # nothing stays half mapped
        short = VmmSegment(seg.base, seg.chunk_sizes + [0x100], seg.server, seg.token)
        with pytest.raises(RuntimeError, match="expected 4 descriptors"):
            importer.map(short)
    finally:
        exporter.close()


class _FakeTensor:
    """Just enough of a CUDA tensor for an address book: an address, a shape, a dtype."""

    is_cuda = True

    def __init__(self, ptr, n_bytes):
        import torch

        self._ptr, self.shape, self.dtype = ptr, (n_bytes,), torch.uint8

    def numel(self):
        return self.shape[0]

    def data_ptr(self):
        return self._ptr

    def stride(self):
        return (1,)


class _BookLib(FakeLib):
    """cudaMalloc allocations at 0x100000 (IPC works) and virtual-memory allocations at 0x1000.. (IPC refused)."""

    def awex_address_range(self, ptr, base, size):
        if 0x100000 <= ptr < 0x200000:
            base._obj.value, size._obj.value = 0x100000, 0x100000
            return 0
        return super().awex_address_range(ptr, base, size)

    def awex_ipc_handle_bytes(self):
        return 64

    def awex_ipc_export(self, base, buf):
        if base != 0x100000:
            return 1  # cudaErrorInvalidValue: not a cudaMalloc allocation
        buf.raw = b"H" * 64
        return 0


def test_address_book_mixes_ipc_segments_and_descriptor_segments(monkeypatch):
    from awex_b200.parallel import peer_memory

    monkeypatch.setattr(peer_memory, "_device_uuid", lambda index: "GPU-fake")
    lib = _BookLib()
    exporter = peer_memory.PeerMemoryExporter.__new__(peer_memory.PeerMemoryExporter)
    exporter.lib, exporter.device_index, exporter.epoch, exporter._last_bases = lib, 0, 0, {}
    exporter._vmm, exporter._vmm_pending = None, {}
    named = [
        ("plain.a", _FakeTensor(0x100100, 0x200)), ("plain.b", _FakeTensor(0x100800, 0x100)),  # one cudaMalloc segment
        ("vm.short", _FakeTensor(0x1100, 0x100)),       # inside the first virtual-memory allocation
        ("vm.long", _FakeTensor(0x1200, 0x900)),        # starts there too but reaches the third allocation
        ("vm.tail", _FakeTensor(0x1900, 0x100)),        # inside the third one alone
    ]
    try:
        book = exporter.export(named)
        seg = {n: book.tensors[n][0] for n, _ in named}
        assert seg["plain.a"] == seg["plain.b"] and seg["plain.a"] not in book.vmm and book.segments[seg["plain.a"]][0] == b"H" * 64
        assert book.vmm[seg["vm.short"]][0] == [0x400]                      # one allocation suffices
        assert seg["vm.long"] != seg["vm.short"] and book.vmm[seg["vm.long"]][0] == [0x400, 0x400, 0x800]  # re-exported to its end
        assert book.vmm[seg["vm.tail"]][0] == [0x800] and book.segments[seg["vm.tail"]][1] == 0x1800
        for name, t in named:
            index, offset = book.tensors[name][:2]
            _handle, base, size = book.segments[index]
            assert base + offset == t.data_ptr() and offset + t.numel() <= size  # every tensor lies inside its segment
        # the importer side: IPC segments are opened, descriptor segments are mapped
        importer = peer_memory.PeerMemoryImporter.__new__(peer_memory.PeerMemoryImporter)
        importer.lib, importer._open, importer._me, importer._vmm = lib, {}, ("elsewhere", 1), None
        lib.awex_ipc_open = lambda handle, out: setattr(out._obj, "value", 0x700000) or 0
        monkeypatch.setattr("torch.cuda.current_device", lambda: 5)
        addrs = importer.resolve(book)
        assert addrs["plain.a"].ptr == 0x700100 and addrs["vm.long"].ptr == 0x9000 + 0x200
        assert all(c[-1] == 5 for c in lib.calls if c[0] == "map")
    finally:
        exporter._vmm.close()


def test_books_of_this_process_on_another_gpu_need_peer_access(monkeypatch):
    """One process that holds the training shard on one GPU and the engine on
    another: the sender uses plain addresses, so the importer enables peer access
    first and refuses when the devices have no peer path (a kernel would fault)."""
    from awex_b200.parallel import peer_memory

    calls = []
    lib = type("Lib", (), {"awex_enable_peer_access": lambda self, a, b: calls.append((a, b)) or (0 if b == 1 else -2)})()
    importer = peer_memory.PeerMemoryImporter.__new__(peer_memory.PeerMemoryImporter)
    importer.lib, importer._open, importer._me = lib, {}, ("here", 7)
    monkeypatch.setattr("torch.cuda.current_device", lambda: 0)

    def book(device):
        b = peer_memory.AddressBook(("here", 7), device, f"GPU-{device}", 1)
        b.segments.append((b"", 0x1000, 0x100))
        b.tensors["w"] = (0, 0x10, (4,), (1,), "float32")
        return b

    assert importer.resolve(book(0))["w"].ptr == 0x1010 and calls == []  # same device: nothing to enable
    assert importer.resolve(book(1))["w"].ptr == 0x1010 and calls == [(0, 1)]
    importer.resolve(book(1))
    assert calls == [(0, 1)]  # once per pair
    with pytest.raises(RuntimeError, match="no peer path"):
        importer.resolve(book(2))
