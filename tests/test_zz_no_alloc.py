"""The allocation-free launch (`awex_fused_transfer_no_alloc`, declared in
awex_b200/ops/csrc/awex_no_alloc.h), called through its exported C symbol, must
write exactly what the regular launcher writes for the same descriptor table,
on two calls in a row that share the library's built-in scratch."""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_DESCS = 2048


def _symbol():
    from awex_b200.ops import native

    fn = native.load().awex_fused_transfer_no_alloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int, ctypes.c_void_p,
                   ctypes.POINTER(ctypes.c_int32), ctypes.c_char_p, ctypes.c_size_t]
    return fn


def _items(rows, cols):
    from awex_b200.converter.rows import ValueOp
    from awex_b200.transfer.lowering import CopyItem

    half = cols // 2
    return [
        # column slabs swapped (strided rows), a contiguous band, and a cast
        CopyItem("a", 0, (0, 0), (rows, half), 0, "a", (0, half), torch.bfloat16, torch.bfloat16),
        CopyItem("a", 0, (0, half), (rows, half), 0, "a", (0, 0), torch.bfloat16, torch.bfloat16),
        CopyItem("b", 0, (0, 0), (rows, cols), 0, "b", (0, 0), torch.bfloat16, torch.bfloat16),
        CopyItem("c", 0, (0, 0), (rows, cols), 0, "c", (0, 0), torch.bfloat16, torch.float32, ValueOp("cast", dtype=torch.float32)),
    ]


def _table(items, srcs, dsts):
    from awex_b200.transfer.descriptors import TensorAddr, encode_items

    table, n_tiles, enc = encode_items(items, {(n, 0): TensorAddr.of(t) for n, t in srcs.items()}, {0: {n: TensorAddr.of(t) for n, t in dsts.items()}})
    return np.ascontiguousarray(table), n_tiles, enc


def _fresh_dsts(rows, cols):
    return {"a": torch.zeros(rows, cols, dtype=torch.bfloat16, device="cuda"), "b": torch.zeros(rows, cols, dtype=torch.bfloat16, device="cuda"),
            "c": torch.zeros(rows, cols, dtype=torch.float32, device="cuda")}


def test_no_alloc_entry_matches_regular_launcher_twice():
    from awex_b200.ops.fused_transfer import TransferProgram

    fn = _symbol()
    rows, cols = 1000, 1536
    items = _items(rows, cols)
    err = ctypes.create_string_buffer(256)
    status = (ctypes.c_int32 * 4)()
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        g = torch.Generator(device="cuda").manual_seed(100 + call)
        srcs = {n: torch.randn(rows, cols, generator=g, device="cuda").to(torch.bfloat16) for n in "abc"}
        want, got = _fresh_dsts(rows, cols), _fresh_dsts(rows, cols)
        table_w, tiles_w, enc_w = _table(items, srcs, want)
        prog = TransferProgram(table_w, tiles_w, "cuda", encoder=enc_w)
        prog.launch(call + 1)
        torch.cuda.synchronize()
        prog.status.raise_if_failed()
        table_g, tiles_g, _ = _table(items, srcs, got)
        assert table_g.dtype.itemsize == 128 and len(table_g) <= MAX_DESCS
        for i in range(4):
            status[i] = -1
        rc = fn(table_g.ctypes.data, len(table_g), tiles_g, 2_000_000_000, 0, stream, status, err, len(err))
        assert rc == 0, err.value.decode()
        assert list(status) == [0, 0, 0, 0]
        for name in want:  # bitwise: the same kernel ran on the same table
            assert torch.equal(got[name], want[name]), (call, name)
        assert torch.equal(got["a"][:, cols // 2 :], srcs["a"][:, : cols // 2])
        assert torch.equal(got["c"], srcs["c"].float())


def test_no_alloc_entry_refuses_oversized_tables():
    fn = _symbol()
    err = ctypes.create_string_buffer(256)
    table = np.zeros(MAX_DESCS + 1, dtype=np.dtype([("raw", np.uint8, 128)]))
    before = torch.cuda.memory_allocated()
    rc = fn(table.ctypes.data, MAX_DESCS + 1, 1, 1_000_000, 0, torch.cuda.current_stream().cuda_stream, None, err, len(err))
    assert rc == 1  # cudaErrorInvalidValue
    assert b"2049" in err.value and b"2048" in err.value
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    assert torch.ones(8, device="cuda").sum().item() == 8


def test_no_alloc_entry_refuses_raw_encoder_tables_with_gathered_rows_and_bad_addresses():
    """A table whose `row_table` still holds the encoder's index, or whose
    addresses are not device memory, is refused on the host: nothing is queued,
    so nothing can fault."""
    fn = _symbol()
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    src = torch.randn(256, 256, device="cuda").to(torch.bfloat16)
    dst = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda")
    from awex_b200.transfer.lowering import CopyItem

    table, n_tiles, _ = _table([CopyItem("a", 0, (0, 0), (256, 256), 0, "a", (0, 0), torch.bfloat16, torch.bfloat16)], {"a": src}, {"a": dst})
    cases = []
    t = table.copy(); t["row_table"][0] = 1; cases.append((t, b"row_table"))          # an index, not an address
    t = table.copy(); t["tensor_map"][0] = 4096; cases.append((t, b"tensor_map"))
    host = np.zeros(256 * 256, dtype=np.uint16)
    t = table.copy(); t["src"][0] = (host.ctypes.data + 15) & ~15; cases.append((t, b"src is not a device address"))
    t = table.copy(); t["dst"][0] = (host.ctypes.data + 15) & ~15; cases.append((t, b"dst is not a device address"))
    for bad, needle in cases:
        rc = fn(np.ascontiguousarray(bad).ctypes.data, len(bad), n_tiles, 1_000_000, 0, stream, None, err, len(err))
        assert rc == 1 and needle in err.value, (needle, err.value)
    torch.cuda.synchronize()
    assert torch.count_nonzero(dst).item() == 0  # nothing ran
    status = (ctypes.c_int32 * 4)()
    assert fn(table.ctypes.data, len(table), n_tiles, 2_000_000_000, 0, stream, status, err, len(err)) == 0, err.value
    assert list(status) == [0, 0, 0, 0] and torch.equal(dst, src)  # the context is intact and the good table runs
