"""Execute a descriptor table on the host, tile by tile, exactly as the fused
transfer kernel defines it (``ops/csrc/xfer_desc.h``): the CPU statement of the
kernel's semantics.

Used to test the encoder without a GPU (tables built over CPU tensors are run
here and compared with the item-level executor) and as the oracle when a table
is transformed (split, reordered): any table that means the same must leave
the same bytes.  Addresses are real host addresses of live CPU tensors; every
access is bounds-checked against the tensors passed in, so a wrong table raises
instead of corrupting memory.
"""

from __future__ import annotations

import ctypes
from typing import Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from awex_b200.converter.weights_converter import FP8_BLOCK, per_block_cast_to_fp8
from awex_b200.transfer.descriptors import (
    _DT_SIZE, DT_BF16, DT_BYTES, DT_F16, DT_F32, DT_FP8_E4M3, FLAG_UE8M0, OP_ADD, OP_CAST, OP_COPY, OP_FP8_BLOCK, _SpanIndex,
)

_TORCH = {DT_BF16: torch.bfloat16, DT_F16: torch.float16, DT_F32: torch.float32, DT_FP8_E4M3: torch.float8_e4m3fn, DT_BYTES: torch.uint8}


class HostMemory:
    """Bounds-checked byte access to a set of live CPU tensors by address."""

    def __init__(self, tensors: Iterable[torch.Tensor]):
        self.keep = [t for t in tensors if t.numel()]
        spans = []
        for t in self.keep:
            if t.device.type != "cpu":
                raise ValueError("the table interpreter runs on CPU tensors")
            storage = t.untyped_storage()
            spans.append((storage.data_ptr(), storage.data_ptr() + storage.nbytes()))
        self.index = _SpanIndex(spans)

    def view(self, addr: int, nbytes: int) -> np.ndarray:
        if nbytes == 0:
            return np.empty(0, dtype=np.uint8)
        if not self.index.contains(addr, addr + nbytes):
            raise IndexError(f"access [{addr:#x}, {addr + nbytes:#x}) is outside every tensor given to the interpreter")
        return np.ctypeslib.as_array((ctypes.c_uint8 * nbytes).from_address(addr))

    def read(self, addr: int, count: int, code: int) -> torch.Tensor:
        raw = torch.from_numpy(self.view(addr, count * _DT_SIZE[code]).copy())
        return raw.view(_TORCH[code])

    def write(self, addr: int, values: torch.Tensor) -> None:
        raw = values.contiguous().view(torch.uint8).reshape(-1).numpy()
        self.view(addr, raw.size)[:] = raw


def run_table(table: np.ndarray, n_tiles: int, memory: HostMemory, row_offsets: Sequence[int] = (),
              tile_order: Optional[Iterable[int]] = None) -> int:
    """Process tiles ``0 .. n_tiles-1`` (or ``tile_order``) and return how many
    were processed.  ``row_offsets`` is the encoder's gathered-row side table
    (descriptors refer to it by ``1 + first index`` while the table has no device
    address)."""
    begins = table["tile_begin"].astype(np.int64)
    done = 0
    for tile in (range(n_tiles) if tile_order is None else tile_order):
        di = int(np.searchsorted(begins, tile, side="right")) - 1
        _run_tile(table[di], tile - int(begins[di]), memory, row_offsets)
        done += 1
    return done


def _src_row_offset(d, row: int, row_offsets: Sequence[int]) -> int:
    ref = int(d["row_table"])
    if ref:
        return int(row_offsets[ref - 1 + row])
    return row * int(d["src_stride"])


def _run_tile(d, k: int, mem: HostMemory, row_offsets: Sequence[int]) -> None:
    op, sdt, ddt = int(d["op"]), int(d["src_dtype"]), int(d["dst_dtype"])
    ses, des = _DT_SIZE[sdt], _DT_SIZE[ddt]
    band, ct = divmod(k, int(d["col_tiles"]))
    row0, col0 = band * int(d["tile_rows"]), ct * int(d["tile_cols"])
    rows = min(int(d["tile_rows"]), int(d["rows"]) - row0)
    cols = min(int(d["tile_cols"]), int(d["row_elems"]) - col0)
    if rows <= 0 or cols <= 0:
        raise IndexError(f"tile {k} lies outside its slab")
    src, dst = int(d["src"]), int(d["dst"])
    block = torch.stack([mem.read(src + _src_row_offset(d, row0 + r, row_offsets) + col0 * ses, cols, sdt) for r in range(rows)])
    if op == OP_COPY:
        out = block
    elif op in (OP_CAST, OP_ADD):
        out = (block.float() + (float(d["aux_f"]) if op == OP_ADD else 0.0)).to(_TORCH[ddt])
    elif op == OP_FP8_BLOCK:
        if int(d["tile_rows"]) != FP8_BLOCK or int(d["tile_cols"]) != FP8_BLOCK:
            raise ValueError("fp8 tiles are one 128x128 block")
        out, scale = per_block_cast_to_fp8(block.contiguous(), bool(int(d["flags"]) & FLAG_UE8M0))
        mem.write(int(d["aux_ptr"]) + (band * int(d["aux_stride"]) + ct) * 4, scale.reshape(-1)[:1])
    else:
        raise ValueError(f"unknown op {op}")
    for r in range(rows):
        mem.write(dst + (row0 + r) * int(d["dst_stride"]) + col0 * des, out[r])


def run_chunked(table: np.ndarray, n_tiles: int, memory: HostMemory, grid: int, chunk_shift: int,
                row_offsets: Sequence[int] = ()) -> List[int]:
    """Process the table in the order the kernel's CTAs would with round-robin
    chunks (CTA 0's tiles first, then CTA 1's ...); returns tiles per CTA.
    Together with :func:`run_table` this shows that the chunk deal is a
    permutation of the tiles."""
    c = 1 << chunk_shift
    n_chunks = (n_tiles + c - 1) // c
    per_cta = []
    for b in range(grid):
        tiles = [t for chunk in range(b, n_chunks, grid) for t in range(chunk * c, min((chunk + 1) * c, n_tiles))]
        run_table(table, n_tiles, memory, row_offsets, tile_order=tiles)
        per_cta.append(len(tiles))
    return per_cta
