"""Encode copy items as the flat descriptor table of the fused transfer kernel,
and check tables on the host before they ever reach a GPU.

The table format is the C struct ``awex::XferDesc`` (``ops/csrc/xfer_desc.h``),
mirrored here as a numpy structured dtype.  Encoding collapses every N-d box
into as few 2-D slabs as the two stride patterns allow, picks a tile shape
that fits one 32 KiB pipeline stage, and decides per slab whether the
bulk-async (16-byte aligned) path applies.

:func:`validate_table` is the host-side stand-in for a device sanitizer: it
proves, from addresses and extents alone, that every slab stays inside the
tensors it names, that no two slabs write the same destination byte, and that
every bulk copy meets the alignment rules of ``cp.async.bulk``; a table that
fails is never launched.

The table takes the place of the per-operation send and receive lists the
reference builds from a plan (`awex/transfer/nccl_comm.py:379-541`).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from awex_b200.converter.weights_converter import FP8_BLOCK
from awex_b200.transfer.lowering import CopyItem

OP_COPY, OP_CAST, OP_ADD, OP_FP8_BLOCK = 0, 1, 2, 3
DT_BYTES, DT_BF16, DT_F16, DT_F32, DT_FP8_E4M3 = 0, 1, 2, 3, 4
FLAG_BULK, FLAG_DST_VEC16, FLAG_UE8M0, FLAG_OUT_BULK = 1, 2, 4, 8
STAGE_BYTES = 32 * 1024
MAX_TX_BYTES = (1 << 20) - 1

PLAN_DTYPE = np.dtype(
    [("tile_begin", "<u8"), ("tile_end", "<u8"), ("rank", "<u4"), ("size", "<u4"), ("chunk_off", "<u4"), ("reserved", "<u4")]
)
assert PLAN_DTYPE.itemsize == 32

DESC_DTYPE = np.dtype(
    [
        ("src", "<u8"), ("dst", "<u8"), ("rows", "<u8"), ("row_elems", "<u8"), ("src_stride", "<i8"),
        ("dst_stride", "<i8"), ("tile_begin", "<u8"), ("aux_ptr", "<u8"), ("aux_stride", "<i8"), ("aux_f", "<f8"),
        ("op", "<u4"), ("flags", "<u4"), ("src_dtype", "<u4"), ("dst_dtype", "<u4"), ("tile_rows", "<u4"),
        ("tile_cols", "<u4"), ("col_tiles", "<u4"), ("reserved", "<u4"), ("row_table", "<u8"), ("tensor_map", "<u8"),
    ]
)
assert DESC_DTYPE.itemsize == 128

_DT_CODE = {torch.bfloat16: DT_BF16, torch.float16: DT_F16, torch.float32: DT_F32, torch.float8_e4m3fn: DT_FP8_E4M3}
_DT_SIZE = {DT_BYTES: 1, DT_BF16: 2, DT_F16: 2, DT_F32: 4, DT_FP8_E4M3: 1}


@dataclass(frozen=True)
class TensorAddr:
    """Where a tensor (or view) lives: address of element 0, shape, strides in
    elements, dtype.  Plain data, so it can be published to other processes."""

    ptr: int
    shape: Tuple[int, ...]
    strides: Tuple[int, ...]
    dtype: torch.dtype

    @staticmethod
    def of(t: torch.Tensor, ptr: Optional[int] = None) -> "TensorAddr":
        return TensorAddr(t.data_ptr() if ptr is None else ptr, tuple(t.shape), tuple(t.stride()), t.dtype)

    def byte_span(self) -> Tuple[int, int]:
        """[low, high) addresses the view can touch."""
        es = self.dtype.itemsize
        lo = hi = 0
        for n, s in zip(self.shape, self.strides):
            if n == 0:
                return self.ptr, self.ptr
            if s >= 0:
                hi += (n - 1) * s
            else:
                lo += (n - 1) * s
        return self.ptr + lo * es, self.ptr + (hi + 1) * es


def collapse_box(extent: Sequence[int], src_strides: Sequence[int], dst_strides: Sequence[int]):
    """Reduce an N-d box to ``(rows, row_elems, src_row_stride, dst_row_stride,
    [(src_off, dst_off), ...])`` in elements: the innermost run that is
    contiguous on both sides becomes a row, the next dim (merged with its
    parents where strides allow) indexes rows, the rest is enumerated."""
    dims = [(e, s, d) for e, s, d in zip(extent, src_strides, dst_strides) if e != 1]
    if any(e == 0 for e in extent):
        return 0, 0, 0, 0, []
    if not dims:
        return 1, 1, 0, 0, [(0, 0)]
    row_elems = 1
    if dims[-1][1] == 1 and dims[-1][2] == 1:
        row_elems = dims[-1][0]
        dims = dims[:-1]
        while dims and dims[-1][1] == row_elems and dims[-1][2] == row_elems:
            row_elems *= dims[-1][0]
            dims = dims[:-1]
    if not dims:
        return 1, row_elems, 0, 0, [(0, 0)]
    rows, s_row, d_row = dims[-1]
    dims = dims[:-1]
    while dims and dims[-1][1] == s_row * rows and dims[-1][2] == d_row * rows:
        rows *= dims[-1][0]
        dims = dims[:-1]
    offsets = [(0, 0)]
    for e, s, d in dims:
        offsets = [(so + i * s, do + i * d) for so, do in offsets for i in range(e)]
    return rows, row_elems, s_row, d_row, offsets


def _aligned16(*values: int) -> bool:
    return all(v % 16 == 0 for v in values)


def _tile_shape(rows: int, row_elems: int, ses: int, staged: bool) -> Tuple[int, int]:
    if staged:
        if row_elems * ses >= STAGE_BYTES:
            return 1, STAGE_BYTES // ses
        pitch = (row_elems * ses + 15) & ~15
        return max(1, min(rows, STAGE_BYTES // pitch, 1024)), row_elems
    # unstaged elementwise: about 8K elements per tile
    if row_elems >= 8192:
        return 1, 8192
    return max(1, min(rows, 8192 // max(row_elems, 1))), row_elems


class DescriptorEncoder:
    def __init__(self):
        self.rows: List[tuple] = []
        # per-row source byte offsets of gathered slabs, concatenated; a descriptor's
        # ``row_table`` holds 1 + its first index here until the table has a device address
        self.row_offsets: List[int] = []
        # descriptors (by index) whose tiles are fetched with one tiled TMA load each
        self.tensor_map_descs: List[int] = []
        # destination rank of every descriptor (the kernel's CTA groups are cut along these)
        self.desc_dst: List[int] = []
        self._dst_rank = 0
        self.n_tiles = 0
        self.bytes_out = 0
        self.bytes_in = 0

    def add_item(self, item: CopyItem, src: TensorAddr, dst: TensorAddr, scale: Optional[TensorAddr] = None) -> None:
        kind = item.value_op.kind
        self._dst_rank = int(item.dst_rank)
        ses, des = src.dtype.itemsize, dst.dtype.itemsize
        if src.dtype != item.src_dtype:
            raise ValueError(f"{item.src_param}: tensor dtype {src.dtype} differs from planned {item.src_dtype}")
        if dst.dtype != item.dst_dtype:
            raise ValueError(f"{item.dst_name}: destination dtype {dst.dtype} differs from planned {item.dst_dtype}")
        src0 = src.ptr + sum(o * s for o, s in zip(item.src_start, src.strides)) * ses
        dst0 = dst.ptr + sum(o * s for o, s in zip(item.dst_start, dst.strides)) * des
        self.bytes_in += item.numel * ses
        self.bytes_out += item.numel * des
        if kind == "fp8_block":
            self._add_fp8(item, src, dst, scale, src0, dst0)
            return
        if kind == "none" and src.dtype == dst.dtype:
            op = OP_COPY
        elif kind in ("none", "cast"):
            op = OP_CAST
        elif kind == "add":
            op = OP_ADD
        else:
            raise NotImplementedError(f"value op {kind!r} has no kernel form")
        rows, row_elems, s_row, d_row, offsets = collapse_box(item.extent, src.strides, dst.strides)
        if rows == 0:
            return
        for s_off, d_off in offsets:
            self._push(op, src0 + s_off * ses, dst0 + d_off * des, rows, row_elems, s_row * ses, d_row * des,
                       _DT_CODE[src.dtype], _DT_CODE[dst.dtype], aux_f=item.value_op.const if op == OP_ADD else 0.0)

    def _push(self, op, src, dst, rows, row_elems, src_stride, dst_stride, sdt, ddt, aux_ptr=0, aux_stride=0, aux_f=0.0, flags=0,
              tile=None, row_offsets: Optional[Sequence[int]] = None) -> None:
        if op == OP_COPY:  # raw bytes
            row_elems *= _DT_SIZE[sdt]
            sdt = ddt = DT_BYTES
        ses, des = _DT_SIZE[sdt], _DT_SIZE[ddt]
        src_ok = _aligned16(src, row_elems * ses) and (rows == 1 or _aligned16(src_stride))
        row_table = 0
        if row_offsets is not None:
            assert len(row_offsets) == rows
            src_ok = _aligned16(src, row_elems * ses, *row_offsets)
            row_table = 1 + len(self.row_offsets)
            self.row_offsets.extend(int(o) for o in row_offsets)
        dst_ok = _aligned16(dst, row_elems * des) and (rows == 1 or _aligned16(dst_stride))
        staged = src_ok and (dst_ok or op != OP_COPY)
        if op == OP_FP8_BLOCK and sdt not in (DT_BF16, DT_F16):
            staged = False  # a 128x128 fp32 block does not fit one stage
        if tile is None:
            tile_rows, tile_cols = _tile_shape(rows, row_elems, ses, staged)
        else:
            tile_rows, tile_cols = tile
        if staged and (tile_cols * ses) % 16 != 0:
            staged = False
        if staged:
            flags |= FLAG_BULK
        if dst_ok:
            flags |= FLAG_DST_VEC16
        col_tiles = -(-row_elems // tile_cols)
        bands = -(-rows // tile_rows)
        if op == OP_FP8_BLOCK and staged and row_offsets is None:
            self.tensor_map_descs.append(len(self.rows))
        self.desc_dst.append(self._dst_rank)
        self.rows.append(
            (src, dst, rows, row_elems, src_stride, dst_stride, self.n_tiles, aux_ptr, aux_stride, aux_f, op, flags, sdt, ddt,
             tile_rows, tile_cols, col_tiles, 0, row_table, 0)
        )
        self.n_tiles += col_tiles * bands

    def _add_fp8(self, item, src, dst, scale, src0, dst0) -> None:
        if scale is None:
            raise ValueError(f"{item.dst_name}: block fp8 needs the address of {item.scale_name}")
        if len(item.extent) != 2 or src.strides[-1] != 1 or dst.strides[-1] != 1:
            raise ValueError(f"{item.dst_name}: block fp8 needs 2-D row-major slabs")
        if scale.dtype != torch.float32 or scale.strides[-1] != 1:
            raise ValueError(f"{item.scale_name}: scales must be row-major float32")
        rows, cols = item.extent
        aux = scale.ptr + (item.scale_start[0] * scale.strides[0] + item.scale_start[1]) * 4
        flags = FLAG_UE8M0 if item.value_op.ue8m0 else 0
        pitch = src.strides[0] * src.dtype.itemsize
        row_offsets = None
        if item.src_rows is not None:
            # src0 was computed with src_start[0] as row 0; offsets are relative to it
            row_offsets = [0] * rows
            for rel, srow, n in item.src_rows:
                if srow < 0 or srow + n > src.shape[0]:
                    raise ValueError(f"{item.dst_name}: gathered rows [{srow}, {srow + n}) exceed the source tensor")
                for i in range(n):
                    row_offsets[rel + i] = (srow + i - item.src_start[0]) * pitch
        self._push(OP_FP8_BLOCK, src0, dst0, rows, cols, pitch, dst.strides[0],
                   _DT_CODE[src.dtype], DT_FP8_E4M3, aux_ptr=aux, aux_stride=scale.strides[0], flags=flags,
                   tile=(FP8_BLOCK, FP8_BLOCK), row_offsets=row_offsets)
        self.bytes_out += 4 * (-(-rows // FP8_BLOCK)) * (-(-cols // FP8_BLOCK))

    def table(self) -> np.ndarray:
        arr = np.zeros(len(self.rows), dtype=DESC_DTYPE)
        for i, row in enumerate(self.rows):
            arr[i] = row
        return arr


def encode_items(items: Iterable[CopyItem], src_addrs: Dict[Tuple[str, int], TensorAddr],
                 dst_addrs: Dict[int, Dict[str, TensorAddr]]) -> Tuple[np.ndarray, int, DescriptorEncoder]:
    enc = DescriptorEncoder()
    for it in items:
        dst_book = dst_addrs[it.dst_rank]
        scale = dst_book.get(it.scale_name) if it.scale_name else None
        enc.add_item(it, src_addrs[(it.src_param, it.vp_stage)], dst_book[it.dst_name], scale)
    return enc.table(), enc.n_tiles, enc


def mark_bulk_output(table: np.ndarray, desc_dst: Sequence[int], remote_ranks: Iterable[int]) -> int:
    """Let the quantised tiles of destinations across NVLink leave through shared
    memory and bulk-async stores (``FLAG_OUT_BULK``) instead of per-thread
    stores.  An option, off by default: one sender to one receiver it measured
    slower (526 against 631 GB/s of fp8 payload; the second barrier per tile and
    the shorter load lookahead cost more than the store path gains).  Needs staged
    tiles and 16-byte aligned destination rows.  Returns the number of descriptors
    marked."""
    remote = np.isin(np.asarray(desc_dst, dtype=np.int64), np.fromiter(remote_ranks, dtype=np.int64))
    if not len(table) or not remote.any():
        return 0
    need = FLAG_BULK | FLAG_DST_VEC16
    mask = remote & (table["op"] == OP_FP8_BLOCK) & ((table["flags"] & need) == need) & (table["dst_stride"] % 16 == 0)
    table["flags"][mask] |= FLAG_OUT_BULK
    return int(mask.sum())


def table_dst_bytes(table: np.ndarray) -> np.ndarray:
    """Bytes every descriptor writes (payload only)."""
    es = np.array([_DT_SIZE[c] for c in range(5)], dtype=np.int64)
    return table["rows"].astype(np.int64) * table["row_elems"].astype(np.int64) * es[table["dst_dtype"].astype(np.int64)]


def build_cta_plan(table: np.ndarray, n_tiles: int, n_ctas: int, chunk_shift: int, desc_group: Optional[Sequence[int]] = None,
                   group_cost: Optional[Dict[int, float]] = None) -> Tuple[np.ndarray, np.ndarray]:
    """The per-CTA plan (``PLAN_DTYPE``) and the chunk index of the fused kernel.

    Descriptors with the same group id that follow one another form a group; a
    group gets CTAs in proportion to the time its tiles take (at least one) and its
    tiles are dealt to them in round-robin chunks of ``2**chunk_shift`` tiles.  The
    estimate: bytes written, times ``group_cost`` for plain copies (a copy that
    stays in this GPU's memory is several times faster per byte than one across
    NVLink), times one for tiles that are computed on (quantised, cast): those
    take a CTA the same time wherever they go.  (With the copy discount applied to
    quantised tiles, the group of the local destination of a block-fp8 layout got
    a quarter of its share of CTAs and finished three times later than the rest.)  Without group ids, or when the table alternates
    between groups more often than there are CTAs to share out, all CTAs form one
    group over the whole table.  The chunk index holds, group after group, the
    descriptor of every chunk's first tile."""
    begins = table["tile_begin"].astype(np.int64)
    n_desc = int(table.shape[0])
    runs: List[Tuple[int, int, float]] = []  # (tile_begin, tile_end, weight)
    if desc_group is not None and n_desc:
        ids = np.asarray(desc_group, dtype=np.int64)
        assert ids.shape[0] == n_desc, "one group id per descriptor"
        cuts = np.flatnonzero(np.diff(ids)) + 1
        first = np.concatenate(([0], cuts))
        last = np.concatenate((cuts, [n_desc]))
        per_byte = np.array([float((group_cost or {}).get(int(g), 1.0)) for g in ids])
        per_byte[table["op"] != OP_COPY] = 1.0
        # a computed tile reads its source too; count what it moves in and out
        es = np.array([_DT_SIZE[c] for c in range(5)], dtype=np.int64)
        moved = table_dst_bytes(table).astype(np.float64)
        moved[table["op"] != OP_COPY] += (table["rows"].astype(np.int64) * table["row_elems"].astype(np.int64)
                                          * es[table["src_dtype"].astype(np.int64)])[table["op"] != OP_COPY]
        csum = np.concatenate(([0.0], np.cumsum(moved * per_byte)))
        for a, b in zip(first.tolist(), last.tolist()):
            tb, te = int(begins[a]), int(begins[b]) if b < n_desc else int(n_tiles)
            if te > tb:
                runs.append((tb, te, float(csum[b] - csum[a])))
    if not runs or len(runs) > max(1, n_ctas // 2):
        runs = [(0, int(n_tiles), 1.0)]
    # apportion the CTAs: at least one each, the rest by largest remainder
    total = sum(w for _, _, w in runs) or 1.0
    spare = n_ctas - len(runs)
    ideal = [spare * w / total for _, _, w in runs]
    share = [1 + int(x) for x in ideal]
    order = sorted(range(len(runs)), key=lambda g: ideal[g] - int(ideal[g]), reverse=True)
    for g in order[: n_ctas - sum(share)]:
        share[g] += 1
    plan = np.zeros(n_ctas, dtype=PLAN_DTYPE)
    index_parts: List[np.ndarray] = []
    cta = off = 0
    for (tb, te, _), size in zip(runs, share):
        starts = np.arange(tb, te, 1 << chunk_shift, dtype=np.int64)
        index_parts.append((np.searchsorted(begins, starts, side="right") - 1).astype(np.uint32))
        for r in range(size):
            plan[cta] = (tb, te, r, size, off, 0)
            cta += 1
        off += len(starts)
    assert cta == n_ctas
    return plan, np.concatenate(index_parts) if index_parts else np.zeros(0, dtype=np.uint32)


def plan_tile_order(plan: np.ndarray, chunk_shift: int) -> List[int]:
    """Every tile number the CTAs of a plan visit, CTA after CTA, computed the
    way the kernel computes it.  A correct plan yields every tile exactly once."""
    order: List[int] = []
    size = 1 << chunk_shift
    for e in plan:
        tb, te, rank, group = int(e["tile_begin"]), int(e["tile_end"]), int(e["rank"]), int(e["size"])
        n_chunks = -(-(te - tb) // size)
        for chunk in range(rank, n_chunks, group):
            first = tb + chunk * size
            order.extend(range(first, min(first + size, te)))
    return order


# ---- host-side checks ------------------------------------------------------------------------------
class _SpanIndex:
    """``[low, high)`` ranges with an O(log n) "is this range inside one of
    them" query: ranges sorted by start, with the running maximum of their ends
    (the range that attains it starts at or before the query and ends at or after it)."""

    def __init__(self, spans: Sequence[Tuple[int, int]]):
        import bisect

        self._bisect = bisect.bisect_right
        ordered = sorted((int(a), int(b)) for a, b in spans)
        self.starts = [a for a, _ in ordered]
        self.reach: List[int] = []
        best = -1
        for _, b in ordered:
            best = max(best, b)
            self.reach.append(best)

    def contains(self, lo: int, hi: int) -> bool:
        i = self._bisect(self.starts, lo) - 1
        return i >= 0 and self.reach[i] >= hi


def validate_table(table: np.ndarray, n_tiles: int, src_spans: Sequence[Tuple[int, int]],
                   dst_spans: Sequence[Tuple[int, int]], check_overlap: bool = True) -> List[str]:
    """Return every violated rule.  ``src_spans`` / ``dst_spans`` are the
    ``[low, high)`` address ranges of the tensors the table may read / write."""
    problems: List[str] = []
    src_spans, dst_spans = _SpanIndex(src_spans), _SpanIndex(dst_spans)

    def inside(lo: int, hi: int, spans: "_SpanIndex") -> bool:
        return spans.contains(lo, hi)

    expect_begin = 0
    written: List[Tuple[int, int, int]] = []
    for i, d in enumerate(table):
        op, flags = int(d["op"]), int(d["flags"])
        rows, row_elems = int(d["rows"]), int(d["row_elems"])
        ses, des = _DT_SIZE.get(int(d["src_dtype"]), 0), _DT_SIZE.get(int(d["dst_dtype"]), 0)
        tag = f"desc[{i}]"
        if op not in (OP_COPY, OP_CAST, OP_ADD, OP_FP8_BLOCK) or not ses or not des:
            problems.append(f"{tag}: unknown op/dtype")
            continue
        if rows <= 0 or row_elems <= 0:
            problems.append(f"{tag}: empty slab")
            continue
        if int(d["tile_begin"]) != expect_begin:
            problems.append(f"{tag}: tile_begin {int(d['tile_begin'])} != running count {expect_begin}")
        tr, tc, ct = int(d["tile_rows"]), int(d["tile_cols"]), int(d["col_tiles"])
        if tr <= 0 or tc <= 0 or ct != -(-row_elems // tc):
            problems.append(f"{tag}: inconsistent tile geometry")
            continue
        expect_begin += ct * -(-rows // tr)
        s_stride, d_stride = int(d["src_stride"]), int(d["dst_stride"])
        src, dst = int(d["src"]), int(d["dst"])
        if src % ses or dst % des or (rows > 1 and (s_stride % ses or d_stride % des)):
            problems.append(f"{tag}: address or stride not aligned to the element size")
        s_lo, s_hi = src + min(0, (rows - 1) * s_stride), src + max(0, (rows - 1) * s_stride) + row_elems * ses
        d_lo, d_hi = dst + min(0, (rows - 1) * d_stride), dst + max(0, (rows - 1) * d_stride) + row_elems * des
        if int(d["row_table"]) == 0 and not inside(s_lo, s_hi, src_spans):
            problems.append(f"{tag}: reads [{s_lo:#x}, {s_hi:#x}) outside every source tensor")
        if not inside(d_lo, d_hi, dst_spans):
            problems.append(f"{tag}: writes [{d_lo:#x}, {d_hi:#x}) outside every destination tensor")
        if rows > 1 and abs(d_stride) < row_elems * des:
            problems.append(f"{tag}: destination rows overlap each other")
        if flags & FLAG_BULK:
            pitch = (tc * ses + 15) & ~15
            if src % 16 or (rows > 1 and s_stride % 16) or (row_elems * ses) % 16 or (tc * ses) % 16:
                problems.append(f"{tag}: bulk source rule (16-byte address, stride and size) violated")
            if op == OP_COPY and (dst % 16 or (rows > 1 and d_stride % 16)):
                problems.append(f"{tag}: bulk destination rule (16-byte address and stride) violated")
            if tr * pitch > STAGE_BYTES or tr * pitch > MAX_TX_BYTES:
                problems.append(f"{tag}: tile of {tr} x {pitch} bytes exceeds one stage")
        if op == OP_FP8_BLOCK:
            if (tr, tc) != (FP8_BLOCK, FP8_BLOCK):
                problems.append(f"{tag}: fp8 tiles must be {FP8_BLOCK}x{FP8_BLOCK}")
            a_lo = int(d["aux_ptr"])
            a_hi = a_lo + ((-(-rows // FP8_BLOCK) - 1) * int(d["aux_stride"]) + ct) * 4
            if a_lo % 4 or not inside(a_lo, a_hi, dst_spans):
                problems.append(f"{tag}: scale range [{a_lo:#x}, {a_hi:#x}) outside every destination tensor")
        written.append((d_lo, d_hi, i))
    if expect_begin != n_tiles:
        problems.append(f"table describes {expect_begin} tiles, launch says {n_tiles}")
    if check_overlap and len(written) > 1:
        # bounding ranges of strided slabs may interleave legitimately (column
        # slabs of one matrix); only flag ranges whose rows really intersect
        written.sort()
        active: List[Tuple[int, int, int]] = []
        for lo, hi, i in written:
            active = [a for a in active if a[1] > lo]
            for a_lo, a_hi, j in active:
                if _slabs_intersect(table[j], table[i]):
                    problems.append(f"desc[{j}] and desc[{i}] write overlapping destination bytes")
            active.append((lo, hi, i))
    return problems


def _slabs_intersect(a, b) -> bool:
    """Exact test for two destination slabs with equal row stride; different
    strides are compared row by row (bounded), else conservatively by range."""
    def rows_of(d):
        des = _DT_SIZE[int(d["dst_dtype"])]
        return int(d["dst"]), int(d["rows"]), int(d["dst_stride"]), int(d["row_elems"]) * des

    a0, ar, astr, aw = rows_of(a)
    b0, br, bstr, bw = rows_of(b)
    if ar == 1 and br == 1:
        return a0 < b0 + bw and b0 < a0 + aw
    if (astr == bstr or ar == 1 or br == 1) and (astr or bstr):
        stride = astr if ar > 1 else bstr
        if stride > 0 and aw <= stride and bw <= stride:
            # same lattice: compare column windows modulo the stride and row windows
            delta = b0 - a0
            shift, col = divmod(delta, stride)
            hits = []
            if col < aw:  # b's row k starts inside a's row k+shift
                hits.append(shift)
            if col + bw > stride:  # ... and spills into a's next row
                hits.append(shift + 1)
            for sh in hits:
                lo, hi = max(0, sh), min(ar, sh + br)
                if lo < hi:
                    return True
            return False
    if ar * br <= 1 << 16:
        for i in range(ar):
            lo = a0 + i * astr
            for j in range(br):
                lo2 = b0 + j * bstr
                if lo < lo2 + bw and lo2 < lo + aw:
                    return True
        return False
    return True
