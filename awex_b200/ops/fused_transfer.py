"""Python launcher of the fused transfer kernel (``csrc/fused_transfer.cu``).

A :class:`TransferProgram` is one training rank's compiled update: a descriptor
table resident on the device, the flags it must see before writing (one per
destination, raised by the reader when its engine is paused) and the flags it
raises when its writes are complete.  :meth:`TransferProgram.launch` is a single
kernel launch on the current stream; nothing is allocated and nothing
synchronises with the host.

One launch stands where the reference slices and converts every parameter,
builds one send per planned operation and issues them as batched NCCL
point-to-point calls (`awex/transfer/nccl_comm.py:379-447,544-624`,
`awex/writer/nccl_writer.py:198-340`).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from awex_b200.ops import native
from awex_b200.transfer.descriptors import DESC_DTYPE

STATUS_NAMES = {
    0: "ok",
    1: "a destination did not announce readiness in time",
    2: "a staged load did not complete in time",
    3: "a sender's completion flag did not arrive in time",
    4: "a descriptor failed a device-side check",
}


class TransferError(RuntimeError):
    def __init__(self, code: int, detail: Sequence[int]):
        self.code, self.detail = code, tuple(detail)
        super().__init__(f"fused transfer failed: {STATUS_NAMES.get(code, code)} (detail={self.detail})")


def _device_array(values, dtype, device) -> torch.Tensor:
    return torch.from_numpy(np.asarray(values, dtype=dtype).view(np.uint8).copy()).to(device)


def _max_chunk_shift(table: np.ndarray, n_tiles: int) -> int:
    """log2 of the largest chunk in tiles.  Measured on B200: tables of plain
    copies run fastest with chunks of 4 tiles (the depth of the load pipeline),
    tables dominated by quantised blocks with 16.  ``AWEX_XFER_CHUNK_MB``
    overrides the choice with a chunk size in MiB of staged source data.  (The
    reference's ``AWEX_CHUNK_MB`` bounds staging memory of its co-located
    exchange; this kernel stages nothing in device memory, so that knob only
    acts on the message transport.)"""
    import os

    from awex_b200.transfer.descriptors import OP_FP8_BLOCK, STAGE_BYTES

    override = os.environ.get("AWEX_XFER_CHUNK_MB")
    if override:
        try:
            tiles = max(1, int(float(override) * 1024 * 1024) // STAGE_BYTES)
            return min(tiles.bit_length() - 1, 12)
        except ValueError:
            pass
    begins = table["tile_begin"].astype(np.int64)
    counts = np.diff(np.append(begins, n_tiles))
    is_fp8 = table["op"] == OP_FP8_BLOCK
    fp8_tiles = int(counts[is_fp8].sum())
    if 2 * fp8_tiles <= n_tiles:
        return 2
    # small slabs (an expert's shard: 64 blocks): a chunk per slab, so that a CTA stays with one tensor map
    # (slabs of 192 x 4096 ran at 2.50 TB/s with chunks of 16 blocks and at 2.87 TB/s with chunks of 64)
    return 6 if float(np.median(counts[is_fp8])) <= 256 else 4


def _pick_variant(table: np.ndarray, n_tiles: int) -> int:
    """0: one 512-thread CTA per SM, deep ring (tables of long contiguous
    copies); 1: two 256-thread CTAs per SM (tables dominated by tiles all warps
    compute on, or by strided copies of short rows, where a single CTA per SM
    leaves the copy engine idle between its many small requests: 2 KiB rows ran
    at 0.63 of the copy peak with one CTA per SM and 0.85 with two).
    ``AWEX_XFER_VARIANT`` overrides."""
    import os

    from awex_b200.transfer.descriptors import OP_COPY

    forced = os.environ.get("AWEX_XFER_VARIANT")
    if forced in ("0", "1", "2"):
        return int(forced)
    if not len(table) or not n_tiles:
        return 0
    begins = table["tile_begin"].astype(np.int64)
    counts = np.diff(np.append(begins, n_tiles))
    is_copy = table["op"] == OP_COPY
    short_rows = is_copy & (table["tile_rows"] > 1) & (table["row_elems"] <= SHORT_ROW_BYTES)  # copies count bytes
    slow = int(counts[~is_copy].sum()) + int(counts[short_rows].sum())
    return 1 if 2 * slow > n_tiles else 0


SHORT_ROW_BYTES = 4096


class StatusWord:
    """Four int32 on the device: code, detail0..2.  Kernels only ever move it
    from OK to an error; the host reads it when it wants a verdict."""

    def __init__(self, device):
        self.t = torch.zeros(4, dtype=torch.int32, device=device)

    @property
    def ptr(self) -> int:
        return self.t.data_ptr()

    def reset(self) -> None:
        self.t.zero_()

    def read(self) -> List[int]:
        return self.t.tolist()

    def raise_if_failed(self) -> None:
        code, *detail = self.read()
        if code != 0:
            self.reset()
            raise TransferError(code, detail)


class FlagPad:
    """``n`` 64-bit flags in this GPU's memory, written by peers."""

    def __init__(self, n_slots: int, device):
        self.n = n_slots
        self.t = torch.zeros(max(n_slots, 1), dtype=torch.int64, device=device)

    @property
    def ptr(self) -> int:
        return self.t.data_ptr()

    def slot_addr(self, slot: int, base: Optional[int] = None) -> int:
        return (self.ptr if base is None else base) + 8 * slot


class TransferProgram:
    def __init__(self, table: np.ndarray, n_tiles: int, device, ready_pad: Optional[FlagPad] = None,
                 ready_slots: Sequence[int] = (), done_flag_addrs: Sequence[int] = (), timeout_ms: int = 2000,
                 grid: int = 0, row_offsets: Sequence[int] = (), tensor_map_descs: Sequence[int] = (), encoder=None,
                 interleave: bool = True, variant: Optional[int] = None, desc_group: Optional[Sequence[int]] = None,
                 group_cost: Optional[Dict[int, float]] = None, _resolved: bool = False, _status: Optional["StatusWord"] = None):
        """``interleave``: deal tiles to CTAs in round-robin chunks instead of one
        contiguous range per CTA.  ``desc_group`` (one id per descriptor, e.g. the
        destination rank; taken from ``encoder`` when it is given and this is
        ``True``) makes one group of CTAs per run of equal ids, sized by the bytes it
        writes times ``group_cost[id]`` (relative time per byte, default 1).

        When no launch shape is forced and a worthwhile part of the table is
        quantised blocks fetched by tiled TMA loads, that part is split off and run
        by the lean block-fp8 kernel (``self.lean``, launched first on the same
        stream); the general kernel then runs the rest and raises the completion
        flags.  ``AWEX_XFER_LEAN_FP8=0`` keeps everything in the general kernel."""
        if encoder is not None:  # side tables produced while encoding
            row_offsets, tensor_map_descs = encoder.row_offsets, encoder.tensor_map_descs
            if desc_group is True:
                desc_group = encoder.desc_dst
        if desc_group is True:
            desc_group = None
        if table.dtype != DESC_DTYPE:
            raise TypeError("descriptor table has the wrong dtype")
        self.lib = native.load()
        assert self.lib.awex_xfer_desc_size() == DESC_DTYPE.itemsize, "descriptor layout mismatch between Python and CUDA"
        self.device = torch.device(device)
        self.n_desc = int(table.shape[0])
        self.n_tiles = int(n_tiles)
        self.row_table_dev = None
        self.lean: Optional["TransferProgram"] = None
        if _resolved:
            row_offsets, tensor_map_descs = (), ()
        if len(row_offsets):
            # descriptors refer to the gathered-row offsets by index + 1; give them addresses
            self.row_table_dev = _device_array(list(row_offsets), np.int64, self.device)
            table = table.copy()
            has = table["row_table"] != 0
            table["row_table"][has] = self.row_table_dev.data_ptr() + (table["row_table"][has] - 1) * 8
        elif not _resolved and self.n_desc and bool((table["row_table"] != 0).any()):
            raise ValueError("descriptor table uses gathered rows but no row offsets were given")
        self.tensor_maps_dev = None
        if len(tensor_map_descs):
            table = self._attach_tensor_maps(table, tensor_map_descs)
        self.status = _status if _status is not None else StatusWord(self.device)
        self.total_tiles = self.n_tiles
        if variant is None and not _resolved:
            table, desc_group = self._split_off_lean_part(table, desc_group, group_cost, ready_pad, ready_slots, timeout_ms, interleave)
        self.table_host = table
        self.table_dev = torch.from_numpy(table.view(np.uint8).reshape(-1).copy()).to(self.device) if self.n_desc else torch.empty(0, dtype=torch.uint8, device=self.device)
        self.ready_pad = ready_pad
        self.ready_slots = _device_array(list(ready_slots), np.uint32, self.device) if len(ready_slots) else None
        self.n_ready = len(ready_slots)
        self.done_flags = _device_array(list(done_flag_addrs), np.uint64, self.device) if len(done_flag_addrs) else None
        self.n_done = len(done_flag_addrs)
        # chunk index for the round-robin deal of tiles to CTAs: chunks of up to 16
        # tiles, smaller when the table is short so that every CTA still gets work
        self.variant = _pick_variant(table, self.n_tiles) if variant is None else int(variant)
        self.chunk_desc, self.chunk_shift, self.cta_plan, self.plan_host = None, 0, None, None
        if interleave and self.n_desc and self.n_tiles:
            from awex_b200.transfer.descriptors import build_cta_plan

            per_sm = 3 if self.variant == 3 else self.variant + 1
            ctas = grid if grid > 0 else torch.cuda.get_device_properties(self.device).multi_processor_count * per_sm
            ctas = max(1, min(ctas, self.n_tiles))
            shift = _max_chunk_shift(table, self.n_tiles)
            while shift > 0 and (self.n_tiles >> shift) < 4 * ctas:
                shift -= 1
            self.plan_host, index = build_cta_plan(table, self.n_tiles, ctas, shift, desc_group, group_cost)
            self.cta_plan = torch.from_numpy(self.plan_host.view(np.uint8).reshape(-1).copy()).to(self.device)
            self.chunk_desc = _device_array(index, np.uint32, self.device)
            self.chunk_shift = shift
            grid = ctas
        self.counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.timeout_ns = int(timeout_ms) * 1_000_000
        self.grid = grid
        self.launches = 0

    def _split_off_lean_part(self, table, desc_group, group_cost, ready_pad, ready_slots, timeout_ms, interleave):
        """Move the descriptors the lean block-fp8 kernel can run (staged
        ``OP_FP8_BLOCK`` slabs of a 2-byte type with a tensor map) into a program of
        their own when they are worth a launch; returns what stays here."""
        import os

        from awex_b200.transfer.descriptors import DT_BF16, DT_F16, FLAG_BULK, FLAG_OUT_BULK, OP_FP8_BLOCK

        if os.environ.get("AWEX_XFER_LEAN_FP8", "1") == "0" or os.environ.get("AWEX_XFER_VARIANT") or not self.n_desc:
            return table, desc_group
        lean = ((table["op"] == OP_FP8_BLOCK) & (table["tensor_map"] != 0) & ((table["flags"] & FLAG_BULK) != 0)
                & ((table["flags"] & FLAG_OUT_BULK) == 0) & np.isin(table["src_dtype"], (DT_BF16, DT_F16)))
        begins = table["tile_begin"].astype(np.int64)
        counts = np.diff(np.append(begins, self.n_tiles))
        lean_tiles = int(counts[lean].sum())
        if lean_tiles < 4096 and 2 * lean_tiles < self.n_tiles:
            return table, desc_group

        def part(mask):
            sub = table[mask].copy()
            sub_counts = counts[mask]
            sub["tile_begin"] = np.concatenate(([0], np.cumsum(sub_counts)[:-1])) if len(sub) else sub["tile_begin"]
            groups = None if desc_group is None else [g for g, m in zip(desc_group, mask) if m]
            return sub, int(sub_counts.sum()), groups

        lean_table, lean_n, lean_groups = part(lean)
        rest_table, rest_n, rest_groups = part(~lean)
        self.lean = TransferProgram(lean_table, lean_n, self.device, ready_pad=ready_pad, ready_slots=ready_slots, done_flag_addrs=(),
                                    timeout_ms=timeout_ms, interleave=interleave, variant=3, desc_group=lean_groups, group_cost=group_cost,
                                    _resolved=True, _status=self.status)
        self.n_desc, self.n_tiles = int(rest_table.shape[0]), rest_n
        return rest_table, rest_groups

    def _attach_tensor_maps(self, table: np.ndarray, indices: Sequence[int]) -> np.ndarray:
        """Encode one CUtensorMap per listed descriptor (its tiles are then fetched
        with a single tiled TMA load each) and store their device addresses."""
        import ctypes

        from awex_b200.transfer.descriptors import _DT_SIZE

        table = table.copy()
        maps = np.zeros((len(indices), 128), dtype=np.uint8)
        for slot, i in enumerate(indices):
            d = table[i]
            es = _DT_SIZE[int(d["src_dtype"])]
            code = self.lib.awex_encode_tensor_map_2d(
                maps[slot].ctypes.data_as(ctypes.c_void_p), es, int(d["src"]), int(d["row_elems"]), int(d["rows"]),
                int(d["src_stride"]) if int(d["rows"]) > 1 else int(d["row_elems"]) * es, int(d["tile_cols"]), int(d["tile_rows"]),
            )
            if code != 0:
                raise RuntimeError(f"cuTensorMapEncodeTiled failed for descriptor {i} (code {code})")
        self.tensor_maps_dev = torch.from_numpy(maps.reshape(-1)).to(self.device)
        base = self.tensor_maps_dev.data_ptr()
        assert base % 128 == 0
        for slot, i in enumerate(indices):
            table["tensor_map"][i] = base + 128 * slot
        return table

    def check(self) -> None:
        """Raise :class:`TransferError` if the last launches reported a failure.
        A failed launch may have counted only some of its CTAs in, so the arrival
        counter is cleared together with the status: the program can be launched
        again (a retried update writes the same bytes to the same addresses)."""
        try:
            self.status.raise_if_failed()
        except TransferError:
            self.counter.zero_()
            if self.lean is not None:
                self.lean.counter.zero_()
            raise

    def launch(self, epoch: int, stream_ptr: Optional[int] = None) -> None:
        stream = native.current_stream_ptr() if stream_ptr is None else stream_ptr
        if self.lean is not None:
            self.lean.launch(epoch, stream)  # same stream: finished before the launch below raises the completion flags
        code = self.lib.awex_launch_fused_transfer(
            self.table_dev.data_ptr() if self.n_desc else None, self.n_desc, self.n_tiles, epoch, self.timeout_ns,
            self.ready_pad.ptr if (self.ready_pad is not None and self.n_ready) else None,
            self.ready_slots.data_ptr() if self.n_ready else None, self.n_ready,
            self.done_flags.data_ptr() if self.n_done else None, self.n_done,
            self.counter.data_ptr(), self.status.ptr, self.grid, stream,
            self.chunk_desc.data_ptr() if self.chunk_desc is not None else None, self.chunk_shift, self.variant,
            self.cta_plan.data_ptr() if self.cta_plan is not None else None,
        )
        native.check(code, "fused_transfer launch")
        self.launches += 1


class FlagWaiter:
    """Receiver side: one tiny kernel that returns when every listed slot of the
    local pad has reached ``epoch`` or the deadline passed (status says which)."""

    def __init__(self, pad: FlagPad, slots: Sequence[int], device, timeout_ms: int = 2000):
        self.lib = native.load()
        self.pad = pad
        self.device = torch.device(device)
        self.n = len(slots)
        self.slots = _device_array(list(slots), np.uint32, self.device) if self.n else None
        self.status = StatusWord(self.device)
        self.timeout_ns = int(timeout_ms) * 1_000_000
        self.launches = 0

    def launch(self, epoch: int, stream_ptr: Optional[int] = None) -> None:
        if not self.n:
            return
        stream = native.current_stream_ptr() if stream_ptr is None else stream_ptr
        code = self.lib.awex_launch_wait_flags(self.pad.ptr, self.slots.data_ptr(), self.n, epoch, self.timeout_ns, self.status.ptr, stream)
        native.check(code, "wait_flags launch")
        self.launches += 1


class FlagPoster:
    """Raise ``epoch`` at a fixed list of (local or peer-mapped) flag addresses."""

    def __init__(self, addrs: Sequence[int], device):
        self.lib = native.load()
        self.device = torch.device(device)
        self.n = len(addrs)
        self.addrs = _device_array(list(addrs), np.uint64, self.device) if self.n else None
        self.launches = 0

    def launch(self, epoch: int, stream_ptr: Optional[int] = None) -> None:
        if not self.n:
            return
        stream = native.current_stream_ptr() if stream_ptr is None else stream_ptr
        native.check(self.lib.awex_launch_post_flags(self.addrs.data_ptr(), self.n, epoch, stream), "post_flags launch")
        self.launches += 1
