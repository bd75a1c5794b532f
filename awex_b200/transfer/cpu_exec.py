"""Reference executor of copy items in plain PyTorch.

It is the oracle for the fused CUDA kernel and the data plane of the CPU
(gloo) backend: the same items, executed with ``copy_`` semantics.  Messages
between processes are flat byte buffers in item order, so that both ends
derive offsets from the published manifest and nothing but payload travels.
The reference states the same semantics in its CPU simulation of a plan
(`awex/tests/test_transfer_plan_cpu_sim.py:94-168`).
"""

from __future__ import annotations

from typing import Dict, Iterable, List, Sequence, Tuple

import torch

from awex_b200.converter.weights_converter import FP8_BLOCK, per_block_cast_to_fp8
from awex_b200.transfer.lowering import CopyItem


def _box(t: torch.Tensor, start: Sequence[int], extent: Sequence[int]) -> torch.Tensor:
    if t.dim() == 0:
        return t
    return t[tuple(slice(s, s + e) for s, e in zip(start, extent))]


def transformed_payload(item: CopyItem, src: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor | None]:
    """(values in destination dtype, block scales or None) for one item."""
    if item.src_rows is not None:
        rows = torch.cat([src.narrow(0, srow, n) for _rel, srow, n in item.src_rows], 0)
        piece = _box(rows, (0,) + tuple(item.src_start[1:]), item.extent)
    else:
        piece = _box(src, item.src_start, item.extent)
    kind = item.value_op.kind
    if kind == "fp8_block":
        q, scale = per_block_cast_to_fp8(piece.contiguous(), item.value_op.ue8m0)
        return q, scale
    if kind == "add":
        # the add is done in fp32 and rounded once to the destination dtype
        return (piece.float() + item.value_op.const).to(item.dst_dtype), None
    if kind in ("none", "cast"):
        return piece.to(item.dst_dtype), None
    raise NotImplementedError(f"value op {kind!r} cannot ride along with a transfer")


def write_payload(views: Dict[str, torch.Tensor], entry: tuple, values: torch.Tensor, scale: torch.Tensor | None) -> None:
    name, start, extent, _dtype, scale_name, scale_start = entry
    _box(views[name], start, extent).copy_(values.view(extent) if values.dim() != len(extent) else values)
    if scale_name is not None:
        blocks = tuple(-(-e // FP8_BLOCK) for e in extent)
        _box(views[scale_name], scale_start, blocks).copy_(scale.view(blocks))


def execute_items(items: Iterable[CopyItem], local_params: Dict[Tuple[str, int], torch.Tensor],
                  views_by_rank: Dict[int, Dict[str, torch.Tensor]]) -> int:
    """Run items whose destinations are addressable in this process.  Returns
    the number of destination bytes written."""
    written = 0
    with torch.no_grad():
        for it in items:
            values, scale = transformed_payload(it, local_params[(it.src_param, it.vp_stage)])
            write_payload(views_by_rank[it.dst_rank], it.manifest_entry(), values, scale)
            written += it.dst_bytes
    return written


# ---- flat messages -------------------------------------------------------------------------------
def entry_nbytes(entry: tuple) -> int:
    _name, _start, extent, dtype, scale_name, _ss = entry
    n = 1
    for e in extent:
        n *= e
    nbytes = n * getattr(torch, dtype.replace("torch.", "")).itemsize
    if scale_name is not None:
        blocks = 1
        for e in extent:
            blocks *= -(-e // FP8_BLOCK)
        nbytes += 4 * blocks
    return nbytes


def pack_message(items: Sequence[CopyItem], local_params: Dict[Tuple[str, int], torch.Tensor]) -> torch.Tensor:
    """Concatenate the payloads of ``items`` (one destination) as bytes."""
    chunks: List[torch.Tensor] = []
    with torch.no_grad():
        for it in items:
            values, scale = transformed_payload(it, local_params[(it.src_param, it.vp_stage)])
            chunks.append(values.contiguous().view(torch.uint8).reshape(-1))
            if scale is not None:
                chunks.append(scale.contiguous().view(torch.uint8).reshape(-1))
    if not chunks:
        return torch.empty(0, dtype=torch.uint8)
    return torch.cat(chunks)


def unpack_message(manifest: Sequence[tuple], message: torch.Tensor, views: Dict[str, torch.Tensor]) -> None:
    pos = 0
    with torch.no_grad():
        for entry in manifest:
            _name, _start, extent, dtype, scale_name, _ss = entry
            torch_dtype = getattr(torch, dtype.replace("torch.", ""))
            n = 1
            for e in extent:
                n *= e
            nbytes = n * torch_dtype.itemsize
            chunk = message[pos : pos + nbytes]
            if chunk.storage_offset() % torch_dtype.itemsize:
                chunk = chunk.clone()  # dtype views need an aligned start
            values = chunk.view(torch_dtype).view(tuple(extent))
            pos += nbytes
            scale = None
            if scale_name is not None:
                blocks = tuple(-(-e // FP8_BLOCK) for e in extent)
                sbytes = 4 * blocks[0] * blocks[1]
                chunk = message[pos : pos + sbytes]
                if chunk.storage_offset() % 4:
                    chunk = chunk.clone()
                scale = chunk.view(torch.float32).view(blocks)
                pos += sbytes
            write_payload(views, entry, values, scale)
    assert pos == message.numel(), f"message has {message.numel()} bytes, manifest describes {pos}"
