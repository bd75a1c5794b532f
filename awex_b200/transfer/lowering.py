"""Lower a transfer plan plus the converter's row maps into copy items.

The planner speaks in *canonical* tensors: "send rows [a, b) of the training
rank's converted tensor".  A converted tensor is never materialised here;
:class:`awex_b200.converter.rows.Rows` says which physical training tensor and
which of its rows each canonical row is.  Lowering intersects every planned
box with those row runs and emits :class:`CopyItem` objects — plain N-d box
copies from a *local training parameter* to a *named destination view* on an
inference rank, with an optional value transform (cast, constant add, block
fp8 quantisation).

Re-homing: when a canonical tensor draws rows from tensor-parallel peers (the
default fused-QKV regroup does), the plan's sender for a box may not hold the
bytes.  Every training rank therefore also walks the plans of its TP peers for
such tensors and keeps the pieces whose rows it physically owns.  The bytes
that reach each destination element are exactly those the planned sender
would have sent after an all-gather, so results are bit-identical to the
gather-then-send pipeline of the reference (`awex/writer/nccl_writer.py:197-304`,
`awex/converter/mcore_converter.py:1040-1052`) without the collective.

Copy items are the common currency of all data planes: the CPU executor
(:mod:`awex_b200.transfer.cpu_exec`) runs them with ``copy_``; the fused CUDA
path encodes them into flat descriptors (:mod:`awex_b200.transfer.descriptors`).
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from awex_b200 import logging
from awex_b200.converter.rows import IDENTITY, Rows, TensorSpec, ValueOp
from awex_b200.converter.weights_converter import FP8_BLOCK, SCALE_SUFFIX
from awex_b200.meta.weight_meta import ParameterMeta, ParameterShardMeta
from awex_b200.sharding.rank_info import RankInfo
from awex_b200.transfer.transfer_plan import CommunicationOperation, TransferPlanBuilder

logger = logging.getLogger(__name__)


@dataclass(slots=True)
class CopyItem:
    """Copy ``extent`` elements starting at ``src_start`` of local training
    parameter ``src_param`` (chunk ``vp_stage``) to ``dst_start`` of the view
    named ``dst_name`` on inference transfer rank ``dst_rank``."""

    src_param: str
    vp_stage: int
    src_start: Tuple[int, ...]
    extent: Tuple[int, ...]
    dst_rank: int
    dst_name: str
    dst_start: Tuple[int, ...]
    src_dtype: torch.dtype
    dst_dtype: torch.dtype
    value_op: ValueOp = IDENTITY
    # fp8_block only: destination of the block scales and the block coordinates
    # of this item's origin inside that scale tensor
    scale_name: Optional[str] = None
    scale_start: Tuple[int, int] = (0, 0)
    # optional gather of dim-0 rows: ((row relative to the item, source row, n), ...)
    # replacing the contiguous run that starts at src_start[0]
    src_rows: Optional[Tuple[Tuple[int, int, int], ...]] = None

    @property
    def numel(self) -> int:
        n = 1
        for e in self.extent:
            n *= e
        return n

    @property
    def dst_bytes(self) -> int:
        return self.numel * self.dst_dtype.itemsize

    def manifest_entry(self) -> tuple:
        return (self.dst_name, self.dst_start, self.extent, str(self.dst_dtype), self.scale_name, self.scale_start)


@dataclass
class LocalParam:
    name: str
    vp_stage: int
    shape: Tuple[int, ...]
    dtype: torch.dtype


# Value operations that need a whole canonical tensor at once (a reduction over
# it) cannot ride along tile by tile.  Their result is kept in a persistent
# sender-side buffer that is refreshed before every update and sent from there
# with plain copies.
WHOLE_TENSOR_OPS = ("l2norm_dim0",)
DERIVED_PREFIX = "__derived__/"


@dataclass
class DerivedTensor:
    """A sender-side tensor computed from local parameters before each update:
    ``value_op(rows.gather(local))`` of one canonical tensor, addressed by items
    as local source ``key`` in canonical coordinates."""

    key: Tuple[str, int]  # (DERIVED_PREFIX + canonical name, vp_stage)
    spec: TensorSpec
    tp_rank: int
    # rows of training TP peers are needed (a collective over the training TP group)
    gathers: bool = False

    def compute(self, local: Dict[Tuple[str, int], torch.Tensor], gather_fn: Optional[Callable] = None) -> torch.Tensor:
        shards: Dict[str, Sequence[torch.Tensor]] = {}
        if self.gathers:
            # every TP rank gathers every source tensor, in one order, whether or not it uses all of them
            if gather_fn is None:
                raise RuntimeError(f"{self.key[0]} draws rows from training TP peers; a gather function is needed")
            for pname in sorted({src[0] for src in self.spec.rows.sources()}):
                shards[pname] = gather_fn(pname, self.key[1])

        def fetch(src):
            pname, tp_rank = src
            if tp_rank == self.tp_rank:
                return local[(pname, self.key[1])]
            if pname not in shards or tp_rank >= len(shards[pname]):
                raise RuntimeError(f"{self.key[0]}: rows of training TP rank {tp_rank} are not held here")
            return shards[pname][tp_rank]

        value = self.spec.rows.gather(fetch)
        return self.spec.value_op.apply(value) if self.spec.value_op.kind in WHOLE_TENSOR_OPS else value

    def compute_into(self, buffer: Optional[torch.Tensor], local: Dict[Tuple[str, int], torch.Tensor],
                     gather_fn: Optional[Callable] = None) -> Optional[torch.Tensor]:
        """Refresh ``buffer`` in place with the device kernel where there is one
        (column normalisation of a 2-D CUDA tensor: no temporary of the tensor's
        size); returns ``None`` when the general path must be taken."""
        if buffer is None or self.gathers or self.spec.value_op.kind != "l2norm_dim0":
            return None
        value = self.spec.rows.gather(lambda src: local[(src[0], self.key[1])])
        if not value.is_cuda or value.dim() != 2 or value.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            return None
        from awex_b200.ops.normalize import col_l2_normalize

        return col_l2_normalize(value, out=buffer, eps=1e-7)


def refresh_derived(derived: Iterable[DerivedTensor], local: Dict[Tuple[str, int], torch.Tensor],
                    gather_fn: Optional[Callable] = None) -> int:
    """Recompute every derived tensor into its buffer in ``local`` (allocated on
    first use, next to the parameters it comes from; never reallocated, so
    descriptor tables that hold its address stay valid).  ``gather_fn(name,
    vp_stage)`` returns the training TP group's shards of a local parameter in TP
    rank order; it is a collective, which every rank of the group reaches in the
    same order because derived tensors are refreshed sorted by name.  Returns the
    number of tensors refreshed."""
    n = 0
    with torch.no_grad():
        for d in sorted(derived, key=lambda d: d.key):
            if d.compute_into(local.get(d.key), local, gather_fn) is not None:
                n += 1
                continue
            value = d.compute(local, gather_fn)
            if d.key not in local:
                local[d.key] = torch.empty_like(value, memory_format=torch.contiguous_format)
            local[d.key].copy_(value)
            n += 1
    return n


def _tp_peers(my: RankInfo, all_ranks: Sequence[RankInfo]) -> List[RankInfo]:
    """Training ranks that hold the other TP shards of what ``my`` holds."""
    if my.tp_size <= 1:
        return [my]
    peers = [
        r for r in all_ranks
        if (r.pp_rank, r.dp_rank, r.cp_rank) == (my.pp_rank, my.dp_rank, my.cp_rank) and r.tp_size == my.tp_size
    ]
    if len({r.tp_rank for r in peers}) != my.tp_size or len(peers) != my.tp_size:
        # EP-style layouts can give several ranks per (pp, dp, cp, tp); keep the
        # ones that also share the expert coordinates, always including ``my``
        peers = [r for r in peers if (r.ep_rank, r.ep_tp_rank) == (my.ep_rank, my.ep_tp_rank) or r.global_rank == my.global_rank]
        by_tp: Dict[int, RankInfo] = {}
        for r in sorted(peers, key=lambda x: x.global_rank != my.global_rank):
            by_tp.setdefault(r.tp_rank, r)
        peers = list(by_tp.values())
    return sorted(peers, key=lambda r: r.tp_rank)


class SendProgramCompiler:
    """Builds the list of :class:`CopyItem` one training rank executes per update."""

    def __init__(
        self,
        rank_info: RankInfo,
        all_train_ranks: Sequence[RankInfo],
        converter_factory: Callable[[RankInfo], object],
        local_params: Sequence[LocalParam],
        infer_meta: Sequence[ParameterMeta],
        train_meta: Sequence[ParameterMeta],
        builder: TransferPlanBuilder,
    ):
        self.rank_info = rank_info
        self.peers = _tp_peers(rank_info, all_train_ranks)
        self.converter_factory = converter_factory
        self.local_params = list(local_params)
        self.infer_meta = {m.name: m for m in infer_meta}
        self.train_meta = {m.name: m for m in train_meta}
        self.infer_meta_list = list(infer_meta)
        self.train_meta_list = list(train_meta)
        self.builder = builder
        self.my_transfer_rank = rank_info.global_rank + builder.infer_world_size
        self._param_by_key = {(p.name, p.vp_stage): p for p in self.local_params}
        # filled by compile(): tensors the sender must compute before each update
        self.derived: Dict[Tuple[str, int], DerivedTensor] = {}
        # canonical names whose quantisation blocks mix rows of several training TP ranks: their
        # owner gathers the rows before each update instead of every rank sending its own
        self.gathered_names: set = set()

    def _names_needing_gather(self, all_specs: Dict[int, Dict[str, Tuple[TensorSpec, LocalParam]]]) -> set:
        """Block-quantised tensors with a planned box whose rows are held by more
        than one training TP rank.  Every rank of the TP group computes this from
        the same peers' plans, so the whole group agrees."""
        names = set()
        for sender in self.peers:
            virtual_rank = sender.global_rank + self.builder.infer_world_size
            for n, (spec, _lp) in all_specs[sender.global_rank].items():
                if n in names or spec.rows is None or spec.value_op.kind != "fp8_block" or spec.scale_of is not None:
                    continue
                if len({src[1] for src in spec.rows.sources()}) < 2:
                    continue
                if n not in self.train_meta or n not in self.infer_meta or n in self.builder.skip_names:
                    continue
                for op in self.builder._build_parameter_communication_plan(
                    n, self.infer_meta[n], self.train_meta[n], global_transfer_rank=virtual_rank
                ):
                    if op.send_rank != virtual_rank:
                        continue
                    owners = {src[1] for _, src, _, _ in spec.rows.segments(op.train_slices[0].start, op.overlap_shape[0])}
                    if len(owners) > 1:
                        names.add(n)
                        break
        return names

    # ---- symbolic conversion for one (possibly virtual) sender ----------------------------
    def _specs_for(self, sender: RankInfo) -> Dict[str, Tuple[TensorSpec, LocalParam]]:
        converter = self.converter_factory(sender)
        tied = bool(getattr(converter.hf_config, "tie_word_embeddings", False))
        out: Dict[str, Tuple[TensorSpec, LocalParam]] = {}
        for lp in self.local_params:
            for spec in converter.plan_param(lp.name, lp.shape, lp.dtype, vp_stage=lp.vp_stage):
                out[spec.name] = (spec, lp)
        if tied and sender.pp_rank == sender.pp_size - 1 and "lm_head.weight" not in out and "model.embed_tokens.weight" in out:
            spec, lp = out["model.embed_tokens.weight"]
            out["lm_head.weight"] = (dataclasses.replace(spec, name="lm_head.weight"), lp)
        return out

    def compile(self) -> List[CopyItem]:
        my_tp = self.rank_info.tp_rank
        items: List[CopyItem] = []
        own_plan = self.builder.build_local_transfer_plan(self.infer_meta_list, self.train_meta_list, self.my_transfer_rank)
        all_specs = {sender.global_rank: self._specs_for(sender) for sender in self.peers}
        self.gathered_names = self._names_needing_gather(all_specs) if len(self.peers) > 1 else set()
        for sender in self.peers:
            specs = all_specs[sender.global_rank]
            is_me = sender.global_rank == self.rank_info.global_rank
            if is_me:
                ops = own_plan.all_operations()
            else:
                # only tensors that draw rows from this rank need the peer's plan
                names = [
                    n for n, (spec, _) in specs.items()
                    if spec.rows is not None and any(src[1] == my_tp for src in spec.rows.sources() if isinstance(src, tuple) and src[0] != "__scale__")
                    and n in self.train_meta and n in self.infer_meta and n not in self.builder.skip_names
                    and n not in self.gathered_names  # the peer sends those itself, from gathered rows
                ]
                virtual_rank = sender.global_rank + self.builder.infer_world_size
                ops = []
                for n in sorted(names):
                    ops.extend(
                        op for op in self.builder._build_parameter_communication_plan(
                            n, self.infer_meta[n], self.train_meta[n], global_transfer_rank=virtual_rank
                        ) if op.send_rank == virtual_rank
                    )
                ops.sort(key=lambda op: (op.recv_rank, op.send_shard_meta.name, op.send_offset, op.recv_offset))
            for op in ops:
                name = op.send_shard_meta.name
                if name not in specs:
                    if is_me:
                        raise KeyError(f"plan asks rank {self.my_transfer_rank} for {name!r}, which its model does not produce")
                    continue
                items.extend(self._lower_op(op, *specs[name], my_tp))
        items.sort(key=lambda it: (it.dst_rank, it.dst_name, it.dst_start, it.src_param, it.src_start))
        return items

    @staticmethod
    def _place_fp8_item(item: CopyItem, spec: TensorSpec, op: CommunicationOperation) -> None:
        """Check that a block-quantised item covers whole blocks of the destination
        shard and point it at its place in the scale tensor."""
        if len(item.extent) != 2:
            raise ValueError(f"{spec.name}: block fp8 needs a 2-D tensor, got extent {item.extent}")
        if item.dst_start[0] % FP8_BLOCK or item.dst_start[1] % FP8_BLOCK:
            raise ValueError(
                f"{spec.name}: a piece starting at {item.dst_start} of the destination shard does not start on a "
                f"{FP8_BLOCK}x{FP8_BLOCK} block; its block would mix rows of several senders"
            )
        shard = op.recv_shard_meta.shape
        for d in (0, 1):
            end = item.dst_start[d] + item.extent[d]
            if end % FP8_BLOCK and end != shard[d]:
                raise ValueError(f"{spec.name}: piece ends inside a block at {end} (dim {d}, shard extent {shard[d]})")
        item.scale_name = spec.name + SCALE_SUFFIX
        item.scale_start = (item.dst_start[0] // FP8_BLOCK, item.dst_start[1] // FP8_BLOCK)

    # ---- one planned box -> copy items ----------------------------------------------------------
    def _lower_op(self, op: CommunicationOperation, spec: TensorSpec, lp: LocalParam, my_tp: int) -> List[CopyItem]:
        if spec.scale_of is not None:
            return []  # scales are produced together with their weight
        dst_dtype = op.recv_shard_meta.dtype
        if spec.rows is None:  # 0-d
            return [CopyItem(lp.name, lp.vp_stage, (), (), op.recv_rank, spec.name, (), spec.src_dtype, dst_dtype, spec.value_op)]
        row0 = op.train_slices[0].start
        n_rows = op.overlap_shape[0]
        tail_src = tuple(s.start for s in op.train_slices[1:])
        tail_dst = tuple(s.start for s in op.inf_slices[1:])
        tail_ext = tuple(op.overlap_shape[1:])
        dst_row0 = op.inf_slices[0].start
        out: List[CopyItem] = []
        if spec.value_op.kind in WHOLE_TENSOR_OPS or spec.name in self.gathered_names:
            gathers = spec.name in self.gathered_names
            owners = {src[1] for src in spec.rows.sources()}
            if owners != {my_tp} and not gathers:
                if my_tp not in owners:
                    return []
                raise NotImplementedError(
                    f"{spec.name}: {spec.value_op.kind} needs the whole tensor on one rank, but its rows come from "
                    f"training TP ranks {sorted(owners)}"
                )
            key = (DERIVED_PREFIX + spec.name, lp.vp_stage)
            self.derived.setdefault(key, DerivedTensor(key, spec, my_tp, gathers))
            whole = spec.value_op.kind in WHOLE_TENSOR_OPS
            item = CopyItem(
                src_param=key[0], vp_stage=key[1], src_start=(row0,) + tail_src, extent=(n_rows,) + tail_ext,
                dst_rank=op.recv_rank, dst_name=spec.name, dst_start=(dst_row0,) + tail_dst,
                src_dtype=spec.value_op.out_dtype(spec.src_dtype) if whole else spec.src_dtype, dst_dtype=dst_dtype,
                value_op=IDENTITY if whole else spec.value_op,
            )
            if item.value_op.kind == "fp8_block":
                self._place_fp8_item(item, spec, op)
            return [item]
        segments = spec.rows.segments(row0, n_rows)
        if spec.value_op.kind == "fp8_block":
            # a quantisation block needs all of its rows at once: keep the box whole
            # and gather its rows, which must all be held by this rank
            owners = {src[1] for _, src, _, _ in segments}
            if owners != {my_tp}:
                if my_tp not in owners:
                    return []
                raise NotImplementedError(
                    f"{spec.name}: a block-quantised box draws rows from several training TP ranks {sorted(owners)}; "
                    "quantising it needs those rows on one rank"
                )
            names = {src[0] for _, src, _, _ in segments}
            if len(names) != 1:
                raise NotImplementedError(f"{spec.name}: a block-quantised box draws rows from several tensors {sorted(names)}")
            whole_blocks = all(rel % FP8_BLOCK == 0 for rel, _, _, _ in segments) and all(n % FP8_BLOCK == 0 for _, _, _, n in segments[:-1])
            if len(segments) > 1 and whole_blocks:
                # every contiguous source run covers whole quantisation blocks of the destination (de-interleaved
                # Q / K / V with head sizes that are multiples of the block): one plain slab per run, which the
                # kernel fetches with one tiled load per tile instead of one copy per gathered row
                segments = [(rel, src, src_row, n, None) for rel, src, src_row, n in segments]
            else:
                segments = [(0, segments[0][1], segments[0][2], n_rows, tuple((rel, srow, n) for rel, _, srow, n in segments))]
        else:
            segments = [(rel, src, src_row, n, None) for rel, src, src_row, n in segments]
        for rel, src, src_row, n, gather in segments:
            pname, tp_rank = src
            if tp_rank != my_tp:
                continue  # a TP peer owns these rows and sends them itself
            lp_src = lp if pname == lp.name else self._param_by_key[(pname, lp.vp_stage)]
            item = CopyItem(
                src_param=lp_src.name, vp_stage=lp_src.vp_stage, src_start=(src_row,) + tail_src,
                extent=(n,) + tail_ext, dst_rank=op.recv_rank, dst_name=spec.name,
                dst_start=(dst_row0 + rel,) + tail_dst, src_dtype=spec.src_dtype, dst_dtype=dst_dtype,
                value_op=spec.value_op,
            )
            if gather is not None and len(gather) > 1:
                item.src_rows = gather
            if spec.value_op.kind == "fp8_block":
                self._place_fp8_item(item, spec, op)
            out.append(item)
        return out


# ---- re-ordering one sender's work across its destinations ------------------------------------------------
def split_item_rows(item: CopyItem, max_rows: int) -> List[CopyItem]:
    """Cut ``item`` along dimension 0 into pieces of at most ``max_rows`` rows that
    together do exactly what ``item`` does.  Block-quantised items are cut on
    quantisation-block boundaries (``max_rows`` is rounded down to a multiple of
    the block, at least one block), and their place in the scale tensor moves
    along; gathered row lists are cut with the rows they cover."""
    if not item.extent or max_rows <= 0:
        return [item]
    if item.value_op.kind == "fp8_block":
        max_rows = max(FP8_BLOCK, max_rows - max_rows % FP8_BLOCK)
    rows = item.extent[0]
    if rows <= max_rows:
        return [item]
    pieces: List[CopyItem] = []
    for r0 in range(0, rows, max_rows):
        r1 = min(rows, r0 + max_rows)
        piece = dataclasses.replace(item, extent=(r1 - r0,) + tuple(item.extent[1:]), dst_start=(item.dst_start[0] + r0,) + tuple(item.dst_start[1:]))
        if item.src_rows is None:
            piece.src_start = (item.src_start[0] + r0,) + tuple(item.src_start[1:])
        else:
            runs = []
            for rel, srow, n in item.src_rows:
                lo, hi = max(rel, r0), min(rel + n, r1)
                if lo < hi:
                    runs.append((lo - r0, srow + (lo - rel), hi - lo))
            piece.src_rows = tuple(runs)
        if item.scale_name is not None:
            piece.scale_start = (item.scale_start[0] + r0 // FP8_BLOCK, item.scale_start[1])
        pieces.append(piece)
    return pieces


def _item_src_bytes(item: CopyItem) -> int:
    return item.numel * item.src_dtype.itemsize


def stripe_by_destination(items: Sequence[CopyItem], stripe_bytes: int) -> List[CopyItem]:
    """The same work in another order: every item is cut into pieces of about
    ``stripe_bytes`` of source data, and the pieces of the different
    destinations are merged so that at every point of the list each destination
    has received the same fraction of its bytes.  A kernel that walks the list
    with all its CTAs inside one narrow window then writes to all destinations
    at once, in proportion to what each is owed, instead of one after the other.
    The order inside a destination is kept."""
    per_dst: Dict[int, List[CopyItem]] = {}
    for it in items:
        row_bytes = max(1, _item_src_bytes(it) // max(it.extent[0], 1)) if it.extent else 1
        per_dst.setdefault(it.dst_rank, []).extend(split_item_rows(it, max(1, stripe_bytes // row_bytes)))
    if len(per_dst) < 2:
        return [p for d in sorted(per_dst) for p in per_dst[d]]
    totals = {d: max(1, sum(_item_src_bytes(p) for p in ps)) for d, ps in per_dst.items()}
    done = {d: 0 for d in per_dst}
    cursor = {d: 0 for d in per_dst}
    out: List[CopyItem] = []
    remaining = sum(len(ps) for ps in per_dst.values())
    while remaining:
        # the destination that is furthest behind (ties: lowest rank) goes next
        d = min((d for d in per_dst if cursor[d] < len(per_dst[d])), key=lambda d: (done[d] / totals[d], d))
        piece = per_dst[d][cursor[d]]
        out.append(piece)
        cursor[d] += 1
        done[d] += _item_src_bytes(piece)
        remaining -= 1
    return out


def manifest_by_destination(items: Iterable[CopyItem]) -> Dict[int, List[tuple]]:
    """What each destination rank will receive from this sender, as plain
    tuples that can be published through the MetaServer."""
    out: Dict[int, List[tuple]] = {}
    for it in items:
        out.setdefault(it.dst_rank, []).append(it.manifest_entry())
    return out


def check_exactly_once(
    manifests: Iterable[Sequence[tuple]],
    views: Dict[str, Tuple[Tuple[int, ...], torch.dtype]],
    required: Optional[Iterable[str]] = None,
) -> List[str]:
    """Host-side race/coverage check of everything that will be written into one
    inference rank: every element of every required view is written exactly once
    and nothing is written out of bounds.  Returns a list of problems.

    Cost depends on the number of boxes, not on the size of the tensors: per
    view the box boundaries cut the index space into a coarse grid whose cells
    are counted (a few cells per box for the regular shardings that occur)."""
    problems: List[str] = []
    boxes: Dict[str, List[Tuple[Tuple[int, ...], Tuple[int, ...], str]]] = {}

    def note(name: str, start, extent, label: str) -> None:
        if name not in views:
            problems.append(f"{label}: write into unknown view {name!r}")
            return
        shape = views[name][0]
        if len(start) != len(shape) or any(s < 0 or e < 0 or s + e > d for s, e, d in zip(start, extent, shape)):
            problems.append(f"{label}: box start={start} extent={extent} exceeds {name!r} of shape {shape}")
            return
        boxes.setdefault(name, []).append((tuple(start), tuple(extent), label))

    for sender, manifest in enumerate(manifests):
        for name, start, extent, dtype, scale_name, scale_start in manifest:
            if name in views and str(views[name][1]) != dtype:
                problems.append(f"sender#{sender}: dtype {dtype} written into {name!r} of dtype {views[name][1]}")
            note(name, tuple(start), tuple(extent), f"sender#{sender}")
            if scale_name is not None:
                blocks = tuple(-(-e // FP8_BLOCK) for e in extent)
                note(scale_name, tuple(scale_start), blocks, f"sender#{sender}(scale)")
    for name, written in boxes.items():
        problems.extend(_cover_problems(name, views[name][0], written))
    for name in required if required is not None else views:
        if name not in boxes and not any(name in p for p in problems):
            problems.append(f"view {name!r} receives nothing")
    return problems


_MAX_GRID_CELLS = 20_000_000


def _cover_problems(name: str, shape: Tuple[int, ...], written) -> List[str]:
    """Overlaps and gaps of in-bounds boxes inside ``shape``."""
    import numpy as np

    if not shape:  # scalar view
        return [] if len(written) == 1 else [f"view {name!r}: scalar written {len(written)} times"]
    nd = len(shape)
    cuts = []
    for d in range(nd):
        edge = {0, shape[d]}
        for start, extent, _ in written:
            edge.add(start[d])
            edge.add(start[d] + extent[d])
        cuts.append(np.array(sorted(edge), dtype=np.int64))
    cells = 1
    for c in cuts:
        cells *= max(len(c) - 1, 1)
    if cells > _MAX_GRID_CELLS:
        return _cover_problems_pairwise(name, shape, written)
    grid = np.zeros([max(len(c) - 1, 1) for c in cuts], dtype=np.int32)
    out: List[str] = []
    for start, extent, label in written:
        if any(e == 0 for e in extent):
            continue
        sl = tuple(slice(int(np.searchsorted(cuts[d], start[d])), int(np.searchsorted(cuts[d], start[d] + extent[d]))) for d in range(nd))
        if grid[sl].any() and len(out) < 8:
            out.append(f"{label}: box start={start} extent={extent} of {name!r} overlaps an earlier write")
        grid[sl] += 1
    if (grid != 1).any():
        volume = np.ones(grid.shape, dtype=np.int64)
        for d, c in enumerate(cuts):
            widths = np.diff(c) if len(c) > 1 else np.array([0])
            volume = volume * widths.reshape([-1 if i == d else 1 for i in range(nd)])
        missing = int(volume[grid == 0].sum())
        if missing:
            total = 1
            for n in shape:
                total *= n
            out.append(f"view {name!r}: {missing} of {total} elements are never written")
    return out


def _cover_problems_pairwise(name: str, shape: Tuple[int, ...], written) -> List[str]:
    """Irregular box sets: disjointness by pairs (sorted by first coordinate) and
    coverage by total volume."""
    out: List[str] = []
    order = sorted(written, key=lambda b: b[0])
    volume = 0
    for i, (s_i, e_i, label) in enumerate(order):
        v = 1
        for e in e_i:
            v *= e
        volume += v
        for s_j, e_j, _ in order[i + 1 :]:
            if s_j[0] >= s_i[0] + e_i[0]:
                break
            if all(a < b + eb and b < a + ea for a, ea, b, eb in zip(s_i, e_i, s_j, e_j)) and len(out) < 8:
                out.append(f"{label}: box start={s_i} extent={e_i} of {name!r} overlaps another write")
    total = 1
    for n in shape:
        total *= n
    if not out and volume != total:
        out.append(f"view {name!r}: {total - volume} of {total} elements are never written")
    return out
