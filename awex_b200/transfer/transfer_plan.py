"""Deterministic peer-to-peer transfer planning.

Every process (training or inference) runs this planner on the same two
metadata lists and obtains the same operations in the same order; that shared
order is the only synchronisation the data plane needs.  The observable
contract is the reference's (`awex/transfer/transfer_plan.py:158-813`):

* transfer ranks: inference shard -> ``global_rank + engine * instance_world``;
  training shard -> ``global_rank + infer_world_size``;
* inference replica *i* (engines outermost) is fed by training replica
  ``i mod n_train_replicas`` (``replica_pairing="spread"`` instead hands each
  inference replica the least-loaded training replica, walking the parameters
  in sorted order, to balance the senders);
* an operation is the N-d box intersection of one inference shard with one
  training shard, with offsets and slices relative to each shard;
* a rank's plan maps peer -> operations sorted by (name, send offset, recv
  offset), peers ascending;
* the plan fingerprint is the sha256 of a canonical JSON of those operations.

The intersection search here walks both shard lists in sorted order along the
sharded dim instead of testing all pairs.
"""

from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field
from hashlib import sha256
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from awex_b200 import logging
from awex_b200.meta.weight_meta import ParameterMeta, ParameterReplicaMeta, ParameterShardMeta
from awex_b200.utils.common import is_allowed_infer_only_alias, to_dict

logger = logging.getLogger(__name__)

PRUNE_SHARD_THRESHOLD = 10000


@dataclass(slots=True)
class CommunicationOperation:
    """Move ``overlap_shape`` elements from ``send_shard[train_slices]`` on
    ``send_rank`` to ``recv_shard[inf_slices]`` on ``recv_rank``."""

    send_rank: int
    send_shard_meta: ParameterShardMeta
    send_offset: Tuple[int, ...]
    recv_rank: int
    recv_shard_meta: ParameterShardMeta
    recv_offset: Tuple[int, ...]
    overlap_shape: Tuple[int, ...]
    train_slices: Tuple[slice, ...]
    inf_slices: Tuple[slice, ...]
    pp_rank: int = 0
    placement_version: int = -1
    param_class: str = "dense_other"


@dataclass(slots=True)
class TransferPlan:
    """peer transfer rank -> operations exchanged with that peer.
    ``operations`` and ``inter_operations`` are two names for one dict."""

    operations: Dict[int, List[CommunicationOperation]] = field(default_factory=dict)
    inter_operations: Dict[int, List[CommunicationOperation]] = field(default_factory=dict)

    def __post_init__(self):
        if self.inter_operations:
            if self.operations and self.operations != self.inter_operations:
                logger.warning("TransferPlan got two different op tables; inter_operations wins")
            self.operations = self.inter_operations
        else:
            self.inter_operations = self.operations

    def all_operations(self) -> List[CommunicationOperation]:
        return [op for peer in sorted(self.inter_operations) for op in self.inter_operations[peer]]


@dataclass(slots=True)
class ShardOffset:
    shard: Any
    start_offset: tuple
    end_offset: tuple
    shape: tuple
    rank: int


@dataclass(slots=True)
class OverlapRegion:
    inference_shard: ShardOffset
    training_shard: ShardOffset
    overlap_start: tuple
    overlap_end: tuple


@dataclass(slots=True)
class NormalizedAxes:
    pp_rank: int
    tp_rank: int
    tp_size: int
    ep_rank: int
    ep_size: int
    ep_tp_rank: int
    ep_tp_size: int
    attn_tp_rank: int
    attn_tp_size: int


def normalize_rank_axes(param_class: str, rank_info: Any, shard_meta: Any = None) -> NormalizedAxes:
    """One view of a rank's axes per parameter class: attention parameters use
    the attention-TP coordinates as their TP axis, everything else plain TP.
    Context-parallel axes are deliberately absent (CP peers are replicas)."""

    def read(obj, key, default):
        return getattr(obj, key, default) if obj is not None else default

    if param_class == "attention":
        tp_rank = read(rank_info, "attn_tp_rank", read(rank_info, "tp_rank", 0))
        tp_size = read(rank_info, "attn_tp_size", read(rank_info, "tp_size", 1))
    else:
        tp_rank, tp_size = read(rank_info, "tp_rank", 0), read(rank_info, "tp_size", 1)
    return NormalizedAxes(
        pp_rank=read(shard_meta, "pp_rank", read(rank_info, "pp_rank", 0)),
        tp_rank=tp_rank,
        tp_size=tp_size,
        ep_rank=read(rank_info, "ep_rank", 0),
        ep_size=read(rank_info, "ep_size", 1),
        ep_tp_rank=read(rank_info, "ep_tp_rank", 0),
        ep_tp_size=read(rank_info, "ep_tp_size", 1),
        attn_tp_rank=read(rank_info, "attn_tp_rank", tp_rank),
        attn_tp_size=read(rank_info, "attn_tp_size", tp_size),
    )


class TransferPlanBuilder:
    def __init__(
        self,
        infer_world_size: int,
        train_world_size: int,
        num_infer_engines: int = 1,
        enable_debug_mode: bool = False,
        strict_param_key_match: bool = False,
        replica_pairing: str = "round_robin",
        skip_names: Iterable[str] = (),
        colocation: Optional[Dict[int, int]] = None,
    ):
        # names that are planned for nobody (aliases of memory another name covers)
        self.skip_names = frozenset(skip_names)
        if replica_pairing not in ("round_robin", "spread", "local"):
            raise ValueError(f"unknown replica_pairing {replica_pairing!r}")
        # "local": like "spread", but an inference shard whose GPU also holds a training replica of the tensor takes
        # it from there.  ``colocation`` maps inference transfer ranks to the training global rank on the same GPU
        # (default: inference transfer rank t sits with training rank t).
        self.locality = replica_pairing == "local"
        self.colocation = None if colocation is None else {int(k): int(v) for k, v in colocation.items()}
        replica_pairing = "spread" if self.locality else replica_pairing
        self.replica_pairing = replica_pairing
        self._replica_choice: Dict[Tuple[str, int], int] = {}
        if num_infer_engines <= 0:
            raise ValueError("num_infer_engines must be positive")
        self.train_world_size = train_world_size
        self.infer_world_size = infer_world_size
        self.world_size = train_world_size + infer_world_size
        self.num_infer_engines = num_infer_engines
        self.infer_instance_world_size = infer_world_size // num_infer_engines
        self.enable_debug_mode = enable_debug_mode
        self.strict_param_key_match = strict_param_key_match

    # ---- key contract ---------------------------------------------------
    def _common_names(self, infer: Dict[str, ParameterMeta], train: Dict[str, ParameterMeta]) -> List[str]:
        ik, tk = set(infer), set(train)
        missing, extra = tk - ik, ik - tk
        bad_extra = {k for k in extra if not is_allowed_infer_only_alias(k, ik, tk)}
        if missing or (extra if self.strict_param_key_match else bad_extra):
            msg = (
                "Train/infer key mismatch for transfer plan: "
                f"train={len(tk)} infer={len(ik)} missing_on_infer={sorted(missing)} "
                f"extra_on_infer={sorted(extra)} unsupported_extra_on_infer={sorted(bad_extra)} "
                f"strict={self.strict_param_key_match}"
            )
            logger.error(msg)
            raise ValueError(msg)
        if extra:
            logger.info(f"Infer metadata has extra keys ignored by the plan: count={len(extra)} sample={sorted(extra)[:8]}")
        return sorted((ik & tk) - self.skip_names)

    # ---- per-shard helpers ----------------------------------------------
    def _compute_shard_transfer_rank(self, shard: ParameterShardMeta, engine_rank: int, is_infer: bool) -> int:
        if is_infer:
            return shard.global_rank + engine_rank * self.infer_instance_world_size
        assert engine_rank == 0, "Training only has one engine instance"
        return shard.global_rank + self.infer_world_size

    def _create_shard_offset_for_replica(
        self,
        replica: ParameterReplicaMeta,
        engine_rank: int,
        is_infer: bool,
        global_transfer_rank: Optional[int] = None,
        reused_shape_obj=None,
    ) -> List[ShardOffset]:
        if not replica.shards:
            raise ValueError("No shards found for replica")
        boxes: List[ShardOffset] = []
        for shard in replica.shards:
            if not shard.global_offset and len(shard.shape) > 0:
                raise ValueError("Shard has empty global_offset")
            if len(shard.global_offset) != len(shard.shape):
                raise ValueError(
                    f"Dimension mismatch for shard in replica: global_offset has {len(shard.global_offset)} dims, "
                    f"shape has {len(shard.shape)} dims"
                )
            rank = self._compute_shard_transfer_rank(shard, engine_rank, is_infer)
            if global_transfer_rank is not None and rank != global_transfer_rank:
                continue
            start = tuple(shard.global_offset)
            boxes.append(
                ShardOffset(
                    shard=shard,
                    start_offset=start,
                    end_offset=tuple(o + n for o, n in zip(start, shard.shape)),
                    shape=tuple(shard.shape),
                    rank=rank,
                )
            )
        return boxes

    @staticmethod
    def _intersect(a: ShardOffset, b: ShardOffset) -> Optional[Tuple[tuple, tuple]]:
        lo, hi = [], []
        for d in range(len(a.start_offset)):
            s = max(a.start_offset[d], b.start_offset[d])
            e = min(a.end_offset[d], b.end_offset[d])
            if s >= e:
                return None
            lo.append(s)
            hi.append(e)
        return tuple(lo), tuple(hi)

    def _find_overlapping_regions(self, inference_map: List[ShardOffset], training_map: List[ShardOffset]) -> List[OverlapRegion]:
        """All intersecting (inference, training) shard pairs, ordered by
        inference shard then training shard as listed."""
        regions: List[OverlapRegion] = []
        if not inference_map or not training_map:
            return regions
        # Pick the dim with the most distinct start offsets on the training side
        # and bisect on it; other dims are checked by the full box test.
        ndim = len(training_map[0].start_offset)
        sweep_dim = max(range(ndim), key=lambda d: len({t.start_offset[d] for t in training_map})) if ndim else 0
        if ndim and len(training_map) > 8:
            order = sorted(range(len(training_map)), key=lambda i: training_map[i].start_offset[sweep_dim])
            starts = [training_map[i].start_offset[sweep_dim] for i in order]
            import bisect

            for inf in inference_map:
                hi = bisect.bisect_left(starts, inf.end_offset[sweep_dim])
                hits = []
                for pos in range(hi):
                    t = training_map[order[pos]]
                    if t.end_offset[sweep_dim] <= inf.start_offset[sweep_dim]:
                        continue
                    box = self._intersect(inf, t)
                    if box is not None:
                        hits.append((order[pos], t, box))
                hits.sort(key=lambda h: h[0])
                regions.extend(OverlapRegion(inf, t, box[0], box[1]) for _, t, box in hits)
            return regions
        for inf in inference_map:
            for t in training_map:
                box = self._intersect(inf, t)
                if box is not None:
                    regions.append(OverlapRegion(inf, t, box[0], box[1]))
        return regions

    def _build_region_communication_plan(self, region: OverlapRegion, reused_shape_obj=None) -> List[CommunicationOperation]:
        inf, trn = region.inference_shard, region.training_shard
        lo, hi = region.overlap_start, region.overlap_end
        extent = tuple(h - l for l, h in zip(lo, hi))
        inf_rel = tuple(l - o for l, o in zip(lo, inf.start_offset))
        trn_rel = tuple(l - o for l, o in zip(lo, trn.start_offset))
        assert trn.rank != inf.rank, "Send and recv rank cannot be the same"
        assert trn.rank >= self.infer_world_size, f"Send rank {trn.rank} is not in the training world"
        assert inf.rank < self.infer_world_size, f"Recv rank {inf.rank} is not in the inference world"
        return [
            CommunicationOperation(
                send_rank=trn.rank,
                send_shard_meta=trn.shard,
                send_offset=trn_rel,
                recv_rank=inf.rank,
                recv_shard_meta=inf.shard,
                recv_offset=inf_rel,
                overlap_shape=extent,
                train_slices=tuple(slice(o, o + n) for o, n in zip(trn_rel, extent)),
                inf_slices=tuple(slice(o, o + n) for o, n in zip(inf_rel, extent)),
            )
        ]

    # ---- per-parameter / global -------------------------------------------
    def _build_parameter_communication_plan(
        self,
        param_name: str,
        inference_meta: ParameterMeta,
        training_meta: ParameterMeta,
        global_transfer_rank: Optional[int] = None,
    ) -> List[CommunicationOperation]:
        infer_replicas = [(e, r) for e in range(self.num_infer_engines) for r in inference_meta.replicas]
        train_replicas = training_meta.replicas
        if not infer_replicas or not train_replicas:
            raise ValueError(f"No replicas found for parameter {param_name}")
        only_infer = global_transfer_rank if (global_transfer_rank is not None and global_transfer_rank < self.infer_world_size) else None
        only_train = global_transfer_rank if (global_transfer_rank is not None and global_transfer_rank >= self.infer_world_size) else None
        ops: List[CommunicationOperation] = []
        home = self._replica_of_train_rank(training_meta) if self.locality and len(train_replicas) > 1 else None
        for i, (engine, inf_replica) in enumerate(infer_replicas):
            chosen = self._pick_train_replica(i, training_meta)
            inf_boxes = self._create_shard_offset_for_replica(inf_replica, engine, True, only_infer)
            groups: Dict[int, List[ShardOffset]] = {chosen: inf_boxes}
            if home is not None:
                # every inference shard takes the tensor from the replica on its own GPU where there is one
                groups = {}
                for box in inf_boxes:
                    mate = box.rank if self.colocation is None else self.colocation.get(box.rank)
                    groups.setdefault(home.get(mate, chosen), []).append(box)
            for k in sorted(groups):
                trn_boxes = self._create_shard_offset_for_replica(train_replicas[k], 0, False, only_train)
                for region in self._find_overlapping_regions(groups[k], trn_boxes):
                    ops.extend(self._build_region_communication_plan(region))
        return ops

    @staticmethod
    def _replica_of_train_rank(training_meta: ParameterMeta) -> Dict[int, int]:
        """training global rank -> index of the replica it holds a shard of."""
        return {int(s.global_rank): k for k, rep in enumerate(training_meta.replicas) for s in rep.shards}

    def _pick_train_replica(self, i: int, training_meta: ParameterMeta) -> int:
        """Index of the training replica that feeds inference replica ``i``.
        ``spread`` looks the answer up in the table made by
        :meth:`_assign_replicas`; a parameter the table does not know (a direct
        call before any plan was built) falls back to the reference's modulo."""
        n = len(training_meta.replicas)
        if self.replica_pairing != "spread" or n == 1:
            return i % n
        return self._replica_choice.get((training_meta.name, i), i % n)

    def _assign_replicas(self, names: Sequence[str], infer: Dict[str, ParameterMeta], train: Dict[str, ParameterMeta]) -> None:
        """``spread``: walk the parameters in sorted order and hand each inference
        replica the training replica that has been given the fewest bytes so far
        (ties: lowest index), so parameters replicated over many data-parallel
        ranks are served by all of them.  The table depends only on the metadata,
        hence every rank computes the same one, and it is kept so that later
        per-parameter calls (plans made on behalf of a TP peer) agree with it."""
        self._replica_choice = {}
        if self.replica_pairing != "spread":
            return
        loads: Dict[int, List[int]] = {}
        for name in names:
            n = len(train[name].replicas)
            if n <= 1:
                continue
            nbytes = 1
            for d in train[name].global_shape:
                nbytes *= int(d)
            per_group = loads.setdefault(n, [0] * n)
            for i in range(self.num_infer_engines * len(infer[name].replicas)):
                k = min(range(n), key=lambda j: (per_group[j], j))
                per_group[k] += nbytes
                self._replica_choice[(name, i)] = k

    def build_weights_mapping_operations(
        self,
        inference_weights_meta: Sequence[ParameterMeta],
        training_weights_meta: Sequence[ParameterMeta],
        global_transfer_rank: Optional[int] = None,
    ) -> List[CommunicationOperation]:
        if not inference_weights_meta or not training_weights_meta:
            logger.warning("Empty weights meta provided, returning empty plan")
            return []
        infer = {m.name: m for m in inference_weights_meta}
        train = {m.name: m for m in training_weights_meta}
        ops: List[CommunicationOperation] = []
        names = self._common_names(infer, train)
        self._assign_replicas(names, infer, train)
        for name in names:
            ops.extend(self._build_parameter_communication_plan(name, infer[name], train[name], global_transfer_rank))
        return ops

    def _group_operations_by_rank(self, operations: Iterable[CommunicationOperation], key_name: str) -> Dict[int, List[CommunicationOperation]]:
        grouped: Dict[int, List[CommunicationOperation]] = {}
        for op in operations:
            grouped.setdefault(getattr(op, key_name), []).append(op)
        for ops in grouped.values():
            ops.sort(key=lambda op: (op.send_shard_meta.name, op.send_offset, op.recv_offset))
        return {peer: grouped[peer] for peer in sorted(grouped)}

    def build_local_transfer_plan(
        self,
        inference_weights_meta: Sequence[ParameterMeta],
        training_weights_meta: Sequence[ParameterMeta],
        global_transfer_rank: int,
    ) -> TransferPlan:
        t0 = time.time()
        is_train = global_transfer_rank >= self.infer_world_size
        side = "train" if is_train else "infer"
        n_shards = sum(len(r.shards) for p in inference_weights_meta for r in p.replicas) * self.num_infer_engines
        n_shards += sum(len(r.shards) for p in training_weights_meta for r in p.replicas)
        # Above the threshold only boxes that involve this rank are intersected.
        prune = n_shards > PRUNE_SHARD_THRESHOLD
        ops = self.build_weights_mapping_operations(
            inference_weights_meta, training_weights_meta, global_transfer_rank if prune else None
        )
        if self.enable_debug_mode:
            self._dump(f"global_communication_plan_{side}_{global_transfer_rank}_{os.getpid()}.json", ops)
        mine_key, peer_key = ("send_rank", "recv_rank") if is_train else ("recv_rank", "send_rank")
        mine = [op for op in ops if getattr(op, mine_key) == global_transfer_rank]
        grouped = self._group_operations_by_rank(mine, peer_key)
        logger.info(
            f"Rank[{global_transfer_rank}] ({side}) local plan: {len(mine)} operations, peers {list(grouped)}, "
            f"{len(ops)} operations considered (pruned={prune}), {time.time() - t0:.2f}s"
        )
        if self.enable_debug_mode:
            self._dump(f"local_communication_plan_{side}_{global_transfer_rank}_{os.getpid()}.json", grouped)
        return TransferPlan(inter_operations=grouped)

    @staticmethod
    def _dump(file_name: str, obj) -> None:
        with open(file_name, "w") as f:
            json.dump(to_dict(obj), f, indent=2)
        logger.info(f"Saved communication plan to {os.path.abspath(file_name)}")


@torch.no_grad()
def slice_tensor(tensor: torch.Tensor, op: CommunicationOperation, is_train, **kwargs) -> torch.Tensor:
    """View of the op's box inside ``tensor``.  The inference view may be
    strided.  A strided training view is made dense (and cached in
    ``slice_context``) because send/recv transports need contiguous messages;
    the fused peer-store path never calls this."""
    view = tensor[op.train_slices if is_train else op.inf_slices]
    if not is_train or view.is_contiguous():
        return view
    cache = kwargs.get("slice_context")
    if cache is None:
        return view.contiguous()
    key = f"{op.send_shard_meta.name}-{op.train_slices}"
    dense = cache.get(key)
    if dense is None:
        dense = cache[key] = view.contiguous()
    return dense


def _slices_as_tuples(slices: Iterable[slice]) -> tuple:
    return tuple((s.start, s.stop, s.step or 1) for s in slices)


def compute_transfer_plan_hash(transfer_plan: TransferPlan) -> str:
    rows = []
    for peer in sorted(transfer_plan.inter_operations):
        for op in transfer_plan.inter_operations[peer]:
            rows.append(
                (
                    peer, op.send_rank, op.recv_rank, op.send_shard_meta.name, op.recv_shard_meta.name,
                    tuple(op.send_offset), tuple(op.recv_offset), tuple(op.overlap_shape),
                    _slices_as_tuples(op.train_slices), _slices_as_tuples(op.inf_slices),
                    op.pp_rank, op.placement_version, op.param_class,
                )
            )
    blob = json.dumps({"inter": rows}, sort_keys=True, separators=(",", ":"))
    return sha256(blob.encode("utf-8")).hexdigest()


def _itemsize(dtype: Any) -> int:
    if isinstance(dtype, str):
        dtype = getattr(torch, dtype.replace("torch.", ""), None)
    return dtype.itemsize if isinstance(dtype, torch.dtype) else 4


def compute_transfer_plan_stats(transfer_plan: TransferPlan) -> Dict[str, Any]:
    n_ops = numel = nbytes = 0
    for ops in transfer_plan.inter_operations.values():
        n_ops += len(ops)
        for op in ops:
            n = 1
            for d in op.overlap_shape:
                n *= int(d)
            numel += n
            nbytes += n * _itemsize(op.send_shard_meta.dtype)
    digest = compute_transfer_plan_hash(transfer_plan)
    return {
        "inter_hash": digest,
        "full_hash": digest,
        "inter": {"peer_count": len(transfer_plan.inter_operations), "op_count": n_ops, "numel": numel, "bytes": nbytes},
        "total": {"op_count": n_ops, "numel": numel, "bytes": nbytes},
    }
