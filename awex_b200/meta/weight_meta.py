"""Shard / replica / parameter metadata exchanged between training and
inference.

The three dataclasses keep the reference's field names, order and defaults
(`awex/meta/weight_meta.py:32-103`) because pickles of them travel through
the MetaServer and are hashed into plan fingerprints.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

import torch

from awex_b200.sharding.param_sharding import ShardingType
from awex_b200.utils.common import to_dict


@dataclass(slots=True)
class ParameterShardMeta:
    """One rank's piece of one canonical parameter.  ``global_offset`` is the
    position of the piece inside the unsharded tensor."""

    tp_rank: int
    attn_tp_rank: int
    pp_rank: int
    ep_rank: int
    ep_tp_rank: int
    global_rank: int
    world_size: int
    engine_rank: int
    name: str
    shape: Tuple[int, ...]
    numel: int
    dtype: torch.dtype
    global_offset: Tuple[int, ...] = field(default_factory=tuple)
    sharding_type: ShardingType = ShardingType.NO_SHARDING
    num_shards: int = 1
    sharding_dim: int = 0
    cp_rank: int = 0
    cp_size: int = 1
    cp_mode: str = "none"


@dataclass(slots=True)
class ParameterReplicaMeta:
    """Shards that together form one full logical copy."""

    shards: List[ParameterShardMeta]


@dataclass(slots=True)
class ParameterMeta:
    name: str
    global_numel: int
    global_shape: Tuple[int, ...]
    dtype: torch.dtype
    shards: List[ParameterShardMeta]  # every shard of every replica
    replicas: List[ParameterReplicaMeta]

    def fast_copy_with_engine_rank(self, engine_rank: int) -> "ParameterMeta":
        """Deep copy of the shard tree with ``engine_rank`` replaced."""
        flat: List[ParameterShardMeta] = []
        replicas: List[ParameterReplicaMeta] = []
        for replica in self.replicas:
            copies = [dataclasses.replace(s, engine_rank=engine_rank) for s in replica.shards]
            flat.extend(copies)
            replicas.append(ParameterReplicaMeta(shards=copies))
        return ParameterMeta(
            name=self.name,
            global_numel=self.global_numel,
            global_shape=self.global_shape,
            dtype=self.dtype,
            shards=flat,
            replicas=replicas,
        )

    def to_local_parameter_meta(self, global_rank: int) -> "ParameterMeta":
        """Restrict to what ``global_rank`` holds: at most one shard in at
        most one replica (experts are absent from most ranks)."""
        local = self.fast_copy_with_engine_rank(self.shards[0].engine_rank)
        local.shards = [s for s in local.shards if s.global_rank == global_rank]
        kept: List[ParameterReplicaMeta] = []
        for replica in local.replicas:
            mine = [s for s in replica.shards if s.global_rank == global_rank]
            assert len(mine) <= 1, (
                f"A tp worker should have at most one shard per replica but got {len(mine)} shards for {global_rank}"
            )
            if mine:
                replica.shards = mine
                kept.append(replica)
        local.replicas = kept
        assert len(local.shards) <= 1, (
            f"A tp worker should have one shard for model parameter but got {local.shards} for {global_rank}"
        )
        assert len(kept) <= 1, f"More than one replica found for global_rank {global_rank}"
        return local


def dump_parameters_meta(params_meta: Sequence[ParameterMeta]) -> list:
    """JSON-ready summary used by debug-mode dumps."""
    return [
        to_dict(
            {
                "name": p.name,
                "global_numel": p.global_numel,
                "global_shape": p.global_shape,
                "dtype": p.dtype,
                "num_shards": len(p.shards),
                "num_replicas": len(p.replicas),
                "replicas": p.replicas,
            }
        )
        for p in params_meta
    ]


def compute_total_model_size(params_meta: Sequence[ParameterMeta]) -> int:
    """Bytes of one full copy of the model."""
    return sum(p.global_numel * p.dtype.itemsize for p in params_meta)
