"""Turn per-rank raw parameter listings into global :class:`ParameterMeta`.

Grouping rules are those of the reference (`awex/meta/meta_resolver.py:93-232`):
un-sharded parameters make one replica per holder; sharded ones are bucketed
by the rank coordinate that the sharding type splits on, replica *k* being
the *k*-th holder of every bucket; the global extent of the sharded dim is
the sum over the first replica and offsets are running sums per replica.
Context-parallel coordinates are not copied into shards.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Dict, List, Tuple

import torch

from awex_b200 import logging
from awex_b200.meta.weight_meta import ParameterMeta, ParameterReplicaMeta, ParameterShardMeta
from awex_b200.sharding.param_sharding import ShardingType
from awex_b200.sharding.rank_info import RankInfo
from awex_b200.utils.common import cfg_get

logger = logging.getLogger(__name__)

_GROUP_KEY = {
    ShardingType.TP_SHARDING: "tp_rank",
    ShardingType.DP_TP_SHARDING: "attn_tp_rank",
    ShardingType.EP_TP_SHARDING: "ep_tp_rank",
    ShardingType.EP_SHARDING: "ep_rank",
}


def get_num_hidden_layers(hf_config) -> int:
    """Decoder depth from a flat config or a composite one (``text_config``)."""
    n = cfg_get(hf_config, "num_hidden_layers")
    if n is None:
        n = cfg_get(cfg_get(hf_config, "text_config"), "num_hidden_layers")
    if n is None:
        raise AttributeError(
            "Hugging Face config must define num_hidden_layers either at the top level or under text_config"
        )
    return int(n)


def _as_dtype(dtype) -> Any:
    if isinstance(dtype, str):
        return getattr(torch, dtype.replace("torch.", ""), dtype)
    return dtype


def group_into_replicas(name: str, shards: List[ParameterShardMeta]) -> List[List[ParameterShardMeta]]:
    kind, num_shards = shards[-1].sharding_type, shards[-1].num_shards
    if kind == ShardingType.NO_SHARDING:
        return [[s] for s in shards]
    if num_shards == 1:
        return [list(shards)]
    key = _GROUP_KEY.get(kind)
    if key is None:
        raise ValueError(f"Unknown sharding_type: {kind}")
    buckets: Dict[int, List[ParameterShardMeta]] = {}
    for s in shards:
        buckets.setdefault(getattr(s, key), []).append(s)
    sizes = [len(b) for b in buckets.values()]
    assert len(set(sizes)) == 1, f"Inconsistent number of replicas across {key}s for param {name}: {sizes}"
    ordered = [buckets[k] for k in sorted(buckets)]
    return [sorted((b[i] for b in ordered), key=lambda s: s.tp_rank) for i in range(sizes[0])]


def assign_global_layout(replicas: List[List[ParameterShardMeta]]) -> Tuple[Tuple[int, ...], int]:
    """Fill ``global_offset`` of every shard; return (global_shape, global_numel)."""
    first = replicas[0]
    dim = first[0].sharding_dim
    ndim = len(first[0].shape)
    shape = tuple(sum(s.shape[i] for s in first) if i == dim else first[0].shape[i] for i in range(ndim))
    for replica in replicas:
        cursor = 0
        for s in replica:
            s.global_offset = tuple(cursor if i == dim else 0 for i in range(ndim))
            if ndim:
                cursor += s.shape[dim]
    return shape, sum(s.numel for s in first)


class ParamMetaResolver(ABC):
    def __init__(self, hf_config):
        self.hf_config = hf_config
        self.num_hidden_layers = get_num_hidden_layers(hf_config)

    @abstractmethod
    def get_model_arch_name(self) -> str: ...

    @abstractmethod
    def get_parameters_meta(self) -> List[ParameterMeta]: ...

    @abstractmethod
    def _get_params_raw_meta(self) -> List[Dict[str, Any]]:
        """One ``{"rank_info", "params_meta": [{"name","numel","shape","dtype"}]}`` per rank."""

    @abstractmethod
    def _get_sharding_info(self, name: str, rank_info: RankInfo, param_meta: Dict[str, Any]) -> Tuple[ShardingType, int, int]: ...

    def _build_params_meta(self) -> List[ParameterMeta]:
        by_name: Dict[str, List[ParameterShardMeta]] = {}
        for rank_meta in self._get_params_raw_meta():
            ri: RankInfo = rank_meta["rank_info"]
            for raw in rank_meta["params_meta"]:
                name = raw["name"]
                kind, dim, count = self._get_sharding_info(name, ri, raw)
                by_name.setdefault(name, []).append(
                    ParameterShardMeta(
                        tp_rank=ri.tp_rank, attn_tp_rank=ri.attn_tp_rank, pp_rank=ri.pp_rank,
                        ep_rank=ri.ep_rank, ep_tp_rank=ri.ep_tp_rank, global_rank=ri.global_rank,
                        world_size=ri.world_size, engine_rank=ri.engine_rank, name=name,
                        shape=raw["shape"], numel=raw["numel"], dtype=_as_dtype(raw["dtype"]),
                        sharding_type=kind, num_shards=count, sharding_dim=dim,
                    )
                )
        result: List[ParameterMeta] = []
        total = 0
        for name, shards in by_name.items():
            replicas = group_into_replicas(name, shards)
            shape, numel = assign_global_layout(replicas)
            total += sum(len(r) for r in replicas)
            result.append(
                ParameterMeta(
                    name=name, global_numel=numel, global_shape=shape, dtype=shards[0].dtype, shards=shards,
                    replicas=[ParameterReplicaMeta(shards=r) for r in replicas],
                )
            )
        logger.info(f"Number of shards: {total}")
        return result
