"""Parallel coordinates of one model worker.

Field order and defaults are the metadata contract shared with the reference
(`awex/sharding/rank_info.py:45-65`): objects of this class are pickled
through the MetaServer and compared field by field.

Context parallelism (``cp_*``) is carried as labels only: CP peers hold
identical weights and are handled as ordinary replicas by the planner.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(slots=True)
class RankInfo:
    tp_rank: int
    tp_size: int
    pp_rank: int
    pp_size: int
    dp_size: int
    dp_rank: int
    ep_rank: int
    ep_size: int
    ep_tp_rank: int
    ep_tp_size: int
    attn_tp_rank: int
    attn_tp_size: int
    attn_dp_rank: int
    world_size: int
    global_rank: int
    local_rank: int
    engine_rank: int
    is_infer: bool
    cp_rank: int = 0
    cp_size: int = 1
    cp_mode: str = "none"

    @staticmethod
    def single(global_rank: int = 0, world_size: int = 1, is_infer: bool = False, **overrides) -> "RankInfo":
        """A rank with every parallel size 1; ``overrides`` replace fields."""
        base = dict(
            tp_rank=0, tp_size=1, pp_rank=0, pp_size=1, dp_size=1, dp_rank=0, ep_rank=0, ep_size=1,
            ep_tp_rank=0, ep_tp_size=1, attn_tp_rank=0, attn_tp_size=1, attn_dp_rank=0,
            world_size=world_size, global_rank=global_rank, local_rank=global_rank, engine_rank=0,
            is_infer=is_infer,
        )
        base.update(overrides)
        return RankInfo(**base)
