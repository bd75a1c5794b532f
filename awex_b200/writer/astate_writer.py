"""RDMA ("astate") mode, writer side.

The reference drives a closed-source RDMA table library
(`awex/writer/astate_writer.py:26-74`): every training rank opens the remote
table ``"weights_exchange"`` with its parallel coordinates, puts its canonical
shards under keys made of (name, global shape, global offset) and completes the
step; the library reshards between what writers put and what readers get.  The
library is not public and cross-node RDMA is out of scope on one NVLink box, so
this class keeps the exact call shape against whatever module named ``astate``
is importable and fails loudly when none is.
"""

from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from awex_b200 import logging
from awex_b200.writer.weights_writer import WeightsExchangeShardingWriter

logger = logging.getLogger(__name__)

TABLE_NAME = "weights_exchange"


def _import_astate():
    try:
        import astate  # type: ignore

        return astate
    except ImportError as exc:
        raise RuntimeError(
            "comm_backend='astate' needs the astate RDMA library, which is not installed; "
            "use 'nccl' (fused NVLink transfer) on a single node"
        ) from exc


def parallel_fields(rank_info, role_size: int, role_rank: int) -> Dict[str, int]:
    """Keyword arguments of ``ParallelConfig.create_{training,inference}_config``."""
    cp_size = int(getattr(rank_info, "cp_size", 1) or 1)
    cp_rank = int(getattr(rank_info, "cp_rank", 0) or 0) if cp_size > 1 else 0
    return dict(
        role_size=role_size, role_rank=role_rank, dp_size=rank_info.dp_size, dp_rank=rank_info.dp_rank, tp_size=rank_info.tp_size,
        tp_rank=rank_info.tp_rank, pp_size=rank_info.pp_size, pp_rank=rank_info.pp_rank, cp_size=max(cp_size, 1), cp_rank=cp_rank,
        ep_size=rank_info.ep_size, ep_rank=rank_info.ep_rank, etp_size=rank_info.ep_tp_size, etp_rank=rank_info.ep_tp_rank,
    )


def sharded_pairs(astate, tensors: Dict[str, torch.Tensor], params_meta, global_rank: int, engine_rank=None) -> List[Tuple[object, torch.Tensor]]:
    """``(sharded key, tensor)`` for every tensor this rank holds a shard of."""
    from astate.utils import create_sharded_key  # type: ignore

    by_name = {m.name: m for m in params_meta}
    pairs = []
    for name, tensor in tensors.items():
        meta = by_name.get(name)
        if meta is None:
            continue
        mine = [s for s in meta.shards if s.global_rank == global_rank and (engine_rank is None or s.engine_rank == engine_rank)]
        if not mine:
            continue
        shard = mine[0]
        if tuple(shard.shape) != tuple(tensor.shape):
            raise ValueError(f"{name}: metadata says shard shape {tuple(shard.shape)}, tensor has {tuple(tensor.shape)}")
        pairs.append((create_sharded_key(name, tuple(meta.global_shape), tuple(shard.global_offset)), tensor))
    return pairs


class AStateWeightsWriter(WeightsExchangeShardingWriter):
    def _initialize(self) -> None:
        astate = _import_astate()
        super()._initialize()
        ri = self.rank_info
        config = astate.ParallelConfig.create_training_config(**parallel_fields(ri, ri.world_size, ri.global_rank))
        self.table = astate.create_remote_table(TABLE_NAME, parallel_config=config)
        logger.info(f"astate writer ready on training rank {ri.global_rank}")

    def write_tensors(self, step_id, tensors: Dict[str, torch.Tensor]) -> int:
        pairs = sharded_pairs(_import_astate(), tensors, self.parameters_meta, self.rank_info.global_rank)
        self.table.multi_put(step_id, pairs)
        return len(pairs)

    def finish_step(self, step_id) -> None:
        self.table.complete(step_id)

    def _write_weights(self, step_id, **kwargs) -> None:
        self.write_tensors(step_id, self.convert_parameters())
        self.finish_step(step_id)
