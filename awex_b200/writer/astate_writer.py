"""RDMA ("astate") mode: API surface only.

The reference drives a closed-source RDMA table library
(`awex/writer/astate_writer.py:26-74`): ``create_remote_table("weights_exchange",
parallel_config)``, ``multi_put(step, [(sharded_key, tensor)])``, ``complete(step)``.
Cross-node RDMA is out of scope on a single NVLink box, so this class keeps
the call shape and fails loudly when the library is absent."""

from __future__ import annotations

from awex_b200.writer.weights_writer import WeightsExchangeShardingWriter


def _import_astate():
    try:
        import astate  # type: ignore

        return astate
    except ImportError as exc:
        raise RuntimeError(
            "comm_backend='astate' needs the astate RDMA library, which is not installed; "
            "use 'nccl' (fused NVLink transfer) on a single node"
        ) from exc


class AStateWeightsWriter(WeightsExchangeShardingWriter):
    def _initialize(self) -> None:
        astate = _import_astate()
        super()._initialize()
        ri = self.rank_info
        parallel_config = dict(
            role_rank=ri.global_rank, role_size=ri.world_size, tp_rank=ri.tp_rank, tp_size=ri.tp_size, pp_rank=ri.pp_rank,
            pp_size=ri.pp_size, dp_rank=ri.dp_rank, dp_size=ri.dp_size, cp_rank=ri.cp_rank, cp_size=ri.cp_size, cp_mode=ri.cp_mode,
        )
        self.table = astate.create_remote_table("weights_exchange", parallel_config)

    def _write_weights(self, step_id, **kwargs) -> None:
        pairs = list(self.convert_parameters().items())
        self.table.multi_put(step_id, pairs)
        self.table.complete(step_id)
