"""RDMA ("astate") mode, reader side (`awex/reader/astate_reader.py:26-85` in
the reference): every inference worker opens the remote table with its
coordinates, gets its canonical shards *in place* by (name, global shape, global
offset) keys and completes the step."""

from __future__ import annotations

from awex_b200 import logging
from awex_b200.reader.nccl_reader import WorkerWeightsReader
from awex_b200.reader.weights_reader import WeightsReader
from awex_b200.writer.astate_writer import TABLE_NAME, _import_astate, parallel_fields, sharded_pairs

logger = logging.getLogger(__name__)


class AStateWorkerWeightsReader(WorkerWeightsReader):
    def initialize(self) -> None:
        super().initialize()
        astate = _import_astate()
        ri = self.rank_info
        role_size = ri.world_size * self.num_engines
        role_rank = ri.global_rank + ri.world_size * self.engine_rank
        config = astate.ParallelConfig.create_inference_config(**parallel_fields(ri, role_size, role_rank))
        self.table = astate.create_remote_table(TABLE_NAME, parallel_config=config)
        logger.info(f"astate reader ready on inference rank {self.engine_rank}-{ri.global_rank}")

    def read_tensors(self, step_id) -> int:
        views = {n: self.parameters[n] for n in self.required_names}
        pairs = sharded_pairs(_import_astate(), views, self.parameters_meta, self.rank_info.global_rank)
        self.table.multi_get(step_id, pairs)  # in place
        return len(pairs)

    def finish_step(self, step_id) -> None:
        self.table.complete(step_id)

    def begin_update(self, step_id) -> None:
        self.epoch += 1

    def finish_update(self, step_id, synchronize: bool = True) -> None:
        self.read_tensors(step_id)
        self.finish_step(step_id)
        self._after_update()

    def close(self) -> None:
        pass


class AStateWeightsReader(WeightsReader):
    def _initialize(self) -> None:
        _import_astate()
        super()._initialize()
