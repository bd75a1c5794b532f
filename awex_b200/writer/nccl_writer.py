"""Writer for the ``nccl`` communication backend name.

The class keeps the reference's name (`awex/writer/nccl_writer.py:43-427`) so
user code is unchanged, but on CUDA devices the data plane is not NCCL: each
``write_weights`` is one launch of the fused transfer kernel that stores this
rank's shards, already converted, into the inference engines' live parameters
over NVLink.  On CPU the same program travels over Gloo.

Per update nothing is converted, sliced, cloned or packed on the host: the
send program is compiled once, on the first update.
"""

from __future__ import annotations

import os
import time

import torch

from awex_b200 import logging
from awex_b200.transfer.lowering import DERIVED_PREFIX, LocalParam, SendProgramCompiler, refresh_derived
from awex_b200.transfer.transfer_plan import TransferPlanBuilder, compute_transfer_plan_stats
from awex_b200.utils.trace import phase
from awex_b200.utils.common import compute_statistics
from awex_b200.writer.weights_writer import WeightsExchangeShardingWriter

logger = logging.getLogger(__name__)


class NCCLWeightsWriter(WeightsExchangeShardingWriter):
    def __init__(self, train_engine):
        super().__init__(train_engine)
        self.transport = None
        self.epoch = 0
        self.grid = int(self.config.get("transfer_grid", 0))

    def _initialize(self) -> None:
        super()._initialize()
        t0 = time.time()
        self.builder = TransferPlanBuilder(
            self.infer_world_size, self.training_world_size, self.num_infer_engines, enable_debug_mode=self.enable_debug_mode,
            replica_pairing=str(self.config.get("replica_pairing", "spread")),
            skip_names=(self.infer_conf.get("aliased_parameters") or {}),
            # with replica_pairing="local": inference transfer rank -> training global rank on the same GPU
            colocation=self.config.get("colocation") or self.infer_conf.get("colocation"),
        )
        local = self.local_tensors()
        params = [LocalParam(name, vp, tuple(t.shape), t.dtype) for (name, vp), t in local.items()]
        compiler = SendProgramCompiler(
            self.rank_info, self.all_train_ranks, self._make_converter, params, self.infer_params_meta,
            self.parameters_meta, self.builder,
        )
        self.items = compiler.compile()
        # tensors that must be computed from whole parameters before each update (a column-normalised
        # head): persistent buffers beside the parameters, sent with plain copies
        self.derived = list(compiler.derived.values())
        self._local = local
        # the parameter objects behind ``local``: a training framework that re-allocates a parameter leaves the
        # detached tensors here pointing at the old storage, which would be sent again and again
        self._watched = [((name, vp), p) for vp, chunk in enumerate(self.model) for name, p in chunk.named_parameters()]
        self._encoded_ptrs = {key: p.data_ptr() for key, p in self._watched}  # the addresses the send table was built from
        refresh_derived(self.derived, local, self._gather_tp_shards)
        self.transfer_plan = self.builder.build_local_transfer_plan(self.infer_params_meta, self.parameters_meta, self.transfer_rank)
        stats = compute_transfer_plan_stats(self.transfer_plan)
        logger.info(f"Rank[{self.transfer_rank}] plan hash {stats['full_hash'][:16]} stats {stats['total']}; {len(self.items)} copy items")
        self.required_param_names = sorted({it.dst_name for it in self.items})
        device = next(iter(local.values())).device if local else torch.device("cpu")
        common = dict(meta=self.meta_server_client, items=self.items, local=local, train_rank=self.rank_info.global_rank,
                      infer_world=self.infer_world_size, device=device, wait_timeout_s=self.timeout)
        from awex_b200.transfer.transports import choose_data_plane

        # the inference side's published choice wins; a contradicting setting here is an error, not a silent mismatch
        mine = os.environ.get("AWEX_DATA_PLANE") or self.config.get("data_plane")
        plane = self.infer_conf.get("data_plane") or choose_data_plane(device.type, self.config.get("data_plane"))
        if mine and mine != plane:
            raise ValueError(f"training side asks for data plane {mine!r} but the inference side published {plane!r}")
        plane = choose_data_plane(device.type, plane)  # refuses peer stores for parameters that are not on a CUDA device
        if plane == "peer_stores":
            from awex_b200.transfer.transports import PeerStoreSender

            self.transport = PeerStoreSender(timeout_ms=self.device_wait_timeout_ms, validate=True, grid=self.grid, **common)
        else:
            from awex_b200.transfer.transports import GlooSender

            self.transport = GlooSender(train_world=self.training_world_size, exchange_timeout_s=self.exchange_timeout_s, **common)
        self.transport.connect()
        logger.info(f"Rank[{self.transfer_rank}] writer ready in {time.time() - t0:.2f}s")

    def _gather_tp_shards(self, name: str, vp_stage: int):
        from awex_b200.converter.mcore_converter import gather_tp_shards

        return gather_tp_shards(self._local[(name, vp_stage)], self.rank_info.tp_size)

    def _follow_moved_sources(self) -> None:
        moved = [key for key, p in self._watched if key in self._local and p.data_ptr() != self._encoded_ptrs[key]]
        if not moved:
            return
        logger.info(f"Rank[{self.transfer_rank}] {len(moved)} training tensors were re-allocated (e.g. {moved[0][0]}); rebuilding the send table")
        kept = {k: t for k, t in self._local.items() if k[0].startswith(DERIVED_PREFIX)}
        fresh = self.local_tensors()
        for key, t in fresh.items():
            old = self._local.get(key)
            if old is not None and (tuple(old.shape) != tuple(t.shape) or old.dtype != t.dtype):
                raise RuntimeError(f"{key[0]} changed shape or dtype ({tuple(old.shape)} {old.dtype} -> {tuple(t.shape)} {t.dtype})")
        self._local.clear()  # the transport holds this very dict
        self._local.update(fresh)
        self._local.update(kept)
        self._encoded_ptrs = {key: p.data_ptr() for key, p in self._watched}
        self.transport.rebind_sources()

    def _write_weights(self, step_id, **kwargs) -> None:
        t0 = time.time()
        self._follow_moved_sources()
        if self.derived:
            with phase("derive_tensors"):
                refresh_derived(self.derived, self._local, self._gather_tp_shards)  # same stream as the transfer: ordered before it
        with phase("send_weights"):
            # the count moves only when an update went out; across processes the transport follows the epoch the
            # inference side announces, so a failed or repeated update on either side cannot put the two out of step
            self.epoch = self.transport.send(self.epoch + 1, synchronize=kwargs.get("synchronize", True))
        compute_statistics(self._history, step_id, time.time() - t0, "Send weights")

    def close(self) -> None:
        if self.transport is not None:
            self.transport.close()
