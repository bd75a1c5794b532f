"""Per-GPU reader that lives inside an inference model worker.

``WorkerWeightsReader.initialize`` maps every parameter of the worker's model
to canonical views (``self.parameters``: canonical name -> live tensor view);
those views are what training ranks write into.  ``NCCLWorkerWeightsReader``
keeps the reference's class name (`awex/reader/nccl_reader.py:49-493`) for the
``nccl`` backend name; on CUDA its data plane is the fused NVLink peer-store
path: it publishes an address book of the views, checks the senders' manifests
for exactly-once coverage and afterwards only raises and waits on flags.
"""

from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch

from awex_b200 import logging
from awex_b200.meta.infer_meta_resolver import canonical_named_views
from awex_b200.meta.meta_server import MetaServerClient
from awex_b200.models.registry import get_infer_weights_converter
from awex_b200.sharding.param_sharding import get_rank_info_extractor
from awex_b200.utils.common import compute_statistics
from awex_b200.utils.trace import phase

logger = logging.getLogger(__name__)


def clear_for_validation(t: torch.Tensor, fill: str = "zero") -> None:
    """Overwrite ``t`` before a validated update: zeros, or with ``fill="poison"``
    NaNs in floating-point tensors (8-bit floats get their NaN bit pattern)."""
    with torch.no_grad():
        if fill == "poison" and t.is_floating_point():
            if t.dtype.itemsize == 1:
                # e4m3fn has no infinities: 0x7f is its NaN; 0x7f is a NaN of e5m2 as well
                t.copy_(torch.full(tuple(t.shape), 0x7F, dtype=torch.uint8, device=t.device).view(t.dtype))
            else:
                t.fill_(float("nan"))
        else:
            t.zero_()


class WorkerWeightsReader:
    def __init__(self, model, model_context: dict, infer_conf: dict, parameters_meta, training_params_meta,
                 engine_rank: int, num_engines: int, meta_server_addr: str, enable_debug_mode: bool = False,
                 debug_mode_config: Optional[dict] = None, enable_colocate_mode: bool = False,
                 device_wait_timeout_ms: int = 2000, **_unused):
        self.model = model
        self.model_context = model_context
        self.scheduler = model_context.get("scheduler")
        self.infer_conf = infer_conf
        self.engine_name = infer_conf["engine_name"]
        self.infer_engine_config = infer_conf["infer_engine_config"]
        self.parameters_meta = parameters_meta
        self.training_params_meta = training_params_meta
        self.engine_rank, self.num_engines = engine_rank, num_engines
        self.meta_server_addr = meta_server_addr
        self.meta_server_client = MetaServerClient(*meta_server_addr.rsplit(":", 1))
        self.enable_debug_mode = enable_debug_mode
        self.debug_mode_config = debug_mode_config or {}
        self.enable_colocate_mode = enable_colocate_mode
        self.device_wait_timeout_ms = device_wait_timeout_ms
        self.rank_info = get_rank_info_extractor(self.engine_name)(model_context, engine_rank)
        self.infer_world_size = int(infer_conf["infer_world_size"])
        self.instance_world_size = self.infer_world_size // num_engines
        self.transfer_rank = engine_rank * self.instance_world_size + self.rank_info.global_rank
        self.training_world_size = training_params_meta[0].shards[0].world_size
        self.timeout = float(self.debug_mode_config.get("host_wait_timeout_s", 10000))
        self.exchange_timeout_s = float(self.debug_mode_config.get("exchange_timeout_s", 1800))
        # what validation leaves in the parameters before the update: "zero" (the reference's choice) or
        # "poison" (NaN bit patterns in floating-point tensors, so that an unwritten shard of a
        # tensor whose true values are zero is caught too)
        self.validation_fill = str(self.debug_mode_config.get("validation_fill", "zero"))
        if self.validation_fill not in ("zero", "poison"):
            raise ValueError(f"debug_mode_config.validation_fill must be 'zero' or 'poison', got {self.validation_fill!r}")
        self.parameters: Dict[str, torch.Tensor] = {}
        self._history: Dict[str, List[float]] = {}
        self._snapshot = None
        self.epoch = 0

    def initialize(self) -> None:
        arch = type(self.model).__name__
        converter = get_infer_weights_converter(
            self.engine_name, arch, hf_config=self.model.config, infer_engine_config=self.infer_engine_config,
            rank_info=self.rank_info,
        )
        self.parameters = dict(canonical_named_views(self.model, converter, self.model_context, convert_params=True))
        train_names = {m.name for m in self.training_params_meta}
        # what training will fill: its names, plus block scales that are produced
        # together with their weights
        aliases = set((self.infer_conf.get("aliased_parameters") or {}))
        self.required_names = [n for n in self.parameters if n in train_names and n not in aliases]
        self.device = next(iter(self.parameters.values())).device if self.parameters else torch.device("cpu")
        self._published_ptrs = self._model_ptrs()

    def _rebind_views(self) -> None:
        """Canonical views of the model as it is now, under the names published before."""
        converter = get_infer_weights_converter(
            self.engine_name, type(self.model).__name__, hf_config=self.model.config, infer_engine_config=self.infer_engine_config,
            rank_info=self.rank_info,
        )
        fresh = dict(canonical_named_views(self.model, converter, self.model_context, convert_params=True))
        if set(fresh) != set(self.parameters):
            raise RuntimeError("the model exposes other parameters than it did when the plan was made")
        for name, t in fresh.items():
            old = self.parameters[name]
            if tuple(t.shape) != tuple(old.shape) or t.dtype != old.dtype:
                raise RuntimeError(f"{name} changed shape or dtype ({tuple(old.shape)} {old.dtype} -> {tuple(t.shape)} {t.dtype})")
        self.parameters = fresh
        self._published_ptrs = self._model_ptrs()
        self._sum_plan = None  # device checksum plans hold the old addresses
        self.transport.rebind(self.parameters)

    def invalidate_addresses(self) -> None:
        """The memory behind the parameters may have been replaced without the
        addresses changing: publish them again before the next update."""
        self._addresses_invalid = True

    def _model_ptrs(self) -> Dict[str, int]:
        """Address of every parameter of the model as it is now.  The canonical
        views keep the storages alive that they were cut from, so only the model
        itself shows whether the engine has re-allocated or re-mapped its weights."""
        return {name: p.data_ptr() for name, p in self.model.named_parameters()}

    def parameters_moved(self) -> List[str]:
        now = self._model_ptrs()
        return [n for n, ptr in self._published_ptrs.items() if now.get(n) != ptr] + [n for n in now if n not in self._published_ptrs]

    # ---- update -----------------------------------------------------------------------------------
    def begin_update(self, step_id) -> None:
        raise NotImplementedError

    def finish_update(self, step_id, synchronize: bool = True) -> None:
        raise NotImplementedError

    def update_weights(self, step_id) -> None:
        t0 = time.time()
        self.begin_update(step_id)
        self.finish_update(step_id)
        compute_statistics(self._history, step_id, time.time() - t0, "Receive weights")

    def _after_update(self) -> None:
        """Caches computed with the old weights are stale."""
        if self.scheduler is not None and hasattr(self.scheduler, "flush_cache"):
            flushed = self.scheduler.flush_cache()
            logger.info(f"Rank[{self.transfer_rank}] flushed the engine's caches after the update (flush_cache returned {flushed!r})")

    def dump_parameters(self, step_id, names, directory: str) -> List[str]:
        """Save the received canonical tensors named in ``names`` (as
        ``reader_<pid>_from_commu_<step>.<name>.pt``, the reference's file names,
        `awex/reader/weights_reader.py:533-545`) for offline comparison with the
        writer's dumps."""
        import os

        os.makedirs(directory, exist_ok=True)
        written = []
        for name in names:
            tensor = self.parameters.get(name)
            if tensor is None:
                continue
            path = os.path.abspath(os.path.join(directory, f"reader_{os.getpid()}_from_commu_{step_id}.{name}.pt"))
            torch.save(tensor.detach().cpu().contiguous(), path)
            written.append(path)
            logger.info(f"[Reader] saved parameter {name} to {path}")
        return written

    # ---- validation detail: what differs in parameters that failed ----------------------------------
    def stash_received(self, names) -> int:
        """Copy the current (received) values of ``names`` to the host."""
        self._stash = {n: self.parameters[n].detach().to("cpu", copy=True) for n in names if n in self.parameters}
        return len(self._stash)

    def diff_against_stash(self) -> Dict[str, bool]:
        """The parameters now hold the oracle again (the checkpoint was re-loaded):
        log how the stashed, received values differ from it, then put the received
        values back."""
        from awex_b200.utils.tensor_util import compare_and_log_tensor_differences

        stash, self._stash = getattr(self, "_stash", {}) or {}, {}
        verdicts = {}
        with torch.no_grad():
            for name, received in stash.items():
                live = self.parameters[name]
                oracle = live.detach().to("cpu", copy=True)
                if received.dtype.itemsize == 1 and received.is_floating_point():  # 8-bit floats: compare what they decode to
                    verdicts[name] = compare_and_log_tensor_differences(received.float(), oracle.float(), name, exact_match=True)
                else:
                    verdicts[name] = compare_and_log_tensor_differences(received, oracle, name, exact_match=True)
                live.copy_(received.to(live.device))
        return verdicts

    # ---- validation: record, clear, compare ----------------------------------------------------------
    def _validation_tensors(self):
        names = sorted(self.required_names)
        return names, [self.parameters[n] for n in names]

    def snapshot_and_clear(self) -> int:
        """Record what every parameter holds (device checksums on CUDA, host
        copies on CPU), then zero it, so that an unwritten shard cannot pass."""
        names, tensors = self._validation_tensors()
        if self.device.type == "cuda":
            from awex_b200.ops.checksum import ChecksumPlan

            if getattr(self, "_sum_plan", None) is None:
                self._sum_plan = ChecksumPlan(tensors, self.device)
            self._snapshot = (names, self._sum_plan.run())
        else:
            self._snapshot = (names, [t.detach().clone() for t in tensors])
        for t in tensors:
            clear_for_validation(t, self.validation_fill)
        return len(names)

    def verify_against_snapshot(self) -> Dict[str, bool]:
        if self._snapshot is None:
            raise RuntimeError("verify_against_snapshot called without snapshot_and_clear")
        names, before = self._snapshot
        _, tensors = self._validation_tensors()
        if self.device.type == "cuda":
            sums, nans = self._sum_plan.run()
            want_sums, _ = before
            result = {n: (s == w and k == 0) for n, s, w, k in zip(names, sums, want_sums, nans)}
        else:
            from awex_b200.utils.tensor_util import check_and_log_nan_values, compare_and_log_tensor_differences

            check_and_log_nan_values(dict(zip(names, tensors)), "infer")
            result = {n: compare_and_log_tensor_differences(t, w, n, exact_match=True) for n, t, w in zip(names, tensors, before)}
        self._snapshot = None
        return result


class NCCLWorkerWeightsReader(WorkerWeightsReader):
    def initialize(self) -> None:
        super().initialize()
        t0 = time.time()
        common = dict(
            meta=self.meta_server_client, views=self.parameters, transfer_rank=self.transfer_rank,
            infer_world=self.infer_world_size, train_world=self.training_world_size, required=self.required_names,
            device=self.device, wait_timeout_s=self.timeout, strict=not self.enable_debug_mode,
        )
        from awex_b200.transfer.transports import choose_data_plane

        plane = self.infer_conf.get("data_plane") or choose_data_plane(self.device.type, self.debug_mode_config.get("data_plane"))
        if plane == "peer_stores":
            from awex_b200.transfer.transports import PeerStoreReceiver

            self.transport = PeerStoreReceiver(timeout_ms=self.device_wait_timeout_ms,
                                               may_move=bool(self.debug_mode_config.get("parameters_may_move", False)), **common)
        else:
            from awex_b200.transfer.transports import GlooReceiver

            self.transport = GlooReceiver(exchange_timeout_s=self.exchange_timeout_s, **common)
        self.transport.connect()
        # epochs only grow, also across a reader that replaces an earlier one of the same rank
        self.epoch = max(self.epoch, int(getattr(self.transport, "epoch_base", 0)))
        logger.info(f"Rank[{self.transfer_rank}] reader ready in {time.time() - t0:.2f}s, {len(self.parameters)} canonical views")

    def begin_update(self, step_id) -> None:
        # Every attempt gets a new epoch, also one that fails below: flags of an abandoned attempt can then
        # never satisfy a later wait.  Senders take the epoch from this side's announcement, so their own
        # count cannot fall out of step with it.
        self.epoch += 1
        moved = self.parameters_moved()
        if moved and getattr(self.transport, "may_move", False):
            # the engine re-allocated or re-mapped its weights (sleep / wake-up): cut the canonical views again;
            # the transport publishes their addresses and the senders rebuild their tables before they write
            logger.info(f"Rank[{self.transfer_rank}] {len(moved)} parameters moved; publishing their new addresses")
            self._rebind_views()
        elif moved:
            raise RuntimeError(
                f"{len(moved)} inference parameters (e.g. {moved[:3]}) moved since they were published; senders hold "
                "stale addresses (re-create the writer and reader after the engine re-maps its weights, or set "
                "debug_mode_config['parameters_may_move'] on the inference side)"
            )
        if getattr(self, "_addresses_invalid", False):
            if not getattr(self.transport, "may_move", False):
                raise RuntimeError("invalidate_addresses() needs debug_mode_config['parameters_may_move'] on the inference side")
            self._rebind_views()
            self.transport.republish_if_moved(force=True)
            self._addresses_invalid = False
        with phase("announce_ready"):
            self.transport.begin(self.epoch)

    def finish_update(self, step_id, synchronize: bool = True) -> None:
        with phase("receive_weights"):
            self.transport.finish(self.epoch, synchronize=synchronize)
        self._after_update()

    def close(self) -> None:
        self.transport.close()
