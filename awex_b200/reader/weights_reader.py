"""Inference-side half of a weight exchange.

:class:`WeightsReader` lives in the inference engine's control process.  It
resolves the inference metadata, trades it with the training side through the
MetaServer and installs one :class:`WorkerWeightsReader` per model worker
(GPU); every update is then a task executed inside the workers.  Behavioural
contract: `awex/reader/weights_reader.py:52-815` in the reference, including
the worker attribute name ``scheduler.awes_weights_reader`` and the cache flush
after each update.

For deployments where a training rank and an inference worker share one
process (one process per GPU doing both jobs), ``begin_update`` /
``finish_update`` split an update so that the caller can launch the training
side's write between them on the same stream; ``update_weights`` is the two
back to back.
"""

from __future__ import annotations

import os
import pickle
import threading
import time
from abc import ABC, abstractmethod
from typing import Dict, List, Optional, Sequence

import torch

from awex_b200 import logging
from awex_b200.meta.infer_meta_resolver import InferParamMetaResolver, canonical_named_views
from awex_b200.meta.meta_server import MetaServerClient
from awex_b200.meta.weight_meta import ParameterMeta
from awex_b200.utils import device as device_util
from awex_b200.utils.common import check_train_infer_params_meta, compute_statistics, simple_hf_config

logger = logging.getLogger(__name__)


def derive_expected_pp_ranks(infer_params_meta: Sequence[ParameterMeta], local_engine_rank: int) -> List[int]:
    """Pipeline stages that hold parameters of engine ``local_engine_rank``."""
    stages = {s.pp_rank for p in infer_params_meta for s in p.shards if s.engine_rank == local_engine_rank}
    if not stages:
        raise ValueError(f"No infer shards found for engine_rank={local_engine_rank}; cannot derive expected_pp_ranks")
    return sorted(stages)


class WeightExchangeReader(ABC):
    def __init__(self, inference_engine):
        self.inference_engine = inference_engine
        self.infer_config = inference_engine.config
        self.enable_colocate_mode = bool(self.infer_config.enable_colocate_mode)
        self.weights_comm_nccl_group_size = self.infer_config.weights_comm_nccl_group_size

    @abstractmethod
    def initialize(self, **kwargs): ...

    @abstractmethod
    def update_weights(self, step_id, **kwargs): ...


class FileWeightExchangeReader(WeightExchangeReader):
    """``comm_backend="file"``: load an HF checkpoint with the engine's loader."""

    def initialize(self, **kwargs):
        pass

    def update_weights(self, step_id, **kwargs):
        path = kwargs.get("path")
        if not path:
            raise ValueError("the file backend needs update_weights(step_id, path=...)")
        self.inference_engine.update_weights_from_disk(path, kwargs.get("load_format"))


def _worker_reader(kwargs):
    return kwargs["model_context"]["scheduler"].awes_weights_reader


class WeightsReader(WeightExchangeReader):
    def __init__(self, inference_engine, meta_resolver: InferParamMetaResolver = None):
        super().__init__(inference_engine)
        config = inference_engine.config
        self.infer_engine_config = config
        self.meta_resolver = meta_resolver or InferParamMetaResolver(
            inference_engine, num_engines=inference_engine.num_engines, engine_rank=inference_engine.engine_rank, convert_params=True
        )
        self.parameters_meta: List[ParameterMeta] = []
        self.hf_config = inference_engine.hf_config
        self.model_arch_name = self.meta_resolver.get_model_arch_name()
        self.meta_server_addr = config.meta_server_addr
        self.meta_server_client = MetaServerClient(*self.meta_server_addr.rsplit(":", 1))
        self.num_engines = config.num_engines
        self.engine_rank = inference_engine.engine_rank
        self.tp_size = config.tp_size or 1
        self.pp_size = config.pp_size or 1
        # one engine with internal data parallelism still contributes dp_size
        # copies of every rank to the exchange
        self.dp_size = max(1, int(getattr(config, "dp_size", 1) or 1))
        self.infer_world_size = self.num_engines * self.tp_size * self.pp_size * self.dp_size
        self.validated_steps = 0
        self.start_step = -1
        self.last_validation_failed: List[str] = []  # names that differed in the most recent validated update
        self.weights_validation_steps = config.weights_validation_steps
        self.validate_weights_every_n_steps = config.validate_weights_every_n_steps
        self.dump_weights_list_for_validation = config.dump_weights_list_for_validation
        self.dump_weights_dir_for_validation = config.dump_weights_dir_for_validation or os.getcwd()
        self.debug_mode_config = config.debug_mode_config or {}
        self.raise_on_validation_fail = self.debug_mode_config.get("raise_on_validation_fail", False)
        self.ipc_backend = config.weights_exchange_ipc_backend
        self.timeout = float(self.debug_mode_config.get("host_wait_timeout_s", 10000))
        self.lock = threading.Lock()
        self.initialized = False
        self.expected_pp_ranks: List[int] = []
        self._history: Dict[str, List[float]] = {}

    # ---- discovery -----------------------------------------------------------------------------
    def initialize(self, **kwargs):
        meta = self.meta_server_client
        meta.put_object("num_infer_engines", self.num_engines)
        if self.enable_colocate_mode:
            self.inference_engine.release_memory_occupation()
        meta.add_object_to_set("num_inited_inference_engines", self.engine_rank)

    def _initialize(self) -> None:
        meta = self.meta_server_client
        self.parameters_meta = self.meta_resolver.get_parameters_meta()
        self.expected_pp_ranks = derive_expected_pp_ranks(self.parameters_meta, self.engine_rank)
        config = self.inference_engine.config
        self.infer_conf = {
            "engine_name": self.inference_engine.engine_name,
            "infer_atten_tp_size": self.meta_resolver.rank0_info.attn_tp_size,
            "router_dtype": self._router_dtype(),
            "infer_engine_config": self.infer_engine_config,
            "hf_config": simple_hf_config(self.hf_config) if hasattr(self.hf_config, "to_dict") else self.hf_config,
            "infer_world_size": self.infer_world_size,
            "expected_pp_ranks": self.expected_pp_ranks,
            "device_backend": device_util.get_device_type(),
            "fp8_block_quant": bool(getattr(config, "fp8_block_quant", False)),
            # how tensors travel (peer stores inside one machine, messages across machines); the training side follows
            "data_plane": self._data_plane(),
            # second names of memory that another name already covers: nobody sends them
            "aliased_parameters": dict(getattr(self.meta_resolver, "aliases", {}) or {}),
        }
        meta.put_object("infer_conf", self.infer_conf)
        if self.engine_rank == 0:
            meta.put_object("infer_params_meta", self.parameters_meta)
        self.training_params_meta = meta.get_object("training_params_meta", timeout=self.timeout)
        self.training_world_size = self.training_params_meta[0].shards[0].world_size
        check_train_infer_params_meta(self.training_params_meta, self.parameters_meta, raise_exception=not config.enable_debug_mode)
        self.inference_engine.execute_task_in_model_worker(
            self._init_in_tp_worker,
            infer_conf_bytes=pickle.dumps(self.infer_conf),
            parameters_meta_bytes=pickle.dumps(self.parameters_meta),
            training_params_meta_bytes=pickle.dumps(self.training_params_meta),
            engine_rank=self.engine_rank,
            num_engines=self.num_engines,
            meta_server_addr=self.meta_server_addr,
            weights_comm_backend=config.comm_backend,
            enable_debug_mode=config.enable_debug_mode,
            debug_mode_config=config.debug_mode_config,
            disable_pipeline=config.disable_weights_exchange_pipeline,
            enable_colocate_mode=self.enable_colocate_mode,
            ipc_backend=self.ipc_backend,
            weights_comm_nccl_group_size=self.weights_comm_nccl_group_size,
            device_wait_timeout_ms=getattr(config, "device_wait_timeout_ms", 2000),
        )

    def _data_plane(self) -> Optional[str]:
        """The configured data plane (``debug_mode_config["data_plane"]`` or
        ``AWEX_DATA_PLANE``), or None: each side then picks by the device its
        tensors live on (peer stores on CUDA, messages on CPU)."""
        from awex_b200.transfer.transports import DATA_PLANES

        choice = os.environ.get("AWEX_DATA_PLANE") or self.debug_mode_config.get("data_plane")
        if choice is not None and choice not in DATA_PLANES:
            raise ValueError(f"data plane must be one of {DATA_PLANES}, got {choice!r}")
        return choice

    def _router_dtype(self) -> str:
        """Dtype the training side casts MoE router weights to: the model
        config's ``router_dtype`` if it names one (as the reference reads it),
        else whatever dtype the engine actually holds its router weights in."""
        named = getattr(self.hf_config, "router_dtype", None)
        if named:
            return named
        for meta in self.parameters_meta:
            if meta.name.endswith(("mlp.gate.weight", "mlp.router.weight")):
                return {torch.float32: "fp32", torch.float16: "fp16"}.get(meta.dtype, "bf16")
        return "bf16"

    @staticmethod
    def _init_in_tp_worker(**kwargs):
        """Runs inside a model worker: build the per-GPU reader and keep it on
        the scheduler."""
        from awex_b200.reader.nccl_reader import NCCLWorkerWeightsReader

        ctx = kwargs["model_context"]
        backend = kwargs.get("weights_comm_backend", "nccl")
        if backend == "astate":
            from awex_b200.reader.astate_reader import AStateWorkerWeightsReader as worker_cls
        elif backend in ("nccl", "p2p", "gloo"):
            worker_cls = NCCLWorkerWeightsReader
        else:
            raise NotImplementedError(f"worker reader for comm_backend {backend!r} is not available")
        reader = worker_cls(
            model=kwargs["model"], model_context=ctx,
            infer_conf=pickle.loads(kwargs["infer_conf_bytes"]),
            parameters_meta=pickle.loads(kwargs["parameters_meta_bytes"]),
            training_params_meta=pickle.loads(kwargs["training_params_meta_bytes"]),
            engine_rank=kwargs["engine_rank"], num_engines=kwargs["num_engines"],
            meta_server_addr=kwargs["meta_server_addr"], enable_debug_mode=kwargs.get("enable_debug_mode", False),
            debug_mode_config=kwargs.get("debug_mode_config") or {}, enable_colocate_mode=kwargs.get("enable_colocate_mode", False),
            device_wait_timeout_ms=kwargs.get("device_wait_timeout_ms", 2000),
        )
        ctx["scheduler"].awes_weights_reader = reader
        reader.initialize()
        return True

    # ---- worker tasks (module-level behaviour, shipped by qualified name) --------------------------
    @staticmethod
    def _begin_update_in_tp_worker(step_id, **kwargs):
        _worker_reader(kwargs).begin_update(step_id)
        return True

    @staticmethod
    def _finish_update_in_tp_worker(step_id, synchronize=True, **kwargs):
        _worker_reader(kwargs).finish_update(step_id, synchronize=synchronize)
        return True

    @staticmethod
    def _invalidate_addresses_in_tp_worker(**kwargs):
        _worker_reader(kwargs).invalidate_addresses()
        return True

    def invalidate_addresses(self) -> None:
        """Tell every worker that the memory behind its parameters may be new even
        where the addresses are the same (an allocator that re-creates physical
        memory at fixed virtual addresses after a sleep / wake-up cycle): the next
        update publishes fresh address books and the senders map them again.  Needs
        ``debug_mode_config["parameters_may_move"]``."""
        if self.initialized:
            self.inference_engine.execute_task_in_model_worker(self._invalidate_addresses_in_tp_worker)

    @staticmethod
    def _update_parameters_in_tp_worker(step_id, **kwargs):
        _worker_reader(kwargs).update_weights(step_id)
        return True

    @staticmethod
    def _pre_validate_weights_on_tp_worker(**kwargs):
        return _worker_reader(kwargs).snapshot_and_clear()

    @staticmethod
    def _verify_weights_on_tp_worker(step_id=None, dump_weights_list_for_validation=None, dump_weights_dir_for_validation=None, **kwargs):
        worker = _worker_reader(kwargs)
        if dump_weights_list_for_validation:
            worker.dump_parameters(step_id, dump_weights_list_for_validation, dump_weights_dir_for_validation or os.getcwd())
        return worker.verify_against_snapshot()

    @staticmethod
    def _stash_for_diff_on_tp_worker(names=None, **kwargs):
        return _worker_reader(kwargs).stash_received(names or [])

    @staticmethod
    def _diff_against_stash_on_tp_worker(**kwargs):
        return _worker_reader(kwargs).diff_against_stash()

    # ---- per step -------------------------------------------------------------------------------------
    def _ensure_initialized(self) -> None:
        if not self.initialized:
            self._initialize()
            self.initialized = True

    def prepare(self) -> None:
        """Run the one-time metadata exchange and worker set-up now instead of
        on the first update (blocks until the training side has published)."""
        with self.lock:
            self._ensure_initialized()

    def begin_update(self, step_id, **kwargs) -> None:
        """First half of an update: pause-side bookkeeping, validation snapshot,
        and the announcement that parameters may be overwritten."""
        self._ensure_initialized()
        if self.enable_colocate_mode:
            self.inference_engine.release_memory_occupation()
            self._pre_update_weights()
        self._validating = self._should_validate(step_id)
        self._validation_path = (kwargs.get("path"), kwargs.get("load_format")) if self._validating else (None, None)
        if self._validating:
            self._pre_validate_weights(step_id, **kwargs)
        self.inference_engine.execute_task_in_model_worker(self._begin_update_in_tp_worker, step_id=step_id)

    def finish_update(self, step_id, **kwargs) -> None:
        """Second half: wait until every sender has finished, flush caches,
        validate."""
        self.inference_engine.execute_task_in_model_worker(
            self._finish_update_in_tp_worker, step_id=step_id, synchronize=kwargs.get("synchronize", True)
        )
        if self._validating:
            self._validate_weights(step_id)
        if self.enable_colocate_mode:
            self._post_update_weights()

    def update_weights(self, step_id, **kwargs):
        with self.lock:
            t0 = time.time()
            try:
                self.begin_update(step_id, **kwargs)
                self.finish_update(step_id, **kwargs)
            except Exception as exc:
                logger.exception(f"Error in update_weights: {exc}")
                raise
            compute_statistics(self._history, step_id, time.time() - t0, "Update weights")

    # ---- co-located hand-off (`awex/reader/weights_reader.py:337-359,589-617`) -------------------------
    def _pre_update_weights(self) -> None:
        meta = self.meta_server_client
        meta.wait_set_until_size("all_training_offloaded_optimizers", 1, timeout=self.timeout)
        self.inference_engine.resume_memory_occupation(tags=["weights"])

    def _post_update_weights(self) -> None:
        self.meta_server_client.add_object_to_set("finished_weights_update_engines", self.engine_rank)
        self.inference_engine.resume_memory_occupation(tags=["kv_cache"])

    # ---- validation (`awex/reader/weights_reader.py:361-587`) ------------------------------------------
    def _should_validate(self, step_id) -> bool:
        if self.start_step < 0:
            self.start_step = step_id
        if self.validated_steps >= self.weights_validation_steps:
            return False
        return (step_id - self.start_step) % max(self.validate_weights_every_n_steps, 1) == 0

    def _pre_validate_weights(self, step_id, **kwargs) -> None:
        """With a ``path`` the engine first loads the file-written checkpoint:
        that load is the oracle.  Either way every worker then records what it
        holds and clears it, so that a shard nobody writes is a visible failure."""
        self.validated_steps += 1
        path = kwargs.get("path")
        meta = self.meta_server_client
        if path:
            deadline = time.time() + self.timeout
            while not meta.has_key("weights_ready_for_load"):
                if time.time() > deadline:
                    raise TimeoutError("training side never published weights_ready_for_load")
                time.sleep(0.2)
            self.inference_engine.update_weights_from_disk(path, kwargs.get("load_format"))
        self.inference_engine.execute_task_in_model_worker(self._pre_validate_weights_on_tp_worker)
        if path:
            meta.add_object_to_set("weights_ready_for_send", self.engine_rank)
            meta.wait_set_until_size("weights_ready_for_send", self.num_engines, timeout=self.timeout)

    def _validate_weights(self, step_id) -> bool:
        results = self.inference_engine.execute_task_in_model_worker(
            self._verify_weights_on_tp_worker, step_id=step_id,
            dump_weights_list_for_validation=list(self.dump_weights_list_for_validation or []),
            dump_weights_dir_for_validation=self.dump_weights_dir_for_validation,
        )
        failed = sorted({name for worker in results for name, ok in worker.items() if not ok})
        verdict = "PASSED" if not failed else "FAILED"
        logger.info(f"[Validation] step {step_id} {verdict}" + (f": {len(failed)} mismatching parameters, e.g. {failed[:8]}" if failed else ""))
        self.last_validation_failed = failed
        if failed:
            self._log_detailed_differences(step_id, failed)
        if failed and self.raise_on_validation_fail:
            raise RuntimeError(f"weights validation failed at step {step_id}: {failed[:8]}")
        return not failed


def _attach_detail_logger():
    def _log_detailed_differences(self, step_id, failed) -> None:
        """What differs in the parameters that failed (the reference logs max / mean
        absolute and relative differences and the first differing positions for each,
        `awex/reader/weights_reader.py:510-587`).  On CUDA the comparison itself only
        moves checksums, so the values it was made against are gone: when the update
        was validated against a checkpoint, the workers set the received values of the
        failed parameters aside on the host, the engine loads the checkpoint once more,
        the workers log the differences, and the received values are put back.  Only
        the failed parameters are copied."""
        path, load_format = getattr(self, "_validation_path", (None, None))
        if not path:
            logger.info(f"[Validation] step {step_id}: no checkpoint to compare with; per-element differences are not available "
                        "(validate with a path, or on CPU, to get them)")
            return
        try:
            self.inference_engine.execute_task_in_model_worker(self._stash_for_diff_on_tp_worker, names=list(failed))
            self.inference_engine.update_weights_from_disk(path, load_format)
            self.inference_engine.execute_task_in_model_worker(self._diff_against_stash_on_tp_worker)
        except Exception as exc:  # the verdict stands; the detail is best effort
            logger.warning(f"[Validation] step {step_id}: could not produce per-element differences: {exc!r}")

    WeightsReader._log_detailed_differences = _log_detailed_differences


_attach_detail_logger()


def get_weights_exchange_reader(inference_engine):
    backend = inference_engine.config.comm_backend
    if backend == "file":
        return FileWeightExchangeReader(inference_engine)
    if backend == "astate":
        from awex_b200.reader.astate_reader import AStateWeightsReader

        return AStateWeightsReader(inference_engine)
    if backend == "hccl":
        raise NotImplementedError("the hccl (Ascend) backend is not part of this CUDA-only framework")
    return WeightsReader(inference_engine)
