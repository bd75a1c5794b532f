"""Training-side half of a weight exchange.

``WeightExchangeWriter`` is the contract (``initialize`` / ``write_weights``);
:class:`FileWeightExchangeWriter` saves a Hugging Face checkpoint on a shared
file system; :class:`WeightsExchangeShardingWriter` does everything that is
independent of the data plane: lazy metadata exchange through the MetaServer,
converter construction, per-step locking, validation hooks and the co-located
memory hand-off.  Behavioural contract: `awex/writer/weights_writer.py:52-522`
in the reference.
"""

from __future__ import annotations

import os
import threading
import time
from abc import ABC, abstractmethod
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from awex_b200 import logging
from awex_b200.meta.meta_server import MetaServerClient
from awex_b200.meta.train_meta_resolver import McoreParamMetaResolver, resolve_train_rank_info
from awex_b200.models.registry import get_train_weights_converter
from awex_b200.utils.common import check_train_infer_params_meta, compute_statistics, from_binary

logger = logging.getLogger(__name__)


class WeightExchangeWriter(ABC):
    def __init__(self, train_engine):
        self.train_engine = train_engine
        self.enable_colocate_mode = bool(getattr(train_engine, "enable_colocate_mode", False))
        self.enable_debug_mode = bool(getattr(train_engine, "enable_debug_mode", False))

    @abstractmethod
    def initialize(self, **kwargs): ...

    @abstractmethod
    def write_weights(self, step_id, **kwargs): ...


class FileWeightExchangeWriter(WeightExchangeWriter):
    """``comm_backend="file"``: the training engine writes an HF checkpoint to
    ``path``; the reader loads it with the engine's own loader."""

    def initialize(self, **kwargs):
        pass

    def write_weights(self, step_id, **kwargs):
        path = kwargs.get("path")
        if not path:
            raise ValueError("the file backend needs write_weights(step_id, path=...)")
        self.train_engine.save_hf_checkpoint(path)


class WeightsExchangeShardingWriter(WeightExchangeWriter):
    def __init__(self, train_engine):
        super().__init__(train_engine)
        self.meta_server_addr = train_engine.meta_server_addr
        self.meta_server_client = MetaServerClient(*self.meta_server_addr.rsplit(":", 1))
        self.infer_conf = None
        self.infer_engine_config = None
        model = train_engine.model
        self.model = list(model) if isinstance(model, (list, tuple)) else [model]
        self.hf_config = train_engine.hf_config
        self.model_arch_name = self.hf_config.architectures[0]
        self.comm_backend = getattr(train_engine, "comm_backend", "nccl")
        self.config: Dict = train_engine.config if isinstance(train_engine.config, dict) else {}
        get = self.config.get
        self.weights_validation_steps = get("weights_validation_steps", 0)
        self.validate_weights_every_n_steps = get("validate_weights_every_n_steps", 1)
        self.dump_weights_for_validation = get("dump_weights_for_validation", False)
        self.dump_weights_list_for_validation = get("dump_weights_list_for_validation", [])
        self.dump_weights_dir_for_validation = get("dump_weights_dir_for_validation", os.getcwd())
        # accepted for compatibility; the fused data plane has no pipeline to disable
        self.disable_pipeline = get("disable_weights_exchange_pipeline", False)
        self.enable_nccl_debug_mode = get("debug_mode_config", {}).get("enable_nccl_debug_mode", False)
        self.raise_on_validation_fail = get("debug_mode_config", {}).get("raise_on_validation_fail", False)
        self.device_wait_timeout_ms = int(get("device_wait_timeout_ms", 2000))
        self.validated_steps = 0
        self.start_step = -1
        self.lock = threading.Lock()
        # how long host-side waits for the other side last (metadata, address books, co-located hand-off)
        self.timeout = float(get("host_wait_timeout_s", 10000))
        # timeout of collectives and messages of the exchange group (message transport)
        self.exchange_timeout_s = float(get("exchange_timeout_s", 1800))
        self.initialized = False
        self.num_infer_engines = None
        self.engine_name = train_engine.engine_name
        self.enable_mem_debug = os.environ.get("AWEX_MEM_DEBUG", "0") == "1"
        self._history: Dict[str, List[float]] = {}
        self.process_group = getattr(train_engine, "process_group", None)

    # ---- helpers ---------------------------------------------------------------------------
    def _train_barrier(self) -> None:
        if dist.is_initialized() and dist.get_world_size(self.process_group) > 1:
            dist.barrier(group=self.process_group)

    def initialize(self, **kwargs):
        """Nothing to do eagerly: the metadata exchange needs a reader that has
        loaded its model, so it happens on the first ``write_weights``."""

    def prepare(self) -> None:
        """Run the one-time metadata exchange and program compilation now
        instead of on the first ``write_weights`` (blocks until a reader has
        published its side)."""
        with self.lock:
            if not self.initialized:
                self._initialize()
                self.initialized = True

    def _initialize(self) -> None:
        meta = self.meta_server_client
        self.infer_conf = meta.get_object("infer_conf", timeout=self.timeout)
        self.infer_engine_config = self.infer_conf.get("infer_engine_config")
        self.rank_info = resolve_train_rank_info(self.train_engine)
        self.infer_world_size = int(self.infer_conf["infer_world_size"])
        self.training_world_size = self.rank_info.world_size
        self.transfer_rank = self.infer_world_size + self.rank_info.global_rank
        resolver = McoreParamMetaResolver(self.train_engine, self.hf_config, self.infer_conf)
        self.meta_resolver = resolver
        self.parameters_meta = resolver.get_parameters_meta()
        self.all_train_ranks = [m["rank_info"] for m in resolver._get_params_raw_meta()]
        if self.rank_info.global_rank == 0:
            meta.put_object("training_params_meta", self.parameters_meta)
            meta.put_object("training_rank_infos", self.all_train_ranks)
        self.infer_params_meta = from_binary(meta.get_binary("infer_params_meta", timeout=self.timeout))
        check_train_infer_params_meta(self.parameters_meta, self.infer_params_meta, raise_exception=not self.enable_debug_mode)
        self.pp_stage_layer_id_map = resolver.get_pp_stage_layer_id_map()
        self.weight_converter = self._make_converter(self.rank_info)
        tp_group = getattr(self.train_engine, "tp_group", None)
        if tp_group is not None:  # materialised conversion (dumps, file oracle) gathers over it
            from awex_b200.converter.mcore_converter import set_train_tp_group

            set_train_tp_group(tp_group, self.rank_info.tp_size)
        self.num_infer_engines = meta.get_object("num_infer_engines", timeout=self.timeout)

    def _make_converter(self, rank_info):
        conf = {**self.infer_conf, "train_pp_stage_layer_id_map": self.pp_stage_layer_id_map}
        return get_train_weights_converter(
            self.engine_name, self.model_arch_name, self.hf_config, rank_info, conf, tf_config=self.meta_resolver._tf_config
        )

    def local_tensors(self) -> Dict:
        from awex_b200.converter.mcore_converter import get_mcore_model_parameters

        return {
            (name, vp): (p.detach() if p.requires_grad else p)
            for vp, chunk in enumerate(self.model)
            for name, p in get_mcore_model_parameters(chunk).items()
        }

    @torch.no_grad()
    def convert_parameters(self, required_names=None) -> Dict[str, torch.Tensor]:
        """Materialised canonical tensors of this rank (collective over the
        training TP group for gathered layouts).  Used by dumps and the file
        oracle; the transfer path does not call it."""
        from awex_b200.converter.mcore_converter import get_mcore_model_parameters

        out: Dict[str, torch.Tensor] = {}
        tied = bool(getattr(self.hf_config, "tie_word_embeddings", False))
        last = self.rank_info.pp_rank == self.rank_info.pp_size - 1
        for vp, chunk in enumerate(self.model):
            for name, p in get_mcore_model_parameters(chunk).items():
                for cname, tensor in self.weight_converter.convert_param(name, p.detach(), vp_stage=vp):
                    if required_names is None or cname in required_names:
                        out[cname] = tensor
        if tied and last and "lm_head.weight" not in out and "model.embed_tokens.weight" in out:
            out["lm_head.weight"] = out["model.embed_tokens.weight"]
        return out

    # ---- per step ------------------------------------------------------------------------------
    @torch.no_grad()
    def write_weights(self, step_id, **kwargs):
        with self.lock:
            try:
                if self.enable_colocate_mode:
                    self._release_memory_for_weights_exchange()
                if not self.initialized:
                    self._initialize()
                    self.initialized = True
                self._validate_weights(step_id, **kwargs)
                t0 = time.time()
                if self.enable_colocate_mode:
                    self.train_engine.resume_memory_occupation(tags=["weights"])
                self._write_weights(step_id, **kwargs)
                self._finish_weights_update()
                compute_statistics(self._history, step_id, time.time() - t0, "Write weights")
            except Exception as exc:
                logger.exception(f"Error in write_weights: {exc}")
                raise

    @abstractmethod
    def _write_weights(self, step_id, **kwargs): ...

    # ---- co-located memory hand-off (`awex/writer/weights_writer.py:329-372`) -----------------------
    def _release_memory_for_weights_exchange(self) -> None:
        meta = self.meta_server_client
        if self.num_infer_engines is None:
            self.num_infer_engines = meta.get_object("num_infer_engines", timeout=self.timeout)
            meta.wait_set_until_size("num_inited_inference_engines", self.num_infer_engines, timeout=self.timeout)
        self.train_engine.release_memory_occupation(tags=["optimizer"])
        self.train_engine.resume_memory_occupation(tags=["weights"])
        self._train_barrier()
        rank = dist.get_rank(self.process_group) if dist.is_initialized() else 0
        if rank == 0:
            meta.add_object_to_set("all_training_offloaded_optimizers", rank)

    def _finish_weights_update(self) -> None:
        if not self.enable_colocate_mode:
            return
        meta = self.meta_server_client
        meta.wait_set_until_size("finished_weights_update_engines", self.num_infer_engines, timeout=self.timeout)
        self._train_barrier()
        rank = dist.get_rank(self.process_group) if dist.is_initialized() else 0
        if rank == 0:
            for key in ("finished_weights_update_engines", "all_training_offloaded_optimizers", "all_training_offloaded_weights"):
                meta.delete_if_exists(key)

    # ---- validation against a file-loaded reference (`weights_writer.py:420-500`) ---------------------
    def _should_validate(self, step_id) -> bool:
        if self.start_step < 0:
            self.start_step = step_id
        if self.validated_steps >= self.weights_validation_steps:
            return False
        return (step_id - self.start_step) % max(self.validate_weights_every_n_steps, 1) == 0

    def _validate_weights(self, step_id, **kwargs) -> None:
        if not self._should_validate(step_id):
            return
        self.validated_steps += 1
        path = kwargs.get("path")
        if self.dump_weights_for_validation or self.dump_weights_list_for_validation:
            self._dump_weights(step_id)
        if not path:
            return  # the reader validates against its own snapshot
        from awex_b200.utils.tensor_util import check_and_log_nan_values

        check_and_log_nan_values({k[0]: v for k, v in self.local_tensors().items()}, "train")
        self.train_engine.save_hf_checkpoint(path)
        self._train_barrier()
        meta = self.meta_server_client
        if self.rank_info.global_rank == 0:
            meta.put_object("weights_ready_for_load", True)
            meta.wait_set_until_size("weights_ready_for_send", self.num_infer_engines, timeout=self.timeout)
            meta.delete_if_exists("weights_ready_for_load")
            meta.delete_if_exists("weights_ready_for_send")
        self._train_barrier()

    def _dump_weights(self, step_id) -> None:
        wanted = set(self.dump_weights_list_for_validation or [])
        os.makedirs(self.dump_weights_dir_for_validation, exist_ok=True)
        native = {k[0]: v.detach().cpu() for k, v in self.local_tensors().items() if not wanted or k[0] in wanted}
        converted = {k: v.detach().cpu() for k, v in self.convert_parameters().items() if not wanted or k in wanted}
        base = os.path.join(self.dump_weights_dir_for_validation, f"train_step{step_id}_rank{self.rank_info.global_rank}")
        torch.save(native, base + "_native.pt")
        torch.save(converted, base + "_converted.pt")
        logger.info(f"dumped {len(native)} native and {len(converted)} converted tensors to {base}_*.pt")


def get_weights_exchange_writer(train_engine):
    backend = getattr(train_engine, "comm_backend", "nccl")
    if backend == "file":
        return FileWeightExchangeWriter(train_engine)
    if backend in ("nccl", "p2p", "gloo"):
        from awex_b200.writer.nccl_writer import NCCLWeightsWriter

        return NCCLWeightsWriter(train_engine)
    if backend == "astate":
        from awex_b200.writer.astate_writer import AStateWeightsWriter

        return AStateWeightsWriter(train_engine)
    if backend == "hccl":
        raise NotImplementedError("the hccl (Ascend) backend is not part of this CUDA-only framework")
    raise ValueError(f"Unknown comm_backend {backend!r}")
