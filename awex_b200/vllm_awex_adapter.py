"""Inference-engine adapter that lives inside a vLLM API server process.

It duck-types the inference-engine contract of :mod:`awex_b200.engine.core` on
top of vLLM's ``AsyncLLM`` / engine-core client: worker tasks travel as
``collective_rpc("awex_execute", ...)`` with the task named by module and
qualified name; metadata collection fans out to *every* internal data-parallel
core, because returning only the first core's answer would lose the shards the
other cores hold; memory hand-off maps to vLLM's sleep / wake_up
(`awex/vllm_awex_adapter.py:28-301` in the reference).
"""

from __future__ import annotations

import asyncio
import inspect
from dataclasses import asdict
from typing import Any, Dict, List, Optional

from awex_b200 import logging
from awex_b200.config import InferenceConfig
from awex_b200.reader.weights_reader import get_weights_exchange_reader

logger = logging.getLogger(__name__)

_META_TASKS = ("collect_worker_param_info", "_get_model_param_info")


def inference_config_from_vllm(parallel_config, **overrides) -> InferenceConfig:
    """Translate vLLM's parallel config.  With expert parallelism enabled the EP
    group spans TP x DP x prefill-CP ranks."""
    pcp = int(getattr(parallel_config, "prefill_context_parallel_size", 1) or 1)
    ep = 1
    if bool(getattr(parallel_config, "enable_expert_parallel", False)):
        ep = parallel_config.tensor_parallel_size * parallel_config.data_parallel_size * pcp
    base = dict(
        tp_size=parallel_config.tensor_parallel_size,
        pp_size=parallel_config.pipeline_parallel_size,
        dp_size=parallel_config.data_parallel_size,
        ep_size=ep,
        enable_dp_attention=False,
        enable_dp_lm_head=False,
        moe_dense_tp_size=None,
        nnodes=getattr(parallel_config, "nnodes", None) or 1,
        node_rank=getattr(parallel_config, "node_rank", None) or 0,
    )
    base.update({k: v for k, v in overrides.items() if v is not None})
    return InferenceConfig(**base)


class AwexVLLMServerAdapter:
    engine_name = "vllm"

    def __init__(
        self,
        engine_client,
        meta_server_addr: str,
        engine_rank: int = 0,
        num_engines: int = 1,
        comm_backend: str = "file",
        enable_debug_mode: bool = False,
        debug_mode_config: Optional[Dict[str, Any]] = None,
        disable_weights_exchange_pipeline: bool = False,
        enable_colocate_mode: bool = False,
        weights_exchange_ipc_backend: str = "cuda",
        weights_comm_nccl_group_size: int = 1,
        nnodes: Optional[int] = None,
        node_rank: Optional[int] = None,
        weights_validation_steps: int = 0,
        validate_weights_every_n_steps: int = 1,
        dump_weights_list_for_validation: Optional[List[str]] = None,
        dump_weights_dir_for_validation: Optional[str] = None,
        loop: Optional[asyncio.AbstractEventLoop] = None,
    ):
        self._engine_client = engine_client
        self._engine_core = getattr(engine_client, "engine_core", None)
        self._initialized = False
        self._initializing = False
        self._loop = loop
        self.hf_config = engine_client.model_config.hf_config
        self._config = inference_config_from_vllm(
            engine_client.vllm_config.parallel_config,
            nnodes=nnodes, node_rank=node_rank, num_engines=num_engines, engine_rank=engine_rank,
            meta_server_addr=meta_server_addr, comm_backend=comm_backend, enable_debug_mode=enable_debug_mode,
            debug_mode_config=debug_mode_config or {}, disable_weights_exchange_pipeline=disable_weights_exchange_pipeline,
            enable_colocate_mode=enable_colocate_mode, weights_exchange_ipc_backend=weights_exchange_ipc_backend,
            weights_comm_nccl_group_size=weights_comm_nccl_group_size, weights_validation_steps=weights_validation_steps,
            validate_weights_every_n_steps=validate_weights_every_n_steps,
            dump_weights_list_for_validation=dump_weights_list_for_validation or [],
            dump_weights_dir_for_validation=dump_weights_dir_for_validation,
        )
        self.weights_exchange_reader = None

    # ---- engine contract -------------------------------------------------------------------
    @property
    def config(self) -> InferenceConfig:
        return self._config

    @property
    def num_engines(self) -> int:
        return self._config.num_engines

    @property
    def engine_rank(self) -> int:
        return self._config.engine_rank

    def initialize(self) -> None:
        if self._initialized or self._initializing:
            return
        self._initializing = True
        try:
            self.weights_exchange_reader = get_weights_exchange_reader(self)
            self.weights_exchange_reader.initialize()
            self._initialized = True
        finally:
            self._initializing = False

    def update_weights(self, step_id: int, **kwargs):
        if not self._initialized:
            raise RuntimeError("Awex adapter not initialized.")
        self.weights_exchange_reader.update_weights(step_id=step_id, **kwargs)

    def update_weights_from_disk(self, model_path: str, load_format: Optional[str] = None):
        self._collective_rpc("awex_update_weights_from_disk", args=(model_path, load_format))

    def release_memory_occupation(self, tags=None) -> None:
        self._call_engine("sleep", 1)

    def resume_memory_occupation(self, tags=None) -> None:
        self._call_engine("wake_up", tags)

    # ---- plumbing ------------------------------------------------------------------------------
    def _run_on_loop(self, coro):
        if self._loop is None:
            raise RuntimeError("No event loop available for async engine calls.")
        return asyncio.run_coroutine_threadsafe(coro, self._loop).result()

    def _maybe_await(self, fn, *args, **kwargs):
        if inspect.iscoroutinefunction(fn):
            return self._run_on_loop(fn(*args, **kwargs))
        return fn(*args, **kwargs)

    def _call_engine(self, method: str, *args):
        fn = getattr(self._engine_client, method, None)
        if fn is None:
            raise RuntimeError(f"Engine client has no method {method}")
        return self._maybe_await(fn, *args)

    def _collective_rpc(self, method: str, timeout: Optional[float] = None, args: tuple = (), kwargs: Optional[dict] = None):
        if hasattr(self._engine_client, "collective_rpc"):
            return self._maybe_await(self._engine_client.collective_rpc, method, timeout, args, kwargs)
        return self._engine_core.collective_rpc(method, timeout=timeout, args=args, kwargs=kwargs)

    def _get_dp_rpc_client(self):
        """The object that can address individual data-parallel cores, if any:
        the client itself or its ``engine_core``."""
        for candidate in (self._engine_client, getattr(self._engine_client, "engine_core", None)):
            if candidate is not None and hasattr(candidate, "core_engines") and hasattr(candidate, "_call_utility_async"):
                return candidate
        return None

    def _collective_rpc_all_dp_cores(self, method: str, timeout: Optional[float] = None, args: tuple = (), kwargs: Optional[dict] = None):
        client = self._get_dp_rpc_client()
        cores = list(getattr(client, "core_engines", []) or []) if client is not None else []
        if not cores:
            return [self._collective_rpc(method, timeout=timeout, args=args, kwargs=kwargs)]
        call = client._call_utility_async
        if inspect.iscoroutinefunction(call):
            async def gather_all():
                return await asyncio.gather(*[call("collective_rpc", method, timeout, args, kwargs, engine=e) for e in cores])

            return self._run_on_loop(gather_all())
        return [call("collective_rpc", method, timeout, args, kwargs, engine=e) for e in cores]

    @staticmethod
    def _is_meta_collection_call(method: str, payload: dict) -> bool:
        if method in _META_TASKS:
            return True
        if method != "awex_execute":
            return False
        qualname = payload.get("task_qualname", "")
        return isinstance(qualname, str) and qualname.endswith(_META_TASKS)

    def execute_task_in_model_worker(self, fn, **kwargs):
        if not self._initialized and not self._initializing:
            raise RuntimeError("Awex adapter not initialized.")
        if isinstance(fn, str):
            method, payload = fn, kwargs
        else:
            if isinstance(kwargs.get("infer_engine_config"), InferenceConfig):
                kwargs = {**kwargs, "infer_engine_config": asdict(kwargs["infer_engine_config"])}
            method = "awex_execute"
            payload = {"task_module": fn.__module__, "task_qualname": fn.__qualname__, "task_kwargs": kwargs}
        if self._is_meta_collection_call(method, payload):
            merged: list = []
            results = self._collective_rpc_all_dp_cores(method, args=(), kwargs=payload)
            for result in results:
                merged.extend(result if isinstance(result, list) else [result])
            logger.info(f"Collected model param meta from {len(results)} DP core(s), merged {len(merged)} entries.")
            return merged
        return self._collective_rpc(method, args=(), kwargs=payload)
