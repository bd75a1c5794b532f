"""vLLM integration: HTTP routes on the OpenAI API server and RPC methods on
the model workers.

Surface (same as the reference, `awex/vllm_plugin.py:114-506`):

* ``POST /areal_awex_init``  — body :class:`AwexInitRequest`; builds an
  :class:`AwexVLLMServerAdapter` around the server's engine client and
  initialises the weights reader in a thread;
* ``POST /areal_awex_update`` — body ``{step_id, kwargs}``;
* responses ``{"success": bool, "message": str}`` with 200 / 400 / 500;
* worker methods added to vLLM's ``WorkerBase``: ``awex_execute`` (import a task
  by module + qualified name, inject ``model`` and ``model_context``),
  ``awex_get_model_context``, ``awex_update_weights_from_disk``, ``flush_cache``
  and one named method per known worker task.

Everything that does not need vLLM (request models, kwarg whitelists, IPC
sanitising, rank discovery from group objects, the router itself) is plain
Python so it can be tested with fakes; vLLM is imported only inside
``patch_vllm_worker`` / ``attach_router_to_vllm``.  The entry point
``vllm.general_plugins: awex_adapter = awex_b200.vllm_plugin:register_awex_plugin``
registers both.
"""

from __future__ import annotations

import asyncio
import importlib
import logging
import os
from typing import Any, Callable, Dict, List, Optional

from awex_b200.config import InferenceConfig

logger = logging.getLogger(__name__)

# worker task name -> (module, qualified name)
AWEX_WORKER_METHODS: Dict[str, tuple] = {
    "_get_model_param_info": ("awex_b200.meta.infer_meta_resolver", "collect_worker_param_info"),
    "_init_in_tp_worker": ("awex_b200.reader.weights_reader", "WeightsReader._init_in_tp_worker"),
    "_update_parameters_in_tp_worker": ("awex_b200.reader.weights_reader", "WeightsReader._update_parameters_in_tp_worker"),
    "_begin_update_in_tp_worker": ("awex_b200.reader.weights_reader", "WeightsReader._begin_update_in_tp_worker"),
    "_finish_update_in_tp_worker": ("awex_b200.reader.weights_reader", "WeightsReader._finish_update_in_tp_worker"),
    "_invalidate_addresses_in_tp_worker": ("awex_b200.reader.weights_reader", "WeightsReader._invalidate_addresses_in_tp_worker"),
    "_pre_validate_weights_on_tp_worker": ("awex_b200.reader.weights_reader", "WeightsReader._pre_validate_weights_on_tp_worker"),
    "_verify_weights_on_tp_worker": ("awex_b200.reader.weights_reader", "WeightsReader._verify_weights_on_tp_worker"),
}

# per task: keyword arguments that must be present / may be present; anything
# else a caller sends is dropped before the task runs inside a worker
AWEX_WORKER_SIGNATURES: Dict[str, Dict[str, List[str]]] = {
    "_get_model_param_info": {"required": ["engine_name", "infer_engine_config"], "optional": ["convert_params", "engine_rank"]},
    "_init_in_tp_worker": {
        "required": [
            "infer_conf_bytes", "parameters_meta_bytes", "training_params_meta_bytes", "engine_rank", "num_engines",
            "meta_server_addr", "weights_comm_backend", "debug_mode_config", "disable_pipeline", "enable_colocate_mode", "ipc_backend",
        ],
        "optional": ["enable_debug_mode", "weights_comm_nccl_group_size", "device_wait_timeout_ms"],
    },
    "_update_parameters_in_tp_worker": {"required": ["step_id"], "optional": []},
    "_begin_update_in_tp_worker": {"required": ["step_id"], "optional": []},
    "_finish_update_in_tp_worker": {"required": ["step_id"], "optional": ["synchronize"]},
    "_invalidate_addresses_in_tp_worker": {"required": [], "optional": []},
    "_pre_validate_weights_on_tp_worker": {"required": [], "optional": ["step_id"]},
    "_verify_weights_on_tp_worker": {
        "required": [], "optional": ["step_id", "dump_weights_list_for_validation", "dump_weights_dir_for_validation"],
    },
}


def filter_awex_kwargs(method_name: str, kwargs: dict) -> dict:
    signature = AWEX_WORKER_SIGNATURES.get(method_name)
    if signature is None:
        return kwargs
    allowed = set(signature["required"]) | set(signature["optional"])
    kept = {k: v for k, v in kwargs.items() if k in allowed}
    missing = [k for k in signature["required"] if k not in kept]
    if missing:
        raise ValueError(f"Missing required args for {method_name}: {missing}")
    return kept


def sanitize_for_ipc(obj):
    """vLLM's engine-core IPC is msgpack: dtypes and devices become strings,
    dataclasses become dicts, tuples become lists."""
    try:
        import torch

        if isinstance(obj, torch.dtype):
            return str(obj).replace("torch.", "")
        if isinstance(obj, torch.device):
            return str(obj)
    except Exception:
        pass
    if isinstance(obj, dict):
        return {k: sanitize_for_ipc(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [sanitize_for_ipc(v) for v in obj]
    if hasattr(obj, "__dataclass_fields__"):
        import dataclasses

        return sanitize_for_ipc(dataclasses.asdict(obj))
    return obj


def resolve_task(task_module: str, task_qualname: str) -> Callable:
    target: Any = importlib.import_module(task_module)
    for attr in task_qualname.split("."):
        target = getattr(target, attr)
    return target


def _group_coords(getter, default=(0, 1)):
    try:
        group = getter()
        return int(group.rank_in_group), int(group.world_size)
    except (AssertionError, Exception):
        return default


def vllm_rank_context(worker, groups: Dict[str, Callable], infer_engine_config: Optional[InferenceConfig] = None) -> dict:
    """Parallel coordinates of a vLLM worker as a ``model_context`` dict.
    ``groups`` maps "tp" / "pp" / "dp" / "ep" (/ "pcp") to vLLM's group getters.
    ``engine_rank`` is the index of the external inference instance, not vLLM's
    internal DP rank; the global rank composes DP rank and in-core rank."""
    pc = worker.model_runner.vllm_config.parallel_config
    tp_rank, tp_size = _group_coords(groups["tp"])
    pp_rank, pp_size = _group_coords(groups["pp"])
    dp_rank, dp_size = _group_coords(groups["dp"], (int(getattr(pc, "data_parallel_rank", 0) or 0), int(getattr(pc, "data_parallel_size", 1) or 1)))
    ep_rank, ep_size = _group_coords(groups["ep"])
    local_world = int(getattr(pc, "world_size", 1) or 1)
    local_rank = int(getattr(pc, "rank", 0) or 0)
    cp_size = int(getattr(pc, "prefill_context_parallel_size", 1) or 1)
    cp_rank = 0
    if cp_size > 1:
        getter = groups.get("pcp")
        cp_rank, cp_size = _group_coords(getter, (local_rank % cp_size, cp_size)) if getter else (local_rank % cp_size, cp_size)
    cp_mode = os.environ.get("AWEX_CP_MODE") or ("ring" if cp_size > 1 else "none")
    global_rank = dp_rank * local_world + local_rank if 0 <= local_rank < local_world else local_rank
    return {
        "tp_rank": tp_rank, "tp_size": tp_size, "pp_rank": pp_rank, "pp_size": pp_size, "dp_rank": dp_rank, "dp_size": dp_size,
        "ep_rank": ep_rank, "ep_size": ep_size, "ep_tp_rank": 0, "ep_tp_size": 1,
        "local_rank": getattr(worker, "local_rank", local_rank), "global_rank": global_rank,
        "world_size": getattr(pc, "world_size_across_dp", local_world * dp_size),
        "engine_rank": int(getattr(infer_engine_config, "engine_rank", 0) or 0) if infer_engine_config is not None else 0,
        "is_infer": True, "attn_tp_rank": tp_rank, "attn_tp_size": tp_size, "attn_dp_rank": 0,
        "cp_rank": cp_rank, "cp_size": cp_size, "cp_mode": cp_mode,
    }


def vllm_model_context(worker, groups, infer_engine_config: Optional[InferenceConfig] = None) -> dict:
    """``model_context`` for a worker task: rank coordinates, the worker itself as
    ``scheduler`` (it offers ``flush_cache``), and the merged engine config."""
    if not hasattr(worker, "_awex_infer_engine_config"):
        from awex_b200.vllm_awex_adapter import inference_config_from_vllm

        pc = worker.model_runner.vllm_config.parallel_config
        backend = getattr(infer_engine_config, "comm_backend", None) or os.environ.get("AWEX_COMM_BACKEND", "file")
        worker._awex_infer_engine_config = inference_config_from_vllm(
            pc, num_engines=int(getattr(infer_engine_config, "num_engines", 1) or 1),
            engine_rank=int(getattr(infer_engine_config, "engine_rank", 0) or 0), comm_backend=backend,
            meta_server_addr=getattr(infer_engine_config, "meta_server_addr", None) or os.environ.get("AWEX_META_SERVER_ADDR"),
        )
    config = worker._awex_infer_engine_config
    if infer_engine_config is not None:
        merged = InferenceConfig.from_dict(dict(vars(config)), False)
        for name in InferenceConfig.field_names():
            value = getattr(infer_engine_config, name, None)
            if value is not None:
                setattr(merged, name, value)
        config = merged
    ctx = vllm_rank_context(worker, groups, config)
    ctx["scheduler"] = worker
    ctx["infer_engine_config"] = config
    return ctx


def execute_task_on_worker(worker, groups, task_module: str, task_qualname: str, task_kwargs: Optional[dict] = None):
    target = resolve_task(task_module, task_qualname)
    kwargs = dict(task_kwargs or {})
    cfg = kwargs.get("infer_engine_config")
    if isinstance(cfg, dict):
        cfg = InferenceConfig.from_dict(cfg)
        kwargs["infer_engine_config"] = cfg
    kwargs["model"] = worker.model_runner.model
    kwargs["model_context"] = vllm_model_context(worker, groups, cfg if isinstance(cfg, InferenceConfig) else None)
    return sanitize_for_ipc(target(**kwargs))


# ---- worker patches (need vLLM) -----------------------------------------------------------------
def reload_load_config(load_config, load_format: Optional[str] = None):
    """The load configuration for re-reading weights from a checkpoint directory:
    the engine's own, with ``load_format`` when the caller names one, and never the
    ``dummy`` format (a server started with random weights would otherwise answer a
    reload with fresh random weights instead of the checkpoint's)."""
    import copy

    current = str(getattr(load_config, "load_format", "auto"))
    current = current.rsplit(".", 1)[-1].lower()  # enum members print as LoadFormat.DUMMY on older releases
    wanted = load_format or ("auto" if current == "dummy" else None)
    if not wanted or wanted == current:
        return load_config
    changed = copy.copy(load_config)
    object.__setattr__(changed, "load_format", wanted)  # the config may be a frozen dataclass
    return changed


def worker_update_weights_from_disk(self, model_path: str, load_format: Optional[str] = None):
    from vllm.model_executor.model_loader import get_model_loader

    self.model_runner.model_config.model = model_path
    vllm_config = self.model_runner.vllm_config
    loader = get_model_loader(reload_load_config(vllm_config.load_config, load_format))
    try:  # newer loaders read the engine configuration from a context that is only set while the engine builds its model
        from vllm.config import set_current_vllm_config
    except Exception:
        set_current_vllm_config = None
    if set_current_vllm_config is None:
        loader.load_weights(self.model_runner.model, model_config=self.model_runner.model_config)
    else:
        with set_current_vllm_config(vllm_config):
            loader.load_weights(self.model_runner.model, model_config=self.model_runner.model_config)
    return True


def worker_flush_cache(self):
    fn = getattr(self.model_runner, "flush_cache", None)
    return fn() if callable(fn) else True


def patch_worker_class(worker_cls, groups: Dict[str, Callable]) -> None:
    """Add the Awex RPC methods to ``worker_cls`` (vLLM's ``WorkerBase`` or a fake)."""

    def awex_get_model_context(self):
        return vllm_rank_context(self, groups, None)

    def awex_execute(self, task_module: str, task_qualname: str, task_kwargs: Optional[dict] = None):
        return execute_task_on_worker(self, groups, task_module, task_qualname, task_kwargs)

    worker_cls.awex_get_model_context = awex_get_model_context
    worker_cls.awex_execute = awex_execute
    worker_cls.awex_update_weights_from_disk = worker_update_weights_from_disk
    worker_cls.flush_cache = worker_flush_cache

    def make(method_name: str, module: str, qualname: str):
        def method(self, **kwargs):
            return execute_task_on_worker(self, groups, module, qualname, filter_awex_kwargs(method_name, kwargs))

        method.__name__ = method_name
        return method

    for method_name, (module, qualname) in AWEX_WORKER_METHODS.items():
        setattr(worker_cls, method_name, make(method_name, module, qualname))


def patch_vllm_worker() -> bool:
    try:
        from vllm.distributed import parallel_state as ps
        from vllm.v1.worker.worker_base import WorkerBase
    except Exception as exc:
        logger.warning("Failed to patch vLLM worker for Awex: %s", exc)
        return False
    groups = {"tp": ps.get_tp_group, "pp": ps.get_pp_group, "dp": ps.get_dp_group, "ep": ps.get_ep_group}
    if callable(getattr(ps, "get_pcp_group", None)):
        groups["pcp"] = ps.get_pcp_group
    patch_worker_class(WorkerBase, groups)
    return True


# ---- HTTP routes ---------------------------------------------------------------------------------------
def _request_models():
    from pydantic import BaseModel

    class AwexInitRequest(BaseModel):
        meta_server_addr: str
        engine_rank: int = 0
        num_engines: int = 1
        comm_backend: str = "file"
        enable_debug_mode: bool = False
        debug_mode_config: Optional[Dict[str, Any]] = None
        disable_weights_exchange_pipeline: bool = False
        enable_colocate_mode: bool = False
        weights_exchange_ipc_backend: str = "cuda"
        weights_comm_nccl_group_size: int = 1
        nnodes: Optional[int] = None
        node_rank: Optional[int] = None
        weights_validation_steps: int = 0
        validate_weights_every_n_steps: int = 1
        dump_weights_list_for_validation: Optional[List[str]] = None
        dump_weights_dir_for_validation: Optional[str] = None

    class AwexUpdateRequest(BaseModel):
        step_id: int
        kwargs: Optional[Dict[str, Any]] = None

    return AwexInitRequest, AwexUpdateRequest


AwexInitRequest, AwexUpdateRequest = _request_models()


def _reply(success: bool, message: str, status_code: Optional[int] = None):
    from fastapi.responses import JSONResponse

    return JSONResponse({"success": success, "message": message}, status_code=status_code or (200 if success else 400))


def build_router(adapter_factory: Optional[Callable[..., Any]] = None):
    """FastAPI router with the two Awex routes.  ``adapter_factory(engine_client,
    **fields, loop=...)`` defaults to :class:`AwexVLLMServerAdapter`."""
    from fastapi import APIRouter, Request

    if adapter_factory is None:
        from awex_b200.vllm_awex_adapter import AwexVLLMServerAdapter as adapter_factory  # noqa: N813

    router = APIRouter()

    async def awex_init(request, raw_request):
        try:
            client = raw_request.app.state.engine_client
            adapter = adapter_factory(client, loop=asyncio.get_running_loop(), **request.model_dump())
            await asyncio.to_thread(adapter.initialize)
            raw_request.app.state.awex_adapter = adapter
            return _reply(True, "Awex initialized")
        except Exception as exc:
            logger.exception("Awex init failed")
            return _reply(False, f"Awex init failed: {exc}", 500)

    async def awex_update(request, raw_request):
        adapter = getattr(raw_request.app.state, "awex_adapter", None)
        if adapter is None:
            return _reply(False, "Awex adapter not initialized. Call /areal_awex_init first.")
        try:
            await asyncio.to_thread(lambda: adapter.update_weights(request.step_id, **(request.kwargs or {})))
            return _reply(True, "Awex update done")
        except Exception as exc:
            logger.exception("Awex update failed")
            return _reply(False, f"Awex update failed: {exc}", 500)

    # annotations are attached as objects: this module postpones annotation
    # evaluation, and FastAPI could not resolve the locally imported Request
    awex_init.__annotations__ = {"request": AwexInitRequest, "raw_request": Request}
    awex_update.__annotations__ = {"request": AwexUpdateRequest, "raw_request": Request}
    router.post("/areal_awex_init")(awex_init)
    router.post("/areal_awex_update")(awex_update)
    return router


_router = None
_build_app_patched = False
_registered = False


def attach_router_to_vllm(router) -> bool:
    """Older vLLM exposes a module-level router that apps include; newer vLLM
    builds its app in ``build_app``, which is wrapped to include ours."""
    global _build_app_patched
    try:
        from vllm.entrypoints.openai import api_server
    except Exception as exc:
        logger.warning("Cannot attach Awex routes to vLLM: %s", exc)
        return False
    shared = getattr(api_server, "router", None)
    if shared is not None:
        shared.include_router(router)
        return True
    if _build_app_patched:
        return True
    original = getattr(api_server, "build_app", None)
    if original is None:
        logger.warning("vLLM api_server has no build_app; Awex routes will not be attached.")
        return False

    def build_app_with_awex(*args, **kwargs):
        app = original(*args, **kwargs)
        app.include_router(router)
        return app

    api_server.build_app = build_app_with_awex
    _build_app_patched = True
    return True


def register_awex_plugin() -> None:
    """Entry point of ``vllm.general_plugins``: idempotent."""
    global _registered, _router
    if _registered:
        return
    _registered = True
    patch_vllm_worker()
    _router = build_router()
    attach_router_to_vllm(_router)


def register_awex_routes() -> None:
    """Register routes and worker patches without vLLM's plugin discovery."""
    register_awex_plugin()
