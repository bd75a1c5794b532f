"""In-process wrapper of a vLLM engine handle (`awex/engine/vllm.py:38-209` in
the reference).

The handle must expose ``call_utility(method, args=, kwargs=, run_on_all=)``
returning ``{"results": [...]}`` per engine core, ``initialize()`` /
``initialized`` and ``_engine.offload()`` / ``_engine.onload(tags=)``.  Callables
are shipped as ``awex_execute`` with module and qualified name, because vLLM
workers live in other processes and the utility channel carries plain data.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional, Union

from awex_b200 import logging
from awex_b200.config import InferenceConfig
from awex_b200.engine.serving import ServingEngineBase

logger = logging.getLogger(__name__)

# method name -> {"required": [...], "optional": [...]}: kwargs outside the
# lists are dropped before the call, missing required ones raise.  Methods
# without an entry pass through unchanged.
VLLM_TASK_SIGNATURES: Dict[str, Dict[str, List[str]]] = {}


def adapt_task_kwargs(method: str, kwargs: Dict[str, Any]) -> Dict[str, Any]:
    signature = VLLM_TASK_SIGNATURES.get(method)
    if signature is None:
        return kwargs
    allowed = set(signature.get("required", ())) | set(signature.get("optional", ()))
    kept = {k: v for k, v in kwargs.items() if k in allowed}
    missing = [k for k in signature.get("required", ()) if k not in kept]
    if missing:
        raise ValueError(f"Missing required args for {method}: {missing}")
    return kept


def load_hf_config(model_path: str):
    from transformers import AutoConfig

    return AutoConfig.from_pretrained(model_path, trust_remote_code=True)


class VLLMEngine(ServingEngineBase):
    engine_name = "vllm"

    def __init__(self, config: Union[Dict[str, Any], InferenceConfig], vllm_engine, hf_config=None):
        if isinstance(config, dict):
            config = InferenceConfig.from_dict(config)
        if hf_config is None:
            if config.model_path is None:
                raise ValueError("hf_config or config.model_path must be provided.")
            hf_config = load_hf_config(config.model_path)
        super().__init__(config, hf_config)
        self._vllm_engine = vllm_engine

    def _before_initialize(self) -> None:
        if not getattr(self._vllm_engine, "initialized", False):
            self._vllm_engine.initialize()

    def _load_from_disk(self, model_path: str, load_format: Optional[str]) -> None:
        if load_format is not None:
            logger.warning(f"vLLM checkpoint reload ignores load_format={load_format}")
        self._vllm_engine.call_utility("awex_update_weights_from_disk", args=[model_path, load_format], kwargs={}, run_on_all=True)

    def _release(self, tags: List[str]) -> None:
        self._vllm_engine._engine.offload()

    def _resume(self, tags: List[str]) -> None:
        self._vllm_engine._engine.onload(tags=tags)

    def _run_in_workers(self, fn, **kwargs):
        run_on_all = kwargs.pop("run_on_all", True)
        if isinstance(fn, str):
            method, payload = fn, kwargs
        else:
            method = "awex_execute"
            payload = {"task_module": fn.__module__, "task_qualname": fn.__qualname__, "task_kwargs": kwargs}
        payload = adapt_task_kwargs(method, payload)
        responses = self._vllm_engine.call_utility(method, args=[], kwargs=payload, run_on_all=run_on_all)
        if not run_on_all:
            return responses.get("results", [])
        merged: list = []
        for response in responses:
            merged.extend(response.get("results", []))
        return merged
