"""Shared behaviour of the in-process SGLang and vLLM engine wrappers.

Both wrappers do the same bookkeeping around a different serving object: only
node 0 of a multi-node engine owns the weights-exchange reader, memory hand-off
tracks which tags are currently released so that release / resume are
idempotent, and worker tasks are refused before ``initialize`` and on non-zero
nodes.  The reference repeats this logic in each wrapper
(`awex/engine/sglang.py:28-157`, `awex/engine/vllm.py:38-183`); here it lives
once and the wrappers supply three hooks.
"""

from __future__ import annotations

import time
from typing import Any, Dict, Iterable, List, Optional, Union

from awex_b200 import logging
from awex_b200.config import InferenceConfig
from awex_b200.engine.core import InferenceEngine

logger = logging.getLogger(__name__)

DEFAULT_MEMORY_TAGS = ("kv_cache", "weights")


def normalize_tags(tags: Union[None, str, Iterable[str]]) -> List[str]:
    if tags is None:
        return list(DEFAULT_MEMORY_TAGS)
    if isinstance(tags, str):
        return [tags]
    return list(tags)


class ServingEngineBase(InferenceEngine):
    """Hooks: ``_release(tags)``, ``_resume(tags)``, ``_run_in_workers(fn, **kw)``,
    ``_load_from_disk(path, load_format)``."""

    engine_name = ""

    def __init__(self, config: Union[Dict[str, Any], InferenceConfig], hf_config):
        if isinstance(config, dict):
            config = InferenceConfig.from_dict(config)
        self._config = config
        self.hf_config = hf_config
        self.node_rank = config.node_rank or 0
        self.released_tags: set = set()
        self.weights_exchange_reader = None
        self.rank_coordinate = f"{config.engine_rank}-{self.node_rank}"
        self.global_step = 0
        self._initialized = False

    @property
    def config(self) -> InferenceConfig:
        return self._config

    # ---- lifecycle -----------------------------------------------------------------------
    def _before_initialize(self) -> None:
        pass

    def initialize(self) -> None:
        self._before_initialize()
        if self.node_rank != 0:
            logger.info(f"Node {self.rank_coordinate} holds no weights-exchange reader")
            return
        from awex_b200.reader.weights_reader import get_weights_exchange_reader

        self._initialized = True
        self.weights_exchange_reader = get_weights_exchange_reader(self)
        self.weights_exchange_reader.initialize()
        logger.info(f"Weights-exchange reader ready on {self.rank_coordinate}")

    def _require_initialized(self):
        if not self._initialized:
            raise RuntimeError("Engine not initialized. Call initialize() first.")

    # ---- weight updates ----------------------------------------------------------------
    def update_weights(self, step_id: Optional[int] = None, **kwargs):
        self._require_initialized()
        if step_id is not None:
            self.global_step = step_id
        started = time.time()
        self.weights_exchange_reader.update_weights(step_id=self.global_step, **kwargs)
        logger.info(f"Updated weights for step {self.global_step} on {self.rank_coordinate} in {time.time() - started:.3f}s")

    def update_weights_from_disk(self, model_path: str, load_format: Optional[str] = None):
        self._require_initialized()
        if self.node_rank != 0:
            logger.info("Non-zero node: checkpoint reload is driven by node 0")
            return
        self._load_from_disk(model_path, load_format)

    # ---- memory hand-off --------------------------------------------------------------
    def release_memory_occupation(self, tags=None) -> None:
        if not (self._initialized and self.node_rank == 0):
            return
        todo = [t for t in normalize_tags(tags) if t not in self.released_tags]
        if not todo:
            logger.info("No memory occupation to release")
            return
        self.released_tags.update(todo)
        self._release(todo)

    def resume_memory_occupation(self, tags=None) -> None:
        if not (self._initialized and self.node_rank == 0):
            return
        todo = [t for t in normalize_tags(tags) if t in self.released_tags]
        if not todo:
            logger.info("No memory occupation to resume")
            return
        self.released_tags.difference_update(todo)
        self._resume(todo)
        may_move = bool((getattr(self.config, "debug_mode_config", None) or {}).get("parameters_may_move", False))
        reader = getattr(self, "weights_exchange_reader", None)
        if "weights" in todo and may_move and hasattr(reader, "invalidate_addresses"):
            # weights that were released and came back may sit in new memory, even at the old addresses
            reader.invalidate_addresses()

    # ---- worker tasks ------------------------------------------------------------------
    def execute_task_in_model_worker(self, fn, **kwargs):
        self._require_initialized()
        if self.node_rank != 0:
            raise RuntimeError(f"Node {self.rank_coordinate} may not execute tasks in model workers")
        return self._run_in_workers(fn, **kwargs)

    # ---- hooks --------------------------------------------------------------------------
    def _release(self, tags: List[str]) -> None:
        raise NotImplementedError

    def _resume(self, tags: List[str]) -> None:
        raise NotImplementedError

    def _run_in_workers(self, fn, **kwargs):
        raise NotImplementedError

    def _load_from_disk(self, model_path: str, load_format: Optional[str]) -> None:
        raise NotImplementedError
