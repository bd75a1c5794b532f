"""Engine contracts (`awex/engine/core.py:26-101` in the reference).

A *training engine* owns the Megatron model and hands the writer
``model`` (module or list of virtual-pipeline chunks), ``hf_config``,
``config`` (dict), ``engine_name == "mcore"``, ``meta_server_addr``,
``comm_backend`` and the memory hooks.  An *inference engine* owns the serving
workers and gives the reader ``config`` (:class:`InferenceConfig`),
``hf_config``, ``engine_name`` ("sglang" | "vllm"), ``num_engines``,
``engine_rank`` and ``execute_task_in_model_worker(fn, **kwargs)``, which runs
``fn(model=..., model_context=..., **kwargs)`` in every worker and returns the
list of results.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, List, Optional


class Engine(ABC):
    hf_config: Any = None
    global_step: int = 0

    def initialize(self) -> None:
        pass

    def set_global_step(self, global_step: int) -> None:
        """The training step the engine's weights belong to (`awex/engine/core.py:44-46`)."""
        self.global_step = global_step

    def release_memory_occupation(self, tags: Optional[List[str]] = None) -> None:
        raise NotImplementedError

    def resume_memory_occupation(self, tags: Optional[List[str]] = None) -> None:
        raise NotImplementedError


class InferenceEngine(Engine):
    engine_name: str = ""

    @abstractmethod
    def execute_task_in_model_worker(self, fn, **kwargs) -> list: ...

    @abstractmethod
    def update_weights_from_disk(self, model_path: str, load_format: Optional[str] = None): ...

    def update_weights(self, step_id: int, **kwargs):
        self.weights_exchange_reader.update_weights(step_id=step_id, **kwargs)

    @property
    def num_engines(self) -> int:
        return self.config.num_engines

    @property
    def engine_rank(self) -> int:
        return self.config.engine_rank


class TrainingEngine(Engine):
    engine_name: str = "mcore"

    def save_hf_checkpoint(self, path: str):
        raise NotImplementedError

    @abstractmethod
    def write_weights(self, **kwargs): ...

    def release_grad_memory(self) -> None:
        pass
