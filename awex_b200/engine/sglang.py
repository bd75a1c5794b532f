"""In-process wrapper of an SGLang ``Engine`` (`awex/engine/sglang.py:28-167`
in the reference).

The SGLang object must expose ``tokenizer_manager.model_config`` (the HF
config), ``update_weights_from_disk``, ``release_memory_occupation`` /
``resume_memory_occupation`` (tags) and ``execute_task_in_model_worker``, as the
fork the reference targets does.
"""

from __future__ import annotations

from typing import Any, Dict, List, Optional, Union

from awex_b200 import logging
from awex_b200.config import InferenceConfig
from awex_b200.engine.serving import ServingEngineBase
from awex_b200.utils.gpu import get_gpu_status

logger = logging.getLogger(__name__)


class SGLangEngine(ServingEngineBase):
    engine_name = "sglang"

    def __init__(self, config: Union[Dict[str, Any], InferenceConfig], sgl_engine):
        super().__init__(config, sgl_engine.tokenizer_manager.model_config)
        self._sgl_engine = sgl_engine

    def _load_from_disk(self, model_path: str, load_format: Optional[str]) -> None:
        self._sgl_engine.update_weights_from_disk(model_path=model_path, load_format=load_format)

    def _release(self, tags: List[str]) -> None:
        logger.info(f"Releasing {tags}; GPU before:\n{get_gpu_status()}")
        self._sgl_engine.release_memory_occupation(tags=tags)
        logger.info(f"GPU after release:\n{get_gpu_status()}")

    def _resume(self, tags: List[str]) -> None:
        logger.info(f"Resuming {tags}; GPU before:\n{get_gpu_status()}")
        self._sgl_engine.resume_memory_occupation(tags=tags)
        logger.info(f"GPU after resume:\n{get_gpu_status()}")

    def _run_in_workers(self, fn, **kwargs):
        return self._sgl_engine.execute_task_in_model_worker(fn, **kwargs)


def extract_sgl_config(config: Dict[str, Any]) -> Dict[str, Any]:
    """The subset of ``config`` that SGLang's ``ServerArgs`` accepts."""
    from sglang.srt.server_args import ServerArgs

    return {k: v for k, v in config.items() if k in ServerArgs.__dataclass_fields__}
