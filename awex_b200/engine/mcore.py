"""Megatron-core training engine adapter (`awex/engine/mcore.py:32-97`)."""

from __future__ import annotations

import os
import time

from awex_b200 import logging
from awex_b200.engine.core import TrainingEngine

logger = logging.getLogger(__name__)


class MegatronEngine(TrainingEngine):
    """``config`` is a plain dict; recognised keys: ``meta_server_addr``,
    ``comm_backend``, ``enable_colocate_mode``, ``enable_debug_mode``,
    ``enable_forward_share_gpu``, validation and dump options, and
    ``device_wait_timeout_ms``.  ``rank_info`` / ``process_group`` / ``tp_group``
    (this rank's training tensor-parallel group, needed only by dumps and
    other materialised conversions) may be given when Megatron's parallel
    state is not importable."""

    engine_name = "mcore"

    def __init__(self, config: dict, hf_config, model, rank_info=None, process_group=None, tp_group=None):
        self.config = config
        self.hf_config = hf_config
        self.model = model
        self.meta_server_addr = config.get("meta_server_addr")
        self.comm_backend = config.get("comm_backend", "nccl")
        self.enable_colocate_mode = config.get("enable_colocate_mode", False)
        self.enable_debug_mode = config.get("enable_debug_mode", False)
        self.enable_forward_share_gpu = config.get("enable_forward_share_gpu", False)
        self.rank_info = rank_info
        self.process_group = process_group
        self.tp_group = tp_group
        if self.meta_server_addr:
            ip, port = self.meta_server_addr.rsplit(":", 1)
            os.environ["AWEX_META_SERVER_ADDR"] = self.meta_server_addr
            os.environ["AWEX_META_SERVER_IP"] = ip
            os.environ["AWEX_META_SERVER_PORT"] = port
        self.weights_exchange_writer = None

    def initialize(self) -> None:
        from awex_b200.writer.weights_writer import get_weights_exchange_writer

        self.weights_exchange_writer = get_weights_exchange_writer(self)
        self.weights_exchange_writer.initialize()

    def save_hf_checkpoint(self, path: str):
        """Host frameworks override this; the synthetic harness provides one."""
        raise NotImplementedError("MegatronEngine.save_hf_checkpoint must be supplied by the training framework")

    def write_weights(self, **kwargs):
        t0 = time.time()
        self.weights_exchange_writer.write_weights(**kwargs)
        logger.info(f"write_weights took {time.time() - t0:.4f}s")

    def release_memory_occupation(self, tags=None) -> None:
        pass

    def resume_memory_occupation(self, tags=None) -> None:
        pass

    def release_grad_memory(self) -> None:
        for chunk in self.model if isinstance(self.model, (list, tuple)) else [self.model]:
            for p in chunk.parameters():
                if getattr(p, "grad", None) is not None:
                    p.grad = None
