"""Inference-side configuration.

Field names, defaults and validation rules follow the reference dataclass
(`awex/config.py:38-189`) so a config dict written for it loads unchanged.
Fields this framework adds are grouped at the bottom and all have defaults.
"""

from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional

VALID_COMM_BACKENDS = frozenset({"file", "nccl", "hccl", "astate", "p2p", "gloo"})
VALID_IPC_BACKENDS = frozenset({"cpu", "cuda"})


class InferenceConfigValidationError(ValueError):
    """One exception carrying every violated rule, one per line."""


@dataclass
class InferenceConfig:
    model_path: Optional[str] = None
    tp_size: Optional[int] = None
    pp_size: Optional[int] = None
    dp_size: Optional[int] = None
    load_balance_method: Optional[str] = None
    ep_size: Optional[int] = None
    enable_dp_attention: Optional[bool] = None
    enable_dp_lm_head: Optional[bool] = None
    deepep_mode: Optional[str] = None
    ep_num_redundant_experts: Optional[int] = None
    enable_eplb: Optional[bool] = None
    enable_memory_saver: Optional[bool] = None
    moe_dense_tp_size: Optional[int] = None
    n_share_experts_fusion: Optional[int] = None
    nnodes: Optional[int] = None
    node_rank: Optional[int] = None
    local_rank: Optional[int] = None
    # number of inference engine instances in the job / index of this one
    num_engines: int = 1
    engine_rank: int = 0
    # "ip:port" of the job-global MetaServer
    meta_server_addr: Optional[str] = None
    # "file" | "nccl" | "hccl" | "astate"; "nccl" selects the fused NVLink
    # peer-store data plane on CUDA devices, "p2p" is an explicit alias for
    # it and "gloo" runs the same plans on CPU tensors.
    comm_backend: str = "file"
    weights_validation_steps: int = 0
    validate_weights_every_n_steps: int = 1
    dump_weights_list_for_validation: List[str] = field(default_factory=list)
    dump_weights_dir_for_validation: Optional[str] = None
    disable_weights_exchange_pipeline: bool = False
    enable_debug_mode: bool = False
    debug_mode_config: Dict = field(default_factory=dict)
    enable_colocate_mode: bool = False
    weights_exchange_ipc_backend: str = "cuda"
    weights_comm_nccl_group_size: int = 1
    # ---- additions (not in the reference) ----
    # upper bound, in milliseconds, of any device-side wait on a peer flag
    device_wait_timeout_ms: int = 2000
    # serve weights as block-scaled fp8 e4m3 (128x128 blocks, fp32 scales)
    fp8_block_quant: bool = False

    def validate(self) -> None:
        problems: List[str] = []

        def need(cond: bool, msg: str) -> None:
            if not cond:
                problems.append(msg)

        need(
            self.comm_backend in VALID_COMM_BACKENDS,
            f"comm_backend must be one of {sorted(VALID_COMM_BACKENDS)}, got {self.comm_backend!r}",
        )
        need(
            self.weights_exchange_ipc_backend in VALID_IPC_BACKENDS,
            f"weights_exchange_ipc_backend must be one of {sorted(VALID_IPC_BACKENDS)}, "
            f"got {self.weights_exchange_ipc_backend!r}",
        )
        if self.num_engines < 1:
            problems.append(f"num_engines must be >= 1, got {self.num_engines}")
        else:
            need(
                0 <= self.engine_rank < self.num_engines,
                f"engine_rank must be in [0, num_engines), got engine_rank={self.engine_rank} "
                f"with num_engines={self.num_engines}",
            )
        for key in ("tp_size", "pp_size", "dp_size", "ep_size", "moe_dense_tp_size", "weights_comm_nccl_group_size"):
            val = getattr(self, key)
            need(val is None or val >= 1, f"{key} must be >= 1 when set, got {val}")
        if self.nnodes is not None:
            if self.nnodes < 1:
                problems.append(f"nnodes must be >= 1 when set, got {self.nnodes}")
            elif self.node_rank is not None:
                need(
                    0 <= self.node_rank < self.nnodes,
                    f"node_rank must be in [0, nnodes), got node_rank={self.node_rank} with nnodes={self.nnodes}",
                )
        need(
            self.validate_weights_every_n_steps >= 1,
            f"validate_weights_every_n_steps must be >= 1, got {self.validate_weights_every_n_steps}",
        )
        need(
            self.weights_validation_steps >= 0,
            f"weights_validation_steps must be >= 0, got {self.weights_validation_steps}",
        )
        need(
            not self.dump_weights_list_for_validation or bool(self.dump_weights_dir_for_validation),
            "dump_weights_dir_for_validation must be set when dump_weights_list_for_validation is non-empty",
        )
        need(
            self.ep_num_redundant_experts is None or self.ep_size is not None,
            "ep_num_redundant_experts requires ep_size to be set",
        )
        need(not self.enable_eplb or self.ep_size is not None, "enable_eplb requires ep_size to be set")
        need(
            not (self.num_engines > 1 and self.comm_backend != "file" and not self.meta_server_addr),
            f"meta_server_addr must be set when num_engines > 1 and comm_backend is {self.comm_backend!r}",
        )
        need(self.device_wait_timeout_ms > 0, "device_wait_timeout_ms must be positive")
        if problems:
            raise InferenceConfigValidationError(
                "InferenceConfig validation failed:\n" + "\n".join(f"  - {p}" for p in problems)
            )

    def validated(self) -> "InferenceConfig":
        self.validate()
        return self

    @classmethod
    def field_names(cls) -> List[str]:
        return [f.name for f in fields(cls)]

    @staticmethod
    def from_dict(config_dict: Dict[str, Any], validate: bool = True) -> "InferenceConfig":
        known = set(InferenceConfig.field_names())
        cfg = InferenceConfig(**{k: v for k, v in config_dict.items() if k in known})
        if validate:
            cfg.validate()
        return cfg

    @staticmethod
    def from_sgl_server_args(server_args, **extra) -> "InferenceConfig":
        picked = {}
        for key in InferenceConfig.field_names():
            val = getattr(server_args, key, None)
            if val is not None:
                picked[key] = val
        picked.update(extra)
        return InferenceConfig(**picked)

    @staticmethod
    def from_sgl_engine(sgl_engine, **extra) -> "InferenceConfig":
        return InferenceConfig.from_sgl_server_args(sgl_engine.server_args, **extra)
