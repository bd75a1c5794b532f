"""Per-engine discovery of :class:`RankInfo` and construction of the model's
sharding strategy (`awex/sharding/{mcore,sglang,vllm}_sharding.py` in the
reference).

Inference workers describe themselves with a ``model_context`` dict built by
the engine adapter; training ranks read ``megatron.core.parallel_state``.
"""

from __future__ import annotations

import os

from awex_b200.sharding.rank_info import RankInfo
from awex_b200.utils import device as device_util


def _cp_mode(explicit, cp_size: int) -> str:
    return explicit or ("ring" if cp_size > 1 else "none")


def _backend_of(infer_engine_config) -> str:
    for key in ("device_backend", "device_type"):
        val = getattr(infer_engine_config, key, None)
        if isinstance(val, str) and val.strip():
            return val.strip().lower()
    return device_util.get_device_type()


def _infer_strategy(engine_name: str, model_name: str, infer_engine_config, rank_info: RankInfo, **kwargs):
    from awex_b200.models.registry import get_sharding_strategy

    return get_sharding_strategy(model_name)(
        engine_name=engine_name,
        enable_dp_attention=infer_engine_config.enable_dp_attention,
        enable_dp_lm_head=infer_engine_config.enable_dp_lm_head,
        moe_dense_tp_size=infer_engine_config.moe_dense_tp_size,
        tp_size=rank_info.tp_size,
        ep_size=infer_engine_config.ep_size,
        ep_tp_size=rank_info.ep_tp_size,
        rank_info=rank_info,
        device_backend=_backend_of(infer_engine_config),
        **kwargs,
    )


def get_sglang_sharding_strategy(model_name: str, infer_engine_config, rank_info: RankInfo, **kwargs):
    return _infer_strategy("sglang", model_name, infer_engine_config, rank_info, **kwargs)


def get_vllm_sharding_strategy(model_name: str, infer_engine_config, rank_info: RankInfo, **kwargs):
    return _infer_strategy("vllm", model_name, infer_engine_config, rank_info, **kwargs)


def get_mcore_sharding_strategy(model_name: str, rank_info: RankInfo, **kwargs):
    from awex_b200.models.registry import get_sharding_strategy

    return get_sharding_strategy(model_name)(
        engine_name="mcore",
        enable_dp_attention=False,
        enable_dp_lm_head=False,
        moe_dense_tp_size=rank_info.tp_size,
        tp_size=rank_info.tp_size,
        ep_size=rank_info.ep_size,
        ep_tp_size=rank_info.ep_tp_size,
        rank_info=rank_info,
        device_backend=device_util.get_device_type(),
        **kwargs,
    )


def _common_infer_fields(ctx: dict, engine_rank: int) -> dict:
    return dict(
        pp_rank=ctx["pp_rank"],
        pp_size=ctx["pp_size"],
        attn_tp_rank=ctx["attn_tp_rank"],
        attn_tp_size=ctx["attn_tp_size"],
        attn_dp_rank=ctx["attn_dp_rank"],
        world_size=ctx["world_size"],
        global_rank=ctx["global_rank"],
        local_rank=ctx["local_rank"],
        engine_rank=engine_rank,
        is_infer=True,
    )


def get_sglang_rank_info(model_context: dict, engine_rank: int) -> RankInfo:
    """SGLang nests expert-TP inside TP: ``ep_tp_size = tp_size // ep_size``
    (`awex/sharding/sglang_sharding.py:52-105`)."""
    args = model_context["scheduler"].server_args
    if args.dp_size != 1 and not args.enable_dp_attention:
        raise ValueError(f"DP size is not 1, but {args.dp_size}. This is not supported yet.")
    tp_size, tp_rank = model_context["tp_size"], model_context["tp_rank"]
    ep_size = int(args.ep_size or 1)
    if ep_size > 1:
        ep_tp_size = tp_size // ep_size
        ep_rank, ep_tp_rank = divmod(tp_rank, ep_tp_size)
    else:
        ep_rank, ep_tp_size, ep_tp_rank = 0, 1, 0
    cp_size = int(model_context.get("cp_size", getattr(args, "context_parallel_size", 1)) or 1)
    return RankInfo(
        tp_rank=tp_rank, tp_size=tp_size, dp_size=model_context["dp_size"], dp_rank=0,
        ep_rank=ep_rank, ep_size=ep_size, ep_tp_rank=ep_tp_rank, ep_tp_size=ep_tp_size,
        cp_rank=int(model_context.get("cp_rank", 0) or 0), cp_size=cp_size,
        cp_mode=_cp_mode(model_context.get("cp_mode", getattr(args, "context_parallel_mode", None)), cp_size),
        **_common_infer_fields(model_context, engine_rank),
    )


def get_vllm_rank_info(model_context: dict, engine_rank: int) -> RankInfo:
    """vLLM's EP group is independent of TP, so expert-TP is taken from the
    context when given and is 1 otherwise (`awex/sharding/vllm_sharding.py:49-92`)."""
    ep_size = int(model_context.get("ep_size", 1) or 1)
    if ep_size > 1:
        ep_rank = model_context.get("ep_rank", 0)
        ep_tp_size = model_context.get("ep_tp_size", 1)
        ep_tp_rank = model_context.get("ep_tp_rank", 0)
    else:
        ep_rank, ep_tp_size, ep_tp_rank = 0, 1, 0
    cp_size = int(model_context.get("cp_size", 1) or 1)
    return RankInfo(
        tp_rank=model_context["tp_rank"], tp_size=model_context["tp_size"],
        dp_size=model_context["dp_size"], dp_rank=model_context["dp_rank"],
        ep_rank=ep_rank, ep_size=ep_size, ep_tp_rank=ep_tp_rank, ep_tp_size=ep_tp_size,
        cp_rank=int(model_context.get("cp_rank", 0) or 0), cp_size=cp_size,
        cp_mode=_cp_mode(model_context.get("cp_mode"), cp_size),
        **_common_infer_fields(model_context, engine_rank),
    )


def get_mcore_rank_info() -> RankInfo:
    """Read Megatron's parallel state (`awex/sharding/mcore_sharding.py:45-94`).
    Attention TP equals TP on the training side."""
    import torch.distributed as dist

    from awex_b200.utils.mindspeed import ensure_mindspeed_patched

    ensure_mindspeed_patched("get_mcore_rank_info")
    from megatron.core import parallel_state as mpu

    def opt(fn_name: str, default: int) -> int:
        fn = getattr(mpu, fn_name, None)
        return int(fn()) if callable(fn) else default

    tp_rank, tp_size = mpu.get_tensor_model_parallel_rank(), mpu.get_tensor_model_parallel_world_size()
    dp_rank = mpu.get_data_parallel_rank()
    cp_size = opt("get_context_parallel_world_size", 1)
    rank = dist.get_rank()
    return RankInfo(
        tp_rank=tp_rank, tp_size=tp_size,
        pp_rank=mpu.get_pipeline_model_parallel_rank(), pp_size=mpu.get_pipeline_model_parallel_world_size(),
        dp_size=mpu.get_data_parallel_world_size(), dp_rank=dp_rank,
        ep_rank=opt("get_expert_model_parallel_rank", 0), ep_size=opt("get_expert_model_parallel_world_size", 1),
        ep_tp_rank=opt("get_expert_tensor_parallel_rank", 0), ep_tp_size=opt("get_expert_tensor_parallel_world_size", 1),
        attn_tp_rank=tp_rank, attn_tp_size=tp_size, attn_dp_rank=dp_rank,
        world_size=dist.get_world_size(), global_rank=rank,
        local_rank=rank % max(device_util.device_count(), 1), engine_rank=0, is_infer=False,
        cp_rank=opt("get_context_parallel_rank", 0), cp_size=cp_size,
        cp_mode=_cp_mode(os.environ.get("AWEX_CP_MODE"), cp_size),
    )
