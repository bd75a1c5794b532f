"""How a canonical parameter name maps to (sharding type, sharded dim, shard count).

Semantics follow the reference (`awex/sharding/param_sharding.py:26-318`):
the same enum values, the same default shard-dimension table and the same
order of name tests, because both ends of an exchange must classify a name
identically.  Here the router is a first-match rule table instead of an
if-chain so model-specific strategies can splice rules in.
"""

from __future__ import annotations

from enum import Enum
from typing import Callable, List, Tuple

from awex_b200.sharding.rank_info import RankInfo


class ShardingType(Enum):
    NO_SHARDING = "NO_SHARDING"  # every holder has the whole tensor
    TP_SHARDING = "TP_SHARDING"  # split along one dim over the TP group
    DP_TP_SHARDING = "DP_TP_SHARDING"  # split over attention-TP, replicated over attention-DP
    EP_SHARDING = "EP_SHARDING"  # whole experts distributed over the EP group
    EP_TP_SHARDING = "EP_TP_SHARDING"  # each expert additionally split over expert-TP


# suffix (last one or two dotted components) -> dim the tensor is split on.
# Row-parallel projections split the input dim (1); everything else dim 0.
_SHARD_DIM = {
    **{
        k: 0
        for k in (
            "word_embeddings.weight", "lm_head.weight", "query_key_value.weight", "q_proj.weight",
            "k_proj.weight", "v_proj.weight", "g_proj.weight", "q_a_proj.weight", "q_b_proj.weight",
            "kv_a_proj_with_mqa.weight", "kv_b_proj.weight", "fused_qkv_a_proj_with_mqa.weight",
            "g_norm.weight", "query_key_value.bias", "q_proj.bias", "k_proj.bias", "v_proj.bias",
            "dense.bias", "experts.w13_weight", "gate_up_proj.weight", "gate_proj.weight",
            "up_proj.weight", "gate_up_proj.bias", "gate_proj.bias", "up_proj.bias", "down_proj.bias",
        )
    },
    "dense.weight": 1,
    "o_proj.weight": 1,
    "experts.w2_weight": 1,
    "down_proj.weight": 1,
}


def get_default_sharding_dim(param_name: str) -> int:
    """Dim along which ``param_name`` is split; block-scale tensors
    (``*_scale_inv``) shard like the weight they belong to.  Unknown names
    default to dim 0."""
    parts = param_name.replace("_scale_inv", "").split(".")
    if len(parts) >= 2:
        dim = _SHARD_DIM.get(f"{parts[-2]}.{parts[-1]}")
        if dim is not None:
            return dim
    return _SHARD_DIM.get(parts[-1], 0)


Decision = Tuple[ShardingType, int, int]


class ShardingStrategy:
    """Default strategy; model files subclass it and override a family method
    or extend :meth:`rules`."""

    def __init__(
        self,
        engine_name: str,
        enable_dp_attention,
        enable_dp_lm_head,
        moe_dense_tp_size,
        tp_size,
        ep_size,
        ep_tp_size,
        rank_info: RankInfo,
        device_backend: str | None = None,
        **_unused,
    ) -> None:
        self.engine_name = engine_name
        self.enable_dp_attention = enable_dp_attention
        self.enable_dp_lm_head = enable_dp_lm_head
        self.moe_dense_tp_size = moe_dense_tp_size
        self.tp_size = tp_size
        self.ep_size = ep_size
        self.ep_tp_size = ep_tp_size
        self.rank_info = rank_info
        self.device_backend = device_backend

    # ---- helpers -------------------------------------------------------
    def _maybe_adjust_sharding_dim(self, parameter_name: str, sharding_dim: int) -> int:
        return sharding_dim

    def _dim(self, name: str) -> int:
        return self._maybe_adjust_sharding_dim(name, get_default_sharding_dim(name))

    @staticmethod
    def _split_or_whole(kind: ShardingType, dim: int, size) -> Decision:
        size = int(size or 1)
        return (kind, dim, size) if size > 1 else (ShardingType.NO_SHARDING, dim, 1)

    def _tp_or_attn_dp(self, name: str, dp_variant: bool) -> Decision:
        dim = self._dim(name)
        if dp_variant:
            return self._split_or_whole(ShardingType.DP_TP_SHARDING, dim, self.rank_info.attn_tp_size)
        return self._split_or_whole(ShardingType.TP_SHARDING, dim, self.rank_info.tp_size)

    # ---- per-family decisions -----------------------------------------
    def get_attention_sharding_strategy(self, parameter_name, **kwargs) -> Decision:
        return self._tp_or_attn_dp(parameter_name, bool(self.enable_dp_attention))

    def get_embedding_sharding_strategy(self, parameter_name, **kwargs) -> Decision:
        return self.get_attention_sharding_strategy(parameter_name, **kwargs)

    def get_lm_head_sharding_strategy(self, parameter_name, **kwargs) -> Decision:
        return self._tp_or_attn_dp(parameter_name, bool(self.enable_dp_lm_head))

    def get_mlp_sharding_strategy(self, parameter_name, **kwargs) -> Decision:
        return self._split_or_whole(ShardingType.TP_SHARDING, self._dim(parameter_name), self.rank_info.tp_size)

    def get_expert_sharding_strategy(self, parameter_name, **kwargs) -> Decision:
        dim = self._dim(parameter_name)
        ep, etp = int(self.ep_size or 1), int(self.ep_tp_size or 1)
        if ep > 1 and etp > 1:
            return ShardingType.EP_TP_SHARDING, dim, etp
        if ep > 1:
            return ShardingType.EP_SHARDING, dim, ep
        return self._split_or_whole(ShardingType.TP_SHARDING, dim, self.tp_size)

    def get_shared_expert_sharding_strategy(self, parameter_name, **kwargs) -> Decision:
        if self.engine_name == "mcore":
            return self._split_or_whole(ShardingType.TP_SHARDING, self._dim(parameter_name), self.tp_size)
        return self.get_expert_sharding_strategy(parameter_name, **kwargs)

    # ---- router --------------------------------------------------------
    def rules(self) -> List[Tuple[Callable[[str], bool], Callable[..., Decision]]]:
        whole = lambda name, **kw: (ShardingType.NO_SHARDING, 0, 1)  # noqa: E731
        has = lambda *keys: (lambda n: any(k in n for k in keys))  # noqa: E731
        return [
            (has("norm"), whole),  # also covers input/post_attention layernorm
            (has("embedding", "embed_tokens"), self.get_embedding_sharding_strategy),
            (has("lm_head"), self.get_lm_head_sharding_strategy),
            (has("expert_bias"), whole),
            (has("shared_experts"), self.get_shared_expert_sharding_strategy),
            (has("expert"), self.get_expert_sharding_strategy),
            (has("gate.weight", "router.weight"), whole),
            (has("mlp"), self.get_mlp_sharding_strategy),
            # "self_attn" names (architectures whose converters keep Hugging Face attention names) follow the
            # attention rule too: under DP attention they are cut over attention TP, not TP
            (has("attention", "self_attn"), self.get_attention_sharding_strategy),
        ]

    def get_sharding_strategy(self, parameter_name, **kwargs) -> Decision:
        if self.rank_info.tp_size == 1:
            return ShardingType.NO_SHARDING, self._dim(parameter_name), 1
        for matches, decide in self.rules():
            if matches(parameter_name):
                return decide(parameter_name, **kwargs)
        return ShardingType.TP_SHARDING, self._dim(parameter_name), self.rank_info.tp_size


class LinearMLAShardingMixin:
    """MLA low-rank ``*_a_proj`` projections and their norms are replicated;
    the Lightning-attention group norm is TP-split
    (`awex/sharding/param_sharding.py:296-318`)."""

    _REPLICATED = (
        "attention.kv_a_proj_with_mqa.weight",
        "attention.q_a_proj.weight",
        "attention.fused_qkv_a_proj_with_mqa.weight",
        "attention.kv_a_layernorm.weight",
        "attention.q_a_layernorm.weight",
    )

    def get_sharding_strategy(self, parameter_name, **kwargs):
        if any(k in parameter_name for k in self._REPLICATED):
            return ShardingType.NO_SHARDING, get_default_sharding_dim(parameter_name), 1
        if "attention.g_norm.weight" in parameter_name:
            dim = get_default_sharding_dim(parameter_name)
            tp = self.rank_info.tp_size
            return (ShardingType.TP_SHARDING, dim, tp) if tp > 1 else (ShardingType.NO_SHARDING, dim, 1)
        return super().get_sharding_strategy(parameter_name, **kwargs)


def get_sharding_strategy_builder(engine_name: str):
    from awex_b200.sharding import extractors

    try:
        return {
            "sglang": extractors.get_sglang_sharding_strategy,
            "vllm": extractors.get_vllm_sharding_strategy,
            "mcore": extractors.get_mcore_sharding_strategy,
        }[engine_name]
    except KeyError:
        raise ValueError(f"Unknown engine_name {engine_name}") from None


def get_rank_info_extractor(engine_name: str):
    from awex_b200.sharding import extractors

    try:
        return {
            "sglang": extractors.get_sglang_rank_info,
            "vllm": extractors.get_vllm_rank_info,
            "mcore": extractors.get_mcore_rank_info,
        }[engine_name]
    except KeyError:
        raise ValueError(f"Unknown engine_name {engine_name}") from None
