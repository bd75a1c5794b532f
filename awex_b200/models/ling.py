"""Bailing-MoE (``BailingMoeForCausalLM``).

Sharding: on the training side the converted fused QKV is the training rank's
chunk of the regrouped tensor, i.e. TP-sharded on dim 0 (never replicated);
embeddings are TP-sharded unless DP attention is on.  fp8: when the HF config
carries ``quantization_config.quant_method == "fp8"`` the listed linear weights
are served block-quantised, with power-of-two (UE8M0) scales for
``attention.dense`` and for routed-expert gate/up projections
(`awex/models/ling.py:32-148` in the reference).  Quantisation itself rides
along with the transfer (fused kernel) instead of running on the training side
before the send.
"""

from __future__ import annotations

import torch

from awex_b200.converter.rows import ValueOp
from awex_b200.converter.sglang_converter import SGlangToHFWeightConverter
from awex_b200.sharding.param_sharding import ShardingStrategy, ShardingType


class BailingMoeShardingStrategy(ShardingStrategy):
    def get_sharding_strategy(self, parameter_name, **kwargs):
        if self.engine_name == "mcore" and "query_key_value" in parameter_name:
            attn_tp = self.rank_info.attn_tp_size
            return (ShardingType.TP_SHARDING, 0, attn_tp) if attn_tp > 1 else (ShardingType.NO_SHARDING, 0, 1)
        return super().get_sharding_strategy(parameter_name, **kwargs)

    def get_embedding_sharding_strategy(self, parameter_name, **kwargs):
        tp = self.rank_info.tp_size
        if not self.enable_dp_attention and tp > 1:
            return ShardingType.TP_SHARDING, 0, tp
        return ShardingType.NO_SHARDING, 0, 1


def _build_mcore_converter_bailing_moe():
    from awex_b200.converter.mcore_converter import McoreToHFWeightConverter

    class McoreToHFWeightConverterBailingMoe(McoreToHFWeightConverter):
        _FP8_KEYS = (
            "up_proj.weight", "down_proj.weight", "gate_proj.weight", "attention.dense.weight",
            "attention.query_key_value.weight",
        )

        def __init__(self, hf_config, rank_info, infer_conf, tf_config):
            super().__init__(hf_config, rank_info, infer_conf, tf_config=tf_config)
            self.quantization_config = getattr(hf_config, "quantization_config", None) or {}
            self.quant_method = self.quantization_config.get("quant_method")
            if self.quant_method:
                assert self.quant_method == "fp8", "Only fp8 quantization is supported"
            self.fp8_weight_keys = set(self._FP8_KEYS) if self.quant_method else set()

        def _fuse_qkv(self, name: str) -> bool:
            return True

        def _fuse_gate_up_proj(self, name: str) -> bool:
            return False

        def _matching_fp8_key(self, canonical_name: str):
            return next((k for k in self.fp8_weight_keys if k in canonical_name), None)

        def _is_fp8_name(self, canonical_name: str) -> bool:
            return self._matching_fp8_key(canonical_name) is not None

        def _fp8_ue8m0(self, canonical_name: str) -> bool:
            key = self._matching_fp8_key(canonical_name)
            if key == "attention.dense.weight":
                return True
            return ".experts." in canonical_name and key is not None and "_proj.weight" in key and "down_proj" not in key

        def _value_op_for(self, canonical_name, spec):
            if self.quant_method == "fp8" and spec.value_op.kind == "none" and len(spec.shape) == 2 and self._is_fp8_name(canonical_name):
                return ValueOp("fp8_block", dtype=torch.float8_e4m3fn, ue8m0=self._fp8_ue8m0(canonical_name))
            return spec.value_op

    return McoreToHFWeightConverterBailingMoe


class SGlangToHFWeightConverterBailingMoe(SGlangToHFWeightConverter):
    def _fuse_qkv(self, name: str) -> bool:
        return True

    def _fuse_gate_up_proj(self, name: str) -> bool:
        return False


CONFIG = {
    "model_name": "BailingMoeForCausalLM",
    "sharding_strategy": BailingMoeShardingStrategy,
    "mcore_converter": _build_mcore_converter_bailing_moe,
    "sglang_converter": SGlangToHFWeightConverterBailingMoe,
}
