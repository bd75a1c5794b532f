"""Bailing-MoE V2 / V2.5 / Linear: layers alternate Lightning (linear)
attention and MLA; ``lm_head`` and the router's ``expert_bias`` are served in
fp32; with fp8 only routed-expert gate/up/down projections are quantised, with
ordinary (not power-of-two) scales; SGLang calls the input embedding
``word_embeddings`` (`awex/models/ling_linear.py:36-140` in the reference)."""

from __future__ import annotations

import torch

from awex_b200.converter.rows import ValueOp
from awex_b200.converter.sglang_converter import LinearMLASGlangConverterMixin, SGlangToHFWeightConverter
from awex_b200.models.ling import BailingMoeShardingStrategy, _build_mcore_converter_bailing_moe
from awex_b200.sharding.param_sharding import LinearMLAShardingMixin


class BailingLinearMoeShardingStrategy(LinearMLAShardingMixin, BailingMoeShardingStrategy):
    pass


def _build_mcore_converter_bailing_moe_linear():
    from awex_b200.converter.mcore_converter import LinearMLAMcoreConverterMixin

    base = _build_mcore_converter_bailing_moe()

    class McoreToHFWeightConverterBailingMoeLinear(LinearMLAMcoreConverterMixin, base):
        def __init__(self, hf_config, rank_info, infer_conf, tf_config):
            super().__init__(hf_config, rank_info, infer_conf, tf_config=tf_config)
            if self.quant_method == "fp8":
                self.fp8_weight_keys = {"up_proj.weight", "down_proj.weight", "gate_proj.weight"}

        def _convert_lm_head_param(self, name, rows):
            return [("lm_head.weight", rows, ValueOp("cast", dtype=torch.float32))]

        def _is_fp8_name(self, canonical_name: str) -> bool:
            return (
                ".experts." in canonical_name
                and "shared_experts" not in canonical_name
                and any(k in canonical_name for k in self.fp8_weight_keys)
            )

        def _fp8_ue8m0(self, canonical_name: str) -> bool:
            return False

    return McoreToHFWeightConverterBailingMoeLinear


class SGlangToHFWeightConverterBailingMoeLinear(LinearMLASGlangConverterMixin, SGlangToHFWeightConverter):
    def convert_param(self, name, parameter):
        if name == "model.word_embeddings.weight":
            name = "model.embed_tokens.weight"
        return super().convert_param(name, parameter)


CONFIG = [
    {
        "model_name": arch,
        "sharding_strategy": BailingLinearMoeShardingStrategy,
        "mcore_converter": _build_mcore_converter_bailing_moe_linear,
        "sglang_converter": SGlangToHFWeightConverterBailingMoeLinear,
    }
    for arch in ("BailingMoeV2ForCausalLM", "BailingMoeLinearForCausalLM", "BailingMoeV2_5ForCausalLM", "BailingMoeV2_5ForCausalLMNextN")
]
