"""Qwen3-VL dense and MoE (``Qwen3VLForConditionalGeneration``,
``Qwen3VLMoeForConditionalGeneration``).

The language model uses the Qwen3 contract under the ``model.language_model.``
namespace; the vision tower maps Megatron ``vision_model.*`` names to
``model.visual.*`` and regroups its MHA QKV per inference TP rank like the
default fused contract.  Vision sharding: patch embedding, biases and norms
replicated; qkv / fc1 split on dim 0, proj / fc2 on dim 1; the learned position
embedding is replicated by training and split by SGLang
(`awex/models/qwen3_vl.py:54-326` in the reference).
"""

from __future__ import annotations

import re
from types import SimpleNamespace
from typing import Any

import torch

from awex_b200.converter.rows import IDENTITY
from awex_b200.models.qwen3_moe import SGlangToHFWeightConverterQwen3Moe, _build_mcore_converter_qwen3_moe
from awex_b200.sharding.param_sharding import ShardingStrategy, ShardingType, get_default_sharding_dim
from awex_b200.utils.common import cfg_get


def get_qwen3_vl_text_config(config: Any) -> Any:
    return cfg_get(config, "text_config", config)


def _uses_tied_embeddings(config: Any) -> bool:
    return bool(cfg_get(get_qwen3_vl_text_config(config), "tie_word_embeddings", False))


_REPLICATED_SUFFIXES = (".bias", ".norm.weight", ".norm.bias", ".norm1.weight", ".norm1.bias", ".norm2.weight", ".norm2.bias")
_DIM0 = ("attn.qkv.weight", "attn.qkv.bias", "mlp.linear_fc1.weight", "mlp.linear_fc1.bias", "merger.linear_fc1.weight", "merger.linear_fc1.bias")
_DIM1 = ("attn.proj.weight", "mlp.linear_fc2.weight", "merger.linear_fc2.weight")


class Qwen3VLShardingStrategy(ShardingStrategy):
    def _vision_tp_strategy(self, sharding_dim: int):
        if self.enable_dp_attention:
            size, kind = self.rank_info.attn_tp_size, ShardingType.DP_TP_SHARDING
        else:
            size, kind = self.rank_info.tp_size, ShardingType.TP_SHARDING
        return (kind, sharding_dim, size) if size > 1 else (ShardingType.NO_SHARDING, sharding_dim, 1)

    def get_sharding_strategy(self, parameter_name: str, **kwargs):
        n = parameter_name
        if not n.startswith("model.visual."):
            return super().get_sharding_strategy(n, **kwargs)
        dim = get_default_sharding_dim(n)
        split_bias = n.endswith(("qkv.bias", "linear_fc1.bias"))
        if n.startswith("model.visual.patch_embed.") or (n.endswith(_REPLICATED_SUFFIXES) and not split_bias):
            return ShardingType.NO_SHARDING, dim, 1
        if n.endswith("pos_embed.weight"):
            return (ShardingType.NO_SHARDING, 0, 1) if self.engine_name == "mcore" else self._vision_tp_strategy(0)
        deepstack = ".deepstack_merger_list." in n
        if n.endswith(_DIM0) or (deepstack and n.endswith(("linear_fc1.weight", "linear_fc1.bias"))):
            return self._vision_tp_strategy(0)
        if n.endswith(_DIM1) or (deepstack and n.endswith("linear_fc2.weight")):
            return self._vision_tp_strategy(1)
        return ShardingType.NO_SHARDING, dim, 1


class Qwen3VLSGlangToHFWeightConverter(SGlangToHFWeightConverterQwen3Moe):
    def __init__(self, model_config, infer_engine_config, rank_info):
        self.vl_model_config = model_config
        super().__init__(get_qwen3_vl_text_config(model_config), infer_engine_config, rank_info)

    @torch.no_grad()
    def convert_param(self, name, parameter):
        if name.startswith("visual."):
            return [(f"model.{name}".replace(".attn.qkv_proj.", ".attn.qkv."), parameter)]
        out = [
            (n.replace("model.", "model.language_model.", 1) if n.startswith("model.") else n, t)
            for n, t in super().convert_param(name, parameter)
        ]
        if name == "model.embed_tokens.weight" and _uses_tied_embeddings(self.vl_model_config):
            out.append(("lm_head.weight", parameter))
        return out


_VISION_LAYER = re.compile(r"vision_model\.decoder\.layers\.(\d+)\.(.+)")
_VISION_DEEPSTACK = re.compile(r"vision_model\.decoder\.deepstack_merger_list\.(\d+)\.(.+)")
_VISION_DIRECT = {
    f"vision_model.{src}": f"model.visual.{dst}"
    for src, dst in (
        ("patch_embed.proj.weight", "patch_embed.proj.weight"), ("patch_embed.proj.bias", "patch_embed.proj.bias"),
        ("pos_embed.weight", "pos_embed.weight"), ("merger.patch_norm.weight", "merger.norm.weight"),
        ("merger.patch_norm.bias", "merger.norm.bias"), ("merger.linear_fc1.weight", "merger.linear_fc1.weight"),
        ("merger.linear_fc1.bias", "merger.linear_fc1.bias"), ("merger.linear_fc2.weight", "merger.linear_fc2.weight"),
        ("merger.linear_fc2.bias", "merger.linear_fc2.bias"),
    )
}
_VISION_LAYER_NAMES = {
    "self_attention.linear_proj.weight": "attn.proj.weight", "self_attention.linear_proj.bias": "attn.proj.bias",
    "self_attention.linear_qkv.layer_norm_weight": "norm1.weight", "self_attention.linear_qkv.layer_norm_bias": "norm1.bias",
    "mlp.linear_fc1.weight": "mlp.linear_fc1.weight", "mlp.linear_fc1.bias": "mlp.linear_fc1.bias",
    "mlp.linear_fc2.weight": "mlp.linear_fc2.weight", "mlp.linear_fc2.bias": "mlp.linear_fc2.bias",
    "mlp.linear_fc1.layer_norm_weight": "norm2.weight", "mlp.linear_fc1.layer_norm_bias": "norm2.bias",
}
_DEEPSTACK_NAMES = {
    "patch_norm.weight": "norm.weight", "patch_norm.bias": "norm.bias", "linear_fc1.weight": "linear_fc1.weight",
    "linear_fc1.bias": "linear_fc1.bias", "linear_fc2.weight": "linear_fc2.weight", "linear_fc2.bias": "linear_fc2.bias",
}


class VisionTowerRoutes:
    """Routing of Megatron ``vision_model.*`` parameters, shared by the
    Qwen3-VL and Qwen3.5 training converters.  Expects ``self.vl_hf_config``."""

    def _vision_qkv_rows(self, src: str, n_rows: int):
        from awex_b200.converter.mcore_converter import mcore_qkv_to_q_k_v, regroup_qkv_for_infer_tp

        vision = cfg_get(self.vl_hf_config, "vision_config")
        heads, hidden = cfg_get(vision, "num_heads"), cfg_get(vision, "hidden_size")
        if heads is None or hidden is None:
            raise ValueError("vision_config.num_heads and hidden_size are required for vision QKV conversion")
        heads, hidden = int(heads), int(hidden)
        if hidden % heads:
            raise ValueError(f"vision hidden_size must be divisible by num_heads: hidden_size={hidden}, num_heads={heads}")
        vcfg = SimpleNamespace(hidden_size=hidden, num_attention_heads=heads, num_query_groups=heads, kv_channels=hidden // heads)
        tp, rank = max(1, int(self.rank_info.attn_tp_size)), int(self.rank_info.attn_tp_rank)
        q, k, v = mcore_qkv_to_q_k_v(self._tp_full(src, n_rows, tp_size=tp), vcfg)
        merged = regroup_qkv_for_infer_tp(q, k, v, self.infer_atten_tp_size, heads)
        return merged.chunk(tp)[rank] if tp > 1 else merged

    def _route_vision(self, name: str, src: str, rows):
        if name in _VISION_DIRECT:
            return [(_VISION_DIRECT[name], rows, IDENTITY)]
        m = _VISION_LAYER.fullmatch(name)
        if m is not None:
            layer, rest = m.groups()
            base_name = f"model.visual.blocks.{layer}"
            if rest in ("self_attention.linear_qkv.weight", "self_attention.linear_qkv.bias"):
                kind = "weight" if rest.endswith("weight") else "bias"
                return [(f"{base_name}.attn.qkv.{kind}", self._vision_qkv_rows(src, len(rows)), IDENTITY)]
            if rest in _VISION_LAYER_NAMES:
                return [(f"{base_name}.{_VISION_LAYER_NAMES[rest]}", rows, IDENTITY)]
        m = _VISION_DEEPSTACK.fullmatch(name)
        if m is not None:
            idx, rest = m.groups()
            if rest in _DEEPSTACK_NAMES:
                return [(f"model.visual.deepstack_merger_list.{idx}.{_DEEPSTACK_NAMES[rest]}", rows, IDENTITY)]
        raise ValueError(f"Unknown vision parameter: {name}")

    def _plan_vision(self, clean: str, src: str, shape, dtype):
        rows = self._own(src, shape[0] if shape else 1)
        return self._finish_specs(self._route_vision(clean, src, rows), shape if shape else (1,), dtype)


def _build_mcore_converter_qwen3_vl():
    base = _build_mcore_converter_qwen3_moe()

    class Qwen3VLMcoreToHFWeightConverter(VisionTowerRoutes, base):
        def __init__(self, hf_config, rank_info, infer_conf, tf_config):
            self.vl_hf_config = hf_config
            super().__init__(get_qwen3_vl_text_config(hf_config), rank_info, infer_conf, tf_config)

        def plan_param(self, name, shape, dtype, vp_stage=None, source_name=None):
            src = source_name or name
            clean = name.replace("module.", "")
            shape = tuple(int(d) for d in shape)
            if clean.startswith("vision_model."):
                return self._plan_vision(clean, src, shape, dtype)
            if not clean.startswith("language_model."):
                raise ValueError(f"Unknown Qwen3-VL parameter: {name}")
            language_name = clean[len("language_model."):]
            specs = super().plan_param(language_name, shape, dtype, vp_stage=vp_stage, source_name=src)
            for spec in specs:
                if spec.name.startswith("model."):
                    spec.name = spec.name.replace("model.", "model.language_model.", 1)
                    if spec.scale_of is not None:
                        spec.scale_of = spec.scale_of.replace("model.", "model.language_model.", 1)
            if language_name == "embedding.word_embeddings.weight" and _uses_tied_embeddings(self.vl_hf_config):
                import dataclasses

                specs.append(dataclasses.replace(specs[0], name="lm_head.weight"))
            return specs

    return Qwen3VLMcoreToHFWeightConverter


CONFIG = [
    {
        "model_name": arch,
        "sharding_strategy": Qwen3VLShardingStrategy,
        "mcore_converter": _build_mcore_converter_qwen3_vl,
        "sglang_converter": Qwen3VLSGlangToHFWeightConverter,
    }
    for arch in ("Qwen3VLForConditionalGeneration", "Qwen3VLMoeForConditionalGeneration")
]
