"""Inference-engine (SGLang-style) parameter layout -> canonical names.

Everything returned is a *view* into the live parameter it was derived from
(``narrow`` / integer indexing only), because the data plane writes received
weights through these views in place.  Observable naming follows the
reference (`awex/converter/sglang_converter.py:313-399`):

* fused ``qkv_proj`` stays fused (default) or is cut into q/k/v in the ratio
  ``n_heads : n_kv : n_kv`` for models that publish split projections;
* ``gate_up_proj`` / ``w13_weight`` are cut into gate (first half) and up;
* fused expert tensors ``w13_weight[E, 2I, H]`` / ``w2_weight[E, H, I]`` become
  one canonical parameter per expert, with global id ``e + ep_rank * E`` under
  expert parallelism; without EP, slots past the routed experts are shared
  experts.
"""

from __future__ import annotations

from typing import List, Tuple

import torch

from awex_b200.converter.weights_converter import append_scale_inv, normalize_scale_inv_name
from awex_b200.utils.common import cfg_get

Named = List[Tuple[str, torch.Tensor]]

_PASS_THROUGH_TOP = {
    "model.embed_tokens.weight": "model.embed_tokens.weight",
    "model.norm.weight": "model.norm.weight",
    "lm_head.weight": "lm_head.weight",
    "model.lm_head.weight": "lm_head.weight",
}


class SGlangToHFWeightConverter:
    def __init__(self, model_config, infer_engine_config, rank_info):
        self.model_config = model_config
        self.total_num_heads = cfg_get(model_config, "num_attention_heads")
        self.total_kv_heads = cfg_get(model_config, "num_key_value_heads")
        self.infer_engine_config = infer_engine_config
        self.rank_info = rank_info
        self.tp_size = cfg_get(infer_engine_config, "tp_size")
        self.tp_rank = rank_info.tp_rank
        self.ep_size = cfg_get(infer_engine_config, "ep_size") or 1
        self.ep_rank = rank_info.ep_rank
        self.device_backend = "cuda"

    # ---- knobs ---------------------------------------------------------------------
    def _fuse_qkv(self, name: str) -> bool:
        return True

    def _fuse_gate_up_proj(self, name: str) -> bool:
        return False

    # ---- pieces ----------------------------------------------------------------------
    @staticmethod
    def _halves(name: str, t: torch.Tensor) -> Named:
        half = t.shape[0] // 2

        def rename(part):
            return name.replace("gate_up_proj", f"{part}_proj").replace("w13_weight", f"{part}_proj.weight")

        return [(rename("gate"), t.narrow(0, 0, half)), (rename("up"), t.narrow(0, half, half))]

    def _split_gate_up(self, name: str, parameter: torch.Tensor) -> Named:
        return self._halves(name, parameter)

    def _convert_attention_param(self, name: str, parameter: torch.Tensor, layer_number: str) -> Named:
        if "qkv_proj" in name or "query_key_value" in name:
            if self._fuse_qkv(name):
                return [(name, parameter)]
            heads = int(self.total_num_heads)
            kv = int(self.total_kv_heads or heads)
            # attention is cut over attention TP, which is smaller than TP under DP attention
            tp = int(getattr(self.rank_info, "attn_tp_size", 0) or self.tp_size or 1)
            if tp > kv and tp % kv == 0 and heads % tp == 0:
                # every rank stores one whole (replicated) KV head beside its query heads
                heads, kv = heads // tp, 1
            units, rows = heads + 2 * kv, parameter.shape[0]
            if (rows * heads) % units or (rows * kv) % units:
                raise ValueError(
                    f"qkv dim0 {rows} of {name} is not divisible into q/k/v with num_heads={heads}, num_kv_heads={kv}"
                )
            q_rows, kv_rows = rows * heads // units, rows * kv // units
            out, start = [], 0
            for part, n in (("q_proj", q_rows), ("k_proj", kv_rows), ("v_proj", kv_rows)):
                out.append((name.replace("qkv_proj", part).replace("query_key_value", part), parameter.narrow(0, start, n)))
                start += n
            return out
        if "o_proj" in name or "dense" in name:
            return [(name, parameter)]
        raise NotImplementedError(f"Unsupported attention parameter name: {name}")

    def _convert_mlp_param(self, name: str, parameter: torch.Tensor, layer_number: str) -> Named:
        if "gate_up_proj" in name:
            return [(name, parameter)] if self._fuse_gate_up_proj(name) else self._split_gate_up(name, parameter)
        if "down_proj" in name:
            return [(name, parameter)]
        if "w13_weight" in name:
            if self._fuse_gate_up_proj(name):
                return [(name.replace("w13_weight", "gate_up_proj.weight"), parameter)]
            return self._split_gate_up(name, parameter)
        if "w2_weight" in name:
            return [(name.replace("w2_weight", "down_proj.weight"), parameter)]
        raise NotImplementedError(f"Unsupported MLP parameter name: {name}")

    def _n_routed_experts(self) -> int:
        return int(cfg_get(self.model_config, "num_experts") or cfg_get(self.model_config, "n_routed_experts"))

    def _convert_expert_tp_param(self, name: str, parameter: torch.Tensor, layer_number: str) -> Named:
        """No expert parallelism: every rank holds a TP slice of every expert."""
        if "expert_bias" in name:
            return [(name, parameter)]
        if "shared_experts" in name:
            return self._convert_mlp_param(name, parameter, layer_number)
        routed = self._n_routed_experts()
        n_shared = parameter.shape[0] - routed
        out: Named = []
        for slot in range(parameter.shape[0]):
            if slot < routed:
                slot_name = name.replace("experts", f"experts.{slot}")
            elif n_shared > 1:
                slot_name = name.replace("experts", f"shared_experts.{slot - routed}")
            else:
                slot_name = name.replace("experts", "shared_experts")
            out.extend(self._convert_mlp_param(slot_name, parameter[slot], layer_number))
        return out

    def _convert_expert_moe_param(self, name: str, parameter: torch.Tensor, layer_number: str) -> Named:
        """Expert parallelism: this rank holds ``parameter.shape[0]`` whole experts."""
        if "expert_bias" in name:
            return [(name, parameter)]
        if "shared_experts" in name:
            return self._convert_mlp_param(name, parameter, layer_number)
        if "w13_weight" not in name and "w2_weight" not in name:
            raise NotImplementedError(f"Unsupported expert parameter name: {name}")
        n_local = parameter.shape[0]
        out: Named = []
        for slot in range(n_local):
            gid = slot + self.ep_rank * n_local
            for sub, view in self._convert_mlp_param(name, parameter[slot], layer_number):
                if sub.startswith("mlp.experts."):
                    sub = sub.replace("mlp.experts.", f"mlp.experts.{gid}.", 1)
                elif sub.startswith("mlp."):
                    sub = sub.replace("mlp.", f"mlp.experts.{gid}.", 1)
                else:
                    sub = f"mlp.experts.{gid}.{sub}"
                out.append((sub, view))
        return out

    def _convert_layer_norm_param(self, name: str, parameter: torch.Tensor, layer_number: str) -> Named:
        if any(k in name for k in ("input_layernorm", "post_attention_layernorm", "query_layernorm", "key_layernorm")):
            return [(name, parameter)]
        raise NotImplementedError(f"Unsupported layer norm parameter name: {name}")

    # ---- entry point -------------------------------------------------------------------------
    @torch.no_grad()
    def convert_param(self, name: str, parameter: torch.Tensor) -> Named:
        if name in _PASS_THROUGH_TOP:
            return [(_PASS_THROUGH_TOP[name], parameter)]
        if "model.layers." not in name:
            return [(name, parameter)]
        parts = name.split(".")
        at = parts.index("layers")
        if at + 1 >= len(parts):
            raise ValueError(f"Could not extract layer number from parameter name: {name}")
        layer = parts[at + 1]
        rest = ".".join(parts[at + 2 :])
        prefix = f"model.layers.{layer}."
        if "layernorm" in rest or "norm" in rest:
            converted = self._convert_layer_norm_param(rest, parameter, layer)
        elif "attention" in rest or "self_attn" in rest:
            converted = self._convert_attention_param(rest, parameter, layer)
        elif "mlp" in rest:
            if "gate.weight" in rest:
                return [(name, parameter)]
            if "router.weight" in rest:
                return [(prefix + "mlp.gate.weight", parameter)]
            if ".expert" in rest or "experts." in rest:
                fn = self._convert_expert_tp_param if self.ep_size == 1 else self._convert_expert_moe_param
                converted = fn(rest, parameter, layer)
            else:
                converted = self._convert_mlp_param(rest, parameter, layer)
        else:
            return [(name, parameter)]
        return [(prefix + n, t) for n, t in converted]


class LinearMLASGlangConverterMixin:
    """Names of the MLA / Lightning-attention family pass through (with
    ``o_proj`` published as ``dense``); block-scale companions
    (``*_scale_inv``) follow their weight
    (`awex/converter/sglang_converter.py:402-477`)."""

    _NORMS = {
        "input_layernorm.weight", "post_attention_layernorm.weight", "attention.g_norm.weight",
        "attention.query_layernorm.weight", "attention.key_layernorm.weight",
        "attention.kv_a_layernorm.weight", "attention.q_a_layernorm.weight",
    }
    _ATTN_SAME = {
        "attention.g_proj.weight", "attention.q_proj.weight", "attention.k_proj.weight", "attention.v_proj.weight",
        "attention.dense.weight", "attention.g_norm.weight", "attention.query_layernorm.weight",
        "attention.key_layernorm.weight", "attention.kv_a_proj_with_mqa.weight", "attention.kv_b_proj.weight",
        "attention.kv_a_layernorm.weight", "attention.q_b_proj.weight", "attention.q_a_layernorm.weight",
        "attention.q_a_proj.weight", "attention.fused_qkv_a_proj_with_mqa.weight",
    }

    def _fuse_qkv(self, name: str) -> bool:
        return True

    def _fuse_gate_up_proj(self, name: str) -> bool:
        return False

    def _convert_layer_norm_param(self, name, parameter, layer_number):
        base, scaled = normalize_scale_inv_name(name)
        if base in self._NORMS:
            return [(append_scale_inv(base, scaled), parameter)]
        return super()._convert_layer_norm_param(name, parameter, layer_number)

    def _convert_attention_param(self, name, parameter, layer_number):
        base, scaled = normalize_scale_inv_name(name)
        if base in self._ATTN_SAME:
            return [(append_scale_inv(base, scaled), parameter)]
        if base == "attention.o_proj.weight":
            return [(append_scale_inv("attention.dense.weight", scaled), parameter)]
        for kind in ("weight", "bias"):
            if base in (f"attention.query_key_value.{kind}", f"self_attn.qkv_proj.{kind}") and self._fuse_qkv(base):
                return [(append_scale_inv(f"attention.query_key_value.{kind}", scaled), parameter)]
        if "o_proj" in base or "dense" in base:
            return [(append_scale_inv(base, scaled), parameter)]
        return super()._convert_attention_param(name, parameter, layer_number)
