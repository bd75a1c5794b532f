"""Qwen3-MoE (``Qwen3MoeForCausalLM``).

Canonical attention names stay ``self_attn.{q,k,v,o}_proj`` and
``self_attn.{q,k}_norm``.  Training side: the rank-local Megatron
``linear_qkv`` (``n_kv / attn_tp`` groups of ``[q_g | k_g | v_g]``) is cut into
Q, K and V locally, with no TP gather.  Inference side: the fused ``qkv_proj``
is cut in the ratio ``n_heads : n_kv : n_kv``
(`awex/models/qwen3_moe.py:28-140` in the reference).
"""

from __future__ import annotations

from awex_b200.converter.rows import IDENTITY, Rows
from awex_b200.converter.sglang_converter import SGlangToHFWeightConverter


class SGlangToHFWeightConverterQwen3Moe(SGlangToHFWeightConverter):
    def _fuse_qkv(self, name: str) -> bool:
        return False

    def _convert_layer_norm_param(self, name, parameter, layer_number):
        if "q_norm" in name or "k_norm" in name:
            return [(name, parameter)]
        return super()._convert_layer_norm_param(name, parameter, layer_number)


def _build_mcore_converter_qwen3_moe():
    from awex_b200.converter.mcore_converter import McoreToHFWeightConverter, split_interleaved_qkv

    class McoreToHFWeightConverterQwen3Moe(McoreToHFWeightConverter):
        def _fuse_qkv(self, name: str) -> bool:
            return False

        @staticmethod
        def _normalize_attn_name(name: str) -> str:
            return name

        def _gqa_head_dim(self) -> int:
            head_dim = getattr(self.hf_config, "head_dim", None)
            return int(head_dim or self.hf_config.hidden_size // self.hf_config.num_attention_heads)

        def _split_gqa_rows(self, rows):
            hf = self.hf_config
            attn_tp = max(1, int(getattr(self.rank_info, "attn_tp_size", 1)))
            if hf.num_key_value_heads % attn_tp != 0:
                raise ValueError(
                    f"num_key_value_heads ({hf.num_key_value_heads}) must be divisible by attn_tp_size ({attn_tp})"
                )
            if hf.num_attention_heads % hf.num_key_value_heads != 0:
                raise ValueError(
                    f"num_attention_heads ({hf.num_attention_heads}) must be divisible by num_key_value_heads "
                    f"({hf.num_key_value_heads})"
                )
            head = self._gqa_head_dim()
            groups = hf.num_key_value_heads // attn_tp
            q_per_group = hf.num_attention_heads // hf.num_key_value_heads
            expected = groups * (q_per_group + 2) * head
            if len(rows) != expected:
                raise ValueError(
                    f"Unexpected linear_qkv rows for GQA split: got {len(rows)}, expected {expected} "
                    f"(kv_heads={hf.num_key_value_heads}, attn_tp={attn_tp}, q_per_group={q_per_group}, head_dim={head})"
                )
            q, k, v = split_interleaved_qkv(rows, groups, q_per_group * head, head)
            # More attention-TP ranks on the inference side than KV heads: every
            # inference rank stores a whole KV head, so each head appears
            # infer_tp / n_kv times in the canonical K and V (the reference
            # refuses this layout, `awex/converter/sglang_converter.py:127-136`).
            infer_tp = int(self.infer_atten_tp_size or 1)
            if infer_tp > hf.num_key_value_heads:
                if infer_tp % hf.num_key_value_heads:
                    raise ValueError(f"inference attention TP {infer_tp} is not a multiple of num_key_value_heads {hf.num_key_value_heads}")
                repeat = infer_tp // hf.num_key_value_heads
                k = Rows.cat([part for part in k.chunk(groups) for _ in range(repeat)])
                v = Rows.cat([part for part in v.chunk(groups) for _ in range(repeat)])
            return q, k, v

        def _convert_attention_param(self, name, src, rows, layer_number):
            for kind in ("weight", "bias"):
                if f"self_attention.linear_qkv.{kind}" in name:
                    return [
                        (f"self_attn.{p}_proj.{kind}", r, IDENTITY) for p, r in zip("qkv", self._split_gqa_rows(rows))
                    ]
            return super()._convert_attention_param(name, src, rows, layer_number)

    return McoreToHFWeightConverterQwen3Moe


CONFIG = {
    "model_name": "Qwen3MoeForCausalLM",
    "mcore_converter": _build_mcore_converter_qwen3_moe,
    "sglang_converter": SGlangToHFWeightConverterQwen3Moe,
}
