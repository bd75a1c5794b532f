"""vLLM parameter names -> canonical names.

vLLM keeps ``self_attn.{qkv_proj,o_proj,q_norm,k_norm}``; the default
canonical contract uses ``attention.{query_key_value_proj,dense,
query_layernorm,key_layernorm}``.  Names are normalised first and then handled
exactly like SGLang's (`awex/converter/vllm_converter.py:35-56`)."""

from __future__ import annotations

from awex_b200.converter.sglang_converter import LinearMLASGlangConverterMixin, SGlangToHFWeightConverter
from awex_b200.converter.weights_converter import append_scale_inv, normalize_scale_inv_name

# longest needles first so that ".self_attn.qkv_proj" is not caught by ".self_attn.qkv"
_RENAMES = (
    (".self_attn.attn.qkv_proj", ".attention.query_key_value_proj"),
    (".self_attn.attn.qkv", ".attention.query_key_value_proj"),
    (".self_attn.qkv_proj", ".attention.query_key_value_proj"),
    (".self_attn.qkv", ".attention.query_key_value_proj"),
    (".self_attn.attn.o_proj", ".attention.dense"),
    (".self_attn.o_proj", ".attention.dense"),
    (".self_attn.proj", ".attention.dense"),
    (".self_attn.q_norm", ".attention.query_layernorm"),
    (".self_attn.k_norm", ".attention.key_layernorm"),
)


class VLLMToHFWeightConverter(LinearMLASGlangConverterMixin, SGlangToHFWeightConverter):
    def _normalize_name(self, name: str) -> str:
        base, scaled = normalize_scale_inv_name(name)
        for needle, repl in _RENAMES:
            if needle in base:
                base = base.replace(needle, repl)
                break
        return append_scale_inv(base, scaled)

    def convert_param(self, name, parameter):
        return super().convert_param(self._normalize_name(name), parameter)
