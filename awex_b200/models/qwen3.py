"""Dense Qwen3 (``Qwen3ForCausalLM``): same attention contract as Qwen3-MoE,
no expert parameters (`awex/models/qwen3.py:17-37` in the reference)."""

from awex_b200.models.qwen3_moe import SGlangToHFWeightConverterQwen3Moe, _build_mcore_converter_qwen3_moe

CONFIG = {
    "model_name": "Qwen3ForCausalLM",
    "mcore_converter": _build_mcore_converter_qwen3_moe,
    "sglang_converter": SGlangToHFWeightConverterQwen3Moe,
}
