"""Architecture presets for synthetic (random-init) models.

No checkpoint or dataset is needed to exercise a weight exchange: what matters
is the set of parameter names, shapes, dtypes and layouts.  A preset describes
a decoder architecture; :mod:`awex_b200.synthetic.models` builds Megatron-layout
training shards and vLLM-layout inference shards for it from per-name seeds.
"""

from __future__ import annotations

from dataclasses import dataclass, field, replace
from types import SimpleNamespace
from typing import Dict, Optional


@dataclass(frozen=True)
class Arch:
    name: str
    architecture: str  # HF class name; selects converters through the registry
    num_layers: int
    hidden: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    ffn: int  # dense MLP intermediate size (0 for pure-MoE layers)
    vocab: int
    qkv_bias: bool = False
    qk_norm: bool = False
    tie_embeddings: bool = False
    num_experts: int = 0
    expert_ffn: int = 0
    top_k: int = 0
    norm_head: bool = False  # lm_head is published with unit-norm columns (`mcore_converter.py:668-675` in the reference)

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def hf_config(self) -> SimpleNamespace:
        cfg = SimpleNamespace(
            architectures=[self.architecture],
            num_hidden_layers=self.num_layers,
            hidden_size=self.hidden,
            num_attention_heads=self.num_heads,
            num_key_value_heads=self.num_kv_heads,
            head_dim=self.head_dim,
            intermediate_size=self.ffn,
            vocab_size=self.vocab,
            tie_word_embeddings=self.tie_embeddings,
            attention_bias=self.qkv_bias,
        )
        if self.norm_head:
            cfg.norm_head = True
        if self.is_moe:
            cfg.num_experts = self.num_experts
            cfg.moe_intermediate_size = self.expert_ffn
            cfg.num_experts_per_tok = self.top_k
        return cfg

    def hf_config_dict(self, dtype: str = "bfloat16") -> dict:
        """A ``config.json`` that Hugging Face loaders and inference engines accept
        for this architecture (random weights are then made by the engine, e.g.
        vLLM's ``--load-format dummy``)."""
        model_types = {"LlamaForCausalLM": "llama", "Qwen2ForCausalLM": "qwen2", "Qwen3ForCausalLM": "qwen3",
                       "Qwen3MoeForCausalLM": "qwen3_moe"}
        if self.architecture not in model_types:
            raise KeyError(f"no config.json template for {self.architecture}")
        cfg = {
            "architectures": [self.architecture], "model_type": model_types[self.architecture],
            "num_hidden_layers": self.num_layers, "hidden_size": self.hidden, "num_attention_heads": self.num_heads,
            "num_key_value_heads": self.num_kv_heads, "head_dim": self.head_dim,
            "intermediate_size": self.ffn or self.expert_ffn, "vocab_size": self.vocab, "hidden_act": "silu",
            "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "max_position_embeddings": 4096,
            "tie_word_embeddings": self.tie_embeddings, "attention_bias": self.qkv_bias, "torch_dtype": dtype,
            "bos_token_id": 1, "eos_token_id": 2,
        }
        if self.is_moe:
            cfg.update(num_experts=self.num_experts, moe_intermediate_size=self.expert_ffn, num_experts_per_tok=self.top_k,
                       decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True)
        return cfg

    def write_model_dir(self, path: str, dtype: str = "bfloat16") -> str:
        """Create ``path`` with this architecture's ``config.json`` (no weights, no tokenizer)."""
        import json
        import os

        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(self.hf_config_dict(dtype), f, indent=1)
        return path

    def tf_config(self) -> SimpleNamespace:
        """The subset of Megatron's TransformerConfig the converters read."""
        return SimpleNamespace(
            hidden_size=self.hidden,
            num_attention_heads=self.num_heads,
            num_query_groups=self.num_kv_heads,
            kv_channels=self.head_dim,
            num_layers=self.num_layers,
        )

    def with_layers(self, n: int) -> "Arch":
        return replace(self, num_layers=n, name=f"{self.name}-L{n}")

    def param_count(self) -> int:
        h = self.hidden
        attn = (self.num_heads + 2 * self.num_kv_heads) * self.head_dim * h + self.num_heads * self.head_dim * h
        if self.qkv_bias:
            attn += (self.num_heads + 2 * self.num_kv_heads) * self.head_dim
        if self.qk_norm:
            attn += 2 * self.head_dim
        mlp = 3 * h * self.ffn if not self.is_moe else self.num_experts * 3 * h * self.expert_ffn + self.num_experts * h
        per_layer = attn + mlp + 2 * h
        embeds = self.vocab * h * (1 if self.tie_embeddings else 2)
        return self.num_layers * per_layer + embeds + h


PRESETS: Dict[str, Arch] = {
    a.name: a
    for a in (
        # 2 layers, hidden 256, 4/2 heads, SwiGLU 512, vocab 1024
        Arch("tiny-llama", "LlamaForCausalLM", 2, 256, 4, 2, 64, 512, 1024),
        Arch("llama3-8b", "LlamaForCausalLM", 32, 4096, 32, 8, 128, 14336, 128256),
        Arch("qwen2.5-32b", "Qwen2ForCausalLM", 64, 5120, 40, 8, 128, 27648, 152064, qkv_bias=True),
        Arch("qwen3-30b-a3b", "Qwen3MoeForCausalLM", 48, 2048, 32, 4, 128, 0, 151936, qk_norm=True,
             num_experts=128, expert_ffn=768, top_k=8),
        Arch("qwen3-235b-a22b", "Qwen3MoeForCausalLM", 94, 4096, 64, 4, 128, 0, 151936, qk_norm=True,
             num_experts=128, expert_ffn=1536, top_k=8),
        Arch("tiny-qwen3-moe", "Qwen3MoeForCausalLM", 2, 256, 8, 4, 32, 0, 1024, qk_norm=True,
             num_experts=8, expert_ffn=128, top_k=2),
        Arch("tiny-qwen2", "Qwen2ForCausalLM", 2, 256, 8, 4, 32, 512, 1024, qkv_bias=True),
        Arch("tiny-llama-norm-head", "LlamaForCausalLM", 2, 256, 4, 2, 64, 512, 1024, norm_head=True),
    )
}


def get_arch(name: str) -> Arch:
    if name not in PRESETS:
        raise KeyError(f"unknown architecture preset {name!r}; known: {sorted(PRESETS)}")
    return PRESETS[name]
