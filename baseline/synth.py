"""Synthetic Llama-style weights for driving the reference: Megatron-layout
training shards and vLLM-layout inference shards cut from canonical tensors
that are generated from per-name seeds.  Self-contained on purpose: nothing
here imports the framework under test."""

import hashlib
from collections import OrderedDict
from types import SimpleNamespace

import torch

ARCHS = {
    "llama3-8b": dict(layers=32, hidden=4096, heads=32, kv=8, head_dim=128, ffn=14336, vocab=128256),
    "tiny-llama": dict(layers=2, hidden=256, heads=4, kv=2, head_dim=64, ffn=512, vocab=1024),
    "qwen2.5-32b": dict(layers=64, hidden=5120, heads=40, kv=8, head_dim=128, ffn=27648, vocab=152064, qkv_bias=True),
    "tiny-qwen2": dict(layers=2, hidden=256, heads=8, kv=8, head_dim=32, ffn=512, vocab=1024, qkv_bias=True),
}


def canonical(name, shape, dtype, device, seed=0):
    g = torch.Generator(device=device)
    g.manual_seed(int.from_bytes(hashlib.sha256(f"{seed}/{name}".encode()).digest()[:7], "little"))
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 0.02).to(dtype)


class Module:
    """Duck-typed module: ordered named tensors and a config."""

    def __init__(self, tensors, config):
        self._t, self.config = tensors, config

    def named_parameters(self):
        return iter(self._t.items())

    def parameters(self):
        return iter(self._t.values())

    def state_dict(self):
        return OrderedDict(self._t)


def _rows(t, n, i):
    k = t.shape[0] // n
    return t[i * k:(i + 1) * k]


def _cols(t, n, i):
    k = t.shape[1] // n
    return t[:, i * k:(i + 1) * k].contiguous()


def layer_tensors(a, l, dtype, device):
    p = f"model.layers.{l}."
    q, kv, h = a["heads"] * a["head_dim"], a["kv"] * a["head_dim"], a["hidden"]
    shapes = {"q": (q, h), "k": (kv, h), "v": (kv, h), "o": (h, q), "gate": (a["ffn"], h), "up": (a["ffn"], h),
              "down": (h, a["ffn"]), "ln1": (h,), "ln2": (h,)}
    if a.get("qkv_bias"):
        shapes.update({"qb": (q,), "kb": (kv,), "vb": (kv,)})
    return {k: canonical(p + k, s, dtype, device) for k, s in shapes.items()}


def megatron_module(arch, tp, rank, dtype, device):
    a = ARCHS[arch]
    out = OrderedDict()
    out["embedding.word_embeddings.weight"] = _rows(canonical("embed", (a["vocab"], a["hidden"]), dtype, device), tp, rank).contiguous()
    g_local, qpg, hd = a["kv"] // tp, a["heads"] // a["kv"], a["head_dim"]
    for l in range(a["layers"]):
        t = layer_tensors(a, l, dtype, device)
        p = f"decoder.layers.{l}."
        parts = []
        for g in range(rank * g_local, (rank + 1) * g_local):
            parts += [t["q"][g * qpg * hd:(g + 1) * qpg * hd], t["k"][g * hd:(g + 1) * hd], t["v"][g * hd:(g + 1) * hd]]
        out[p + "self_attention.linear_qkv.layer_norm_weight"] = t["ln1"]
        out[p + "self_attention.linear_qkv.weight"] = torch.cat(parts, 0)
        if a.get("qkv_bias"):
            bias = []
            for g in range(rank * g_local, (rank + 1) * g_local):
                bias += [t["qb"][g * qpg * hd:(g + 1) * qpg * hd], t["kb"][g * hd:(g + 1) * hd], t["vb"][g * hd:(g + 1) * hd]]
            out[p + "self_attention.linear_qkv.bias"] = torch.cat(bias, 0)
        out[p + "self_attention.linear_proj.weight"] = _cols(t["o"], tp, rank)
        out[p + "mlp.linear_fc1.layer_norm_weight"] = t["ln2"]
        out[p + "mlp.linear_fc1.weight"] = torch.cat([_rows(t["gate"], tp, rank), _rows(t["up"], tp, rank)], 0)
        out[p + "mlp.linear_fc2.weight"] = _cols(t["down"], tp, rank)
    out["decoder.final_layernorm.weight"] = canonical("norm", (a["hidden"],), dtype, device)
    out["output_layer.weight"] = _rows(canonical("lm_head", (a["vocab"], a["hidden"]), dtype, device), tp, rank).contiguous()
    cfg = SimpleNamespace(hidden_size=a["hidden"], num_attention_heads=a["heads"], num_query_groups=a["kv"],
                          kv_channels=a["head_dim"], num_layers=a["layers"], add_qkv_bias=bool(a.get("qkv_bias")))
    return Module(out, cfg)


def vllm_module(arch, tp, rank, dtype, device, hf_config, zero=False):
    a = ARCHS[arch]
    out = OrderedDict()
    out["model.embed_tokens.weight"] = _rows(canonical("embed", (a["vocab"], a["hidden"]), dtype, device), tp, rank).contiguous()
    hl, kl, hd = a["heads"] // tp, max(a["kv"] // tp, 1), a["head_dim"]
    k0 = rank * a["kv"] // tp
    for l in range(a["layers"]):
        t = layer_tensors(a, l, dtype, device)
        p = f"model.layers.{l}."
        out[p + "input_layernorm.weight"] = t["ln1"]
        out[p + "self_attn.qkv_proj.weight"] = torch.cat(
            [t["q"][rank * hl * hd:(rank + 1) * hl * hd], t["k"][k0 * hd:(k0 + kl) * hd], t["v"][k0 * hd:(k0 + kl) * hd]], 0)
        if a.get("qkv_bias"):
            out[p + "self_attn.qkv_proj.bias"] = torch.cat(
                [t["qb"][rank * hl * hd:(rank + 1) * hl * hd], t["kb"][k0 * hd:(k0 + kl) * hd], t["vb"][k0 * hd:(k0 + kl) * hd]], 0)
        out[p + "self_attn.o_proj.weight"] = _cols(t["o"], tp, rank)
        out[p + "post_attention_layernorm.weight"] = t["ln2"]
        out[p + "mlp.gate_up_proj.weight"] = torch.cat([_rows(t["gate"], tp, rank), _rows(t["up"], tp, rank)], 0)
        out[p + "mlp.down_proj.weight"] = _cols(t["down"], tp, rank)
    out["model.norm.weight"] = canonical("norm", (a["hidden"],), dtype, device)
    out["lm_head.weight"] = _rows(canonical("lm_head", (a["vocab"], a["hidden"]), dtype, device), tp, rank).contiguous()
    if zero:
        for v in out.values():
            v.zero_()
    cls = type(hf_config.architectures[0], (Module,), {})
    return cls(out, hf_config)


def hf_config_for(arch):
    from transformers import LlamaConfig

    a = ARCHS[arch]
    if a.get("qkv_bias"):
        from transformers import Qwen2Config

        return Qwen2Config(hidden_size=a["hidden"], num_attention_heads=a["heads"], num_key_value_heads=a["kv"],
                           num_hidden_layers=a["layers"], intermediate_size=a["ffn"], vocab_size=a["vocab"],
                           architectures=["Qwen2ForCausalLM"], tie_word_embeddings=False)
    return LlamaConfig(hidden_size=a["hidden"], num_attention_heads=a["heads"], num_key_value_heads=a["kv"],
                       num_hidden_layers=a["layers"], intermediate_size=a["ffn"], vocab_size=a["vocab"],
                       head_dim=a["head_dim"], architectures=["LlamaForCausalLM"], tie_word_embeddings=False)
