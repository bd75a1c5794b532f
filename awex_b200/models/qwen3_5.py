"""Qwen3.5 / Qwen3.6 dense, MoE and multimodal (``Qwen3_5*`` architectures).

Layers alternate full attention and Gated DeltaNet (GDN).  What differs from
Qwen3 (`awex/models/qwen3_5.py:52-638` in the reference):

* full-attention ``linear_qkv`` is stored per KV group as ``[Q | gate | K | V]``;
  the canonical tensor stays fused as ``[Q-with-gate | K | V]`` per inference TP
  rank, each query head followed by its gate head, KV heads repeated when the
  inference TP exceeds their number;
* GDN ``in_proj`` is stored rank-locally as ``[Q,K,V,Z,B,A]`` and published as
  fused ``in_proj_qkvz`` and ``in_proj_ba`` in inference-rank order; the conv1d
  channels ``[Q,K,V]`` are re-ordered the same way;
* ``out_norm.weight`` is published as ``linear_attn.norm.weight + 1``;
* ``shared_experts`` is spelled ``shared_expert``; MTP (draft head) parameters
  are frozen during RL and never published;
* language weights live under ``model.*`` (not ``model.language_model.*``),
  the vision tower under ``model.visual.*``.

All layout changes are row permutations, expressed on :class:`Rows`, so that
none of them needs a TP all-gather at transfer time.
"""

from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from awex_b200.converter.rows import IDENTITY, Rows, ValueOp
from awex_b200.models.qwen3_moe import SGlangToHFWeightConverterQwen3Moe, _build_mcore_converter_qwen3_moe
from awex_b200.models.qwen3_vl import Qwen3VLShardingStrategy, VisionTowerRoutes
from awex_b200.sharding.param_sharding import ShardingType, get_default_sharding_dim


def text_config(config):
    return getattr(config, "text_config", config)


def head_dim_of(config) -> int:
    config = text_config(config)
    value = getattr(config, "head_dim", None)
    return int(value) if value else int(config.hidden_size // config.num_attention_heads)


def _even_chunks(rows: Rows, parts: int, what: str) -> List[Rows]:
    if parts <= 0 or len(rows) % parts != 0:
        raise ValueError(f"{what} rows ({len(rows)}) must be divisible by parallel size ({parts})")
    return rows.chunk(parts)


def pack_output_gated_qkv_rows(full: Rows, config, infer_tp_size: int) -> Rows:
    """``[Q | gate | K | V]`` per KV group -> ``[Q-with-gate | K | V]`` per
    inference TP rank."""
    config = text_config(config)
    n_heads, n_kv, hd = int(config.num_attention_heads), int(config.num_key_value_heads), head_dim_of(config)
    if n_heads % n_kv != 0:
        raise ValueError(f"attention heads ({n_heads}) must be divisible by KV heads ({n_kv})")
    if n_heads % infer_tp_size != 0:
        raise ValueError(f"attention heads ({n_heads}) must be divisible by inference TP ({infer_tp_size})")
    q_rows = (n_heads // n_kv) * hd
    group_rows = 2 * q_rows + 2 * hd
    if len(full) != n_kv * group_rows:
        raise ValueError(f"unexpected gated QKV rows: got {len(full)}, expected {n_kv * group_rows}")
    heads: List[Rows] = []
    keys: List[Rows] = []
    values: List[Rows] = []
    for group in full.chunk(n_kv):
        q, gate, k, v = group.split([q_rows, q_rows, hd, hd])
        heads += [Rows.cat([qh, gh]) for qh, gh in zip(q.blocks(hd), gate.blocks(hd))]
        keys.append(k)
        values.append(v)
    per_rank = n_heads // infer_tp_size
    if infer_tp_size >= n_kv:
        if infer_tp_size % n_kv != 0:
            raise ValueError(f"inference TP ({infer_tp_size}) must be divisible by KV heads ({n_kv})")
        rep = infer_tp_size // n_kv
        key_parts = [k for k in keys for _ in range(rep)]
        value_parts = [v for v in values for _ in range(rep)]
    else:
        if n_kv % infer_tp_size != 0:
            raise ValueError(f"KV heads ({n_kv}) must be divisible by inference TP ({infer_tp_size})")
        key_parts = Rows.cat(keys).chunk(infer_tp_size)
        value_parts = Rows.cat(values).chunk(infer_tp_size)
    return Rows.cat(
        [Rows.cat(heads[r * per_rank : (r + 1) * per_rank] + [key_parts[r], value_parts[r]]) for r in range(infer_tp_size)]
    )


def split_gdn_input_rows(full: Rows, config, train_tp_size: int) -> Tuple[Rows, ...]:
    """Undo the rank-local ``[Q,K,V,Z,B,A]`` packing: six global categories."""
    config = text_config(config)
    qk = int(config.linear_num_key_heads * config.linear_key_head_dim)
    val = int(config.linear_num_value_heads * config.linear_value_head_dim)
    vh = int(config.linear_num_value_heads)
    dims = (qk, qk, val, val, vh, vh)
    if any(d % train_tp_size for d in dims):
        raise ValueError("GDN input dimensions must be divisible by training TP")
    local = [d // train_tp_size for d in dims]
    if len(full) != sum(local) * train_tp_size:
        raise ValueError(f"unexpected GDN input rows: got {len(full)}, expected {sum(local) * train_tp_size}")
    pieces: List[List[Rows]] = [[] for _ in dims]
    for block in full.chunk(train_tp_size):
        for bucket, piece in zip(pieces, block.split(local)):
            bucket.append(piece)
    return tuple(Rows.cat(p) for p in pieces)


def pack_gdn_input_rows(full: Rows, config, train_tp_size: int, infer_tp_size: int) -> Tuple[Rows, Rows]:
    cats = split_gdn_input_rows(full, config, train_tp_size)
    shards = [_even_chunks(c, infer_tp_size, f"GDN input category {i}") for i, c in enumerate(cats)]
    qkvz = Rows.cat([Rows.cat([shards[i][r] for i in range(4)]) for r in range(infer_tp_size)])
    ba = Rows.cat([Rows.cat([shards[i][r] for i in (4, 5)]) for r in range(infer_tp_size)])
    return qkvz, ba


def pack_gdn_conv_rows(full: Rows, config, train_tp_size: int, infer_tp_size: int) -> Rows:
    config = text_config(config)
    qk = int(config.linear_num_key_heads * config.linear_key_head_dim)
    val = int(config.linear_num_value_heads * config.linear_value_head_dim)
    if qk % train_tp_size or val % train_tp_size:
        raise ValueError("GDN convolution dimensions must divide training TP")
    local = [qk // train_tp_size, qk // train_tp_size, val // train_tp_size]
    if len(full) != sum(local) * train_tp_size:
        raise ValueError("unexpected GDN convolution rows")
    pieces: List[List[Rows]] = [[], [], []]
    for block in full.chunk(train_tp_size):
        for bucket, piece in zip(pieces, block.split(local)):
            bucket.append(piece)
    shards = [_even_chunks(Rows.cat(p), infer_tp_size, f"GDN conv category {i}") for i, p in enumerate(pieces)]
    return Rows.cat([Rows.cat([shards[i][r] for i in range(3)]) for r in range(infer_tp_size)])


# tensor forms for callers that hold materialised full tensors -----------------------------------
def _apply(rows: Rows, tensor: torch.Tensor) -> torch.Tensor:
    out = rows.gather(lambda _src: tensor)
    return out.contiguous()


class _Qwen3_5Layout:
    text_config = staticmethod(text_config)
    head_dim = staticmethod(head_dim_of)

    @staticmethod
    def pack_output_gated_qkv(parameter, config, infer_tp_size):
        return _apply(pack_output_gated_qkv_rows(Rows.full("w", parameter.shape[0]), config, infer_tp_size), parameter)

    @staticmethod
    def split_gdn_input(parameter, config, train_tp_size):
        return tuple(_apply(r, parameter) for r in split_gdn_input_rows(Rows.full("w", parameter.shape[0]), config, train_tp_size))

    @staticmethod
    def pack_gdn_input(parameter, config, train_tp_size, infer_tp_size):
        qkvz, ba = pack_gdn_input_rows(Rows.full("w", parameter.shape[0]), config, train_tp_size, infer_tp_size)
        return _apply(qkvz, parameter), _apply(ba, parameter)

    @staticmethod
    def pack_gdn_conv(parameter, config, train_tp_size, infer_tp_size):
        return _apply(pack_gdn_conv_rows(Rows.full("w", parameter.shape[0]), config, train_tp_size, infer_tp_size), parameter)


class Qwen3_5ShardingStrategy(Qwen3VLShardingStrategy):
    def get_sharding_strategy(self, parameter_name: str, **kwargs):
        n = parameter_name
        if ".linear_attn." in n:
            if ".norm." in n:
                return ShardingType.NO_SHARDING, 0, 1
            return self.get_attention_sharding_strategy(n, sharding_dim=1 if n.endswith("out_proj.weight") else 0, **kwargs)
        if ".self_attn." in n:
            if "_norm." in n:
                return ShardingType.NO_SHARDING, 0, 1
            return self.get_attention_sharding_strategy(n, **kwargs)
        if "shared_expert_gate" in n:
            return ShardingType.NO_SHARDING, 0, 1
        if "shared_expert" in n:
            return self.get_shared_expert_sharding_strategy(n, **kwargs)
        if ".experts." in n:
            # expert parallelism is its own axis: describe ownership even when dense TP is 1
            return self.get_expert_sharding_strategy(n, **kwargs)
        return super().get_sharding_strategy(n, **kwargs)

    def get_attention_sharding_strategy(self, parameter_name, **kwargs):
        explicit = kwargs.pop("sharding_dim", None)
        if explicit is None:
            return super().get_attention_sharding_strategy(parameter_name, **kwargs)
        if self.enable_dp_attention:
            size, kind = self.rank_info.attn_tp_size, ShardingType.DP_TP_SHARDING
        else:
            size, kind = self.rank_info.tp_size, ShardingType.TP_SHARDING
        return (kind, explicit, size) if size > 1 else (ShardingType.NO_SHARDING, explicit, 1)

    def get_shared_expert_sharding_strategy(self, parameter_name, **kwargs):
        dim = get_default_sharding_dim(parameter_name)
        return (ShardingType.TP_SHARDING, dim, self.tp_size) if self.tp_size > 1 else (ShardingType.NO_SHARDING, dim, 1)


class SGlangToHFWeightConverterQwen3_5(SGlangToHFWeightConverterQwen3Moe):
    def __init__(self, model_config, infer_engine_config, rank_info):
        super().__init__(text_config(model_config), infer_engine_config, rank_info)

    def _fuse_qkv(self, name: str) -> bool:
        return True

    @staticmethod
    def _normalize_shared_expert(name: str) -> str:
        return name.replace(".shared_experts.", ".shared_expert.")

    @torch.no_grad()
    def convert_param(self, name, parameter):
        name = name.replace("model.language_model.", "model.")
        if name.startswith(("mtp.", "model.mtp.")):
            return []
        if name.startswith("model.visual."):
            name = name.replace("model.visual.", "visual.", 1)
        if name.startswith("visual."):
            return [("model." + name.replace(".attn.qkv_proj.", ".attn.qkv."), parameter)]
        parts = name.split(".")
        if len(parts) >= 5 and parts[:2] == ["model", "layers"]:
            layer, rest = parts[2], ".".join(parts[3:])
            if rest.startswith(("qkv_proj.", "o_proj.", "q_norm.", "k_norm.")):
                return [(f"model.layers.{layer}.self_attn.{rest}", parameter)]
            if rest.startswith("linear_attn.") or rest.startswith("mlp.shared_expert_gate."):
                return [(self._normalize_shared_expert(name), parameter)]
        return [(self._normalize_shared_expert(n), t) for n, t in super().convert_param(name, parameter)]


class _Qwen3_5McoreConverterFactory:
    def __call__(self):
        base = _build_mcore_converter_qwen3_moe()

        class McoreToHFWeightConverterQwen3_5(VisionTowerRoutes, base):
            def __init__(self, hf_config, rank_info, infer_conf, tf_config):
                self.root_config = hf_config
                self.vl_hf_config = hf_config
                self.vision_config = getattr(hf_config, "vision_config", None)
                super().__init__(text_config(hf_config), rank_info, infer_conf, tf_config=tf_config)

            def _train_chunk(self, rows: Rows) -> Rows:
                tp = max(1, int(self.rank_info.attn_tp_size))
                return rows if tp == 1 else _even_chunks(rows, tp, "converted parameter")[int(self.rank_info.attn_tp_rank)]

            def _convert_attention_param(self, name, src, rows, layer_number):
                train_tp = max(1, int(self.rank_info.attn_tp_size))
                infer_tp = max(1, int(self.infer_atten_tp_size))
                n = len(rows)
                full = lambda: self._tp_full(src, n, tp_size=train_tp)  # noqa: E731
                for kind in ("weight", "bias"):
                    if f"self_attention.linear_qkv.{kind}" in name:
                        packed = pack_output_gated_qkv_rows(full(), self.hf_config, infer_tp)
                        return [(f"self_attn.qkv_proj.{kind}", self._train_chunk(packed), IDENTITY)]
                if "self_attention.in_proj.layer_norm_weight" in name:
                    return [("input_layernorm.weight", rows, IDENTITY)]
                if "self_attention.in_proj.weight" in name:
                    qkvz, ba = pack_gdn_input_rows(full(), self.hf_config, train_tp, infer_tp)
                    return [
                        ("linear_attn.in_proj_qkvz.weight", self._train_chunk(qkvz), IDENTITY),
                        ("linear_attn.in_proj_ba.weight", self._train_chunk(ba), IDENTITY),
                    ]
                if "self_attention.conv1d.weight" in name:
                    packed = pack_gdn_conv_rows(full(), self.hf_config, train_tp, infer_tp)
                    return [("linear_attn.conv1d.weight", self._train_chunk(packed), IDENTITY)]
                if "self_attention.out_proj.weight" in name:
                    return [("linear_attn.out_proj.weight", rows, IDENTITY)]
                if "self_attention.out_norm.weight" in name:
                    return [("linear_attn.norm.weight", rows, ValueOp("add", const=1.0))]
                if "self_attention.A_log" in name:
                    return [("linear_attn.A_log", rows, IDENTITY)]
                if "self_attention.dt_bias" in name:
                    return [("linear_attn.dt_bias", rows, IDENTITY)]
                return super()._convert_attention_param(name, src, rows, layer_number)

            def _convert_mlp_param(self, name, rows, layer_number):
                return [
                    (n.replace(".shared_experts.", ".shared_expert."), r, op)
                    for n, r, op in super()._convert_mlp_param(name, rows, layer_number)
                ]

            def plan_param(self, name, shape, dtype, vp_stage=None, source_name=None):
                src = source_name or name
                clean = name.replace("module.", "")
                if clean.startswith(("language_model.mtp.", "model.mtp.", "mtp.")):
                    return []
                shape = tuple(int(d) for d in shape)
                if clean.startswith("vision_model."):
                    return self._plan_vision(clean, src, shape, dtype)
                if clean.startswith("language_model."):
                    clean = clean[len("language_model."):]
                return super().plan_param(clean, shape, dtype, vp_stage=vp_stage, source_name=src)

        return McoreToHFWeightConverterQwen3_5


_MCORE_CONVERTER_FACTORY = _Qwen3_5McoreConverterFactory()

CONFIG = [
    {
        "model_name": arch,
        "sharding_strategy": Qwen3_5ShardingStrategy,
        "mcore_converter": _MCORE_CONVERTER_FACTORY,
        "sglang_converter": SGlangToHFWeightConverterQwen3_5,
    }
    for arch in ("Qwen3_5ForCausalLM", "Qwen3_5MoeForCausalLM", "Qwen3_5ForConditionalGeneration", "Qwen3_5MoeForConditionalGeneration")
]
