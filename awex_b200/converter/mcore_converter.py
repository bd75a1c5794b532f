"""Megatron-core (training) layout -> canonical HF-style names and layouts.

The converter is *symbolic first*: :meth:`McoreToHFWeightConverter.plan_param`
maps a Megatron parameter (name, shape, dtype) to :class:`TensorSpec` objects
whose dim-0 rows are described by a :class:`Rows` permutation over physical
training tensors.  :meth:`convert_param` keeps the reference's public contract
(`awex/converter/mcore_converter.py:692-739`: ``(name, tensor[, vp_stage]) ->
[(canonical_name, tensor)]``) by materialising those specs; the fused transfer
kernel instead consumes the permutations directly.

Name mapping and layout rules implemented here (same observable result as the
reference, `mcore_converter.py:475-690,1055-1352`):

* ``linear_qkv`` is stored by Megatron as ``[q_g | k_g | v_g]`` per KV group.
  The default contract re-groups it as ``[Q_r | K_r | V_r]`` per *inference*
  attention-TP rank ``r`` (each KV head repeated ``tp_i / n_kv`` times when
  ``tp_i > n_kv``) and publishes the training rank's equal chunk of that; the
  rows of a chunk may physically live on another TP peer.
* ``linear_fc1`` is ``[gate; up]`` and is published as two tensors.
* experts get global ids ``local + ep_rank * (num_experts / ep_size)``.
* router weights are cast to ``router_dtype``; ``expert_bias`` to fp32.
"""

from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from awex_b200 import logging
from awex_b200.converter.pp_layout import (  # noqa: F401  (re-exported helpers)
    normalize_pp_stage_layer_id_map,
    process_mcore_pp_name,
    resolve_pp_stage_global_layer_ids,
    stage_counts_from_layout,
    stage_counts_from_split_config,
)
from awex_b200.converter.rows import IDENTITY, Rows, TensorSpec, ValueOp
from awex_b200.converter.weights_converter import FP8_BLOCK, SCALE_SUFFIX, block_scale_shape, per_block_cast_to_fp8
from awex_b200.sharding.rank_info import RankInfo
from awex_b200.utils.common import cfg_get, divide

logger = logging.getLogger(__name__)

_ROUTER_DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}

# A training TP group registered by the host program when Megatron's
# parallel_state is not importable (tests, synthetic benchmarks).
_TRAIN_TP_GROUP = {"group": None, "size": 1}


def set_train_tp_group(group, size: int) -> None:
    _TRAIN_TP_GROUP["group"], _TRAIN_TP_GROUP["size"] = group, size


def _train_tp_group():
    """(group, size) of the training tensor-parallel group: the one the host
    program registered, else Megatron's."""
    if _TRAIN_TP_GROUP["group"] is not None or _TRAIN_TP_GROUP["size"] != 1:
        return _TRAIN_TP_GROUP["group"], _TRAIN_TP_GROUP["size"]
    try:
        from megatron.core import parallel_state as mpu

        return mpu.get_tensor_model_parallel_group(), mpu.get_tensor_model_parallel_world_size()
    except Exception:
        return None, 1


def get_full_tensor(weight: torch.Tensor, dim: int = 0) -> torch.Tensor:
    """Concatenate the TP peers' shards of ``weight`` (collective).  Only used
    when a caller asks for materialised converted tensors; the transfer path
    never gathers."""
    group, size = _train_tp_group()
    if size == 1:
        return weight
    parts = [torch.empty_like(weight) for _ in range(size)]
    dist.all_gather(parts, weight.contiguous(), group=group)
    return torch.cat(parts, dim=dim)


def gather_tp_shards(weight: torch.Tensor, expected: int) -> List[torch.Tensor]:
    """The training TP group's shards of ``weight`` in TP rank order
    (collective).  ``expected`` is the TP size the caller's rank coordinates
    name; a missing or differently sized group is an error, not a silent
    single-shard answer."""
    group, size = _train_tp_group()
    if size != expected:
        raise RuntimeError(
            f"a gather over {expected} training TP ranks is needed, but the known training TP group has size {size} "
            "(initialise Megatron's parallel_state, pass tp_group= to the training engine, or call set_train_tp_group())"
        )
    if size == 1:
        return [weight]
    parts = [torch.empty_like(weight, memory_format=torch.contiguous_format) for _ in range(size)]
    dist.all_gather(parts, weight.contiguous(), group=group)
    return parts


def head_size_of(tf_config) -> int:
    kv_channels = cfg_get(tf_config, "kv_channels")
    if kv_channels is not None:
        return int(kv_channels)
    return divide(cfg_get(tf_config, "hidden_size"), cfg_get(tf_config, "num_attention_heads"))


# ---- QKV row algebra ---------------------------------------------------------------
def split_interleaved_qkv(full: Rows, n_groups: int, q_rows: int, kv_rows: int) -> Tuple[Rows, Rows, Rows]:
    """``[q_g | k_g | v_g] * n_groups`` -> (all Q, all K, all V)."""
    qs, ks, vs = [], [], []
    for group in full.chunk(n_groups):
        q, k, v = group.split([q_rows, kv_rows, kv_rows])
        qs.append(q)
        ks.append(k)
        vs.append(v)
    return Rows.cat(qs), Rows.cat(ks), Rows.cat(vs)


def mcore_qkv_to_q_k_v(full: Rows, tf_config) -> Tuple[Rows, Rows, Rows]:
    """De-interleave a *full* (all TP shards concatenated) Megatron QKV.

    Three storage formats are told apart by the row count, compact first
    because for MHA it coincides with the replicated size:
    compact GQA ``(q_per_group + 2) * head * n_kv``; replicated KV ``3 * hidden``
    (K and V stored once per query head; one copy per KV group is kept);
    and a ``4 * hidden`` variant whose head size is ``hidden / n_kv``.
    """
    hidden = int(cfg_get(tf_config, "hidden_size"))
    n_heads = int(cfg_get(tf_config, "num_attention_heads"))
    n_kv = int(cfg_get(tf_config, "num_query_groups") or n_heads)
    head = head_size_of(tf_config)
    q_per_group = divide(n_heads, n_kv)
    rows = len(full)
    if rows == (q_per_group + 2) * head * n_kv:
        return split_interleaved_qkv(full, n_kv, q_per_group * head, head)
    if rows == 3 * hidden:
        q, k, v = full.split([hidden, hidden, hidden])
        pick = lambda t: Rows.cat([t.narrow(g * q_per_group * head, head) for g in range(n_kv)])  # noqa: E731
        return q, pick(k), pick(v)
    if rows == 4 * hidden:
        wide_head = divide(hidden, n_kv)
        return split_interleaved_qkv(full, n_kv, q_per_group * wide_head, wide_head)
    raise ValueError(
        "QKV size mismatch - unsupported format: "
        f"rows={rows}, compact={(q_per_group + 2) * head * n_kv}, replicated={3 * hidden}, "
        f"hidden_size={hidden}, num_heads={n_heads}, num_kv_heads={n_kv}, head_size={head}"
    )


def regroup_qkv_for_infer_tp(q: Rows, k: Rows, v: Rows, infer_tp: int, n_kv: int) -> Rows:
    """``[Q_0|K_0|V_0 | Q_1|K_1|V_1 | ...]`` for ``infer_tp`` attention ranks."""
    q_parts = q.chunk(infer_tp)
    if infer_tp >= n_kv:
        repeat = divide(infer_tp, n_kv)
        k_parts = [part for part in k.chunk(n_kv) for _ in range(repeat)]
        v_parts = [part for part in v.chunk(n_kv) for _ in range(repeat)]
    else:
        k_parts, v_parts = k.chunk(infer_tp), v.chunk(infer_tp)
    return Rows.cat([piece for trio in zip(q_parts, k_parts, v_parts) for piece in trio])


def pack_fused_qkv_a_rows(q_rows: Rows, kv_rows: Rows, infer_tp_size: int) -> Rows:
    """MLA ``q_a``/``kv_a`` laid out ``[q_0; kv_0; q_1; kv_1; ...]`` so that a
    dim-0 cut into ``infer_tp_size`` gives each rank ``[q_i; kv_i]``."""
    if infer_tp_size <= 0:
        raise ValueError(f"infer_tp_size must be positive, got {infer_tp_size}")
    if len(q_rows) % infer_tp_size or len(kv_rows) % infer_tp_size:
        raise ValueError(
            f"MLA projection rows must be divisible by infer_tp_size, got q={len(q_rows)}, kv={len(kv_rows)}, "
            f"infer_tp_size={infer_tp_size}"
        )
    return Rows.cat([p for pair in zip(q_rows.chunk(infer_tp_size), kv_rows.chunk(infer_tp_size)) for p in pair])


def pack_fused_qkv_a_proj_for_tp(q_proj: torch.Tensor, kv_proj: torch.Tensor, infer_tp_size: int) -> torch.Tensor:
    """Tensor form of :func:`pack_fused_qkv_a_rows`
    (`awex/converter/mcore_converter.py:994-1037`)."""
    if q_proj.dim() != 2 or kv_proj.dim() != 2:
        raise ValueError(f"Expected 2D MLA projection weights, got q_proj.dim={q_proj.dim()}, kv_proj.dim={kv_proj.dim()}")
    if q_proj.shape[1] != kv_proj.shape[1]:
        raise ValueError(f"MLA q/kv projection input dims must match, got {tuple(q_proj.shape)} and {tuple(kv_proj.shape)}")
    rows = pack_fused_qkv_a_rows(Rows.full("q", q_proj.shape[0]), Rows.full("kv", kv_proj.shape[0]), infer_tp_size)
    return rows.gather({"q": q_proj, "kv": kv_proj}.__getitem__)


# tensor-level forms kept for callers that hold materialised tensors ------------------
def _rows_to_tensor(rows: Rows, tensor: torch.Tensor) -> torch.Tensor:
    return rows.gather(lambda _src: tensor)


def transform_mcore_qkv_weight(weight: torch.Tensor, tf_config):
    full = get_full_tensor(weight, dim=0)
    q, k, v = mcore_qkv_to_q_k_v(Rows.full("w", full.shape[0]), tf_config)
    return _rows_to_tensor(q, full), _rows_to_tensor(k, full), _rows_to_tensor(v, full)


transform_mcore_qkv_bias = transform_mcore_qkv_weight


def convert_qkv_weight_along_tp_attention(weight, infer_atten_tp_size, tf_config, train_tp_rank=None, train_tp_size=None):
    full = get_full_tensor(weight, dim=0)
    q, k, v = mcore_qkv_to_q_k_v(Rows.full("w", full.shape[0]), tf_config)
    n_kv = int(cfg_get(tf_config, "num_query_groups") or cfg_get(tf_config, "num_attention_heads"))
    merged = regroup_qkv_for_infer_tp(q, k, v, infer_atten_tp_size, n_kv)
    if train_tp_size and train_tp_size > 1:
        if train_tp_rank is None:
            raise ValueError("train_tp_rank is required when train_tp_size > 1")
        merged = merged.chunk(train_tp_size)[train_tp_rank]
    return _rows_to_tensor(merged, full)


convert_qkv_bias_along_tp_attention = convert_qkv_weight_along_tp_attention


def get_mcore_model_parameters(model) -> Dict[str, torch.Tensor]:
    """Named parameters plus the router ``expert_bias`` buffers, which Megatron
    keeps in ``state_dict()`` only."""
    params = dict(model.named_parameters())
    for name, value in model.state_dict().items():
        if "expert_bias" in name and name not in params:
            params[name] = value
    return params


class McoreToHFWeightConverter:
    """Default converter (Llama / Qwen2-style and any unregistered architecture)."""

    def __init__(self, hf_config, rank_info: RankInfo, infer_conf: Dict, tf_config):
        from awex_b200.utils.mindspeed import ensure_mindspeed_patched

        ensure_mindspeed_patched("mcore_converter")
        self.hf_config = hf_config
        self.tf_config = tf_config
        self.rank_info = rank_info
        self.infer_conf = infer_conf
        self._pp_stage_layer_id_map = normalize_pp_stage_layer_id_map(infer_conf.get("train_pp_stage_layer_id_map"))
        router = infer_conf.get("router_dtype", "bf16")
        if router not in _ROUTER_DTYPES:
            raise ValueError(f"Unsupported router dtype: {router}")
        self.router_dtype = _ROUTER_DTYPES[router]
        if "infer_atten_tp_size" not in infer_conf:
            raise ValueError("infer_atten_tp_size must be specified")
        self.infer_atten_tp_size = int(infer_conf["infer_atten_tp_size"])
        self._infer_device_backend = "cuda"

    # ---- knobs subclasses override -------------------------------------------------
    def _fuse_qkv(self, name: str) -> bool:
        return True

    def _fuse_gate_up_proj(self, name: str) -> bool:
        return False

    @staticmethod
    def _normalize_attn_name(name: str) -> str:
        for old, new in (
            ("self_attn.qkv_proj", "attention.query_key_value_proj"),
            ("self_attn.o_proj", "attention.dense"),
            ("self_attn.q_norm", "attention.query_layernorm"),
            ("self_attn.k_norm", "attention.key_layernorm"),
        ):
            name = name.replace(old, new)
        return name.replace("query_key_value_proj_proj", "query_key_value_proj")

    # ---- symbolic sources -------------------------------------------------------------
    def _own(self, param_name: str, n_rows: int) -> Rows:
        return Rows.full((param_name, self.rank_info.tp_rank), n_rows)

    def _tp_full(self, param_name: str, n_rows: int, tp_size: Optional[int] = None) -> Rows:
        """All TP peers' shards of ``param_name`` concatenated along dim 0."""
        tp = int(self.rank_info.attn_tp_size if tp_size is None else tp_size)
        return Rows.cat([Rows.full((param_name, r), n_rows) for r in range(tp)])

    # ---- families -----------------------------------------------------------------------
    def _fused_qkv_rows(self, src: str, n_rows: int) -> Rows:
        tp, rank = int(self.rank_info.attn_tp_size), int(self.rank_info.attn_tp_rank)
        q, k, v = mcore_qkv_to_q_k_v(self._tp_full(src, n_rows), self.tf_config)
        n_kv = int(cfg_get(self.tf_config, "num_query_groups") or cfg_get(self.tf_config, "num_attention_heads"))
        merged = regroup_qkv_for_infer_tp(q, k, v, self.infer_atten_tp_size, n_kv)
        return merged.chunk(tp)[rank] if tp > 1 else merged

    def _convert_attention_param(self, name: str, src: str, rows: Rows, layer_number: str) -> List[Tuple[str, Rows, ValueOp]]:
        n = len(rows)
        for kind in ("weight", "bias"):
            if f"self_attention.linear_qkv.{kind}" in name:
                if self._fuse_qkv(name):
                    return [(f"self_attn.qkv_proj.{kind}", self._fused_qkv_rows(src, n), IDENTITY)]
                if kind == "weight":
                    third = n // 3
                    parts = rows.split([third, third, n - 2 * third])
                else:
                    parts = mcore_qkv_to_q_k_v(self._tp_full(src, n), self.tf_config)
                return [(f"self_attn.{p}_proj.{kind}", r, IDENTITY) for p, r in zip("qkv", parts)]
        simple = {
            "self_attention.linear_qkv.layer_norm_weight": "input_layernorm.weight",
            "self_attention.linear_proj.weight": "self_attn.o_proj.weight",
            "self_attention.linear_proj.bias": "self_attn.o_proj.bias",
            "self_attention.q_layernorm.weight": "self_attn.q_norm.weight",
            "self_attention.k_layernorm.weight": "self_attn.k_norm.weight",
        }
        for key, target in simple.items():
            if key in name:
                return [(target, rows, IDENTITY)]
        raise NotImplementedError(f"Unsupported parameter name: {name}")

    def _convert_linear(self, name: str, rows: Rows) -> List[Tuple[str, Rows, ValueOp]]:
        for kind in ("weight", "bias"):
            if f"linear_fc1.{kind}" in name:
                if self._fuse_gate_up_proj(name):
                    return [(f"gate_up_proj.{kind}", rows, IDENTITY)]
                half = len(rows) // 2
                return [
                    (f"gate_proj.{kind}", rows.narrow(0, half), IDENTITY),
                    (f"up_proj.{kind}", rows.narrow(half, half), IDENTITY),
                ]
            if f"linear_fc2.{kind}" in name:
                return [(f"down_proj.{kind}", rows, IDENTITY)]
        raise NotImplementedError(f"Unsupported parameter name: {name}")

    def _expert_global_id(self, name: str) -> int:
        if "local_experts" in name:  # ...experts.local_experts.<e>.linear_fc1.weight
            local = int(name.rsplit(".", 3)[-3])
        else:  # grouped GEMM naming ...experts.linear_fc1.weight<e>
            local = int(name.rsplit("weight", 1)[-1])
        n_experts = getattr(self.hf_config, "num_experts", None) or getattr(self.hf_config, "n_routed_experts")
        return local + int(self.rank_info.ep_rank) * (int(n_experts) // int(self.rank_info.ep_size))

    def _convert_mlp_param(self, name: str, rows: Rows, layer_number: str) -> List[Tuple[str, Rows, ValueOp]]:
        assert "attention" not in name, f"{name} should be handled as an attention parameter"
        if "pre_mlp_layernorm" in name or "linear_fc1.layer_norm_weight" in name:
            return [("post_attention_layernorm.weight", rows, IDENTITY)]
        if "input_layernorm.weight" in name:
            return [("input_layernorm.weight", rows, IDENTITY)]
        if "shared_experts.gate_weight" in name:
            return [("mlp.shared_expert_gate.weight", rows, IDENTITY)]
        if "shared_experts.linear_fc" in name:
            prefix = "mlp.shared_experts."
        elif "mlp.experts." in name:
            prefix = f"mlp.experts.{self._expert_global_id(name)}."
        elif "linear_fc1." in name or "linear_fc2." in name:
            prefix = "mlp."
        else:
            raise NotImplementedError(f"Unsupported parameter name: {name}")
        return [(prefix + n, r, op) for n, r, op in self._convert_linear(name, rows)]

    def _convert_lm_head_param(self, name: str, rows: Rows) -> List[Tuple[str, Rows, ValueOp]]:
        op = ValueOp("l2norm_dim0") if getattr(self.hf_config, "norm_head", False) else IDENTITY
        return [("lm_head.weight", rows, op)]

    # ---- routing --------------------------------------------------------------------------
    def _route(self, name: str, src: str, rows: Rows) -> List[Tuple[str, Rows, ValueOp]]:
        if name == "embedding.word_embeddings.weight":
            return [("model.embed_tokens.weight", rows, IDENTITY)]
        if name == "decoder.final_layernorm.weight":
            return [("model.norm.weight", rows, IDENTITY)]
        if "output_layer.weight" in name:
            return self._convert_lm_head_param(name, rows)
        if not name.startswith("decoder.layers."):
            raise NotImplementedError(f"Unsupported parameter name: {name}")
        layer, rest = name[len("decoder.layers.") :].split(".", 1)
        at = f"model.layers.{layer}."
        if "self_attention" in rest:
            return [
                (at + self._normalize_attn_name(n), r, op)
                for n, r, op in self._convert_attention_param(rest, src, rows, layer)
            ]
        if "mlp" in rest:
            if "mlp.gate.weight" in name or "mlp.router.weight" in name:
                return [(at + "mlp.gate.weight", rows, ValueOp("cast", dtype=self.router_dtype))]
            if "expert_bias" in name:
                return [(at + "mlp.gate.expert_bias", rows, ValueOp("cast", dtype=torch.float32))]
            return [(at + n, r, op) for n, r, op in self._convert_mlp_param(rest, rows, layer)]
        return self._route_other(name, layer, rest, src, rows)

    def _route_other(self, name, layer, rest, src, rows):
        raise NotImplementedError(f"Unsupported parameter name: {name}")

    def _canonical_source_name(self, name: str, vp_stage: Optional[int]) -> str:
        return process_mcore_pp_name(
            name.replace("module.", ""), self.rank_info, self.hf_config, self.tf_config,
            vp_stage=vp_stage, pp_stage_layer_id_map=self._pp_stage_layer_id_map,
        )

    # ---- public API --------------------------------------------------------------------------
    def plan_param(self, name: str, shape: Sequence[int], dtype: torch.dtype, vp_stage: Optional[int] = None,
                   source_name: Optional[str] = None) -> List[TensorSpec]:
        """Describe the canonical tensors produced from training parameter
        ``name`` without touching data.  Sources in the returned row maps are
        ``(source_name or name, tp_rank)``; ``source_name`` lets a subclass
        route a rewritten name while still pointing at the real parameter."""
        shape = tuple(int(d) for d in shape)
        src = source_name or name
        routed = self._canonical_source_name(name, vp_stage)
        if not shape:
            out = self._route(routed, src, Rows.full((src, self.rank_info.tp_rank), 1))
            return [TensorSpec(n, None, (), dtype, op) for n, _, op in out]
        rows = self._own(src, shape[0])
        return self._finish_specs(self._route(routed, src, rows), shape, dtype)

    def _finish_specs(self, routed, shape, dtype) -> List[TensorSpec]:
        specs: List[TensorSpec] = []
        for cname, crow, op in routed:
            spec = TensorSpec(cname, crow, tuple(shape[1:]), dtype, op)
            spec.value_op = self._value_op_for(cname, spec)
            specs.append(spec)
            if spec.value_op.kind == "fp8_block":
                specs.append(self._scale_spec(spec))
        return specs

    def _infer_tp_size(self) -> int:
        return int(cfg_get(self.infer_conf.get("infer_engine_config"), "tp_size", None) or self.infer_atten_tp_size or 1)

    def _dest_split(self, canonical_name: str) -> int:
        """How many destination shards one of this rank's slices of
        ``canonical_name`` covers along the sharded dim (>= 1)."""
        engine_cfg = self.infer_conf.get("infer_engine_config")
        tp_i = self._infer_tp_size()
        if ".experts." in canonical_name:
            ep_i = int(cfg_get(engine_cfg, "ep_size", None) or 1)
            if ep_i > 1:
                etp_i = tp_i // ep_i if self.infer_conf.get("engine_name") == "sglang" else 1
            else:
                etp_i = tp_i
            return max(etp_i // max(int(self.rank_info.ep_tp_size), 1), 1)
        if "attention" in canonical_name or "self_attn" in canonical_name:
            tp_i = self.infer_atten_tp_size
        return max(tp_i // max(int(self.rank_info.tp_size), 1), 1)

    def _source_split(self, canonical_name: str) -> int:
        """How many of this side's slices share one destination shard of
        ``canonical_name`` along the sharded dim (>= 1): the mirror of
        :meth:`_dest_split`."""
        engine_cfg = self.infer_conf.get("infer_engine_config")
        tp_i = self._infer_tp_size()
        if ".experts." in canonical_name:
            ep_i = int(cfg_get(engine_cfg, "ep_size", None) or 1)
            if ep_i > 1:
                etp_i = tp_i // ep_i if self.infer_conf.get("engine_name") == "sglang" else 1
            else:
                etp_i = tp_i
            return max(max(int(self.rank_info.ep_tp_size), 1) // max(etp_i, 1), 1)
        if "attention" in canonical_name or "self_attn" in canonical_name:
            tp_i = self.infer_atten_tp_size
        return max(max(int(self.rank_info.tp_size), 1) // max(tp_i, 1), 1)

    # ---- block fp8 serving -----------------------------------------------------------------
    _FP8_SUFFIXES = (
        "q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight", "dense.weight", "query_key_value_proj.weight",
        "gate_proj.weight", "up_proj.weight", "down_proj.weight", "gate_up_proj.weight",
    )

    def _is_fp8_name(self, canonical_name: str) -> bool:
        """Which tensors the inference engine serves quantised: the linear
        layers inside decoder blocks; embeddings, output head, norms and router
        weights stay in the training dtype."""
        return ".layers." in canonical_name and canonical_name.endswith(self._FP8_SUFFIXES)

    def _fp8_ue8m0(self, canonical_name: str) -> bool:
        return False

    def _value_op_for(self, canonical_name: str, spec: TensorSpec) -> ValueOp:
        if (
            self.infer_conf.get("fp8_block_quant")
            and spec.value_op.kind == "none"
            and len(spec.shape) == 2
            and self._is_fp8_name(canonical_name)
        ):
            return ValueOp("fp8_block", dtype=torch.float8_e4m3fn, ue8m0=self._fp8_ue8m0(canonical_name))
        return spec.value_op

    def _scale_spec(self, weight: TensorSpec) -> TensorSpec:
        """Scale tensor of a block-quantised weight.  Blocks are laid on the
        *destination* shard grid, so the scale extent along the sharded dim is
        ``k * ceil(extent / k / 128)`` when this rank's slice covers ``k``
        destination shards, else ``ceil(extent / 128)``."""
        from awex_b200.sharding.param_sharding import get_default_sharding_dim

        extent = list(weight.shape)
        dim = get_default_sharding_dim(weight.name)
        k = self._dest_split(weight.name)
        if extent[dim] % k != 0:
            k = 1
        if self._source_split(weight.name) > 1 and extent[dim] % FP8_BLOCK:
            # several training ranks share one destination shard and this rank's slice ends inside a
            # quantisation block: that block would need rows (or columns) from two ranks on one
            raise NotImplementedError(
                f"{weight.name}: this rank's slice ({extent[dim]} along dim {dim}) is not a whole number of {FP8_BLOCK}-wide "
                "quantisation blocks while several training ranks feed one inference shard; quantising those blocks needs "
                "their data on one rank (use a training TP that keeps slices block aligned, or an inference TP >= training TP)"
            )
        along = k * block_scale_shape(extent[dim] // k, 1)[0]
        other = block_scale_shape(extent[1 - dim], 1)[0]
        shape = (along, other) if dim == 0 else (other, along)
        return TensorSpec(
            weight.name + SCALE_SUFFIX, Rows.full(("__scale__", weight.name), shape[0]), (shape[1],),
            torch.float32, IDENTITY, scale_of=weight.name,
        )

    @torch.no_grad()
    def convert_param(self, name: str, parameter: torch.Tensor, vp_stage: Optional[int] = None) -> List[Tuple[str, torch.Tensor]]:
        """Materialised form of :meth:`plan_param`.  Collective over the
        training TP group when a spec draws rows from TP peers."""
        specs = self.plan_param(name, parameter.shape, parameter.dtype, vp_stage)
        return self.realize(specs, {name: parameter})

    def realize(self, specs: Sequence[TensorSpec], local: Dict[str, torch.Tensor]) -> List[Tuple[str, torch.Tensor]]:
        my_tp = self.rank_info.tp_rank
        gathered: Dict[str, List[torch.Tensor]] = {}

        def fetch(src):
            pname, tp_rank = src
            if tp_rank == my_tp:
                return local[pname]
            if pname not in gathered:
                full = get_full_tensor(local[pname], dim=0)
                n = local[pname].shape[0]
                gathered[pname] = [full.narrow(0, r * n, n) for r in range(full.shape[0] // n)]
            if tp_rank >= len(gathered[pname]):
                raise RuntimeError(
                    f"{pname}: the canonical tensor draws rows from training TP rank {tp_rank}, but no training TP group of "
                    f"that size is known here (Megatron's parallel_state is not initialised and set_train_tp_group() was not "
                    "called); materialised conversion needs it, the transfer path does not"
                )
            return gathered[pname][tp_rank]

        out: List[Tuple[str, torch.Tensor]] = []
        quantised: Dict[str, torch.Tensor] = {}
        for spec in specs:
            if spec.scale_of is not None:
                out.append((spec.name, quantised[spec.scale_of]))
                continue
            if spec.rows is None:
                tensor = local[next(iter(local))]
            else:
                tensor = spec.rows.gather(fetch)
            if spec.value_op.kind == "fp8_block":
                tensor, scale = self._quantise_like_destination(spec, tensor)
                quantised[spec.name] = scale
            else:
                tensor = spec.value_op.apply(tensor)
            out.append((spec.name, tensor))
        return out

    def _quantise_like_destination(self, spec: TensorSpec, tensor: torch.Tensor):
        from awex_b200.sharding.param_sharding import get_default_sharding_dim

        dim = get_default_sharding_dim(spec.name)
        ratio = self._dest_split(spec.name)
        if tensor.shape[dim] % ratio != 0:
            ratio = 1
        qs, ss = zip(*(per_block_cast_to_fp8(part.contiguous(), spec.value_op.ue8m0) for part in tensor.chunk(ratio, dim=dim)))
        return torch.cat(qs, dim=dim), torch.cat(ss, dim=dim)


class LinearMLAMcoreConverterMixin:
    """Bailing-linear family: layers alternate Lightning (linear) attention and
    MLA.  Layer ``l`` is linear unless ``(l + 1) % layer_group_size == 0``; MLA
    parameters are also recognised by name so that metadata resolution works
    before global layer ids are known (`awex/converter/mcore_converter.py:742-991`).
    MLA ``q_a``/``kv_a`` down-projections are split over the training TP group
    but served whole: TP rank 0 publishes the concatenation of all peers'
    shards, fused into one tensor when the model has a q LoRA."""

    _MLA_MARKERS = ("linear_q_down_proj", "linear_q_up_proj", "linear_kv_down_proj", "linear_kv_up_proj", "linear_q_proj")
    _MLA_NAMES = {
        "input_layernorm.weight": "input_layernorm.weight",
        "self_attention.linear_proj.weight": "attention.dense.weight",
        "self_attention.linear_q_proj.weight": "attention.q_proj.weight",
        "self_attention.linear_kv_down_proj.weight": "attention.kv_a_proj_with_mqa.weight",
        "self_attention.linear_q_down_proj.weight": "attention.q_a_proj.weight",
        "self_attention.linear_kv_up_proj.weight": "attention.kv_b_proj.weight",
        "self_attention.linear_kv_up_proj.layer_norm_weight": "attention.kv_a_layernorm.weight",
        "self_attention.linear_q_up_proj.weight": "attention.q_b_proj.weight",
        "self_attention.linear_q_up_proj.layer_norm_weight": "attention.q_a_layernorm.weight",
    }
    _LIGHTNING_NAMES = {
        "self_attention.input_layernorm.weight": "input_layernorm.weight",
        "self_attention.linear_gate.weight": "attention.g_proj.weight",
        "self_attention.linear_proj.weight": "attention.dense.weight",
        "self_attention.q_layernorm.weight": "attention.query_layernorm.weight",
        "self_attention.k_layernorm.weight": "attention.key_layernorm.weight",
    }

    def __init__(self, hf_config, rank_info, infer_conf, tf_config):
        super().__init__(hf_config, rank_info, infer_conf, tf_config=tf_config)
        self.layer_group_size = int(cfg_get(tf_config, "layer_group_size") or getattr(hf_config, "layer_group_size", None) or 1)
        self.linear_attn_norm_group_size = (
            cfg_get(tf_config, "linear_attn_norm_group_size")
            or getattr(hf_config, "linear_attn_norm_group_size", None)
            or getattr(hf_config, "group_norm_size", None)
        )
        self.fuse_qkv_a_proj = getattr(hf_config, "q_lora_rank", None) is not None
        self.qkv_a_proj_cache: Dict[str, Dict[str, Tuple[Rows, Tuple[int, ...]]]] = {}

    def _is_linear_layer(self, layer_number: int) -> bool:
        return self.layer_group_size > 1 and (layer_number + 1) % self.layer_group_size != 0

    def _is_mla_param(self, name: str) -> bool:
        return any(m in name for m in self._MLA_MARKERS)

    def _lightning(self, name, src, rows, layer):
        if "self_attention.pre_gate_norm.te_norm.weight" in name:
            return []
        if "self_attention.pre_gate_norm.weight" in name or "self_attention.gate_norm.weight" in name:
            return [("attention.g_norm.weight", rows, IDENTITY)]  # stays 1-D
        for key, target in self._LIGHTNING_NAMES.items():
            if key in name:
                return [(target, rows, IDENTITY)]
        if "self_attention.linear_qkv.weight" in name:
            return [("attention.query_key_value.weight", self._fused_qkv_rows(src, len(rows)), IDENTITY)]
        return McoreToHFWeightConverter._convert_attention_param(self, name, src, rows, layer)

    def _mla(self, name, src, rows, layer):
        for key, target in self._MLA_NAMES.items():
            if key not in name:
                continue
            if target in ("attention.kv_a_proj_with_mqa.weight", "attention.q_a_proj.weight"):
                # served un-sharded: rank 0 publishes all TP peers' rows
                if self.rank_info.tp_rank != 0:
                    return []
                full = self._tp_full(src, len(rows), tp_size=self.rank_info.tp_size)
                if self.fuse_qkv_a_proj:
                    return self._fuse_a_proj(target, full, layer)
                return [(target, full, IDENTITY)]
            return [(target, rows, IDENTITY)]
        return McoreToHFWeightConverter._convert_attention_param(self, name, src, rows, layer)

    def _fuse_a_proj(self, target: str, rows: Rows, layer: str):
        slot, other = ("kv_a_proj", "q_a_proj") if target.endswith("kv_a_proj_with_mqa.weight") else ("q_a_proj", "kv_a_proj")
        cache = self.qkv_a_proj_cache.setdefault(layer, {})
        cache[slot] = rows
        if other not in cache:
            return []
        q, kv = cache["q_a_proj"], cache["kv_a_proj"]
        del self.qkv_a_proj_cache[layer]
        # uncut at the receiver when training has no attention TP: plain concat;
        # otherwise interleave so every dim-0 chunk is [q_i; kv_i]
        fused = Rows.cat([q, kv]) if self.rank_info.attn_tp_size == 1 else pack_fused_qkv_a_rows(q, kv, self.infer_atten_tp_size)
        return [("attention.fused_qkv_a_proj_with_mqa.weight", fused, IDENTITY)]

    def _convert_attention_param(self, name, src, rows, layer_number):
        if self._is_mla_param(name) or not self._is_linear_layer(int(layer_number)):
            return self._mla(name, src, rows, layer_number)
        return self._lightning(name, src, rows, layer_number)

    def _route_other(self, name, layer, rest, src, rows):
        if "input_layernorm.weight" in rest or "g_norm.weight" in rest:
            return [(f"model.layers.{layer}.{rest}", rows, IDENTITY)]
        return super()._route_other(name, layer, rest, src, rows)
