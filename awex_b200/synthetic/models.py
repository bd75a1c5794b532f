"""Random-init models in the two layouts a weight exchange connects.

* :func:`build_megatron_model` — what a Megatron-core training rank holds:
  interleaved ``linear_qkv`` per KV group, ``linear_fc1 = [gate; up]``,
  row/column-parallel shards, pipeline-local layer numbering, rank-local
  experts.
* :func:`build_vllm_model` — what a vLLM worker holds: ``qkv_proj = [Q_r; K_r;
  V_r]`` (KV heads repeated when TP exceeds their number), ``gate_up_proj``,
  fused expert tensors ``w13_weight[E_local, 2I, H]`` / ``w2_weight[E_local, H, I]``,
  optionally block-scaled fp8 with ``*_scale_inv`` companions.

Both are cut from the same canonical (HF-layout) tensors, generated on the
fly as N(0, 0.02) from a seed derived from the tensor's name, so any rank can
regenerate any shard — the inference layout built directly from the canonical
tensors is the oracle a transfer result is compared with.
"""

from __future__ import annotations

import hashlib
import os
from collections import OrderedDict
from typing import Dict, Iterator, List, Optional, Tuple

import torch

from awex_b200.converter.weights_converter import per_block_cast_to_fp8
from awex_b200.sharding.rank_info import RankInfo
from awex_b200.synthetic.arch import Arch


class CanonicalWeights:
    """Canonical tensors by name, regenerated deterministically on demand."""

    def __init__(self, arch: Arch, dtype: torch.dtype, device, seed: int = 0, step: int = 0):
        self.arch, self.dtype, self.device, self.seed, self.step = arch, dtype, torch.device(device), seed, step

    def _seed_of(self, name: str) -> int:
        digest = hashlib.sha256(f"{self.seed}/{self.step}/{name}".encode()).digest()
        return int.from_bytes(digest[:7], "little")

    def get(self, name: str, shape: Tuple[int, ...]) -> torch.Tensor:
        if self.device.type == "meta":  # shapes only: planning studies of models too large to hold
            return torch.empty(shape, dtype=self.dtype, device=self.device)
        gen = torch.Generator(device=self.device)
        gen.manual_seed(self._seed_of(name))
        if name.endswith("norm.weight"):
            # norm gains around 1 so that constant-offset transforms are visible
            base = torch.randn(shape, generator=gen, device=self.device, dtype=torch.float32) * 0.02 + 1.0
        else:
            base = torch.randn(shape, generator=gen, device=self.device, dtype=torch.float32) * 0.02
        return base.to(self.dtype)

    # canonical shapes ------------------------------------------------------------------
    def layer(self, l: int, what: str) -> torch.Tensor:
        a = self.arch
        q_rows, kv_rows = a.num_heads * a.head_dim, a.num_kv_heads * a.head_dim
        shapes = {
            "self_attn.q_proj.weight": (q_rows, a.hidden),
            "self_attn.k_proj.weight": (kv_rows, a.hidden),
            "self_attn.v_proj.weight": (kv_rows, a.hidden),
            "self_attn.q_proj.bias": (q_rows,),
            "self_attn.k_proj.bias": (kv_rows,),
            "self_attn.v_proj.bias": (kv_rows,),
            "self_attn.o_proj.weight": (a.hidden, q_rows),
            "self_attn.q_norm.weight": (a.head_dim,),
            "self_attn.k_norm.weight": (a.head_dim,),
            "input_layernorm.weight": (a.hidden,),
            "post_attention_layernorm.weight": (a.hidden,),
            "mlp.gate_proj.weight": (a.ffn, a.hidden),
            "mlp.up_proj.weight": (a.ffn, a.hidden),
            "mlp.down_proj.weight": (a.hidden, a.ffn),
            "mlp.gate.weight": (a.num_experts, a.hidden),
        }
        return self.get(f"model.layers.{l}.{what}", shapes[what])

    def expert(self, l: int, e: int, what: str) -> torch.Tensor:
        a = self.arch
        shape = (a.hidden, a.expert_ffn) if what == "down_proj" else (a.expert_ffn, a.hidden)
        return self.get(f"model.layers.{l}.mlp.experts.{e}.{what}.weight", shape)

    def embed(self) -> torch.Tensor:
        return self.get("model.embed_tokens.weight", (self.arch.vocab, self.arch.hidden))

    def lm_head(self) -> torch.Tensor:
        if self.arch.tie_embeddings:
            return self.embed()
        return self.get("lm_head.weight", (self.arch.vocab, self.arch.hidden))

    def final_norm(self) -> torch.Tensor:
        return self.get("model.norm.weight", (self.arch.hidden,))


class ZeroWeights(CanonicalWeights):
    """Right shapes, no values: for models that are only allocated."""

    def get(self, name: str, shape: Tuple[int, ...]) -> torch.Tensor:
        return torch.zeros(shape, dtype=self.dtype, device=self.device)


class StoredCanonicalWeights(CanonicalWeights):
    """Canonical tensors read from a name -> tensor mapping (a loaded HF
    checkpoint) instead of being generated."""

    def __init__(self, arch: Arch, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device):
        super().__init__(arch, dtype, device)
        self.tensors = tensors

    def get(self, name: str, shape: Tuple[int, ...]) -> torch.Tensor:
        t = self.tensors[name]
        if tuple(t.shape) != tuple(shape):
            raise ValueError(f"{name}: checkpoint shape {tuple(t.shape)} != expected {tuple(shape)}")
        return t.to(device=self.device, dtype=self.dtype)


def canonical_state_dict(arch: Arch, weights: CanonicalWeights) -> "OrderedDict[str, torch.Tensor]":
    """Every canonical (HF-layout) tensor of the model, by name."""
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    out["model.embed_tokens.weight"] = weights.embed()
    for l in range(arch.num_layers):
        p = f"model.layers.{l}."
        names = ["input_layernorm.weight", "self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
                 "self_attn.o_proj.weight", "post_attention_layernorm.weight"]
        if arch.qkv_bias:
            names += ["self_attn.q_proj.bias", "self_attn.k_proj.bias", "self_attn.v_proj.bias"]
        if arch.qk_norm:
            names += ["self_attn.q_norm.weight", "self_attn.k_norm.weight"]
        if arch.is_moe:
            names += ["mlp.gate.weight"]
        else:
            names += ["mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight"]
        for n in names:
            out[p + n] = weights.layer(l, n)
        for e in range(arch.num_experts):
            for what in ("gate_proj", "up_proj", "down_proj"):
                out[f"{p}mlp.experts.{e}.{what}.weight"] = weights.expert(l, e, what)
    out["model.norm.weight"] = weights.final_norm()
    if not arch.tie_embeddings:
        out["lm_head.weight"] = weights.lm_head()
    return out


class FlatModule:
    """Minimal stand-in for an ``nn.Module``: ordered named tensors (names may
    contain dots) plus a ``config``."""

    def __init__(self, tensors: "OrderedDict[str, torch.Tensor]", config, buffers: Optional[Dict[str, torch.Tensor]] = None):
        self._tensors = tensors
        self._buffers = buffers or {}
        self.config = config

    def named_parameters(self) -> Iterator[Tuple[str, torch.Tensor]]:
        return iter(self._tensors.items())

    def parameters(self) -> Iterator[torch.Tensor]:
        return iter(self._tensors.values())

    def state_dict(self) -> Dict[str, torch.Tensor]:
        out = OrderedDict(self._tensors)
        out.update(self._buffers)
        return out

    def get_parameter(self, name: str) -> torch.Tensor:
        return self._tensors[name]

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._tensors.values())


def _chunk(t: torch.Tensor, n: int, i: int, dim: int = 0) -> torch.Tensor:
    size = t.shape[dim] // n
    return t.narrow(dim, i * size, size)


def pp_layer_range(num_layers: int, pp_rank: int, pp_size: int) -> range:
    per = num_layers // pp_size
    return range(pp_rank * per, (pp_rank + 1) * per)


# ---- Megatron layout ---------------------------------------------------------------------------
def vpp_layer_range(num_layers: int, pp_rank: int, pp_size: int, vp_stage: int, vp_size: int) -> range:
    """Layers of model chunk ``vp_stage`` on pipeline rank ``pp_rank`` with
    interleaved (virtual) pipelining: chunks are numbered virtual stage
    outermost, pipeline rank innermost."""
    per_chunk = num_layers // (pp_size * vp_size)
    first = (vp_stage * pp_size + pp_rank) * per_chunk
    return range(first, first + per_chunk)


def build_megatron_model(arch: Arch, rank_info: RankInfo, dtype=torch.bfloat16, device="cpu", seed: int = 0,
                         step: int = 0, layers: Optional[range] = None, weights: Optional[CanonicalWeights] = None,
                         virtual_stage: Optional[Tuple[int, int]] = None) -> FlatModule:
    """``virtual_stage=(vp_stage, vp_size)`` builds one chunk of an interleaved
    pipeline: its layers, the embedding only in the very first chunk and the
    output layer only in the very last."""
    w = weights or CanonicalWeights(arch, dtype, device, seed, step)
    tp, r = rank_info.tp_size, rank_info.tp_rank
    ep, er = rank_info.ep_size, rank_info.ep_rank
    etp, etr = rank_info.ep_tp_size, rank_info.ep_tp_rank
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    first_stage, last_stage = rank_info.pp_rank == 0, rank_info.pp_rank == rank_info.pp_size - 1
    if virtual_stage is not None:
        vp_stage, vp_size = virtual_stage
        first_stage, last_stage = first_stage and vp_stage == 0, last_stage and vp_stage == vp_size - 1
        if layers is None:
            layers = vpp_layer_range(arch.num_layers, rank_info.pp_rank, rank_info.pp_size, vp_stage, vp_size)
    if first_stage:
        out["embedding.word_embeddings.weight"] = _chunk(w.embed(), tp, r).contiguous()
    global_layers = layers if layers is not None else pp_layer_range(arch.num_layers, rank_info.pp_rank, rank_info.pp_size)
    groups_local = arch.num_kv_heads // tp
    q_per_group = arch.num_heads // arch.num_kv_heads
    hd = arch.head_dim
    for local, l in enumerate(global_layers):
        p = f"decoder.layers.{local}."

        def interleave(kind: str) -> torch.Tensor:
            q, k, v = (w.layer(l, f"self_attn.{x}_proj.{kind}") for x in "qkv")
            parts = []
            for g in range(r * groups_local, (r + 1) * groups_local):
                parts += [q.narrow(0, g * q_per_group * hd, q_per_group * hd), k.narrow(0, g * hd, hd), v.narrow(0, g * hd, hd)]
            return torch.cat(parts, 0)

        out[p + "self_attention.linear_qkv.layer_norm_weight"] = w.layer(l, "input_layernorm.weight")
        out[p + "self_attention.linear_qkv.weight"] = interleave("weight")
        if arch.qkv_bias:
            out[p + "self_attention.linear_qkv.bias"] = interleave("bias")
        if arch.qk_norm:
            out[p + "self_attention.q_layernorm.weight"] = w.layer(l, "self_attn.q_norm.weight")
            out[p + "self_attention.k_layernorm.weight"] = w.layer(l, "self_attn.k_norm.weight")
        out[p + "self_attention.linear_proj.weight"] = _chunk(w.layer(l, "self_attn.o_proj.weight"), tp, r, 1).contiguous()
        if arch.is_moe:
            out[p + "pre_mlp_layernorm.weight"] = w.layer(l, "post_attention_layernorm.weight")
            out[p + "mlp.router.weight"] = w.layer(l, "mlp.gate.weight")
            n_local = arch.num_experts // ep
            for le in range(n_local):
                e = er * n_local + le
                fc1 = torch.cat([_chunk(w.expert(l, e, "gate_proj"), etp, etr), _chunk(w.expert(l, e, "up_proj"), etp, etr)], 0)
                out[p + f"mlp.experts.local_experts.{le}.linear_fc1.weight"] = fc1
                out[p + f"mlp.experts.local_experts.{le}.linear_fc2.weight"] = _chunk(w.expert(l, e, "down_proj"), etp, etr, 1).contiguous()
        else:
            out[p + "mlp.linear_fc1.layer_norm_weight"] = w.layer(l, "post_attention_layernorm.weight")
            out[p + "mlp.linear_fc1.weight"] = torch.cat(
                [_chunk(w.layer(l, "mlp.gate_proj.weight"), tp, r), _chunk(w.layer(l, "mlp.up_proj.weight"), tp, r)], 0
            )
            out[p + "mlp.linear_fc2.weight"] = _chunk(w.layer(l, "mlp.down_proj.weight"), tp, r, 1).contiguous()
    if last_stage:
        out["decoder.final_layernorm.weight"] = w.final_norm()
        # tied embeddings: one tensor when this stage also holds the embedding; with
        # pipeline stages apart, the last stage keeps its own (synchronised) copy
        if not arch.tie_embeddings or not first_stage:
            out["output_layer.weight"] = _chunk(w.lm_head(), tp, r).contiguous()
    model = FlatModule(out, arch.tf_config())
    model.transformer_config = model.config
    return model


# ---- vLLM layout ----------------------------------------------------------------------------------
def _maybe_fp8(out, name: str, t: torch.Tensor, fp8: bool, parts: int = 1, zero: bool = False) -> None:
    """Store ``t`` under ``name``; with ``fp8`` as e4m3 + ``_scale_inv``, each of
    the ``parts`` equal dim-0 sub-tensors (gate/up, q/k/v are quantised as a
    whole: parts=1) carrying its own block grid.  ``zero`` only allocates."""
    if not fp8 or t.dim() < 2:
        out[name] = t.contiguous()
        return
    if zero:
        rows, cols = t.shape[-2], t.shape[-1]
        grid = (parts * -(-(rows // parts) // 128), -(-cols // 128))
        out[name] = torch.zeros(t.shape, dtype=torch.float8_e4m3fn, device=t.device)
        out[name + "_scale_inv"] = torch.zeros(tuple(t.shape[:-2]) + grid, dtype=torch.float32, device=t.device)
        return
    if t.dim() == 3:  # fused experts: quantise every expert slot separately
        qs, ss = zip(*(_quant_parts(t[e], parts) for e in range(t.shape[0])))
        out[name] = torch.stack(qs)
        out[name + "_scale_inv"] = torch.stack(ss)
    else:
        out[name], out[name + "_scale_inv"] = _quant_parts(t, parts)


def _quant_parts(t2d: torch.Tensor, parts: int):
    # Quantise on the CPU: it is the stated oracle.  CUDA PyTorch divides by the
    # scalar 448 as a multiplication by its reciprocal, which moves some scales by
    # one ulp relative to the true division of the CPU path and of the kernels.
    # For models of hundreds of GB the CPU is too slow; AWEX_SYNTH_FP8_ORACLE=kernel
    # switches to the stand-alone quantisation kernel, which the GPU tests hold
    # bit-identical to the CPU path.
    if t2d.is_cuda and os.environ.get("AWEX_SYNTH_FP8_ORACLE", "cpu") == "kernel":
        from awex_b200.ops.fp8 import block_quant

        qs, ss = zip(*(block_quant(c.contiguous()) for c in t2d.chunk(parts, 0)))
        return torch.cat(qs, 0), torch.cat(ss, 0)
    qs, ss = zip(*(per_block_cast_to_fp8(c.detach().cpu().contiguous(), False) for c in t2d.chunk(parts, 0)))
    return torch.cat(qs, 0).to(t2d.device), torch.cat(ss, 0).to(t2d.device)


def build_vllm_model(arch: Arch, rank_info: RankInfo, dtype=torch.bfloat16, device="cpu", seed: int = 0,
                     step: int = 0, fp8: bool = False, zero: bool = False, layers: Optional[range] = None,
                     weights: Optional[CanonicalWeights] = None, dp_lm_head: bool = False) -> FlatModule:
    """``zero=True`` allocates the same tensors filled with zeros (a freshly
    paused engine whose weights are about to be overwritten)."""
    w = weights or (ZeroWeights(arch, dtype, device) if zero else CanonicalWeights(arch, dtype, device, seed, step))
    tp, r = rank_info.tp_size, rank_info.tp_rank
    # attention, embeddings and (with ``dp_lm_head``) the head follow attention TP, which
    # equals TP unless the engine runs DP attention
    atp, ar = rank_info.attn_tp_size, rank_info.attn_tp_rank
    htp, hr = (atp, ar) if dp_lm_head else (tp, r)
    ep, er = rank_info.ep_size, rank_info.ep_rank
    etp, etr = rank_info.ep_tp_size, rank_info.ep_tp_rank
    if ep == 1:  # no expert parallelism: experts are TP-sliced
        etp, etr = tp, r
    out: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    hd = arch.head_dim
    heads_local = arch.num_heads // atp
    kv_local = max(arch.num_kv_heads // atp, 1)
    kv_first = (ar * arch.num_kv_heads) // atp  # index of this rank's first KV head
    first_stage, last_stage = rank_info.pp_rank == 0, rank_info.pp_rank == rank_info.pp_size - 1
    if first_stage:
        out["model.embed_tokens.weight"] = _chunk(w.embed(), atp, ar).contiguous()
    for l in layers if layers is not None else pp_layer_range(arch.num_layers, rank_info.pp_rank, rank_info.pp_size):
        p = f"model.layers.{l}."

        def fused(kind: str) -> torch.Tensor:
            q, k, v = (w.layer(l, f"self_attn.{x}_proj.{kind}") for x in "qkv")
            return torch.cat(
                [q.narrow(0, ar * heads_local * hd, heads_local * hd), k.narrow(0, kv_first * hd, kv_local * hd),
                 v.narrow(0, kv_first * hd, kv_local * hd)], 0,
            )

        out[p + "input_layernorm.weight"] = w.layer(l, "input_layernorm.weight")
        _maybe_fp8(out, p + "self_attn.qkv_proj.weight", fused("weight"), fp8, zero=zero)
        if arch.qkv_bias:
            out[p + "self_attn.qkv_proj.bias"] = fused("bias")
        if arch.qk_norm:
            out[p + "self_attn.q_norm.weight"] = w.layer(l, "self_attn.q_norm.weight")
            out[p + "self_attn.k_norm.weight"] = w.layer(l, "self_attn.k_norm.weight")
        _maybe_fp8(out, p + "self_attn.o_proj.weight", _chunk(w.layer(l, "self_attn.o_proj.weight"), atp, ar, 1), fp8, zero=zero)
        out[p + "post_attention_layernorm.weight"] = w.layer(l, "post_attention_layernorm.weight")
        if arch.is_moe:
            out[p + "mlp.gate.weight"] = w.layer(l, "mlp.gate.weight")
            n_local = arch.num_experts // ep
            w13, w2 = [], []
            for le in range(n_local):
                e = er * n_local + le
                w13.append(torch.cat([_chunk(w.expert(l, e, "gate_proj"), etp, etr), _chunk(w.expert(l, e, "up_proj"), etp, etr)], 0))
                w2.append(_chunk(w.expert(l, e, "down_proj"), etp, etr, 1))
            _maybe_fp8(out, p + "mlp.experts.w13_weight", torch.stack(w13), fp8, parts=2, zero=zero)
            _maybe_fp8(out, p + "mlp.experts.w2_weight", torch.stack(w2), fp8, zero=zero)
        else:
            gate_up = torch.cat([_chunk(w.layer(l, "mlp.gate_proj.weight"), tp, r), _chunk(w.layer(l, "mlp.up_proj.weight"), tp, r)], 0)
            _maybe_fp8(out, p + "mlp.gate_up_proj.weight", gate_up, fp8, parts=2, zero=zero)
            _maybe_fp8(out, p + "mlp.down_proj.weight", _chunk(w.layer(l, "mlp.down_proj.weight"), tp, r, 1), fp8, zero=zero)
    if last_stage:
        out["model.norm.weight"] = w.final_norm()
        if not arch.tie_embeddings or not first_stage:  # as on the training side
            out["lm_head.weight"] = _chunk(w.lm_head(), htp, hr).contiguous()
    if zero:
        for t in out.values():
            t.zero_()
    cls = type(arch.architecture, (FlatModule,), {})
    return cls(out, arch.hf_config())


def vllm_model_context(rank_info: RankInfo, scheduler=None, **extra) -> dict:
    """The ``model_context`` dict an engine adapter hands to worker tasks."""
    ctx = dict(
        tp_rank=rank_info.tp_rank, tp_size=rank_info.tp_size, pp_rank=rank_info.pp_rank, pp_size=rank_info.pp_size,
        dp_rank=rank_info.dp_rank, dp_size=rank_info.dp_size, ep_rank=rank_info.ep_rank, ep_size=rank_info.ep_size,
        ep_tp_rank=rank_info.ep_tp_rank, ep_tp_size=rank_info.ep_tp_size, attn_tp_rank=rank_info.attn_tp_rank,
        attn_tp_size=rank_info.attn_tp_size, attn_dp_rank=rank_info.attn_dp_rank, world_size=rank_info.world_size,
        global_rank=rank_info.global_rank, local_rank=rank_info.local_rank, cp_rank=rank_info.cp_rank,
        cp_size=rank_info.cp_size, cp_mode=rank_info.cp_mode, scheduler=scheduler,
    )
    ctx.update(extra)
    return ctx
