"""A whole exchange inside one process.

:class:`SimulatedJob` holds every training rank's Megatron-layout shards and
every inference rank's (zeroed) vLLM-layout parameters of a synthetic model,
resolves both metadata lists, compiles every training rank's send program and
can run it with the CPU executor.  It is how multi-rank logic is tested
without a cluster, and how a single GPU emulates all ranks of a layout with
one kernel launch over all ranks' data.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from awex_b200.config import InferenceConfig
from awex_b200.meta.infer_meta_resolver import InferParamMetaResolver, canonical_named_views
from awex_b200.meta.train_meta_resolver import RawTrainMetaResolver, list_local_train_params
from awex_b200.meta.weight_meta import ParameterMeta
from awex_b200.models.registry import get_infer_weights_converter, get_train_weights_converter
from awex_b200.sharding.rank_info import RankInfo
from awex_b200.synthetic.arch import Arch
from awex_b200.synthetic.models import FlatModule, build_megatron_model, build_vllm_model, vllm_model_context
from awex_b200.synthetic.topology import infer_rank_infos, train_rank_infos
from awex_b200.transfer.cpu_exec import execute_items
from awex_b200.transfer.lowering import (
    CopyItem, LocalParam, SendProgramCompiler, check_exactly_once, manifest_by_destination, refresh_derived,
)
from awex_b200.transfer.transfer_plan import TransferPlanBuilder
from awex_b200.utils.common import check_train_infer_params_meta


@dataclass
class TrainLayout:
    tp: int = 1
    pp: int = 1
    dp: int = 1
    ep: int = 1
    etp: int = 1

    @property
    def world(self) -> int:
        return self.tp * self.pp * self.dp

    def label(self) -> str:
        return "".join(f"{k}{v}" for k, v in (("tp", self.tp), ("pp", self.pp), ("dp", self.dp), ("ep", self.ep)) if v > 1) or "tp1"


@dataclass
class InferLayout:
    tp: int = 1
    ep: int = 1
    num_engines: int = 1
    engine_name: str = "vllm"
    fp8: bool = False
    pp: int = 1
    attn_tp: int = 0  # SGLang DP attention: attention TP inside TP (0: same as tp)
    dp_lm_head: bool = False

    @property
    def attention_tp(self) -> int:
        return self.attn_tp or self.tp

    @property
    def instance_world(self) -> int:
        return self.tp * self.pp

    @property
    def world(self) -> int:
        return self.tp * self.pp * self.num_engines

    def label(self) -> str:
        base = f"tp{self.tp}" + (f"attn{self.attn_tp}" if self.attn_tp not in (0, self.tp) else "") + (f"pp{self.pp}" if self.pp > 1 else "") + (f"ep{self.ep}" if self.ep > 1 else "") + ("-fp8" if self.fp8 else "")
        return f"{self.num_engines}x{base}" if self.num_engines > 1 else base


class _Scheduler:
    """What the worker reader needs from an inference scheduler."""

    def __init__(self, server_args):
        self.server_args = server_args
        self.flushes = 0

    def flush_cache(self):
        self.flushes += 1
        return True


class LocalInferenceEngine:
    """Inference engine whose model workers are objects in this process."""

    def __init__(self, arch: Arch, layout: InferLayout, ranks: Sequence[RankInfo], models: Sequence[FlatModule],
                 engine_rank: int = 0, **config_overrides):
        self.engine_name = layout.engine_name
        self.hf_config = models[0].config
        cfg = dict(
            tp_size=layout.tp, pp_size=layout.pp, dp_size=layout.tp // layout.attention_tp, ep_size=layout.ep,
            enable_dp_attention=layout.attention_tp != layout.tp, enable_dp_lm_head=layout.dp_lm_head, moe_dense_tp_size=None, num_engines=layout.num_engines, engine_rank=engine_rank,
            comm_backend="nccl", fp8_block_quant=layout.fp8,
        )
        cfg.update(config_overrides)
        self.config = InferenceConfig(**cfg)
        self.num_engines = layout.num_engines
        self.engine_rank = engine_rank
        self.ranks, self.models = list(ranks), list(models)
        self.schedulers = [_Scheduler(self.config) for _ in ranks]

    def model_context(self, i: int) -> dict:
        return vllm_model_context(self.ranks[i], scheduler=self.schedulers[i], infer_engine_config=self.config)

    def execute_task_in_model_worker(self, fn, **kwargs):
        return [fn(model=m, model_context=self.model_context(i), **kwargs) for i, m in enumerate(self.models)]

    def release_memory_occupation(self, tags=None):
        pass

    def resume_memory_occupation(self, tags=None):
        pass

    def update_weights_from_disk(self, path, load_format=None):
        raise NotImplementedError


class SimulatedJob:
    def __init__(self, arch: Arch, train: TrainLayout, infer: InferLayout, dtype=torch.float32, device="cpu",
                 seed: int = 0, build_models: bool = True):
        self.arch, self.train, self.infer, self.dtype, self.device, self.seed = arch, train, infer, dtype, device, seed
        self.hf_config = arch.hf_config()
        self.train_ranks = train_rank_infos(train.tp, train.pp, train.dp, train.ep, train.etp)
        self.infer_ranks = [infer_rank_infos(infer.tp, infer.ep, engine_rank=e, pp=infer.pp, flavour=infer.engine_name, attn_tp=infer.attn_tp) for e in range(infer.num_engines)]
        self.train_models: List[FlatModule] = []
        self.infer_models: List[List[FlatModule]] = []
        if build_models:
            self.train_models = [build_megatron_model(arch, ri, dtype, device, seed) for ri in self.train_ranks]
            self.infer_models = [
                [build_vllm_model(arch, ri, dtype, device, seed, fp8=infer.fp8, zero=True, dp_lm_head=infer.dp_lm_head) for ri in ranks] for ranks in self.infer_ranks
            ]
        self.engines = [
            LocalInferenceEngine(arch, infer, self.infer_ranks[e], self.infer_models[e], engine_rank=e) for e in range(infer.num_engines)
        ] if build_models else []
        self.infer_world_size = infer.world
        self.builder = TransferPlanBuilder(self.infer_world_size, train.world, infer.num_engines)
        self._resolve_metadata()

    # ---- metadata ---------------------------------------------------------------------------------
    def _resolve_metadata(self) -> None:
        resolver = InferParamMetaResolver(self.engines[0], convert_params=True, num_engines=self.infer.num_engines, engine_rank=0)
        self.infer_meta: List[ParameterMeta] = resolver.get_parameters_meta()
        self.aliases = dict(getattr(resolver, "aliases", {}) or {})
        self.builder.skip_names = frozenset(self.aliases)
        self.infer_conf = {
            "engine_name": self.infer.engine_name,
            "infer_atten_tp_size": self.infer.attention_tp,
            "router_dtype": "bf16" if self.dtype == torch.bfloat16 else ("fp16" if self.dtype == torch.float16 else "fp32"),
            "infer_engine_config": self.engines[0].config,
            "hf_config": self.hf_config,
            "infer_world_size": self.infer_world_size,
            "fp8_block_quant": self.infer.fp8,
            "aliased_parameters": self.aliases,
        }
        raw = [
            list_local_train_params([m], self._train_converter(ri, with_pp_map=False), ri, self.hf_config, self.arch.architecture)
            for ri, m in zip(self.train_ranks, self.train_models)
        ]
        tr = RawTrainMetaResolver(self.hf_config, self.arch.architecture, raw, self.train_ranks[0])
        self.train_meta: List[ParameterMeta] = tr.get_parameters_meta()
        self.pp_map = tr.get_pp_stage_layer_id_map()
        check_train_infer_params_meta(self.train_meta, self.infer_meta, raise_exception=True)

    def _train_converter(self, ri: RankInfo, with_pp_map: bool = True):
        conf = dict(self.infer_conf)
        if with_pp_map:
            conf["train_pp_stage_layer_id_map"] = self.pp_map
        return get_train_weights_converter("mcore", self.arch.architecture, self.hf_config, ri, conf, tf_config=self.arch.tf_config())

    # ---- programs -----------------------------------------------------------------------------------
    def local_params(self, train_rank: int) -> List[LocalParam]:
        return [LocalParam(n, 0, tuple(t.shape), t.dtype) for n, t in self.train_models[train_rank].named_parameters()]

    def compile_send_program(self, train_rank: int) -> List[CopyItem]:
        ri = self.train_ranks[train_rank]
        compiler = SendProgramCompiler(
            ri, self.train_ranks, self._train_converter, self.local_params(train_rank), self.infer_meta, self.train_meta, self.builder
        )
        items = compiler.compile()
        if not hasattr(self, "derived"):
            self.derived, self._derived_buffers = {}, {}
        self.derived[train_rank] = list(compiler.derived.values())
        return items

    def local_tensors(self, train_rank: int) -> Dict[Tuple[str, int], torch.Tensor]:
        """(name, chunk) -> tensor for everything ``train_rank``'s items read: its
        parameters and, freshly recomputed, its derived tensors."""
        local = {(n, 0): t for n, t in self.train_models[train_rank].named_parameters()}
        derived = getattr(self, "derived", {}).get(train_rank, [])
        if derived:
            local.update(self._derived_buffers.setdefault(train_rank, {}))
            from awex_b200.transfer.lowering import _tp_peers

            peers = _tp_peers(self.train_ranks[train_rank], self.train_ranks)

            def gather(name, _vp):  # all ranks live in this process: read the TP peers' shards directly
                return [dict(self.train_models[p.global_rank].named_parameters())[name] for p in peers]

            refresh_derived(derived, local, gather)
            self._derived_buffers[train_rank] = {d.key: local[d.key] for d in derived}
        return local

    def source_tensors(self) -> List[torch.Tensor]:
        """Every tensor any rank's items read: all training parameters and derived buffers."""
        return [t for r in range(self.train.world) for t in self.local_tensors(r).values()]

    def compile_all(self) -> Dict[int, List[CopyItem]]:
        self.programs = {r: self.compile_send_program(r) for r in range(self.train.world)}
        return self.programs

    def destination_views(self) -> Dict[int, Dict[str, torch.Tensor]]:
        """transfer rank -> canonical name -> live view, for every inference worker."""
        out: Dict[int, Dict[str, torch.Tensor]] = {}
        for e, (ranks, models) in enumerate(zip(self.infer_ranks, self.infer_models)):
            for ri, model in zip(ranks, models):
                conv = get_infer_weights_converter(self.infer.engine_name, self.arch.architecture, self.hf_config, ri, self.engines[e].config)
                ctx = vllm_model_context(ri)
                out[ri.global_rank + e * self.infer.instance_world] = dict(canonical_named_views(model, conv, ctx))
        return out

    def check_coverage(self) -> List[str]:
        """Exactly-once check of all programs against all destination views."""
        views = self.destination_views()
        problems: List[str] = []
        trained = {m.name for m in self.train_meta}
        for rank, rank_views in views.items():
            manifests = [manifest_by_destination(items).get(rank, []) for items in self.programs.values()]
            shapes = {n: (tuple(v.shape), v.dtype) for n, v in rank_views.items()}
            required = [n for n in shapes if (n in trained or n.endswith("_scale_inv")) and n not in self.aliases]
            problems += [f"rank {rank}: {p}" for p in check_exactly_once(manifests, shapes, required)]
        return problems

    def run_cpu(self) -> int:
        views = self.destination_views()
        total = 0
        for rank, items in self.programs.items():
            total += execute_items(items, self.local_tensors(rank), views)
        return total

    # ---- single-GPU emulation of all ranks ------------------------------------------------------------
    def encode_all(self, validate: bool = True):
        """Encode every rank's program against addresses in this process.
        Returns ``{train_rank: (table, n_tiles, encoder)}``."""
        from awex_b200.transfer.descriptors import TensorAddr, encode_items, validate_table

        views = self.destination_views()
        dst_addrs = {rank: {n: TensorAddr.of(v) for n, v in vs.items()} for rank, vs in views.items()}
        dst_spans = [TensorAddr.of(p).byte_span() for models in self.infer_models for m in models for p in m.parameters()]
        out = {}
        for rank, items in self.programs.items():
            src_addrs = {key: TensorAddr.of(t) for key, t in self.local_tensors(rank).items()}
            table, n_tiles, enc = encode_items(items, src_addrs, dst_addrs)
            if validate:
                problems = validate_table(table, n_tiles, [a.byte_span() for a in src_addrs.values()], dst_spans)
                if problems:
                    raise ValueError(f"rank {rank}: descriptor table rejected: {problems[:5]}")
            out[rank] = (table, n_tiles, enc)
        self.encoded = out
        return out

    def build_gpu_programs(self, timeout_ms: int = 2000, grid: int = 0):
        """One TransferProgram per training rank plus one done-flag pad and a
        waiter, all on this job's device (every "rank" shares the GPU, so the
        launches simply run in stream order and no wait ever spins)."""
        from awex_b200.ops.fused_transfer import FlagPad, FlagWaiter, TransferProgram

        if not hasattr(self, "encoded"):
            self.encode_all()
        self.done_pad = FlagPad(self.train.world, self.device)
        self.gpu_programs = {
            rank: TransferProgram(table, n_tiles, self.device, done_flag_addrs=[self.done_pad.slot_addr(rank)],
                                  timeout_ms=timeout_ms, grid=grid, encoder=enc)
            for rank, (table, n_tiles, enc) in self.encoded.items()
        }
        self.waiter = FlagWaiter(self.done_pad, list(range(self.train.world)), self.device, timeout_ms=timeout_ms)
        return self.gpu_programs

    def run_gpu(self, epoch: int) -> None:
        for rank, derived in getattr(self, "derived", {}).items():
            if derived:
                self.local_tensors(rank)  # recompute derived tensors in place, ahead of the transfer in stream order
        for prog in self.gpu_programs.values():
            prog.launch(epoch)
        self.waiter.launch(epoch)

    def gpu_status(self) -> None:
        for prog in self.gpu_programs.values():
            prog.status.raise_if_failed()
        self.waiter.status.raise_if_failed()

    def mismatches(self) -> List[str]:
        """Names of inference parameters that differ from the layout built
        directly from the canonical weights."""
        bad = []
        for e, (ranks, models) in enumerate(zip(self.infer_ranks, self.infer_models)):
            for ri, model in zip(ranks, models):
                oracle = build_vllm_model(self.arch, ri, self.dtype, self.device, self.seed, fp8=self.infer.fp8, dp_lm_head=self.infer.dp_lm_head)
                for (name, got), (_, want) in zip(model.named_parameters(), oracle.named_parameters()):
                    same = torch.equal(got.view(torch.uint8), want.view(torch.uint8)) if got.dtype == torch.float8_e4m3fn else torch.equal(got, want)
                    if not same:
                        bad.append(f"engine{e}/rank{ri.global_rank}/{name}")
        return bad
