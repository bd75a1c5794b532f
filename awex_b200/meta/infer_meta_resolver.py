"""Inference-side metadata: one task runs in every model worker, lists the
worker's parameters as canonical views, and the control process groups the
per-worker listings into :class:`ParameterMeta`
(`awex/meta/infer_meta_resolver.py:37-309` in the reference).

The worker task is :func:`collect_worker_param_info`; it is a module-level
function so engines can ship it to workers by module + qualified name.
"""

from __future__ import annotations

import json
import os
from datetime import datetime
from typing import Any, Dict, List, Tuple

import torch

from awex_b200 import logging
from awex_b200.meta.meta_resolver import ParamMetaResolver
from awex_b200.meta.weight_meta import ParameterMeta, compute_total_model_size, dump_parameters_meta
from awex_b200.models.registry import get_infer_weights_converter
from awex_b200.sharding.param_sharding import ShardingType, get_rank_info_extractor, get_sharding_strategy_builder
from awex_b200.sharding.rank_info import RankInfo
from awex_b200.utils.common import to_dict

logger = logging.getLogger(__name__)


def canonical_named_views(model, converter, model_context: dict | None = None, convert_params: bool = True):
    """``[(canonical_name, view)]`` for every parameter of ``model``; with tied
    embeddings the last pipeline stage also answers for ``lm_head.weight``
    through the embedding tensor."""
    out: List[Tuple[str, torch.Tensor]] = []
    for name, param in model.named_parameters():
        if convert_params:
            out.extend(converter.convert_param(name, param))
        else:
            out.append((name, param))
    if not convert_params:
        return out
    hf_config = getattr(model, "config", None) or (model_context or {}).get("hf_config")
    if getattr(hf_config, "tie_word_embeddings", False):
        ctx = model_context or {}
        last_stage = ctx.get("pp_rank", 0) == ctx.get("pp_size", 1) - 1
        names = {n for n, _ in out}
        if last_stage and "lm_head.weight" not in names and "model.embed_tokens.weight" in names:
            embed = next(t for n, t in out if n == "model.embed_tokens.weight")
            out.append(("lm_head.weight", embed))
    return out


def find_aliases(views) -> Dict[str, str]:
    """Canonical names that are second names of the very same memory in this
    worker (tied ``lm_head.weight`` served by the embedding tensor): alias ->
    first name.  Writing the first name fills the alias too."""
    first: Dict[tuple, str] = {}
    out: Dict[str, str] = {}
    for name, t in views:
        if t.numel() == 0 or t.device.type == "meta":  # shape-only tensors have no memory to share
            continue
        key = (t.data_ptr(), tuple(t.shape), tuple(t.stride()), str(t.dtype))
        if key in first:
            out[name] = first[key]
        else:
            first[key] = name
    return out


def collect_worker_param_info(engine_name, infer_engine_config, convert_params=False, engine_rank=0, **kwargs):
    """Runs inside a model worker; ``kwargs`` carries ``model`` and
    ``model_context``.  dtypes are sent as strings without the ``torch.``
    prefix so the result survives msgpack transports."""
    model, ctx = kwargs["model"], kwargs["model_context"]
    rank_info = get_rank_info_extractor(engine_name)(ctx, engine_rank)
    arch = type(model).__name__
    converter = get_infer_weights_converter(
        engine_name, arch, hf_config=model.config, infer_engine_config=infer_engine_config, rank_info=rank_info
    )
    views = canonical_named_views(model, converter, ctx, convert_params)
    if os.environ.get("AWEX_DEBUG_INFER_META", "0") == "1":
        names = [n for n, _ in views]
        logger.info(
            f"Infer meta debug: engine={engine_name} engine_rank={engine_rank} pp_rank={ctx.get('pp_rank')}/"
            f"{ctx.get('pp_size')} tp_rank={ctx.get('tp_rank')} convert_params={convert_params} "
            f"has_lm_head={any(n.endswith('lm_head.weight') for n in names)} "
            f"has_embed={any(n.endswith('embed_tokens.weight') for n in names)} total_params={len(names)}"
        )
    strided = [(n, tuple(t.shape)) for n, t in views if not t.is_contiguous()]
    if strided:
        logger.info(f"Infer meta rank {rank_info.global_rank} has {len(strided)} non-contiguous params, e.g. {strided[:8]}")
    return {
        "rank_info": rank_info,
        "model_arch_name": arch,
        "aliases": find_aliases(views),
        "params_meta": [
            {"name": n, "numel": t.numel(), "shape": tuple(t.shape), "dtype": str(t.dtype).replace("torch.", "")}
            for n, t in views
        ],
    }


class InferParamMetaResolver(ParamMetaResolver):
    def __init__(self, inference_engine, convert_params=False, num_engines=1, engine_rank=0):
        super().__init__(inference_engine.hf_config)
        self._inference_engine = inference_engine
        self.infer_engine_config = inference_engine.config
        self.engine_name = inference_engine.engine_name
        self.convert_params = convert_params
        self.num_engines = num_engines
        self.engine_rank = engine_rank
        debug = bool(getattr(self.infer_engine_config, "enable_debug_mode", False))
        suffix = f"{engine_rank}_{os.getpid()}_{datetime.now().strftime('%Y_%m_%d_%H_%M_%S')}.json"

        def run(convert: bool):
            return inference_engine.execute_task_in_model_worker(
                self._get_model_param_info, engine_name=self.engine_name, infer_engine_config=self.infer_engine_config,
                engine_rank=engine_rank, convert_params=convert,
            )

        if debug:
            self._dump(f"infer_params_non_converted_raw_meta_{suffix}", to_dict(run(False)))
        self._params_raw_meta = run(self.convert_params)
        for info in self._params_raw_meta:  # some RPC layers flatten dataclasses to dicts
            if isinstance(info.get("rank_info"), dict):
                info["rank_info"] = RankInfo(**info["rank_info"])
        if debug:
            self._dump(f"infer_params_raw_meta_{suffix}", to_dict(self._params_raw_meta))
        # a name is an alias for the job only if every worker that reports it holds it as one
        reported, aliased = {}, {}
        for info in self._params_raw_meta:
            for pm in info["params_meta"]:
                reported[pm["name"]] = reported.get(pm["name"], 0) + 1
            for alias, target in (info.get("aliases") or {}).items():
                aliased.setdefault(alias, []).append(target)
        self.aliases: Dict[str, str] = {a: ts[0] for a, ts in aliased.items() if len(ts) == reported.get(a) and len(set(ts)) == 1}
        self._rank0_meta = self._select_canonical_rank0_meta(self._params_raw_meta)
        self.rank0_info = self._rank0_meta["rank_info"]
        self._world_size = self.rank0_info.world_size
        self._model_arch_name = self._rank0_meta["model_arch_name"]
        self._sharding_strategy = get_sharding_strategy_builder(self.engine_name)(
            self._model_arch_name, self.infer_engine_config, self.rank0_info
        )
        self._params_meta = self._build_params_meta()
        if debug:
            self._dump(f"infer_params_meta_{suffix}", dump_parameters_meta(self._params_meta))
        self.total_numel = sum(p.global_numel for p in self._params_meta)
        self.total_size = compute_total_model_size(self._params_meta)
        logger.info(f"Total number of elements in the model: {self.total_numel}, total size: {self.total_size} bytes")

    @staticmethod
    def _dump(filename: str, payload) -> None:
        path = os.path.abspath(filename)
        with open(path, "w") as f:
            json.dump(payload, f, indent=4)
        logger.info(f"debug dump written: {path}")

    _get_model_param_info = staticmethod(collect_worker_param_info)

    def get_model_arch_name(self) -> str:
        return self._model_arch_name

    def get_parameters_meta(self) -> List[ParameterMeta]:
        return self._params_meta

    def _get_params_raw_meta(self) -> List[Dict[str, Any]]:
        return self._params_raw_meta

    @staticmethod
    def _meta_identity_key(info: Dict[str, Any]):
        ri = info["rank_info"]
        return (ri.global_rank, ri.dp_rank, ri.tp_rank, ri.pp_rank, ri.ep_rank, ri.attn_tp_rank, ri.attn_dp_rank)

    @classmethod
    def _select_canonical_rank0_meta(cls, params_raw_meta: List[Dict[str, Any]]) -> Dict[str, Any]:
        """With internal data parallelism several cores report a global rank
        0; the one with the smallest (dp, tp, pp, ep, attn_tp, attn_dp) is the
        reference worker."""
        if not params_raw_meta:
            raise ValueError("No inference parameter metadata collected.")
        zeros = {cls._meta_identity_key(i): i for i in params_raw_meta if i["rank_info"].global_rank == 0}
        if zeros:
            if len(zeros) > 1:
                logger.warning(f"Found {len(zeros)} distinct rank0 metas; selecting canonical by (dp,tp,pp,ep,attn_tp,attn_dp).")
            return zeros[min(zeros, key=lambda k: k[1:])]
        logger.warning("No global_rank==0 meta found; falling back to minimum rank identity.")
        return min(params_raw_meta, key=cls._meta_identity_key)

    def _get_sharding_info(self, name: str, rank_info: RankInfo, param_meta: Dict[str, Any]) -> Tuple[ShardingType, int, int]:
        return self._sharding_strategy.get_sharding_strategy(name, rank_info=rank_info, param_meta=param_meta)
