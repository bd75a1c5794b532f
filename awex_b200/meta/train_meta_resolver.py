"""Training-side metadata: every rank lists its canonical tensors, the lists
are all-gathered over the training world, pipeline-local layer ids are
rewritten to global ids, and the result is grouped into :class:`ParameterMeta`.

Differences from the reference (`awex/meta/train_meta_resolver.py:43-314`):
shapes come from the converter's symbolic :meth:`plan_param`, so no layout
transform (and no TP all-gather) runs just to learn a shape; the training
engine may pass its own ``rank_info`` and ``process_group`` when Megatron's
parallel state is not importable.
"""

from __future__ import annotations

import json
import os
import re
from datetime import datetime
from typing import Any, Dict, List, Optional, Tuple

from torch import distributed as dist

from awex_b200 import logging
from awex_b200.meta.meta_resolver import ParamMetaResolver, get_num_hidden_layers
from awex_b200.meta.weight_meta import ParameterMeta, compute_total_model_size, dump_parameters_meta
from awex_b200.models.registry import get_train_weights_converter
from awex_b200.sharding.param_sharding import ShardingType
from awex_b200.sharding.rank_info import RankInfo
from awex_b200.utils.common import to_dict

logger = logging.getLogger(__name__)

_LAYER_ID = re.compile(r"(?<=\.layers\.)(\d+)(?=\.)")


def maybe_get_tf_config(models):
    for model in models if isinstance(models, (list, tuple)) else [models]:
        for attr in ("transformer_config", "config"):
            cfg = getattr(model, attr, None)
            if cfg is not None:
                return cfg
    return None


def _local_layer_id(name: str) -> Optional[int]:
    m = _LAYER_ID.search(name)
    return int(m.group(1)) if m else None


def build_pp_stage_layer_id_map(global_metadata: List[Dict[str, Any]]) -> Dict[Tuple[int, int], Dict[int, int]]:
    """(pp_rank, vp_stage) -> {local layer id -> global layer id}.  Stages are
    numbered virtual stage outermost, pipeline rank innermost; inside a stage
    local ids keep their order."""
    seen: Dict[Tuple[int, int], set] = {}
    pp_size = None
    for rank_meta in global_metadata:
        ri: RankInfo = rank_meta["rank_info"]
        pp_size = int(ri.pp_size) if pp_size is None else pp_size
        for pm in rank_meta["params_meta"]:
            local = _local_layer_id(pm["name"])
            if local is not None:
                seen.setdefault((int(ri.pp_rank), int(pm.get("vp_stage", 0))), set()).add(local)
    if not seen:
        return {}
    out: Dict[Tuple[int, int], Dict[int, int]] = {}
    next_global = 0
    for vp in sorted({k[1] for k in seen}):
        for pp in range(pp_size):
            ids = sorted(seen.get((pp, vp), ()))
            if ids:
                out[(pp, vp)] = {local: next_global + i for i, local in enumerate(ids)}
                next_global += len(ids)
    return out


def canonicalize_pp_layer_names(global_metadata, stage_map):
    if not stage_map:
        return global_metadata
    for rank_meta in global_metadata:
        ri: RankInfo = rank_meta["rank_info"]
        for pm in rank_meta["params_meta"]:
            local = _local_layer_id(pm["name"])
            if local is None:
                continue
            key = (int(ri.pp_rank), int(pm.get("vp_stage", 0)))
            layer_map = stage_map.get(key)
            if layer_map is None or local not in layer_map:
                raise ValueError(
                    f"pp stage layer map has no entry for stage={key}, local_layer_id={local}, "
                    f"param={pm['name']}, rank={ri.global_rank}"
                )
            pm["name"] = _LAYER_ID.sub(str(layer_map[local]), pm["name"], count=1)
    return global_metadata


# names kept for readers of the reference
_build_pp_stage_layer_id_map = build_pp_stage_layer_id_map
_canonicalize_pp_layer_names_in_global_meta = canonicalize_pp_layer_names
_maybe_get_tf_config = maybe_get_tf_config


def resolve_train_rank_info(train_engine) -> RankInfo:
    ri = getattr(train_engine, "rank_info", None)
    if ri is not None:
        return ri
    from awex_b200.sharding.extractors import get_mcore_rank_info

    return get_mcore_rank_info()


def list_local_train_params(models, converter, rank_info: RankInfo, hf_config, arch_name: str, convert_params: bool = True) -> Dict[str, Any]:
    """This rank's raw listing: canonical (or native) names with shapes, before
    the all-gather.  Layer ids are still pipeline-local."""
    from awex_b200.converter.mcore_converter import get_mcore_model_parameters

    listing: List[Dict[str, Any]] = []
    tied = bool(getattr(hf_config, "tie_word_embeddings", False))
    for vp_stage, chunk in enumerate(models):
        for name, param in get_mcore_model_parameters(chunk).items():
            if convert_params:
                specs = converter.plan_param(name, tuple(param.shape), param.dtype, vp_stage=vp_stage)
                entries = [(s.name, s.shape, s.numel, s.dtype) for s in specs]
                names = {e[0] for e in entries}
                # tied embeddings: the last pipeline stage also answers for lm_head
                if tied and rank_info.pp_rank == rank_info.pp_size - 1 and "model.embed_tokens.weight" in names and "lm_head.weight" not in names:
                    entries += [("lm_head.weight",) + e[1:] for e in entries if e[0] == "model.embed_tokens.weight"]
            else:
                entries = [(name, tuple(param.shape), param.numel(), param.dtype)]
            for cname, shape, numel, dtype in entries:
                listing.append({"name": cname, "numel": numel, "shape": tuple(shape), "dtype": dtype, "vp_stage": vp_stage})
    return {"rank_info": rank_info, "params_meta": listing, "model_arch_name": arch_name}


class RawTrainMetaResolver(ParamMetaResolver):
    """Builds training metadata from already collected per-rank listings
    (simulation, tests, offline analysis of debug dumps)."""

    def __init__(self, hf_config, arch_name: str, raw_metas: List[Dict[str, Any]], rank_info: RankInfo):
        super().__init__(hf_config)
        from awex_b200.sharding.extractors import get_mcore_sharding_strategy

        self._arch = arch_name
        self._strategy = get_mcore_sharding_strategy(arch_name, rank_info)
        self._pp_stage_layer_id_map = build_pp_stage_layer_id_map(raw_metas)
        self._raw = canonicalize_pp_layer_names(raw_metas, self._pp_stage_layer_id_map)
        self._meta = self._build_params_meta()

    def get_model_arch_name(self) -> str:
        return self._arch

    def get_parameters_meta(self) -> List[ParameterMeta]:
        return self._meta

    def get_pp_stage_layer_id_map(self):
        return self._pp_stage_layer_id_map

    def _get_params_raw_meta(self):
        return self._raw

    def _get_sharding_info(self, name, rank_info, param_meta):
        return self._strategy.get_sharding_strategy(name, rank_info=rank_info, param_meta=param_meta)


class McoreParamMetaResolver(ParamMetaResolver):
    def __init__(self, train_engine, hf_config, infer_conf: Dict):
        super().__init__(hf_config)
        self._train_engine = train_engine
        model = train_engine.model
        self._mcore_model = list(model) if isinstance(model, (list, tuple)) else [model]
        self._model_arch_name = self.hf_config.architectures[0]
        self._tf_config = maybe_get_tf_config(self._mcore_model)
        from awex_b200.sharding.extractors import get_mcore_sharding_strategy

        self._rank_info = resolve_train_rank_info(train_engine)
        self._group = getattr(train_engine, "process_group", None)
        self._sharding_strategy = get_mcore_sharding_strategy(self._model_arch_name, self._rank_info)
        self._infer_conf = infer_conf
        self.infer_hf_config = infer_conf["hf_config"]
        self.num_hidden_layers = get_num_hidden_layers(self.infer_hf_config)
        self._pp_stage_layer_id_map: Dict[Tuple[int, int], Dict[int, int]] = {}
        debug = bool(getattr(train_engine, "enable_debug_mode", False))
        rank = self._rank_info.global_rank
        suffix = f"_{rank}_{os.getpid()}_{datetime.now().strftime('%Y_%m_%d_%H_%M_%S')}.json"
        if debug:
            self._dump(f"train_params_non_converted_raw_meta{suffix}", to_dict(self._collect_model_param_raw_info(False)))
        self._params_raw_meta = self._collect_model_param_raw_info(True)
        if debug:
            self._dump(f"train_params_raw_meta{suffix}", to_dict(self._params_raw_meta))
        self._params_meta = self._build_params_meta()
        if debug:
            self._dump(f"train_params_meta{suffix}", dump_parameters_meta(self._params_meta))
        self.total_numel = sum(p.global_numel for p in self._params_meta)
        self.total_size = compute_total_model_size(self._params_meta)
        logger.info(f"Total number of elements in the model: {self.total_numel}, total size: {self.total_size} bytes")

    @staticmethod
    def _dump(filename: str, payload) -> None:
        path = os.path.abspath(filename)
        with open(path, "w") as f:
            json.dump(payload, f, indent=4)
        logger.info(f"debug dump written: {path}")

    def get_model_arch_name(self) -> str:
        return self._model_arch_name

    def get_parameters_meta(self) -> List[ParameterMeta]:
        return self._params_meta

    def _get_params_raw_meta(self) -> List[Dict[str, Any]]:
        return self._params_raw_meta

    def get_pp_stage_layer_id_map(self) -> Dict[Tuple[int, int], Dict[int, int]]:
        return self._pp_stage_layer_id_map

    def _collect_model_param_raw_info(self, convert_params: bool = False, **_kw) -> List[Dict[str, Any]]:
        converter = get_train_weights_converter(
            self._train_engine.engine_name, self._model_arch_name, self.hf_config, self._rank_info, self._infer_conf,
            tf_config=self._tf_config,
        )
        meta = list_local_train_params(self._mcore_model, converter, self._rank_info, self.hf_config, self._model_arch_name, convert_params)
        world = dist.get_world_size(self._group) if dist.is_initialized() else 1
        if world > 1:
            gathered: List[Any] = [None] * world
            dist.all_gather_object(gathered, meta, group=self._group)
        else:
            gathered = [meta]
        if convert_params:
            self._pp_stage_layer_id_map = build_pp_stage_layer_id_map(gathered)
            gathered = canonicalize_pp_layer_names(gathered, self._pp_stage_layer_id_map)
        else:
            self._pp_stage_layer_id_map = {}
        return gathered

    def _get_sharding_info(self, name: str, rank_info: RankInfo, param_meta: Dict[str, Any]) -> Tuple[ShardingType, int, int]:
        return self._sharding_strategy.get_sharding_strategy(name, rank_info=rank_info, param_meta=param_meta)
