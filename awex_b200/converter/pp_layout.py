"""Pipeline-parallel layer numbering.

A Megatron pipeline stage numbers its decoder layers locally; canonical names
use global layer ids.  Two sources give the local->global map:

* the map built from the all-gathered training metadata and handed to the
  converter as ``train_pp_stage_layer_id_map`` (keys ``(pp_rank, vp_stage)`` or
  ``"pp:vp"`` strings), used at transfer time;
* an analytic layout from the Megatron config (even split, explicit first/last
  stage sizes, embedding/loss accounted as layers, or an explicit
  ``pipeline_model_parallel_layout``), mirroring what the reference accepts
  (`awex/converter/mcore_converter.py:48-364`).

Stage order for global numbering is virtual stage outermost, pipeline rank
innermost (Megatron's interleaved schedule).
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

from awex_b200.utils.common import cfg_get

StageKey = Tuple[int, int]


def normalize_pp_stage_layer_id_map(raw_map: Optional[Dict]) -> Dict[StageKey, Dict[int, int]]:
    out: Dict[StageKey, Dict[int, int]] = {}
    for key, layers in (raw_map or {}).items():
        if isinstance(key, tuple) and len(key) == 2:
            stage = (int(key[0]), int(key[1]))
        elif isinstance(key, str) and ":" in key:
            pp, vp = key.split(":", 1)
            stage = (int(pp), int(vp))
        elif isinstance(key, str):
            raise ValueError(f"Invalid pp stage map key, expected '<pp_rank>:<vp_stage>': {key}")
        else:
            raise ValueError(f"Unsupported pp stage map key type: {type(key)}")
        if not isinstance(layers, dict):
            raise ValueError(f"Invalid pp stage map value, expected dict: key={key}, value_type={type(layers)}")
        out[stage] = {int(local): int(glob) for local, glob in layers.items()}
    return out


def _is_decoder_entry(entry) -> bool:
    label = str(getattr(entry, "name", entry)).strip().lower()
    return label in ("decoder", "t") or label.endswith(".decoder")


def stage_counts_from_layout(pipeline_layout, pp_size: int) -> List[List[int]]:
    """``counts[pp_rank][vp_stage]`` of decoder layers from an explicit layout,
    given either as ``[pp][vp][layers]`` or as a flat list of stages in
    schedule order (``stage = vp * pp_size + pp_rank``)."""
    layout = getattr(pipeline_layout, "layout", pipeline_layout)
    if not isinstance(layout, list) or not layout:
        raise ValueError("pipeline_model_parallel_layout must be a non-empty list")
    if not isinstance(layout[0], list):
        raise ValueError("pipeline_model_parallel_layout must contain stage layer lists")
    nested = bool(layout[0]) and isinstance(layout[0][0], list)
    if not nested:
        if len(layout) % pp_size != 0:
            raise ValueError(
                f"pipeline_model_parallel_layout stage count must be divisible by pp_size: stages={len(layout)}, pp_size={pp_size}"
            )
        vp = len(layout) // pp_size
        layout = [[layout[v * pp_size + p] for v in range(vp)] for p in range(pp_size)]
    if len(layout) != pp_size:
        raise ValueError(f"pipeline_model_parallel_layout pp dimension mismatch: layout_pp={len(layout)}, pp_size={pp_size}")
    vp = len(layout[0])
    if vp == 0:
        raise ValueError("pipeline_model_parallel_layout has empty vp dimension")
    if any(len(row) != vp for row in layout):
        raise ValueError("pipeline_model_parallel_layout has inconsistent vp dimension across pp ranks")
    return [[sum(1 for e in stage if _is_decoder_entry(e)) for stage in row] for row in layout]


def stage_counts_from_split_config(num_hidden_layers: int, pp_size: int, tf_config) -> List[List[int]]:
    first = cfg_get(tf_config, "num_layers_in_first_pipeline_stage")
    last = cfg_get(tf_config, "num_layers_in_last_pipeline_stage")
    embed_counts = bool(cfg_get(tf_config, "account_for_embedding_in_pipeline_split", False))
    loss_counts = bool(cfg_get(tf_config, "account_for_loss_in_pipeline_split", False))
    vp_cfg = cfg_get(tf_config, "virtual_pipeline_model_parallel_size")
    vp = int(vp_cfg) if vp_cfg is not None and pp_size > 1 else 1
    if vp <= 0:
        raise ValueError(f"virtual_pipeline_model_parallel_size must be positive, got {vp}")
    uneven = first is not None or last is not None
    if uneven and (embed_counts or loss_counts):
        raise ValueError(
            "num_layers_in_first/last_pipeline_stage cannot be mixed with account_for_embedding/loss_in_pipeline_split"
        )
    if uneven:
        for label, val in (("first", first), ("last", last)):
            if val is not None and int(val) <= 0:
                raise ValueError(f"num_layers_in_{label}_pipeline_stage must be positive, got {val}")
        n_first, n_last = int(first or 0), int(last or 0)
        middle_total = num_hidden_layers - n_first - n_last
        middle_ranks = pp_size - (first is not None) - (last is not None)
        if middle_total < 0:
            raise ValueError(
                "Invalid uneven pipeline setup: specified first/last layers exceed total layers "
                f"(total={num_hidden_layers}, first={n_first}, last={n_last})"
            )
        if middle_ranks > 0 and middle_total % middle_ranks != 0:
            raise ValueError(
                f"Uneven pipeline middle layers must be divisible by middle pp size: middle_layers={middle_total}, middle_pp_size={middle_ranks}"
            )
        each = middle_total // middle_ranks if middle_ranks > 0 else 0
        per_rank = [each] * pp_size
        if first is not None:
            per_rank[0] = n_first
        if last is not None:
            per_rank[-1] = n_last
    else:
        effective = num_hidden_layers + int(embed_counts) + int(loss_counts)
        if effective % pp_size != 0:
            raise ValueError(
                "PP split is not divisible under account_for_embedding/loss settings: "
                f"effective_layers={effective}, pp_size={pp_size}, num_hidden_layers={num_hidden_layers}, "
                f"account_for_embedding={embed_counts}, account_for_loss={loss_counts}"
            )
        per_rank = [effective // pp_size] * pp_size
    counts = []
    for p, n in enumerate(per_rank):
        if vp > 1 and n % vp != 0:
            raise ValueError(f"Layers per pp rank must be divisible by virtual pipeline size: pp_rank={p}, layers={n}, vp_size={vp}")
        counts.append([n // vp] * vp if vp > 1 else [n])
    if embed_counts:
        counts[0][0] -= 1
    if loss_counts:
        counts[-1][-1] -= 1
    for p, row in enumerate(counts):
        for v, n in enumerate(row):
            if n < 0:
                raise ValueError(f"Negative decoder layer count after account_for_* adjustment: pp_rank={p}, vp_stage={v}, count={n}")
    return counts


def resolve_pp_stage_global_layer_ids(rank_info, hf_config, tf_config, vp_stage: Optional[int] = None) -> List[int]:
    """Global ids of the decoder layers held by (``rank_info.pp_rank``, ``vp_stage``)."""
    n_layers = getattr(hf_config, "num_hidden_layers", None)
    if n_layers is None:
        n_layers = cfg_get(tf_config, "num_layers")
    if n_layers is None:
        raise ValueError("num_hidden_layers is required for PP layer mapping (missing in hf_config and tf_config)")
    n_layers = int(n_layers)
    pp_size, pp_rank = max(int(rank_info.pp_size), 1), int(rank_info.pp_rank)
    if not 0 <= pp_rank < pp_size:
        raise ValueError(f"Invalid pp_rank={pp_rank} for pp_size={pp_size}")
    layout = cfg_get(tf_config, "pipeline_model_parallel_layout")
    counts = stage_counts_from_layout(layout, pp_size) if layout is not None else stage_counts_from_split_config(n_layers, pp_size, tf_config)
    vp_size = len(counts[0])
    vp = 0 if vp_stage is None else int(vp_stage)
    if not 0 <= vp < vp_size:
        raise ValueError(f"Invalid vp_stage={vp} for vp_size={vp_size}, pp_rank={pp_rank}")
    total = sum(map(sum, counts))
    if total != n_layers:
        raise ValueError(
            f"Resolved PP stage layer counts do not match num_hidden_layers: resolved_total={total}, "
            f"num_hidden_layers={n_layers}, pp_size={pp_size}, stage_counts={counts}"
        )
    before = sum(counts[p][v] for v in range(vp_size) for p in range(pp_size) if (v, p) < (vp, pp_rank))
    return list(range(before, before + counts[pp_rank][vp]))


def process_mcore_pp_name(name: str, rank_info, hf_config=None, tf_config=None, vp_stage: Optional[int] = None,
                          pp_stage_layer_id_map: Optional[Dict[StageKey, Dict[int, int]]] = None) -> str:
    """Rewrite ``...layers.<local>.rest`` to ``...layers.<global>.rest`` using
    the stage map; names without a layer index, or calls without a map, pass
    through unchanged."""
    if ".layers." not in name and not name.startswith("layers."):
        return name
    if not pp_stage_layer_id_map:
        return name
    head, tail = name.rsplit("layers.", 1)
    local_txt, _, rest = tail.partition(".")
    local = int(local_txt)
    vp = 0 if vp_stage is None else int(vp_stage)
    layer_map = pp_stage_layer_id_map.get((int(rank_info.pp_rank), vp))
    if layer_map is None:
        raise ValueError(f"Missing pp stage layer map for current rank/stage: pp_rank={rank_info.pp_rank}, vp_stage={vp}, name={name}")
    if local not in layer_map:
        raise ValueError(
            f"Local layer id missing in pp stage layer map: local_layer_id={local}, pp_rank={rank_info.pp_rank}, "
            f"pp_size={rank_info.pp_size}, vp_stage={vp}, known_local_ids={sorted(layer_map)}, name={name}"
        )
    return f"{head}layers.{layer_map[local]}.{rest}"
