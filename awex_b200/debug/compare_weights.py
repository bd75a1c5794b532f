"""Compare two sources of named tensors and report missing names, shape, dtype
and value mismatches.

A source is a directory of safetensors files (an HF checkpoint or a dump made
with :func:`dump_named_tensors`), a ``.pt`` file holding a ``{name: tensor}``
dict, or an in-memory mapping.  Typical uses, which the reference covers with
three scripts (`awex/tests/experimental/compare_megatron_vllm_weights.py`,
`compare_megatron_vllm_weights_multi.py`, `compare_vllm_sglang_weights.py`):

* training side vs inference side: every training rank dumps the canonical
  tensors its converter produces (:func:`dump_converted_training_shards`), every
  inference worker dumps its canonical views
  (:func:`dump_converted_inference_shards`); :func:`assemble_from_shards` glues
  the shards back with the published metadata and the two full models are
  compared;
* vLLM vs SGLang: dump both engines' canonical views and compare.

    python -m awex_b200.debug.compare_weights LEFT RIGHT [--atol 0 --rtol 0] [--json report.json]
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Any, Dict, Iterable, Mapping, Optional, Sequence

import torch


# ---- sources ---------------------------------------------------------------------------------------
def load_named_tensors(source) -> Dict[str, torch.Tensor]:
    if isinstance(source, Mapping):
        return dict(source)
    if os.path.isdir(source):
        from awex_b200.utils.safetensors_io import load_checkpoint

        return load_checkpoint(source)
    if str(source).endswith(".pt"):
        data = torch.load(source, map_location="cpu", weights_only=True)
        if not isinstance(data, dict):
            raise ValueError(f"{source} does not hold a dict of tensors")
        return data
    raise ValueError(f"do not know how to read tensors from {source!r}")


def dump_named_tensors(path: str, tensors: Mapping[str, torch.Tensor]) -> None:
    from awex_b200.utils.safetensors_io import save_checkpoint

    save_checkpoint(path, {k: v.detach().cpu().contiguous() for k, v in tensors.items()})


def dump_converted_training_shards(path: str, models, converter, rank_info) -> str:
    """This training rank's canonical tensors (after its converter) under
    ``path/train_rank_<global rank>``."""
    from awex_b200.converter.mcore_converter import get_mcore_model_parameters

    out: Dict[str, torch.Tensor] = {}
    for vp, chunk in enumerate(models if isinstance(models, (list, tuple)) else [models]):
        for name, p in get_mcore_model_parameters(chunk).items():
            for cname, tensor in converter.convert_param(name, p.detach(), vp_stage=vp):
                out[cname] = tensor
    target = os.path.join(path, f"train_rank_{rank_info.global_rank}")
    dump_named_tensors(target, out)
    return target


def dump_converted_inference_shards(path: str, model, converter, model_context: dict, engine_rank: int = 0) -> str:
    from awex_b200.meta.infer_meta_resolver import canonical_named_views

    target = os.path.join(path, f"infer_engine_{engine_rank}_rank_{model_context.get('global_rank', 0)}")
    dump_named_tensors(target, dict(canonical_named_views(model, converter, model_context)))
    return target


def assemble_from_shards(params_meta: Sequence, shard_tensors: Mapping[int, Mapping[str, torch.Tensor]], engine_rank: Optional[int] = None
                         ) -> Dict[str, torch.Tensor]:
    """Full tensors from per-rank shards, placed by the metadata's global
    offsets (first replica).  ``shard_tensors`` maps global rank -> name -> shard."""
    out: Dict[str, torch.Tensor] = {}
    for meta in params_meta:
        full = torch.zeros(meta.global_shape, dtype=meta.dtype)
        for s in meta.replicas[0].shards:
            if engine_rank is not None and s.engine_rank != engine_rank:
                continue
            piece = shard_tensors[s.global_rank][meta.name]
            full[tuple(slice(o, o + n) for o, n in zip(s.global_offset, s.shape))] = piece.to(full.dtype)
        out[meta.name] = full
    return out


# ---- comparison -----------------------------------------------------------------------------------
def compare_named_tensors(left: Mapping[str, torch.Tensor], right: Mapping[str, torch.Tensor], atol: float = 0.0, rtol: float = 0.0,
                          ignore: Iterable[str] = (), max_listed: int = 50) -> Dict[str, Any]:
    ignore = tuple(ignore)
    skip = lambda n: any(pat in n for pat in ignore)  # noqa: E731
    lk, rk = {k for k in left if not skip(k)}, {k for k in right if not skip(k)}
    shape, dtype, value = [], [], []
    for name in sorted(lk & rk):
        a, b = left[name], right[name]
        if tuple(a.shape) != tuple(b.shape):
            shape.append({"name": name, "left": list(a.shape), "right": list(b.shape)})
            continue
        if a.dtype != b.dtype:
            dtype.append({"name": name, "left": str(a.dtype), "right": str(b.dtype)})
        af, bf = a.detach().float().cpu(), b.detach().float().cpu()
        if atol == 0.0 and rtol == 0.0:
            bad = af != bf
            bad &= ~(torch.isnan(af) & torch.isnan(bf))
        else:
            bad = ~torch.isclose(af, bf, atol=atol, rtol=rtol, equal_nan=True)
        n_bad = int(bad.sum())
        if n_bad:
            diff = (af - bf).abs()
            value.append({"name": name, "mismatched": n_bad, "numel": a.numel(), "max_abs": float(diff.max()),
                          "first_index": bad.nonzero()[0].tolist()})
    report = {
        "summary": {"left": len(lk), "right": len(rk), "common": len(lk & rk), "missing_on_right": len(lk - rk),
                    "missing_on_left": len(rk - lk), "shape_mismatch": len(shape), "dtype_mismatch": len(dtype),
                    "value_mismatch": len(value), "atol": atol, "rtol": rtol},
        "missing_on_right": sorted(lk - rk)[:max_listed], "missing_on_left": sorted(rk - lk)[:max_listed],
        "shape_mismatch": shape[:max_listed], "dtype_mismatch": dtype[:max_listed], "value_mismatch": value[:max_listed],
    }
    s = report["summary"]
    report["ok"] = not (s["missing_on_right"] or s["missing_on_left"] or s["shape_mismatch"] or s["dtype_mismatch"] or s["value_mismatch"])
    return report


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("left")
    ap.add_argument("right")
    ap.add_argument("--atol", type=float, default=0.0)
    ap.add_argument("--rtol", type=float, default=0.0)
    ap.add_argument("--ignore", action="append", default=[], help="skip names containing this text (repeatable)")
    ap.add_argument("--json")
    args = ap.parse_args(argv)
    report = compare_named_tensors(load_named_tensors(args.left), load_named_tensors(args.right), args.atol, args.rtol, args.ignore)
    print(json.dumps(report["summary"], indent=2))
    if args.json:
        with open(args.json, "w") as f:
            json.dump(report, f, indent=2)
    return 0 if report["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
