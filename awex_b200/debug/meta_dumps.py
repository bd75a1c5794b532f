"""Compare a training-side and an inference-side metadata dump
(``*_params_meta_*.json`` written in debug mode by the resolvers, i.e. the output
of ``dump_parameters_meta``): key sets under the alias rule, global shape / dtype
/ element count per common key, the TP divisibility rule and differing sharding
types (`awex/tests/experimental/analyze_meta_dumps.py:66-170` in the reference).

    python -m awex_b200.debug.meta_dumps train_params_meta_*.json infer_params_meta_*.json [--strict] [--json out.json]
"""

from __future__ import annotations

import argparse
import json
import sys
from typing import Any, Dict, List

from awex_b200.utils.common import is_allowed_infer_only_alias


def load_meta(path: str) -> List[Dict[str, Any]]:
    with open(path) as f:
        data = json.load(f)
    if not isinstance(data, list) or any("name" not in item for item in data):
        raise ValueError(f"{path} is not a parameter metadata dump (a list of objects with a 'name')")
    return data


def _first_replica_shards(item: Dict[str, Any]) -> List[Dict[str, Any]]:
    replicas = item.get("replicas") or []
    return list((replicas[0] or {}).get("shards") or []) if replicas else []


def tp_size_of(item: Dict[str, Any]) -> int:
    return len(_first_replica_shards(item))


def sharding_types_of(item: Dict[str, Any]) -> List[str]:
    return sorted({str(s.get("sharding_type")) for r in item.get("replicas") or [] for s in (r or {}).get("shards") or []})


def analyze_meta(train_meta: List[Dict[str, Any]], infer_meta: List[Dict[str, Any]], strict_key_match: bool = False) -> Dict[str, Any]:
    train, infer = {i["name"]: i for i in train_meta}, {i["name"]: i for i in infer_meta}
    tk, ik = set(train), set(infer)
    missing, extra = sorted(tk - ik), sorted(ik - tk)
    bad_extra = [k for k in extra if not is_allowed_infer_only_alias(k, ik, tk)]
    shape, dtype, numel, tp_rule, kinds = [], [], [], [], []
    for name in sorted(tk & ik):
        t, i = train[name], infer[name]
        if list(t.get("global_shape") or []) != list(i.get("global_shape") or []):
            shape.append((name, t.get("global_shape"), i.get("global_shape")))
        if t.get("dtype") != i.get("dtype"):
            dtype.append((name, t.get("dtype"), i.get("dtype")))
        if t.get("global_numel") != i.get("global_numel"):
            numel.append((name, t.get("global_numel"), i.get("global_numel")))
        a, b = tp_size_of(t), tp_size_of(i)
        if a and b and max(a, b) % min(a, b):
            tp_rule.append((name, a, b))
        if sharding_types_of(t) != sharding_types_of(i):
            kinds.append((name, sharding_types_of(t), sharding_types_of(i)))
    key_error = bool(missing or (extra if strict_key_match else bad_extra))
    critical = int(key_error) + len(shape) + len(dtype) + len(numel) + len(tp_rule)
    return {
        "summary": {
            "train_params": len(train), "infer_params": len(infer), "common_params": len(tk & ik),
            "missing_on_infer_count": len(missing), "extra_on_infer_count": len(extra),
            "unsupported_extra_on_infer_count": len(bad_extra), "shape_mismatch_count": len(shape),
            "dtype_mismatch_count": len(dtype), "numel_mismatch_count": len(numel), "tp_rule_violation_count": len(tp_rule),
            "sharding_type_diff_count": len(kinds), "critical_errors": critical, "strict_key_match": strict_key_match,
        },
        "missing_on_infer": missing, "extra_on_infer": extra, "unsupported_extra_on_infer": bad_extra,
        "shape_mismatch": shape, "dtype_mismatch": dtype, "numel_mismatch": numel, "tp_rule_violations": tp_rule,
        "sharding_type_diff": kinds,
    }


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("train_meta")
    ap.add_argument("infer_meta")
    ap.add_argument("--strict", action="store_true", help="inference keys must equal training keys")
    ap.add_argument("--json", help="write the full report here")
    args = ap.parse_args(argv)
    report = analyze_meta(load_meta(args.train_meta), load_meta(args.infer_meta), args.strict)
    print(json.dumps(report["summary"], indent=2))
    if args.json:
        with open(args.json, "w") as f:
            json.dump(report, f, indent=2)
    return 1 if report["summary"]["critical_errors"] else 0


if __name__ == "__main__":
    sys.exit(main())
