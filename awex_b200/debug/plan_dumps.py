"""Check transfer-plan dumps (``local_communication_plan_{train,infer}_<rank>_<pid>.json``
and ``global_communication_plan_*.json``, written by the plan builder in debug
mode):

* every operation stays inside its sending and its receiving shard;
* what a receiving rank is sent tiles each of its shards exactly once (an exact
  box cover, not only a sum of element counts: two overlapping operations cannot
  hide a gap; cf. `awex/tests/experimental/analyze_transfer_plan_dumps.py:161-184`);
* when both sides' local dumps are given, each (sender, receiver) pair lists the
  same operations.

    python -m awex_b200.debug.plan_dumps DIR_OR_FILES... [--json out.json]
"""

from __future__ import annotations

import argparse
import glob
import json
import os
import sys
from typing import Any, Dict, Iterable, List, Tuple

from awex_b200.transfer.lowering import _cover_problems


def load_operations(path: str) -> List[Dict[str, Any]]:
    """Operations of one dump file, whichever of the two layouts it has."""
    with open(path) as f:
        data = json.load(f)
    if isinstance(data, dict):  # local plan: peer -> operations
        return [op for ops in data.values() for op in ops]
    return list(data)


def _op_id(op: Dict[str, Any]) -> Tuple:
    return (op["send_rank"], op["recv_rank"], op["send_shard_meta"]["name"], tuple(op["send_offset"]), tuple(op["recv_offset"]),
            tuple(op["overlap_shape"]))


def bounds_problems(op: Dict[str, Any]) -> List[str]:
    out = []
    for side, offset_key in (("send", "send_offset"), ("recv", "recv_offset")):
        shard = op[f"{side}_shard_meta"]
        shape, offset, extent = shard["shape"], op[offset_key], op["overlap_shape"]
        if not (len(shape) == len(offset) == len(extent)):
            out.append(f"{side} side of {shard['name']}: rank mismatch shape={shape} offset={offset} extent={extent}")
        elif any(o < 0 or e <= 0 or o + e > d for o, e, d in zip(offset, extent, shape)):
            out.append(f"{side} side of {shard['name']} ({op['send_rank']}->{op['recv_rank']}): box offset={offset} extent={extent} leaves shard {shape}")
    if op["send_shard_meta"]["name"] != op["recv_shard_meta"]["name"]:
        out.append(f"operation joins {op['send_shard_meta']['name']} to {op['recv_shard_meta']['name']}")
    return out


def analyze_operations(ops: Iterable[Dict[str, Any]], receivers: Iterable[int] = ()) -> Dict[str, Any]:
    """``receivers``: ranks whose complete receive plan is in ``ops`` (coverage is
    only meaningful for those)."""
    ops = list({_op_id(op): op for op in ops}.values())
    problems: List[str] = []
    for op in ops:
        problems.extend(bounds_problems(op))
    receivers = set(receivers)
    per_shard: Dict[Tuple[int, str], Dict[str, Any]] = {}
    for op in ops:
        if op["recv_rank"] in receivers:
            entry = per_shard.setdefault((op["recv_rank"], op["recv_shard_meta"]["name"]), {"shape": tuple(op["recv_shard_meta"]["shape"]), "boxes": []})
            entry["boxes"].append((tuple(op["recv_offset"]), tuple(op["overlap_shape"]), f"from {op['send_rank']}"))
    for (rank, name), entry in sorted(per_shard.items()):
        in_bounds = [b for b in entry["boxes"] if len(b[0]) == len(entry["shape"]) and all(o >= 0 and o + e <= d for o, e, d in zip(b[0], b[1], entry["shape"]))]
        problems.extend(f"receiver {rank}: {p}" for p in _cover_problems(name, entry["shape"], in_bounds))
    return {"operations": len(ops), "receivers_checked": sorted(receivers), "shards_checked": len(per_shard), "problems": problems}


def _side_and_rank(path: str):
    parts = os.path.basename(path).split("_")
    try:
        i = parts.index("plan")
        return parts[0], parts[i + 1], int(parts[i + 2])
    except (ValueError, IndexError):
        return None, None, None


def analyze_files(paths: Iterable[str]) -> Dict[str, Any]:
    files = []
    for p in paths:
        files.extend(sorted(glob.glob(os.path.join(p, "*communication_plan_*.json"))) if os.path.isdir(p) else [p])
    ops: List[Dict[str, Any]] = []
    receivers, by_pair = set(), {"train": {}, "infer": {}}
    for path in files:
        scope, side, rank = _side_and_rank(path)
        loaded = load_operations(path)
        ops.extend(loaded)
        if scope == "local" and side in by_pair:
            for op in loaded:
                by_pair[side].setdefault((op["send_rank"], op["recv_rank"]), set()).add(_op_id(op))
            if side == "infer":
                receivers.add(rank)
    report = analyze_operations(ops, receivers)
    for pair in sorted(set(by_pair["train"]) & set(by_pair["infer"])):
        if by_pair["train"][pair] != by_pair["infer"][pair]:
            report["problems"].append(f"sender {pair[0]} and receiver {pair[1]} disagree on their operations "
                                      f"({len(by_pair['train'][pair])} vs {len(by_pair['infer'][pair])})")
    report["files"] = files
    return report


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("paths", nargs="+", help="dump files or directories that contain them")
    ap.add_argument("--json", help="write the report here")
    args = ap.parse_args(argv)
    report = analyze_files(args.paths)
    print(json.dumps({k: v for k, v in report.items() if k != "files"}, indent=2))
    if args.json:
        with open(args.json, "w") as f:
            json.dump(report, f, indent=2)
    return 1 if report["problems"] else 0


if __name__ == "__main__":
    sys.exit(main())
