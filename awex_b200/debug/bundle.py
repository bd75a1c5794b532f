"""Run the metadata and the plan analysis over one directory of debug-mode dumps
(`awex/tests/experimental/analyze_awex_debug_bundle.py` in the reference).

    python -m awex_b200.debug.bundle DIR [--strict] [--json out.json]
"""

from __future__ import annotations

import argparse
import glob
import json
import os
import sys
from typing import Any, Dict

from awex_b200.debug import meta_dumps, plan_dumps


def _latest(directory: str, pattern: str):
    found = sorted(glob.glob(os.path.join(directory, pattern)), key=os.path.getmtime)
    return found[-1] if found else None


def analyze_bundle(directory: str, strict_key_match: bool = False) -> Dict[str, Any]:
    report: Dict[str, Any] = {"directory": os.path.abspath(directory)}
    train, infer = _latest(directory, "train_params_meta_*.json"), _latest(directory, "infer_params_meta_*.json")
    if train and infer:
        report["meta"] = meta_dumps.analyze_meta(meta_dumps.load_meta(train), meta_dumps.load_meta(infer), strict_key_match)
        report["meta"]["files"] = [train, infer]
    else:
        report["meta"] = {"skipped": "need one train_params_meta_*.json and one infer_params_meta_*.json"}
    report["plans"] = plan_dumps.analyze_files([directory])
    critical = report["meta"].get("summary", {}).get("critical_errors", 0) + len(report["plans"]["problems"])
    report["critical_errors"] = critical
    return report


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("directory")
    ap.add_argument("--strict", action="store_true")
    ap.add_argument("--json")
    args = ap.parse_args(argv)
    report = analyze_bundle(args.directory, args.strict)
    print(json.dumps({"critical_errors": report["critical_errors"], "meta": report["meta"].get("summary", report["meta"]),
                      "plans": {k: v for k, v in report["plans"].items() if k != "files"}}, indent=2))
    if args.json:
        with open(args.json, "w") as f:
            json.dump(report, f, indent=2)
    return 1 if report["critical_errors"] else 0


if __name__ == "__main__":
    sys.exit(main())
