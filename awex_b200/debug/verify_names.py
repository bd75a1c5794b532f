"""Check that the canonical names an inference-side converter produces exist in
a Hugging Face checkpoint (by its safetensors index), i.e. that the name contract
between engine layout and checkpoint layout holds for a model
(`awex/tests/experimental/verify_weight_conversion.py` in the reference).

    python -m awex_b200.debug.verify_names CHECKPOINT_DIR --engine vllm --arch Qwen3ForCausalLM --names names.txt
"""

from __future__ import annotations

import argparse
import json
import sys
from typing import Dict, Iterable, List

from awex_b200.utils.safetensors_io import checkpoint_weight_map

# fused engine tensors are views of several checkpoint tensors
_FUSED = {
    "attention.query_key_value_proj": ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"],
    "self_attn.qkv_proj": ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"],
    "mlp.gate_up_proj": ["mlp.gate_proj", "mlp.up_proj"],
    "attention.dense": ["self_attn.o_proj"],
    "attention.query_layernorm": ["self_attn.q_norm"],
    "attention.key_layernorm": ["self_attn.k_norm"],
}


def checkpoint_equivalents(canonical_name: str) -> List[str]:
    """Checkpoint names that a canonical name stands for."""
    for fused, parts in _FUSED.items():
        if fused in canonical_name:
            return [canonical_name.replace(fused, part) for part in parts]
    return [canonical_name]


def verify_names(canonical_names: Iterable[str], checkpoint_names: Iterable[str]) -> Dict[str, object]:
    have = set(checkpoint_names)
    missing, found = [], 0
    for name in canonical_names:
        if name.endswith("_scale_inv"):
            continue  # produced by quantisation, not stored in a bf16 checkpoint
        wanted = checkpoint_equivalents(name)
        absent = [w for w in wanted if w not in have]
        if absent:
            missing.append({"canonical": name, "absent": absent})
        else:
            found += 1
    return {"checked": found + len(missing), "found": found, "missing": missing, "ok": not missing}


def canonical_names_of(model, converter, model_context=None) -> List[str]:
    from awex_b200.meta.infer_meta_resolver import canonical_named_views

    return [name for name, _ in canonical_named_views(model, converter, model_context)]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("checkpoint")
    ap.add_argument("--names", required=True, help="text file with one canonical name per line")
    ap.add_argument("--json")
    args = ap.parse_args(argv)
    with open(args.names) as f:
        names = [line.strip() for line in f if line.strip()]
    report = verify_names(names, checkpoint_weight_map(args.checkpoint))
    print(json.dumps({k: v for k, v in report.items() if k != "missing"} | {"missing_count": len(report["missing"])}, indent=2))
    if args.json:
        with open(args.json, "w") as f:
            json.dump(report, f, indent=2)
    return 0 if report["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
