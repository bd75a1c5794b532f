"""Plan a layout without weights: build shape-only models of a named
architecture, run the planner and the lowering for every training rank, and
report items, bytes per link and the time the update cannot beat.

    python -m awex_b200.debug.plan_study --model qwen3-30b-a3b --train tp1,dp8,ep8 --infer tp4,ep4,engines2 --placement colocated
    python -m awex_b200.debug.plan_study --model llama3-8b --train tp4 --infer tp2,engines2 --placement separated --layers 4

``--placement separated`` puts training ranks and inference workers on disjoint
GPUs (every byte crosses NVLink); ``colocated`` puts training rank r and
inference transfer rank r on GPU r (bytes between them stay in local memory);
``colocated-best`` chooses which inference worker shares a GPU with which
training rank so that as many bytes as possible stay local (an assignment
problem over the bytes each training rank sends to each inference worker) and
prints the pairing.
Peak rates default to what was measured on an 8xB200 box and can be overridden.
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from typing import Dict, List

import torch


def parse_layout(text: str) -> Dict[str, int]:
    out: Dict[str, int] = {}
    for part in filter(None, text.split(",")):
        key = part.rstrip("0123456789")
        if not key or key == part:
            raise SystemExit(f"cannot read layout element {part!r} (expected e.g. tp4, ep8, engines2, fp8)")
        out[key] = int(part[len(key):])
    return out


def study(model: str, train: Dict[str, int], infer: Dict[str, int], placement: str = "colocated", layers: int = 0,
          fp8: bool = False, pairing: str = "spread", nvlink_gbps: float = 770.0, hbm_gbps: float = 6540.0,
          fp8_gbps: float = 2680.0) -> Dict[str, object]:
    from awex_b200 import logging
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout
    from awex_b200.transfer.transfer_plan import TransferPlanBuilder

    logging.setLevel("WARNING")
    arch = get_arch(model)
    if layers:
        arch = arch.with_layers(layers)
    t_layout = TrainLayout(tp=train.get("tp", 1), pp=train.get("pp", 1), dp=train.get("dp", 1), ep=train.get("ep", 1), etp=train.get("etp", 1))
    i_layout = InferLayout(tp=infer.get("tp", 1), ep=infer.get("ep", 1), num_engines=infer.get("engines", 1), fp8=fp8)
    started = time.time()
    job = SimulatedJob(arch, t_layout, i_layout, dtype=torch.bfloat16, device="meta")
    skip = job.builder.skip_names
    job.builder = TransferPlanBuilder(job.infer_world_size, t_layout.world, i_layout.num_engines,
                                      replica_pairing="spread" if pairing == "local" else pairing, skip_names=skip)
    meta_s = time.time() - started
    ranks: List[Dict[str, object]] = []
    job.programs = {r: None for r in range(t_layout.world)}
    gpu_of_infer = {i: i for i in range(job.infer_world_size)}  # inference transfer rank -> GPU (= training rank it sits with)
    if placement == "colocated-best":
        import numpy as np
        from scipy.optimize import linear_sum_assignment

        n = max(t_layout.world, job.infer_world_size)
        sent = np.zeros((n, n))
        for r in range(t_layout.world):
            job.programs[r] = job.compile_send_program(r)
            for it in job.programs[r]:
                sent[r, it.dst_rank] += it.dst_bytes
        rows, cols = linear_sum_assignment(-sent)  # maximise the bytes that stay on their GPU
        gpu_of_infer = {int(i): int(r) for r, i in zip(rows, cols)}
    if pairing == "local":
        # the placement above was found with least-loaded pairing; now let every shard prefer the replica on its own GPU
        mates = gpu_of_infer if placement.startswith("colocated") else {}
        job.builder = TransferPlanBuilder(job.infer_world_size, t_layout.world, i_layout.num_engines, replica_pairing="local",
                                          skip_names=skip, colocation=mates)
        job.programs = {r: None for r in range(t_layout.world)}
    ingress = [0] * job.infer_world_size
    local_in = [0] * job.infer_world_size
    compile_s = 0.0
    for r in range(t_layout.world):
        t0 = time.time()
        items = job.programs[r] = job.programs[r] or job.compile_send_program(r)
        compile_s += time.time() - t0
        remote = local = read = quantised = 0
        for it in items:
            same_gpu = placement.startswith("colocated") and gpu_of_infer.get(it.dst_rank) == r
            if same_gpu:
                local += it.dst_bytes
                local_in[it.dst_rank] += it.dst_bytes
            else:
                remote += it.dst_bytes
                ingress[it.dst_rank] += it.dst_bytes
            read += it.numel * it.src_dtype.itemsize
            if it.value_op.kind == "fp8_block":
                quantised += it.numel * it.src_dtype.itemsize + it.dst_bytes
        ranks.append({"rank": r, "items": len(items), "destinations": len({it.dst_rank for it in items}), "read": read,
                      "remote_egress": remote, "local_written": local, "quantised_in_plus_out": quantised})
    problems = job.check_coverage()
    per_gpu_ms = {
        "nvlink_egress": max(x["remote_egress"] for x in ranks) / (nvlink_gbps * 1e9) * 1e3,
        "nvlink_ingress": max(ingress) / (nvlink_gbps * 1e9) * 1e3,
        "hbm": max((x["read"] + x["local_written"]) for x in ranks) / (hbm_gbps * 1e9) * 1e3,
        "quantisation_at_measured_rate": max(x["quantised_in_plus_out"] for x in ranks) / (fp8_gbps * 1e9) * 1e3,
    }
    bound = max(per_gpu_ms, key=per_gpu_ms.get)
    return {
        "model": arch.name, "train": t_layout.label(), "infer": i_layout.label(), "placement": placement, "pairing": pairing,
        "gpu_of_inference_rank": gpu_of_infer,
        "parameters": arch.param_count(), "coverage_problems": problems[:5], "senders": ranks,
        "ingress_per_inference_rank": ingress, "bound_ms": per_gpu_ms, "bound": bound, "lower_bound_ms": per_gpu_ms[bound],
        "host_seconds": {"metadata_all_ranks": round(meta_s, 2), "plan_and_lowering_per_rank": round(compile_s / max(t_layout.world, 1), 2)},
        "rates_GBps": {"nvlink": nvlink_gbps, "hbm": hbm_gbps, "fp8_in_plus_out": fp8_gbps},
    }


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--train", default="tp1", help="e.g. tp4 or tp1,dp8,ep8 or tp2,pp2")
    ap.add_argument("--infer", default="tp1", help="e.g. tp2,engines2 or tp4,ep4,engines2")
    ap.add_argument("--fp8", action="store_true", help="inference side serves block-scaled fp8")
    ap.add_argument("--placement", default="colocated", choices=["colocated", "colocated-best", "separated"])
    ap.add_argument("--pairing", default="spread", choices=["spread", "round_robin", "local"])
    ap.add_argument("--layers", type=int, default=0, help="truncate the model (quick look)")
    ap.add_argument("--nvlink-gbps", type=float, default=770.0)
    ap.add_argument("--hbm-gbps", type=float, default=6540.0)
    ap.add_argument("--json", action="store_true", help="print the full report as JSON")
    args = ap.parse_args(argv)
    report = study(args.model, parse_layout(args.train), parse_layout(args.infer), args.placement, args.layers, args.fp8,
                   args.pairing, args.nvlink_gbps, args.hbm_gbps)
    if args.json:
        print(json.dumps(report, indent=2))
        return 0
    gb = lambda b: f"{b / 1e9:8.3f}"  # noqa: E731
    print(f"{report['model']}: training {report['train']} -> inference {report['infer']} ({report['placement']}, pairing {report['pairing']})")
    print(" rank  items  dests   read GB  egress GB   local GB")
    for x in report["senders"]:
        print(f"{x['rank']:5d} {x['items']:6d} {x['destinations']:6d} {gb(x['read'])} {gb(x['remote_egress'])}  {gb(x['local_written'])}")
    if report["placement"] == "colocated-best":
        print("inference transfer rank -> GPU (training rank it shares):", report["gpu_of_inference_rank"])
    print("ingress GB per inference rank:", [round(b / 1e9, 3) for b in report["ingress_per_inference_rank"]])
    print("lower bounds (ms):", {k: round(v, 2) for k, v in report["bound_ms"].items()}, "->", report["bound"])
    print("host seconds:", report["host_seconds"], "coverage problems:", report["coverage_problems"])
    return 1 if report["coverage_problems"] else 0


if __name__ == "__main__":
    sys.exit(main())
