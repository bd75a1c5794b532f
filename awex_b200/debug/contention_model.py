"""A fluid model of one update on an NVSwitch box: who is slowed down by whom.

    python -m awex_b200.debug.contention_model --model llama3-8b --train tp4 --infer tp2,engines2 --placement separated
    python -m awex_b200.debug.contention_model --model qwen3-30b-a3b --train tp1,dp8,ep8 --infer tp4,ep4,engines2

Every sender's kernel is a set of CTAs that walk the sender's table of copy
items; a CTA moves bytes at the rate its tile kind allows, all CTAs of a GPU
share the GPU's NVLink egress, all CTAs writing to one GPU share that GPU's
NVLink ingress, and everything a GPU reads or writes locally shares its memory
bandwidth.  Rates are max-min fair under those limits and are re-solved every
time step.  What differs between the orders compared here is only which part of
the table each CTA walks:

* ``contiguous``: CTA j owns the j-th of G equal byte ranges;
* ``chunks``: chunks of the table are dealt round-robin, so all CTAs work inside
  one narrow window of the table;
* ``striped``: the table is first re-ordered by :func:`stripe_by_destination`
  (every window feeds all destinations), then dealt in chunks;
* ``rotated``: chunks, but sender r starts its walk at its (r mod n)-th
  destination, so that senders with equal tables take turns at each receiver.

The model has no launch or flag latency and no per-tile overheads: it explains
ratios (two senders meeting at one receiver run at half rate), not microseconds.
On the 8-GPU measurements it was checked against it gives, model / measured in
ms: Llama-3-8B separated 10.4 / 12.2 with contiguous ranges and 20.9 / 21.7
with chunks; Qwen3-30B-A3B co-located (modulo replica pairing) 23.1 / 28.2 and
39.7 / 41.9.  Measured times are 1.17 to 1.22 times the model's where the links
are the bound (links run at 0.82 to 0.86 of their copy rate under many writers).
Striped orders can resonate: a stripe of 8 chunks with 148 CTAs makes CTAs
alternate between two receivers in step and costs 20%; stripes of 2 chunks (CTAs
pinned to one receiver each) or of 32 and more (no common period) do not.
Rotation by rank only helps while all senders have the same destination set: in
the Llama layout two senders also hold a few replicated norm weights for a third
receiver, their rotation lands on the neighbour's first receiver, and that pair
runs at half rate (20.9 ms) while the other pair is done in 10.4 ms.
"""

from __future__ import annotations

import argparse
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np

# per-CTA rates in source bytes per second, from the single-GPU micro-benchmarks (148 CTAs):
# plain copies 6.42 TB/s read + written, block fp8 2.68 TB/s in + out, casts 1.59 TB/s
CTA_RATE = {"copy": 6.42e12 / 2 / 148, "fp8_block": 2.68e12 * (2 / 3) / 148, "cast": 1.59e12 / 3 / 148}


def segments_of(items: Sequence, gpu_of_dst: Dict[int, int]) -> np.ndarray:
    """One row per item: (destination GPU, source bytes, wire bytes per source byte, per-CTA rate)."""
    rows = np.zeros((len(items), 4))
    for i, it in enumerate(items):
        src = it.numel * it.src_dtype.itemsize
        kind = "fp8_block" if it.value_op.kind == "fp8_block" else ("copy" if it.src_dtype == it.dst_dtype and it.value_op.kind == "none" else "cast")
        rows[i] = (gpu_of_dst[it.dst_rank], max(src, 1), it.dst_bytes / max(src, 1), CTA_RATE[kind])
    return rows


def _fair_rates(cap: np.ndarray, groups: List[Tuple[np.ndarray, np.ndarray, np.ndarray]]) -> np.ndarray:
    """Max-min fair rates.  ``cap``: per-agent ceiling.  ``groups``: (index of the
    shared resource per agent or -1, weight per agent, capacity per resource)."""
    n = cap.shape[0]
    rate = np.zeros(n)
    free = cap > 0
    for _ in range(64):
        if not free.any():
            break
        step = np.min(cap[free] - rate[free])
        tight = []
        for idx, w, capacity in groups:
            member = free & (idx >= 0)
            if not member.any():
                tight.append(None)
                continue
            used = np.bincount(idx[idx >= 0], weights=(rate * w)[idx >= 0], minlength=capacity.shape[0])
            grow = np.bincount(idx[member], weights=w[member], minlength=capacity.shape[0])
            with np.errstate(divide="ignore", invalid="ignore"):
                room = np.where(grow > 0, (capacity - used) / grow, np.inf)
            tight.append(room)
            step = min(step, float(room.min()))
        step = max(step, 0.0)
        rate[free] += step
        newly = free & (rate >= cap - 1e-6 * cap)
        for (idx, _w, _capacity), room in zip(groups, tight):
            if room is None:
                continue
            full = room <= step * (1 + 1e-9)
            newly |= free & (idx >= 0) & full[np.clip(idx, 0, None)]
        if not newly.any():
            break
        free &= ~newly
    return rate


def simulate(tables: Dict[int, np.ndarray], order: str, n_gpus: int, grid: int = 148, chunk_bytes: int = 4 * 32768,
             nvlink: float = 770e9, hbm: float = 6.54e12, dt: float = 20e-6, t_max: float = 1.0) -> Dict[str, object]:
    """``tables``: sender GPU -> segment rows in table order.  Returns finish times in ms."""
    senders = sorted(tables)
    cum = {s: np.concatenate([[0.0], np.cumsum(tables[s][:, 1])]) for s in senders}
    total = {s: cum[s][-1] for s in senders}
    agent_sender = np.repeat(np.array(senders), grid)
    agent_cta = np.tile(np.arange(grid), len(senders))
    n = agent_sender.shape[0]
    length = np.zeros(n)
    for k, s in enumerate(senders):
        sl = slice(k * grid, (k + 1) * grid)
        if order == "contiguous":
            length[sl] = total[s] / grid
        else:
            n_chunks = int(np.ceil(total[s] / chunk_bytes))
            mine = (n_chunks - np.arange(grid) + grid - 1) // grid
            length[sl] = np.clip(mine, 0, None) * chunk_bytes
    pos = np.zeros(n)
    done_at = np.full(n, np.nan)
    t = 0.0
    peak_ingress = np.zeros(n_gpus)
    while t < t_max:
        active = pos < length
        if not active.any():
            break
        dst = np.zeros(n, dtype=np.int64)
        wire = np.ones(n)
        cap = np.zeros(n)
        for k, s in enumerate(senders):
            sl = slice(k * grid, (k + 1) * grid)
            if order == "contiguous":
                where = agent_cta[sl] * (total[s] / grid) + pos[sl]
            else:
                k_chunk = np.floor(pos[sl] / chunk_bytes)
                where = (agent_cta[sl] + k_chunk * grid) * chunk_bytes + (pos[sl] - k_chunk * chunk_bytes)
            seg = np.clip(np.searchsorted(cum[s], where, side="right") - 1, 0, tables[s].shape[0] - 1)
            over = where >= total[s]
            dst[sl], wire[sl], cap[sl] = tables[s][seg, 0].astype(np.int64), tables[s][seg, 2], tables[s][seg, 3]
            act = active[sl] & ~over
            cap[sl] = np.where(act, cap[sl], 0.0)
            pos[sl] = np.where(active[sl] & over, length[sl], pos[sl])  # the table's short last chunk
        remote = dst != agent_sender
        egress_idx = np.where(remote, agent_sender, -1)
        ingress_idx = np.where(remote, dst, -1)
        hbm_w = 1.0 + np.where(remote, 0.0, wire)  # what the sender's memory sees: the read, plus the write when local
        rate = _fair_rates(cap, [
            (egress_idx, wire, np.full(n_gpus, nvlink)), (ingress_idx, wire, np.full(n_gpus, nvlink)),
            (agent_sender.astype(np.int64), hbm_w, np.full(n_gpus, hbm)),
        ])
        peak_ingress = np.maximum(peak_ingress, np.bincount(ingress_idx[remote], weights=(rate * wire)[remote], minlength=n_gpus))
        pos = pos + rate * dt
        t += dt
        finished = np.isnan(done_at) & (pos >= length)
        done_at[finished] = t
    per_sender = {int(s): float(np.nanmax(done_at[k * grid:(k + 1) * grid]) * 1e3) for k, s in enumerate(senders)}
    return {"order": order, "ms": max(per_sender.values()), "ms_per_sender": per_sender, "peak_ingress_GBps": (peak_ingress / 1e9).round(1).tolist()}


def _rotated(items: Sequence, rank: int) -> List:
    dests = sorted({it.dst_rank for it in items})
    if len(dests) < 2:
        return list(items)
    shift = rank % len(dests)
    order = {d: (i - shift) % len(dests) for i, d in enumerate(dests)}
    return sorted(items, key=lambda it: order[it.dst_rank])


def study(model: str, train: Dict[str, int], infer: Dict[str, int], placement: str = "colocated", layers: int = 0, fp8: bool = False,
          pairing: str = "spread", orders: Sequence[str] = ("contiguous", "chunks", "striped"), stripe_mb: float = 1.0,
          chunk_tiles: int = 4, grid: int = 148, nvlink_gbps: float = 770.0, hbm_gbps: float = 6540.0) -> List[Dict[str, object]]:
    import torch

    from awex_b200 import logging
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout
    from awex_b200.transfer.lowering import stripe_by_destination
    from awex_b200.transfer.transfer_plan import TransferPlanBuilder

    logging.setLevel("WARNING")
    arch = get_arch(model)
    if layers:
        arch = arch.with_layers(layers)
    t_layout = TrainLayout(tp=train.get("tp", 1), pp=train.get("pp", 1), dp=train.get("dp", 1), ep=train.get("ep", 1), etp=train.get("etp", 1))
    i_layout = InferLayout(tp=infer.get("tp", 1), ep=infer.get("ep", 1), num_engines=infer.get("engines", 1), fp8=fp8)
    job = SimulatedJob(arch, t_layout, i_layout, dtype=torch.bfloat16, device="meta")
    skip = job.builder.skip_names
    job.builder = TransferPlanBuilder(job.infer_world_size, t_layout.world, i_layout.num_engines,
                                      replica_pairing="spread" if pairing == "local" else pairing, skip_names=skip)
    programs = {r: job.compile_send_program(r) for r in range(t_layout.world)}
    if placement.startswith("colocated"):
        n_gpus = max(t_layout.world, job.infer_world_size)
        gpu_of_dst = {i: i for i in range(job.infer_world_size)}
        if placement == "colocated-best":  # every inference worker beside the training rank that sends it most
            from scipy.optimize import linear_sum_assignment

            sent = np.zeros((n_gpus, n_gpus))
            for r, items in programs.items():
                for it in items:
                    sent[r, it.dst_rank] += it.dst_bytes
            rows, cols = linear_sum_assignment(-sent)
            gpu_of_dst = {int(i): int(r) for r, i in zip(rows, cols)}
    else:
        n_gpus = t_layout.world + job.infer_world_size
        gpu_of_dst = {i: t_layout.world + i for i in range(job.infer_world_size)}
    if pairing == "local" and placement.startswith("colocated"):
        # the placement was found with least-loaded pairing; now every shard prefers the replica on its own GPU
        job.builder = TransferPlanBuilder(job.infer_world_size, t_layout.world, i_layout.num_engines, replica_pairing="local",
                                          skip_names=skip, colocation=gpu_of_dst)
        programs = {r: job.compile_send_program(r) for r in range(t_layout.world)}
    out = []
    for order in orders:
        items = {r: (stripe_by_destination(p, int(stripe_mb * 2**20)) if order == "striped" else _rotated(p, r) if order == "rotated" else p)
                 for r, p in programs.items()}
        tables = {r: segments_of(p, gpu_of_dst) for r, p in items.items() if len(p)}
        result = simulate(tables, "contiguous" if order == "contiguous" else "chunks", n_gpus, grid=grid, chunk_bytes=chunk_tiles * 32768,
                          nvlink=nvlink_gbps * 1e9, hbm=hbm_gbps * 1e9)
        result["order"] = order
        out.append(result)
    return out


def main(argv=None) -> int:
    from awex_b200.debug.plan_study import parse_layout

    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--train", default="tp1")
    ap.add_argument("--infer", default="tp1")
    ap.add_argument("--fp8", action="store_true")
    ap.add_argument("--placement", default="colocated", choices=["colocated", "colocated-best", "separated"])
    ap.add_argument("--pairing", default="spread", choices=["spread", "round_robin", "local"])
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--stripe-mb", type=float, default=1.0)
    ap.add_argument("--chunk-tiles", type=int, default=4)
    ap.add_argument("--orders", default="contiguous,chunks,striped")
    args = ap.parse_args(argv)
    results = study(args.model, parse_layout(args.train), parse_layout(args.infer), args.placement, args.layers, args.fp8, args.pairing,
                    [o for o in args.orders.split(",") if o], args.stripe_mb, args.chunk_tiles)
    for r in results:
        slowest = max(r["ms_per_sender"], key=r["ms_per_sender"].get)
        fastest = min(r["ms_per_sender"], key=r["ms_per_sender"].get)
        print(f"{r['order']:>10}: {r['ms']:7.2f} ms  (senders finish between {r['ms_per_sender'][fastest]:.2f} and {r['ms_per_sender'][slowest]:.2f} ms; "
              f"peak ingress GB/s {r['peak_ingress_GBps']})")
    return 0


if __name__ == "__main__":
    sys.exit(main())
