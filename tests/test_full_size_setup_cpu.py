"""Host-side set-up of the largest benchmark configuration (Qwen3-235B-A22B
architecture, all 94 layers, training EP8 -> inference TP8 serving block fp8) on
shape-only models: plan, lowering, descriptor encoding, table validation, the
per-CTA plan and the receiver's exactly-once coverage check all run to
completion in seconds.  Nothing here touches weight data; it keeps set-up cost
from growing back to the point where it eats a benchmark run."""

import time

import numpy as np
import pytest
import torch


@pytest.mark.timeout(900)
def test_full_235b_fp8_layout_sets_up_in_bounded_time():
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout
    from awex_b200.transfer.descriptors import OP_FP8_BLOCK, TensorAddr, build_cta_plan, encode_items, plan_tile_order, validate_table
    from awex_b200.transfer.lowering import check_exactly_once, manifest_by_destination

    arch = get_arch("qwen3-235b-a22b")
    assert arch.num_layers == 94
    job = SimulatedJob(arch, TrainLayout(tp=1, dp=8, ep=8), InferLayout(tp=8, fp8=True), dtype=torch.bfloat16, device="meta")
    views = job.destination_views()
    cursor = [1 << 30]

    def place(t):  # shape-only tensors have no address: lay them out one after the other
        addr = TensorAddr(cursor[0], tuple(t.shape), tuple(t.stride()), t.dtype)
        cursor[0] += (t.numel() * t.element_size() + 255) // 256 * 256
        return addr

    dsts = {r: {n: place(t) for n, t in v.items()} for r, v in views.items()}
    dst_spans = [a.byte_span() for d in dsts.values() for a in d.values()]
    started = time.time()
    manifests = []
    for rank in range(8):
        items = job.compile_send_program(rank)
        manifests.append(manifest_by_destination(items))
        if rank not in (0, 7):
            continue
        local = {(n, 0): place(t) for n, t in job.train_models[rank].named_parameters()}
        for key, t in job.local_tensors(rank).items():
            local.setdefault(key, place(t))
        table, n_tiles, enc = encode_items(items, local, dsts)
        assert validate_table(table, n_tiles, [a.byte_span() for a in local.values()], dst_spans, check_overlap=False) == []
        assert int((table["op"] == OP_FP8_BLOCK).sum()) > 0.5 * len(table)  # the experts dominate and are quantised
        plan, index = build_cta_plan(table, n_tiles, 296, 4, enc.desc_dst, {rank: 0.25})
        assert len({(int(e["tile_begin"]), int(e["tile_end"])) for e in plan}) == 8  # one CTA group per destination
        assert int(plan["size"].min()) >= 1 and len(index) >= (n_tiles >> 4)
        order = np.asarray(plan_tile_order(plan, 4))
        assert order.size == n_tiles and np.array_equal(np.sort(order), np.arange(n_tiles))
    # receiver 0 checks that the eight senders' writes tile its parameters exactly once
    shapes = {n: (tuple(v.shape), v.dtype) for n, v in views[0].items()}
    required = sorted(n for n in views[0] if n not in job.aliases)
    entries = [m.get(0, []) for m in manifests]
    assert check_exactly_once([e for e in entries if e], shapes, required) == []
    elapsed = time.time() - started
    assert elapsed < 600, f"set-up of the full layout took {elapsed:.0f}s"
