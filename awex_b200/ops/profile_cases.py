"""Small, self-terminating workloads of each kernel for profilers and quick
timing:  ``python -m awex_b200.ops.profile_cases <case> [--mb N] [--iters K]``.

Cases: ``transfer_copy`` (contiguous slabs, bulk path), ``transfer_strided``
(column slabs with 2 KiB runs), ``transfer_cast`` (bf16 -> fp32 elementwise),
``transfer_fp8`` (fused block quantisation), ``transfer_peer`` (contiguous
slabs stored into the memory of a second GPU of this process over NVLink; needs
two devices), ``transfer_peer_fp8`` (block quantisation into the second GPU's
memory; ``AWEX_XFER_OUT_BULK=1`` sends the result through shared memory and
bulk stores instead of per-thread stores), ``fp8_quant`` / ``fp8_dequant`` (stand-alone kernels),
``checksum``.  Every case holds a few hundred MB (more
than L2) and prints achieved GB/s from CUDA-event timings.
"""

from __future__ import annotations

import argparse
import json

import torch


def _time(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters


def _transfer_case(kind: str, mb: int):
    from awex_b200.converter.rows import ValueOp
    from awex_b200.ops.fused_transfer import TransferProgram
    from awex_b200.transfer.descriptors import TensorAddr, encode_items, validate_table
    from awex_b200.transfer.lowering import CopyItem

    cols = 4096
    rows = mb * 1024 * 1024 // (cols * 2)
    g = torch.Generator(device="cuda").manual_seed(0)
    src = torch.randn(rows, cols, generator=g, device="cuda").to(torch.bfloat16)
    views = {}
    if kind in ("transfer_peer", "transfer_peer_fp8"):
        if torch.cuda.device_count() < 2:
            raise SystemExit("transfer_peer needs two GPUs")
        from awex_b200.ops import native

        code = native.load().awex_enable_peer_access(0, 1)
        if code != 0:
            raise SystemExit(f"no peer access from device 0 to device 1 (code {code})")
        if kind == "transfer_peer_fp8":
            dst = torch.zeros(rows, cols, dtype=torch.float8_e4m3fn, device="cuda:1")
            scale = torch.zeros(-(-rows // 128), cols // 128, dtype=torch.float32, device="cuda:1")
            items = [CopyItem("w", 0, (0, 0), (rows, cols), 0, "w", (0, 0), torch.bfloat16, torch.float8_e4m3fn,
                              ValueOp("fp8_block", dtype=torch.float8_e4m3fn), scale_name="w_scale_inv", scale_start=(0, 0))]
            views["w"], views["w_scale_inv"] = dst, scale
            moved = src.numel()  # fp8 bytes that cross the link
        else:
            dst = torch.zeros(rows, cols, dtype=torch.bfloat16, device="cuda:1")
            items = [CopyItem("w", 0, (0, 0), (rows, cols), 0, "w", (0, 0), torch.bfloat16, torch.bfloat16)]
            views["w"] = dst
            moved = src.numel() * 2  # bytes that cross the link, one direction
    elif kind == "transfer_copy":
        dst = torch.zeros_like(src)
        items = [CopyItem("w", 0, (0, 0), (rows, cols), 0, "w", (0, 0), torch.bfloat16, torch.bfloat16)]
        views["w"] = dst
        moved = 2 * src.numel() * 2
    elif kind == "transfer_strided":
        dst = torch.zeros(rows, cols, dtype=torch.bfloat16, device="cuda")
        items = [
            CopyItem("w", 0, (0, c), (rows, 1024), 0, "w", (0, (c + 1024) % cols), torch.bfloat16, torch.bfloat16)
            for c in range(0, cols, 1024)
        ]
        views["w"] = dst
        moved = 2 * src.numel() * 2
    elif kind == "transfer_cast":
        dst = torch.zeros(rows, cols, dtype=torch.float32, device="cuda")
        items = [CopyItem("w", 0, (0, 0), (rows, cols), 0, "w", (0, 0), torch.bfloat16, torch.float32, ValueOp("cast", dtype=torch.float32))]
        views["w"] = dst
        moved = src.numel() * 6
    elif kind == "transfer_fp8":
        dst = torch.zeros(rows, cols, dtype=torch.float8_e4m3fn, device="cuda")
        scale = torch.zeros(-(-rows // 128), cols // 128, dtype=torch.float32, device="cuda")
        items = [CopyItem("w", 0, (0, 0), (rows, cols), 0, "w", (0, 0), torch.bfloat16, torch.float8_e4m3fn,
                          ValueOp("fp8_block", dtype=torch.float8_e4m3fn), scale_name="w_scale_inv", scale_start=(0, 0))]
        views["w"], views["w_scale_inv"] = dst, scale
        moved = src.numel() * 3
    else:
        raise SystemExit(f"unknown case {kind}")
    srcs = {("w", 0): TensorAddr.of(src)}
    dsts = {0: {n: TensorAddr.of(t) for n, t in views.items()}}
    table, n_tiles, enc = encode_items(items, srcs, dsts)
    if kind == "transfer_peer_fp8":
        import os

        from awex_b200.transfer.descriptors import mark_bulk_output

        if os.environ.get("AWEX_XFER_OUT_BULK", "0") == "1":
            mark_bulk_output(table, enc.desc_dst, [0])
    problems = validate_table(table, n_tiles, [a.byte_span() for a in srcs.values()], [a.byte_span() for a in dsts[0].values()])
    assert not problems, problems
    prog = TransferProgram(table, n_tiles, "cuda", encoder=enc)
    epoch = [0]

    def run():
        epoch[0] += 1
        prog.launch(epoch[0])

    def check():
        prog.status.raise_if_failed()
        if kind == "transfer_peer":
            torch.cuda.synchronize(1)
            assert torch.equal(views["w"].to("cuda:0"), src), "peer destination differs from the source"
        if kind == "transfer_peer_fp8":
            from awex_b200.ops.fp8 import block_quant

            torch.cuda.synchronize(1)
            q_ref, s_ref = block_quant(src)
            assert torch.equal(views["w"].to("cuda:0").view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(views["w_scale_inv"].to("cuda:0"), s_ref)

    return run, moved, check


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--mb", type=int, default=512, help="size of the source tensor in MiB")
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    check = lambda: None  # noqa: E731
    if args.case.startswith("transfer_"):
        run, moved, check = _transfer_case(args.case, args.mb)
    elif args.case == "checksum":
        from awex_b200.ops.checksum import ChecksumPlan

        n = args.mb * 1024 * 1024 // 2
        tensors = [torch.randn(n // 4, device="cuda").to(torch.bfloat16) for _ in range(4)]
        plan = ChecksumPlan(tensors)
        run, moved = plan.launch, sum(t.numel() * 2 for t in tensors)
    elif args.case in ("fp8_quant", "fp8_dequant"):
        from awex_b200.ops import fp8 as fp8_ops

        cols = 4096
        rows = args.mb * 1024 * 1024 // (cols * 2)
        x = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
        q, s = fp8_ops.block_quant(x)
        if args.case == "fp8_quant":
            out_q, out_s = torch.empty_like(q), torch.empty_like(s)
            run, moved = (lambda: fp8_ops.block_quant(x, out=(out_q, out_s))), x.numel() * 3
        else:
            out = torch.empty_like(x)
            run, moved = (lambda: fp8_ops.block_dequant(q, s, out=out)), x.numel() * 3
    else:
        raise SystemExit(f"unknown case {args.case}")
    ms = _time(run, args.iters)
    check()
    print(json.dumps({"case": args.case, "mb": args.mb, "ms": ms, "GBps": moved / ms / 1e6}))


if __name__ == "__main__":
    main()
