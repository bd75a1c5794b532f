"""Every tile body and launch shape of the fused transfer kernel against the
plain PyTorch statement of the same op (fp32 math on the CPU for quantisation)."""

import numpy as np
import pytest
import torch

from awex_b200.converter.weights_converter import per_block_cast_to_fp8

pytestmark = pytest.mark.gpu

F = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


def _run(items, srcs, dsts, **program_kwargs):
    from awex_b200.ops.fused_transfer import TransferProgram
    from awex_b200.transfer.descriptors import TensorAddr, encode_items, validate_table

    src_addrs = {(n, 0): TensorAddr.of(t) for n, t in srcs.items()}
    dst_addrs = {rank: {n: TensorAddr.of(t) for n, t in views.items()} for rank, views in dsts.items()}
    table, n_tiles, enc = encode_items(items, src_addrs, dst_addrs)
    if program_kwargs.pop("out_bulk", False):  # as for destinations across NVLink: quantised tiles leave through shared memory
        from awex_b200.transfer.descriptors import mark_bulk_output

        assert mark_bulk_output(table, enc.desc_dst, list(dst_addrs)) > 0
    spans = [a.byte_span() for views in dst_addrs.values() for a in views.values()]
    assert validate_table(table, n_tiles, [a.byte_span() for a in src_addrs.values()], spans) == []
    prog = TransferProgram(table, n_tiles, "cuda", encoder=enc, **program_kwargs)
    prog.launch(1)
    torch.cuda.synchronize()
    prog.check()
    return prog, table


@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("src_dt,dst_dt", [("bf16", "f32"), ("f32", "bf16"), ("f16", "bf16"), ("bf16", "f16"), ("f32", "f16"), ("f16", "f32")])
def test_vector_cast_and_add_paths(src_dt, dst_dt, variant):
    """16-byte chunks from the stage, packed converts, vector stores: many short
    rows, a few long rows (tiles of one row), and a column slab with a pitch."""
    from awex_b200.converter.rows import ValueOp
    from awex_b200.transfer.lowering import CopyItem

    s, d = F[src_dt], F[dst_dt]
    g = torch.Generator(device="cuda").manual_seed(11)
    a = (torch.randn(333, 1024, generator=g, device="cuda") * 3).to(s)
    b = (torch.randn(3, 40000, generator=g, device="cuda") * 3).to(s)
    out_a = torch.zeros(333, 1024, dtype=d, device="cuda")
    out_b = torch.zeros(3, 40000, dtype=d, device="cuda")
    out_c = torch.zeros(333, 2048, dtype=d, device="cuda")
    items = [
        CopyItem("a", 0, (0, 0), (333, 1024), 0, "a", (0, 0), s, d, ValueOp("cast", dtype=d)),
        CopyItem("b", 0, (0, 0), (3, 40000), 0, "b", (0, 0), s, d, ValueOp("cast", dtype=d)),
        CopyItem("a", 0, (0, 512), (333, 512), 0, "c", (0, 1024), s, d, ValueOp("cast", dtype=d)),
    ]
    _run(items, {"a": a, "b": b}, {0: {"a": out_a, "b": out_b, "c": out_c}}, variant=variant)
    assert torch.equal(out_a, a.float().to(d))
    assert torch.equal(out_b, b.float().to(d))
    want_c = torch.zeros_like(out_c)
    want_c[:, 1024:1536] = a[:, 512:].float().to(d)
    assert torch.equal(out_c, want_c)


@pytest.mark.parametrize("variant", [0, 1])
def test_constant_add_rides_along(variant):
    from awex_b200.converter.rows import ValueOp
    from awex_b200.transfer.lowering import CopyItem

    g = torch.Generator(device="cuda").manual_seed(12)
    a = torch.randn(200, 4096, generator=g, device="cuda").to(torch.bfloat16)
    out = torch.zeros_like(a)
    _run([CopyItem("a", 0, (0, 0), (200, 4096), 0, "a", (0, 0), torch.bfloat16, torch.bfloat16, ValueOp("add", const=1.0))],
         {"a": a}, {0: {"a": out}}, variant=variant)
    assert torch.equal(out, (a.float() + 1.0).to(torch.bfloat16))


@pytest.mark.parametrize("variant", [0, 1, 2])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(512, 1024), (130, 136), (257, 384)])
@pytest.mark.parametrize("ue8m0", [False, True])
@pytest.mark.parametrize("out_bulk", [False, True])
def test_fused_block_fp8_matches_cpu_statement(shape, dtype, variant, ue8m0, out_bulk):
    """Block quantisation inside the transfer kernel: whole blocks, edge blocks in
    both directions, both thread counts (8 and 4 chunks per thread)."""
    from awex_b200.converter.rows import ValueOp
    from awex_b200.transfer.lowering import CopyItem

    g = torch.Generator(device="cuda").manual_seed(13)
    x = (torch.randn(shape, generator=g, device="cuda") * 0.05).to(dtype)
    x[0, 0] = 3.0
    x[shape[0] - 1, shape[1] - 1] = -7.0
    q = torch.zeros(shape, dtype=torch.float8_e4m3fn, device="cuda")
    s = torch.zeros(-(-shape[0] // 128), -(-shape[1] // 128), dtype=torch.float32, device="cuda")
    item = CopyItem("x", 0, (0, 0), shape, 0, "q", (0, 0), dtype, torch.float8_e4m3fn,
                    ValueOp("fp8_block", dtype=torch.float8_e4m3fn, ue8m0=ue8m0), scale_name="s", scale_start=(0, 0))
    if out_bulk and shape[1] % 16:
        pytest.skip("rows of the destination are not 16-byte aligned: such slabs never take the bulk-store exit")
    _run([item], {"x": x}, {0: {"q": q, "s": s}}, variant=variant, out_bulk=out_bulk)
    q_ref, s_ref = per_block_cast_to_fp8(x.cpu(), ue8m0)
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))


def test_fused_block_fp8_with_gathered_rows():
    """Blocks whose rows are collected through the per-row offset table (row by
    row bulk copies into the stage; rows past the block's edge are not loaded and
    must not leak from the stage's previous contents)."""
    from awex_b200.converter.rows import ValueOp
    from awex_b200.transfer.lowering import CopyItem

    g = torch.Generator(device="cuda").manual_seed(14)
    x = (torch.randn(600, 256, generator=g, device="cuda") * 0.1).to(torch.bfloat16)
    # destination rows 0..199 come from source rows 400..499 then 100..199
    runs = ((0, 400, 100), (100, 100, 100))
    q = torch.zeros(200, 256, dtype=torch.float8_e4m3fn, device="cuda")
    s = torch.zeros(2, 2, dtype=torch.float32, device="cuda")
    item = CopyItem("x", 0, (0, 0), (200, 256), 0, "q", (0, 0), torch.bfloat16, torch.float8_e4m3fn,
                    ValueOp("fp8_block", dtype=torch.float8_e4m3fn), scale_name="s", scale_start=(0, 0), src_rows=runs)
    # a plain copy of large values first, so that stale stage contents would show in the maxima
    big = torch.full((512, 4096), 100.0, dtype=torch.bfloat16, device="cuda")
    big_out = torch.zeros_like(big)
    items = [CopyItem("big", 0, (0, 0), (512, 4096), 0, "big", (0, 0), torch.bfloat16, torch.bfloat16), item]
    for variant in (0, 1, 2):
        q.zero_(), s.zero_(), big_out.zero_()
        _run(items, {"x": x, "big": big}, {0: {"q": q, "s": s, "big": big_out}}, variant=variant, grid=3)
        gathered = torch.cat([x[400:500], x[100:200]]).cpu()
        q_ref, s_ref = per_block_cast_to_fp8(gathered, False)
        assert torch.equal(s.cpu(), s_ref) and torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
        assert torch.equal(big_out, big)


@pytest.mark.parametrize("variant", [0, 1, 2])
@pytest.mark.parametrize("interleave", [False, True])
def test_destination_groups_and_mixed_tiles(variant, interleave):
    """Three destinations of very different sizes and tile kinds (copies, strided
    copies, casts, quantised blocks): one CTA group per destination, chunks dealt
    round-robin inside a group; every tile is done exactly once."""
    from awex_b200.converter.rows import ValueOp
    from awex_b200.transfer.descriptors import plan_tile_order
    from awex_b200.transfer.lowering import CopyItem

    g = torch.Generator(device="cuda").manual_seed(15)
    w = torch.randn(1024, 2048, generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn(96, 512, generator=g, device="cuda").to(torch.bfloat16)
    d0 = {"w": torch.zeros(1024, 2048, dtype=torch.bfloat16, device="cuda"), "v32": torch.zeros(96, 512, dtype=torch.float32, device="cuda")}
    d1 = {"wq": torch.zeros(1024, 2048, dtype=torch.float8_e4m3fn, device="cuda"), "ws": torch.zeros(8, 16, dtype=torch.float32, device="cuda")}
    d2 = {"wt": torch.zeros(1024, 4096, dtype=torch.bfloat16, device="cuda")}
    items = [
        CopyItem("w", 0, (0, 0), (1024, 2048), 0, "w", (0, 0), torch.bfloat16, torch.bfloat16),
        CopyItem("v", 0, (0, 0), (96, 512), 0, "v32", (0, 0), torch.bfloat16, torch.float32, ValueOp("cast", dtype=torch.float32)),
        CopyItem("w", 0, (0, 0), (1024, 2048), 1, "wq", (0, 0), torch.bfloat16, torch.float8_e4m3fn,
                 ValueOp("fp8_block", dtype=torch.float8_e4m3fn), scale_name="ws", scale_start=(0, 0)),
        CopyItem("w", 0, (0, 0), (1024, 1024), 2, "wt", (0, 3072), torch.bfloat16, torch.bfloat16),
        CopyItem("w", 0, (0, 1024), (1024, 1024), 2, "wt", (0, 0), torch.bfloat16, torch.bfloat16),
    ]
    prog, table = _run(items, {"w": w, "v": v}, {0: d0, 1: d1, 2: d2}, variant=variant, interleave=interleave, desc_group=True,
                       group_cost={0: 0.25}, grid=37, out_bulk=True)
    if interleave:
        groups = sorted({(int(e["tile_begin"]), int(e["tile_end"]), int(e["size"])) for e in prog.plan_host})
        assert len(groups) == 3 and sum(size for _, _, size in groups) == 37
        assert sorted(plan_tile_order(prog.plan_host, prog.chunk_shift)) == list(range(prog.n_tiles))
    else:
        assert prog.plan_host is None
    assert torch.equal(d0["w"], w) and torch.equal(d0["v32"], v.float())
    q_ref, s_ref = per_block_cast_to_fp8(w.cpu(), False)
    assert torch.equal(d1["ws"].cpu(), s_ref) and torch.equal(d1["wq"].cpu().view(torch.uint8), q_ref.view(torch.uint8))
    want = torch.zeros_like(d2["wt"])
    want[:, 3072:], want[:, :1024] = w[:, :1024], w[:, 1024:]
    assert torch.equal(d2["wt"], want)


def test_a_launch_that_timed_out_leaves_the_program_reusable():
    """Many CTAs give up waiting for a destination that never announces itself:
    no byte is written, no flag raised, and the arrival counter is back at zero, so
    the very next launch (without any host-side reset but the status) completes."""
    from awex_b200.ops.fused_transfer import FlagPad, TransferError, TransferProgram
    from awex_b200.transfer.descriptors import TensorAddr, encode_items
    from awex_b200.transfer.lowering import CopyItem

    src = torch.randn(2048, 4096, device="cuda").to(torch.bfloat16)
    dst = torch.zeros_like(src)
    table, n_tiles, enc = encode_items([CopyItem("w", 0, (0, 0), (2048, 4096), 0, "w", (0, 0), torch.bfloat16, torch.bfloat16)],
                                       {("w", 0): TensorAddr.of(src)}, {0: {"w": TensorAddr.of(dst)}})
    ready, done = FlagPad(1, "cuda"), FlagPad(1, "cuda")
    prog = TransferProgram(table, n_tiles, "cuda", ready_pad=ready, ready_slots=[0], done_flag_addrs=[done.slot_addr(0)], timeout_ms=30, encoder=enc)
    prog.launch(epoch=7)
    torch.cuda.synchronize()
    with pytest.raises(TransferError) as err:
        prog.status.raise_if_failed()  # resets the status only
    assert err.value.code == 1 and int(prog.counter.item()) == 0
    assert torch.count_nonzero(dst).item() == 0 and done.t.item() == 0
    ready.t.fill_(7)
    prog.launch(epoch=7)
    torch.cuda.synchronize()
    prog.status.raise_if_failed()
    assert torch.equal(dst, src) and done.t.item() == 7


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(1000, 512), (257, 1030), (19008, 2048)])
def test_column_normalisation_matches_the_pytorch_statement(shape, dtype):
    """``F.normalize(x, dim=0)``: everything but the summation order is the same
    arithmetic, so elements agree exactly except where a column's norm lands on
    the other side of a rounding boundary of the dtype (then by one unit in the
    last place)."""
    from awex_b200.ops.normalize import col_l2_normalize

    g = torch.Generator(device="cuda").manual_seed(21)
    x = (torch.randn(shape, generator=g, device="cuda") * 0.02).to(dtype)
    x[:, 3] = 0  # an all-zero column: divided by eps, stays zero
    got = col_l2_normalize(x)
    want = torch.nn.functional.normalize(x.cpu(), dim=0, p=2, eps=1e-7)
    if dtype == torch.bfloat16:  # with more mantissa bits the norm carries the summation order's last bits into more elements
        assert (got.cpu() == want).float().mean().item() > 0.98
    ulp = {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10, torch.float32: 2.0 ** -18}[dtype]
    assert torch.allclose(got.cpu().float(), want.float(), rtol=4 * ulp, atol=1e-7)
    assert bool((got[:, 3] == 0).all())
    # in place, and into a buffer with a pitch
    wide = torch.zeros(shape[0], shape[1] + 8, dtype=dtype, device="cuda")
    col_l2_normalize(x, out=wide[:, : shape[1]])
    assert torch.equal(wide[:, : shape[1]], got) and bool((wide[:, shape[1]:] == 0).all())
    again = x.clone()
    col_l2_normalize(again, out=again)
    assert torch.equal(again, got)


def test_column_normalisation_is_exact_where_the_norm_is_exact():
    from awex_b200.ops.normalize import col_l2_normalize

    x = torch.zeros(300, 64, dtype=torch.bfloat16, device="cuda")
    rows = torch.arange(64, device="cuda") * 3
    x[rows, torch.arange(64, device="cuda")] = torch.linspace(-4, 4, 64, device="cuda").to(torch.bfloat16)  # one value per column
    got = col_l2_normalize(x)
    want = torch.nn.functional.normalize(x.cpu(), dim=0, p=2, eps=1e-7)
    assert torch.equal(got.cpu(), want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("ue8m0", [False, True])
def test_lean_block_fp8_kernel_on_many_small_slabs_with_copies_beside_them(dtype, ue8m0):
    """A table like a block-fp8 serving layout: many expert-sized slabs (row and
    column slices with half-filled edge blocks) plus plain copies.  With no launch
    shape forced, the quantised slabs run in the lean kernel and the rest in the
    general one; one completion flag is raised, after both."""
    from awex_b200.converter.rows import ValueOp
    from awex_b200.ops.fused_transfer import FlagPad
    from awex_b200.transfer.lowering import CopyItem

    g = torch.Generator(device="cuda").manual_seed(31)
    experts, hid, ffn, tp = 6, 1024, 384, 2
    w13 = (torch.randn(experts, 2 * ffn, hid, generator=g, device="cuda") * 0.05).to(dtype)
    w2 = (torch.randn(experts, hid, ffn, generator=g, device="cuda") * 0.05).to(dtype)
    emb = torch.randn(4096, hid, generator=g, device="cuda").to(dtype)
    srcs, dsts, items = {"emb": emb}, {0: {"emb": torch.zeros_like(emb)}}, []
    items.append(CopyItem("emb", 0, (0, 0), (4096, hid), 0, "emb", (0, 0), dtype, dtype))
    part = ffn // tp  # 192 rows / columns per shard: one and a half blocks
    for e in range(experts):
        srcs[f"w13_{e}"], srcs[f"w2_{e}"] = w13[e], w2[e]
        for j in range(tp):
            for kind, base in (("gate", 0), ("up", ffn)):
                name = f"{kind}{e}_{j}"
                dsts[0][name] = torch.zeros(part, hid, dtype=torch.float8_e4m3fn, device="cuda")
                dsts[0][name + "_s"] = torch.zeros(2, hid // 128, dtype=torch.float32, device="cuda")
                items.append(CopyItem(f"w13_{e}", 0, (base + part * j, 0), (part, hid), 0, name, (0, 0), dtype, torch.float8_e4m3fn,
                                      ValueOp("fp8_block", dtype=torch.float8_e4m3fn, ue8m0=ue8m0), scale_name=name + "_s", scale_start=(0, 0)))
            name = f"down{e}_{j}"
            dsts[0][name] = torch.zeros(hid, part, dtype=torch.float8_e4m3fn, device="cuda")
            dsts[0][name + "_s"] = torch.zeros(hid // 128, 2, dtype=torch.float32, device="cuda")
            items.append(CopyItem(f"w2_{e}", 0, (0, part * j), (hid, part), 0, name, (0, 0), dtype, torch.float8_e4m3fn,
                                  ValueOp("fp8_block", dtype=torch.float8_e4m3fn, ue8m0=ue8m0), scale_name=name + "_s", scale_start=(0, 0)))
    done = FlagPad(1, "cuda")
    prog, _ = _run(items, srcs, dsts, done_flag_addrs=[done.slot_addr(0)])
    assert prog.lean is not None and prog.lean.variant == 3 and prog.lean.n_tiles > 0 and prog.n_tiles > 0
    assert prog.lean.n_tiles + prog.n_tiles == prog.total_tiles
    assert done.t.item() == 1 and int(prog.counter.item()) == 0 and int(prog.lean.counter.item()) == 0
    assert torch.equal(dsts[0]["emb"], emb)
    for e in range(experts):
        for j in range(tp):
            for kind, base in (("gate", 0), ("up", ffn)):
                q_ref, s_ref = per_block_cast_to_fp8(w13[e, base + part * j: base + part * (j + 1)].cpu(), ue8m0)
                name = f"{kind}{e}_{j}"
                assert torch.equal(dsts[0][name + "_s"].cpu(), s_ref), name
                assert torch.equal(dsts[0][name].cpu().view(torch.uint8), q_ref.view(torch.uint8)), name
            q_ref, s_ref = per_block_cast_to_fp8(w2[e, :, part * j: part * (j + 1)].cpu().contiguous(), ue8m0)
            assert torch.equal(dsts[0][f"down{e}_{j}_s"].cpu(), s_ref)
            assert torch.equal(dsts[0][f"down{e}_{j}"].cpu().view(torch.uint8), q_ref.view(torch.uint8))
    # a second launch of the same programs (the counters reset themselves)
    for t in dsts[0].values():
        t.zero_()
    prog.launch(2)
    torch.cuda.synchronize()
    prog.check()
    assert done.t.item() == 2 and torch.equal(dsts[0]["emb"], emb)
    q_ref, _ = per_block_cast_to_fp8(w2[0, :, :part].cpu().contiguous(), ue8m0)
    assert torch.equal(dsts[0]["down0_0"].cpu().view(torch.uint8), q_ref.view(torch.uint8))


def test_lean_kernel_gives_up_cleanly_when_a_destination_never_announces():
    from awex_b200.converter.rows import ValueOp
    from awex_b200.ops.fused_transfer import FlagPad, TransferError, TransferProgram
    from awex_b200.transfer.descriptors import TensorAddr, encode_items
    from awex_b200.transfer.lowering import CopyItem

    x = (torch.randn(4096, 1024, device="cuda") * 0.05).to(torch.bfloat16)
    q = torch.zeros(4096, 1024, dtype=torch.float8_e4m3fn, device="cuda")
    s = torch.zeros(32, 8, dtype=torch.float32, device="cuda")
    item = CopyItem("x", 0, (0, 0), (4096, 1024), 0, "q", (0, 0), torch.bfloat16, torch.float8_e4m3fn,
                    ValueOp("fp8_block", dtype=torch.float8_e4m3fn), scale_name="s", scale_start=(0, 0))
    table, n_tiles, enc = encode_items([item], {("x", 0): TensorAddr.of(x)}, {0: {"q": TensorAddr.of(q), "s": TensorAddr.of(s)}})
    ready, done = FlagPad(1, "cuda"), FlagPad(1, "cuda")
    prog = TransferProgram(table, n_tiles, "cuda", ready_pad=ready, ready_slots=[0], done_flag_addrs=[done.slot_addr(0)], timeout_ms=30, encoder=enc)
    assert prog.lean is not None
    prog.launch(3)
    torch.cuda.synchronize()
    with pytest.raises(TransferError) as err:
        prog.status.raise_if_failed()
    assert err.value.code == 1 and int(prog.lean.counter.item()) == 0 and int(prog.counter.item()) == 0
    assert torch.count_nonzero(q.view(torch.uint8)).item() == 0 and done.t.item() == 0
    ready.t.fill_(3)
    prog.launch(3)
    torch.cuda.synchronize()
    prog.status.raise_if_failed()
    q_ref, s_ref = per_block_cast_to_fp8(x.cpu(), False)
    assert done.t.item() == 3 and torch.equal(s.cpu(), s_ref) and torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
