"""Descriptor tables executed on the host: whatever layout is simulated, running
the encoded tables tile by tile (the CPU statement of the kernel's semantics)
must give the same inference weights as the item-level executor and the oracle."""

import numpy as np
import pytest
import torch

from awex_b200.synthetic.arch import get_arch
from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout
from awex_b200.transfer.table_interpreter import HostMemory, run_chunked, run_table

CASES = [
    ("tiny-llama", TrainLayout(tp=2), InferLayout(tp=1), torch.float32, False),
    ("tiny-qwen2", TrainLayout(tp=4), InferLayout(tp=2, num_engines=2), torch.bfloat16, False),
    ("tiny-qwen2", TrainLayout(tp=2), InferLayout(tp=8), torch.bfloat16, False),
    ("tiny-qwen3-moe", TrainLayout(tp=1, dp=4, ep=4), InferLayout(tp=2, ep=2, num_engines=2), torch.bfloat16, False),
    ("tiny-qwen3-moe", TrainLayout(tp=1, dp=2, ep=2), InferLayout(tp=1, fp8=True), torch.bfloat16, False),
    ("tiny-llama", TrainLayout(tp=1), InferLayout(tp=2, fp8=True), torch.bfloat16, True),
]


def _memory(job):
    tensors = [p for m in job.train_models for p in m.parameters()]
    tensors += [p for models in job.infer_models for m in models for p in m.parameters()]
    return HostMemory(tensors)


@pytest.mark.parametrize("arch,train,infer,dtype,chunked", CASES, ids=lambda v: v.label() if hasattr(v, "label") else str(v))
def test_encoded_tables_mean_what_the_items_mean(arch, train, infer, dtype, chunked):
    job = SimulatedJob(get_arch(arch), train, infer, dtype=dtype)
    job.compile_all()
    assert job.check_coverage() == []
    encoded = job.encode_all(validate=True)
    mem = _memory(job)
    for rank, (table, n_tiles, enc) in encoded.items():
        if chunked:
            per_cta = run_chunked(table, n_tiles, mem, grid=5, chunk_shift=2, row_offsets=enc.row_offsets)
            assert sum(per_cta) == n_tiles
        else:
            assert run_table(table, n_tiles, mem, enc.row_offsets) == n_tiles
    assert job.mismatches() == []


def test_interpreter_refuses_accesses_outside_the_given_tensors():
    from awex_b200.transfer.descriptors import TensorAddr, encode_items
    from awex_b200.transfer.lowering import CopyItem

    src, dst, stranger = torch.arange(64, dtype=torch.float32), torch.zeros(64), torch.zeros(64)
    item = CopyItem("w", 0, (0,), (64,), 0, "w", (0,), torch.float32, torch.float32)
    table, n_tiles, _ = encode_items([item], {("w", 0): TensorAddr.of(src)}, {0: {"w": TensorAddr.of(stranger)}})
    with pytest.raises(IndexError):
        run_table(table, n_tiles, HostMemory([src, dst]))
    table, n_tiles, _ = encode_items([item], {("w", 0): TensorAddr.of(src)}, {0: {"w": TensorAddr.of(dst)}})
    run_table(table, n_tiles, HostMemory([src, dst]))
    assert torch.equal(dst, src)
    bad = table.copy()
    bad["row_elems"][0] = 10_000
    bad["col_tiles"][0] = -(-10_000 // int(bad["tile_cols"][0]))
    with pytest.raises(IndexError):
        run_table(bad, int(bad["col_tiles"][0]), HostMemory([src, dst]))


def _random_case(rng, case):
    """One random copy item between two 2-D or 3-D tensors with odd sizes,
    offsets and (sometimes) non-contiguous destinations."""
    from awex_b200.converter.rows import ValueOp
    from awex_b200.transfer.lowering import CopyItem

    nd = rng.choice([1, 2, 2, 3])
    extent = tuple(rng.choice([1, 2, 3, 5, 7, 8, 16, 33, 64, 130]) for _ in range(nd))
    src_pad = tuple(rng.randrange(0, 4) for _ in range(nd))
    dst_pad = tuple(rng.randrange(0, 4) for _ in range(nd))
    src_shape = tuple(e + p + rng.randrange(0, 3) for e, p in zip(extent, src_pad))
    dst_shape = tuple(e + p + rng.randrange(0, 3) for e, p in zip(extent, dst_pad))
    kind = rng.choice(["copy", "copy", "cast", "add"])
    src_dtype = rng.choice([torch.bfloat16, torch.float16, torch.float32])
    dst_dtype = src_dtype if kind == "copy" else rng.choice([torch.bfloat16, torch.float32])
    g = torch.Generator().manual_seed(case)
    src = torch.randn(src_shape, generator=g).to(src_dtype)
    dst = torch.full(dst_shape, -7.0, dtype=dst_dtype)
    if nd >= 2 and rng.random() < 0.3:  # a destination view with a non-unit outer stride
        dst = torch.full((dst_shape[0], 2) + dst_shape[1:], -7.0, dtype=dst_dtype)[:, 1]
    op = {"copy": ValueOp("none") if src_dtype == dst_dtype else ValueOp("cast", dtype=dst_dtype),
          "cast": ValueOp("cast", dtype=dst_dtype), "add": ValueOp("add", dtype=dst_dtype, const=1.0)}[kind]
    item = CopyItem("w", 0, src_pad, extent, 0, "w", dst_pad, src_dtype, dst_dtype, op)
    return item, src, dst


def test_random_odd_shaped_items_encode_to_equivalent_tables():
    import random

    from awex_b200.transfer.cpu_exec import execute_items
    from awex_b200.transfer.descriptors import TensorAddr, encode_items, validate_table

    rng = random.Random(11)
    for case in range(150):
        item, src, dst = _random_case(rng, case)
        want = dst.clone()
        execute_items([item], {("w", 0): src}, {0: {"w": want}})
        table, n_tiles, enc = encode_items([item], {("w", 0): TensorAddr.of(src)}, {0: {"w": TensorAddr.of(dst)}})
        problems = validate_table(table, n_tiles, [TensorAddr.of(src).byte_span()], [TensorAddr.of(dst).byte_span()])
        assert problems == [], (case, item, problems)
        base = dst._base if dst._base is not None else dst
        run_table(table, n_tiles, HostMemory([src, base]), enc.row_offsets)
        assert torch.equal(dst.float(), want.float()), (case, item)
        # and in the order round-robin chunks would visit the tiles
        dst.fill_(-7.0)
        run_chunked(table, n_tiles, HostMemory([src, base]), grid=3, chunk_shift=1, row_offsets=enc.row_offsets)
        assert torch.equal(dst.float(), want.float()), (case, item)


def test_derived_sender_buffers_are_ordinary_sources_of_the_table():
    """A column-normalised head lives in a sender-side buffer; the table reads it
    like any parameter and address validation covers it."""
    import dataclasses

    arch = dataclasses.replace(get_arch("tiny-llama"), norm_head=True, name="tiny-llama-norm-head")
    job = SimulatedJob(arch, TrainLayout(tp=2), InferLayout(tp=2), dtype=torch.bfloat16)
    job.compile_all()
    encoded = job.encode_all(validate=True)
    buffers = [job.local_tensors(r)[("__derived__/lm_head.weight", 0)] for r in encoded]
    tensors = [p for m in job.train_models for p in m.parameters()] + buffers
    tensors += [p for models in job.infer_models for m in models for p in m.parameters()]
    mem = HostMemory(tensors)
    for rank, (table, n_tiles, enc) in encoded.items():
        assert run_table(table, n_tiles, mem, enc.row_offsets) == n_tiles
    assert {m.rsplit("/", 1)[1] for m in job.mismatches()} == {"lm_head.weight"}
    for r, model in enumerate(job.infer_models[0]):
        got = dict(model.named_parameters())["lm_head.weight"]
        assert torch.equal(got, buffers[r])  # training TP2 -> inference TP2: shard r is sender r's buffer


@pytest.mark.parametrize("arch,train,infer,dtype", [
    ("tiny-qwen2", TrainLayout(tp=2), InferLayout(tp=2, num_engines=2), torch.bfloat16),
    ("tiny-qwen3-moe", TrainLayout(tp=1, dp=2, ep=2), InferLayout(tp=1, fp8=True, num_engines=2), torch.bfloat16),
    ("tiny-llama", TrainLayout(tp=1), InferLayout(tp=4, fp8=True), torch.bfloat16),
], ids=lambda v: v.label() if hasattr(v, "label") else str(v))
def test_striped_order_does_the_same_work(arch, train, infer, dtype):
    """Cutting items into stripes and merging the destinations' stripes changes
    the order only: same bytes to the same places, exactly once, through the CPU
    executor and through the encoded tables; and every window of the striped list
    serves all destinations."""
    from awex_b200.transfer.cpu_exec import execute_items
    from awex_b200.transfer.lowering import check_exactly_once, manifest_by_destination, stripe_by_destination

    job = SimulatedJob(get_arch(arch), train, infer, dtype=dtype)
    programs = job.compile_all()
    views = job.destination_views()
    stripe = 16 * 1024
    striped = {r: stripe_by_destination(items, stripe) for r, items in programs.items()}
    for r, items in striped.items():
        assert sum(it.numel for it in items) == sum(it.numel for it in programs[r])
        dests = sorted({it.dst_rank for it in items})
        if len(dests) > 1 and len(items) > 8 * len(dests):
            quarter = len(items) // 4
            for k in range(3):  # any quarter of the list touches every destination
                assert sorted({it.dst_rank for it in items[k * quarter:(k + 1) * quarter]}) == dests
    # coverage of every receiver by the striped manifests
    for rank, rank_views in views.items():
        manifests = [manifest_by_destination(items).get(rank, []) for items in striped.values()]
        shapes = {n: (tuple(v.shape), v.dtype) for n, v in rank_views.items()}
        required = [n for n in shapes if n not in job.aliases]
        assert check_exactly_once(manifests, shapes, required) == []
    for r, items in striped.items():
        execute_items(items, job.local_tensors(r), views)
    assert job.mismatches() == []
    # and through descriptor tables
    for models in job.infer_models:
        for m in models:
            for p in m.parameters():
                p.view(torch.uint8).zero_() if p.dtype == torch.float8_e4m3fn else p.zero_()
    job.programs = striped
    encoded = job.encode_all(validate=True)
    mem = HostMemory(job.source_tensors() + [p for ms in job.infer_models for m in ms for p in m.parameters()])
    for table, n_tiles, enc in encoded.values():
        assert run_chunked(table, n_tiles, mem, grid=7, chunk_shift=2, row_offsets=enc.row_offsets)
    assert job.mismatches() == []


def test_no_alloc_entry_refuses_malformed_tables_before_any_cuda_call():
    """The allocation-free entry point checks the structure of a caller-built table
    on the host first (tile numbering, geometry, bulk alignment, stage size), so a
    malformed table is refused even on a machine without a GPU."""
    import ctypes

    from awex_b200.ops import native
    from awex_b200.transfer.descriptors import FLAG_BULK, OP_FP8_BLOCK, TensorAddr, encode_items
    from awex_b200.transfer.lowering import CopyItem

    fn = native.load().awex_fused_transfer_no_alloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int, ctypes.c_void_p,
                   ctypes.POINTER(ctypes.c_int32), ctypes.c_char_p, ctypes.c_size_t]
    src = torch.zeros(300, 512, dtype=torch.bfloat16)
    dst = torch.zeros(300, 512, dtype=torch.bfloat16)
    items = [CopyItem("a", 0, (0, 0), (300, 256), 0, "a", (0, 256), torch.bfloat16, torch.bfloat16),
             CopyItem("a", 0, (0, 256), (300, 256), 0, "a", (0, 0), torch.bfloat16, torch.bfloat16)]
    table, n_tiles, _ = encode_items(items, {("a", 0): TensorAddr.of(src)}, {0: {"a": TensorAddr.of(dst)}})
    assert len(table) == 2 and int(table["flags"][0]) & FLAG_BULK
    err = ctypes.create_string_buffer(256)

    def refused(t, tiles):
        t = np.ascontiguousarray(t)
        rc = fn(t.ctypes.data, len(t), tiles, 1000, 0, None, None, err, len(err))
        assert rc == 1, "cudaErrorInvalidValue expected"
        return err.value.decode()

    assert "n_tiles does not match" in refused(table, n_tiles + 1)
    t = table.copy(); t["tile_begin"][0] = 3
    assert "descriptor 0" in refused(t, n_tiles) and "must be 0" in err.value.decode()
    t = table.copy(); t["tile_begin"][1] += 1
    assert "descriptor 1: tile_begin must continue" in refused(t, n_tiles)
    for field in ("tile_rows", "tile_cols", "col_tiles"):
        t = table.copy(); t[field][1] = 0
        assert "non-zero" in refused(t, n_tiles)
    t = table.copy(); t["col_tiles"][0] = 7
    assert "col_tiles does not match" in refused(t, n_tiles)
    t = table.copy(); t["tile_rows"][0] = 4096; t["tile_begin"][1] = 1  # 4096 rows x 512 bytes do not fit a 32 KiB stage
    assert "exceeds one pipeline stage" in refused(t, 1 + int(n_tiles - table["tile_begin"][1]))
    t = table.copy(); t["src"][0] += 2
    assert "bulk source rule" in refused(t, n_tiles)
    t = table.copy(); t["op"][0] = OP_FP8_BLOCK + 1
    assert "unknown op" in refused(t, n_tiles)
    t = table.copy(); t["rows"][1] = 0
    assert "empty slab" in refused(t, n_tiles)
