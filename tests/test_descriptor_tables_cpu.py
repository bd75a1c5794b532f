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
