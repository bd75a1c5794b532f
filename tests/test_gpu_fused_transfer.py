"""GPU tests of the fused transfer kernel: every rank of a layout is emulated
on one device (one launch per training rank over that rank's data), and the
inference parameters must equal, bit for bit, the layout built directly from
the canonical weights (the plain-PyTorch oracle)."""

import pytest
import torch

from awex_b200.synthetic.arch import get_arch
from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout

pytestmark = pytest.mark.gpu

LAYOUTS = [
    ("tiny-llama", TrainLayout(tp=2), InferLayout(tp=1), torch.float32),
    ("tiny-llama", TrainLayout(tp=1), InferLayout(tp=1), torch.bfloat16),
    ("tiny-qwen2", TrainLayout(tp=4), InferLayout(tp=2, num_engines=2), torch.bfloat16),
    ("tiny-qwen2", TrainLayout(tp=2), InferLayout(tp=8), torch.bfloat16),
    ("tiny-qwen2", TrainLayout(tp=2, pp=2), InferLayout(tp=4), torch.float16),
    ("tiny-qwen3-moe", TrainLayout(tp=1, dp=4, ep=4), InferLayout(tp=2, ep=2, num_engines=2), torch.bfloat16),
    ("tiny-qwen3-moe", TrainLayout(tp=2, dp=2, ep=4), InferLayout(tp=4), torch.bfloat16),
]


@pytest.mark.parametrize("arch,train,infer,dtype", LAYOUTS, ids=lambda v: v.label() if hasattr(v, "label") else str(v))
def test_fused_transfer_bitwise(arch, train, infer, dtype):
    job = SimulatedJob(get_arch(arch), train, infer, dtype=dtype, device="cuda")
    job.compile_all()
    assert job.check_coverage() == []
    job.build_gpu_programs()
    for epoch in (1, 2):
        if epoch == 2:  # second update must overwrite, not accumulate
            for models in job.infer_models:
                for m in models:
                    for p in m.parameters():
                        p.fill_(7)
        job.run_gpu(epoch)
        torch.cuda.synchronize()
        job.gpu_status()
        assert job.mismatches() == []


def test_wait_times_out_and_reports():
    """A flag nobody raises: the wait returns within its deadline, records the
    slot, and the CUDA context stays usable."""
    from awex_b200.ops.fused_transfer import FlagPad, FlagWaiter, TransferError

    pad = FlagPad(4, "cuda")
    waiter = FlagWaiter(pad, [0, 3], "cuda", timeout_ms=50)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    waiter.launch(epoch=5)
    stop.record()
    torch.cuda.synchronize()
    assert start.elapsed_time(stop) < 1000
    with pytest.raises(TransferError) as err:
        waiter.status.raise_if_failed()
    assert err.value.code == 3 and err.value.detail[0] in (0, 3)
    pad.t.fill_(5)
    waiter.launch(epoch=5)
    torch.cuda.synchronize()
    waiter.status.raise_if_failed()
    assert torch.ones(4, device="cuda").sum().item() == 4


def test_sender_gives_up_when_destination_never_ready():
    from awex_b200.ops.fused_transfer import FlagPad, TransferError, TransferProgram
    from awex_b200.transfer.descriptors import TensorAddr, encode_items
    from awex_b200.transfer.lowering import CopyItem

    src = torch.arange(4096, dtype=torch.float32, device="cuda")
    dst = torch.zeros_like(src)
    item = CopyItem("w", 0, (0,), (4096,), 0, "w", (0,), torch.float32, torch.float32)
    table, n_tiles, _ = encode_items([item], {("w", 0): TensorAddr.of(src)}, {0: {"w": TensorAddr.of(dst)}})
    ready, done = FlagPad(1, "cuda"), FlagPad(1, "cuda")
    prog = TransferProgram(table, n_tiles, "cuda", ready_pad=ready, ready_slots=[0], done_flag_addrs=[done.slot_addr(0)], timeout_ms=50)
    prog.launch(epoch=1)
    torch.cuda.synchronize()
    with pytest.raises(TransferError) as err:
        prog.status.raise_if_failed()
    assert err.value.code == 1
    assert dst.abs().sum().item() == 0 and done.t.item() == 0  # nothing written, nothing signalled
    ready.t.fill_(1)
    prog.launch(epoch=1)
    torch.cuda.synchronize()
    prog.status.raise_if_failed()
    assert torch.equal(dst, src) and done.t.item() == 1


@pytest.mark.parametrize("shape,dtype", [((1000, 1000), torch.bfloat16), ((4097,), torch.float32), ((33, 17), torch.float32), ((5, 3, 64), torch.float16)])
def test_checksum_matches_numpy(shape, dtype):
    from awex_b200.ops.checksum import ChecksumPlan, checksum_reference

    g = torch.Generator(device="cuda").manual_seed(1)
    full = torch.randn(shape, generator=g, device="cuda").to(dtype)
    tensors = [full]
    if len(shape) == 2:
        tensors.append(full[:, : shape[1] // 2])  # strided rows
        tensors.append(full[1:])
    sums, nans = ChecksumPlan(tensors).run()
    assert sums == [checksum_reference(t) for t in tensors]
    assert nans == [0] * len(tensors)
    # position sensitivity: swapping two rows changes the sum; NaNs are counted
    if len(shape) == 2:
        swapped = full.clone()
        swapped[[0, 1]] = swapped[[1, 0]]
        assert ChecksumPlan([swapped]).run()[0][0] != sums[0]
    poisoned = full.clone()
    poisoned.view(-1)[3] = float("nan")
    assert ChecksumPlan([poisoned]).run()[1][0] == 1


def test_unaligned_and_cast_paths():
    """Odd sizes and offsets take the element path; dtype casts and constant
    adds ride along."""
    from awex_b200.converter.rows import ValueOp
    from awex_b200.ops.fused_transfer import TransferProgram
    from awex_b200.transfer.descriptors import TensorAddr, encode_items, validate_table
    from awex_b200.transfer.lowering import CopyItem

    g = torch.Generator(device="cuda").manual_seed(2)
    src = torch.randn(37, 101, generator=g, device="cuda").to(torch.bfloat16)
    dst_copy = torch.zeros(40, 120, dtype=torch.bfloat16, device="cuda")
    dst_f32 = torch.zeros(37, 101, dtype=torch.float32, device="cuda")
    dst_add = torch.zeros(37, 101, dtype=torch.bfloat16, device="cuda")
    big = torch.randn(512, 4096, generator=g, device="cuda").to(torch.bfloat16)
    big_f32 = torch.zeros(512, 4096, dtype=torch.float32, device="cuda")
    items = [
        CopyItem("s", 0, (3, 5), (30, 90), 0, "copy", (2, 7), torch.bfloat16, torch.bfloat16),
        CopyItem("s", 0, (0, 0), (37, 101), 0, "f32", (0, 0), torch.bfloat16, torch.float32, ValueOp("cast", dtype=torch.float32)),
        CopyItem("s", 0, (0, 0), (37, 101), 0, "add", (0, 0), torch.bfloat16, torch.bfloat16, ValueOp("add", const=1.0)),
        CopyItem("b", 0, (0, 0), (512, 4096), 0, "bigf32", (0, 0), torch.bfloat16, torch.float32, ValueOp("cast", dtype=torch.float32)),
    ]
    srcs = {("s", 0): TensorAddr.of(src), ("b", 0): TensorAddr.of(big)}
    dsts = {0: {"copy": TensorAddr.of(dst_copy), "f32": TensorAddr.of(dst_f32), "add": TensorAddr.of(dst_add), "bigf32": TensorAddr.of(big_f32)}}
    table, n_tiles, _ = encode_items(items, srcs, dsts)
    assert validate_table(table, n_tiles, [a.byte_span() for a in srcs.values()], [a.byte_span() for a in dsts[0].values()]) == []
    prog = TransferProgram(table, n_tiles, "cuda")
    prog.launch(1)
    torch.cuda.synchronize()
    prog.status.raise_if_failed()
    want = torch.zeros_like(dst_copy)
    want[2:32, 7:97] = src[3:33, 5:95]
    assert torch.equal(dst_copy, want)
    assert torch.equal(dst_f32, src.float())
    assert torch.equal(dst_add, (src.float() + 1.0).to(torch.bfloat16))
    assert torch.equal(big_f32, big.float())
