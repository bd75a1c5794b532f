"""Block fp8 kernels against the plain-PyTorch fp32 statement of the same op."""

import pytest
import torch

from awex_b200.converter.weights_converter import per_block_cast_to_fp8, per_block_dequant_from_fp8

pytestmark = pytest.mark.gpu


def _same_fp8(a, b):
    return torch.equal(a.view(torch.uint8), b.view(torch.uint8))


@pytest.mark.parametrize("shape", [(256, 512), (192, 4096), (130, 136), (1, 128), (384, 72)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("ue8m0", [False, True])
def test_block_quant_matches_torch(shape, dtype, ue8m0):
    from awex_b200.ops.fp8 import block_quant

    g = torch.Generator(device="cuda").manual_seed(3)
    x = (torch.randn(shape, generator=g, device="cuda") * 0.05).to(dtype)
    x[0, 0] = 3.0  # a block whose amax is far from the bulk
    q, s = block_quant(x, ue8m0)
    q_ref, s_ref = per_block_cast_to_fp8(x.cpu(), ue8m0)
    torch.cuda.synchronize()
    assert torch.equal(s.cpu(), s_ref)
    assert _same_fp8(q.cpu(), q_ref)


def test_block_quant_special_values():
    from awex_b200.ops.fp8 import block_quant

    x = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda")
    x[:128, :128] = 0.0                      # all-zero block: scale is the 1e-4 floor
    x[:128, 128:] = 2.0 ** -3                # exact power of two
    x[128:, :128] = torch.linspace(-4, 4, 128 * 128, device="cuda").view(128, 128).to(torch.bfloat16)
    x[130, 130] = float("nan")               # NaN poisons its block, as torch.amax does
    x[200, 200] = 1.0
    for ue8m0 in (False, True):
        q, s = block_quant(x, ue8m0)
        q_ref, s_ref = per_block_cast_to_fp8(x.cpu(), ue8m0)
        torch.cuda.synchronize()
        assert torch.equal(torch.nan_to_num(s.cpu(), nan=-1.0), torch.nan_to_num(s_ref, nan=-1.0))
        assert _same_fp8(q.cpu(), q_ref)


@pytest.mark.parametrize("ue8m0", [False, True])
def test_scale_rule_is_exact_for_every_16_bit_amax(ue8m0):
    """Every block maximum a bf16 or fp16 tensor can have (all non-negative bit
    patterns, infinity and NaN included) through the kernels' scale rule, against
    PyTorch's fp32 statement on the CPU."""
    from awex_b200.ops.fp8 import quant_scales

    bf16 = (torch.arange(0, 0x8000, dtype=torch.int32) << 16).view(torch.float32)
    fp16 = torch.arange(0, 0x8000, dtype=torch.int32).to(torch.int16).view(torch.float16).float()
    for amax in (bf16, fp16):
        want = amax.clamp(min=1e-4) / 448.0
        if ue8m0:
            want = want.clamp(min=1e-10).log2().ceil().exp2()
        got = quant_scales(amax.cuda(), ue8m0).cpu()
        assert torch.equal(torch.isnan(got), torch.isnan(want))
        assert torch.equal(torch.nan_to_num(got, nan=0.0), torch.nan_to_num(want, nan=0.0))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_division_free_quotient_is_exact_for_every_value_and_every_scale(dtype):
    """The kernels quantise 16-bit sources without a division (one correction step on
    x * RN(1 / scale)).  Every value of the type against every block maximum of the
    type, plain and power-of-two scales: the e4m3 byte must equal what the true
    division gives.  (The fp32 quotient itself may differ in its last bit in rare
    cases; the count is returned for information.)"""
    from awex_b200.ops.fp8 import quotient_check

    bad_bytes, bad_quotients, checked = quotient_check(dtype)
    assert checked > 2_000_000_000
    assert bad_bytes == 0, getattr(quotient_check, "example", None)
    assert bad_quotients < checked // 1000


def test_unaligned_rows_take_the_transfer_kernel_path():
    from awex_b200.ops.fp8 import block_quant

    base = (torch.randn(200, 1001, device="cuda") * 0.1).to(torch.bfloat16)
    x = base[:, 1:]  # pitch 2002 bytes and a 2-byte offset: not TMA-loadable
    q, s = block_quant(x)
    q_ref, s_ref = per_block_cast_to_fp8(x.cpu().contiguous(), False)
    torch.cuda.synchronize()
    assert torch.equal(s.cpu(), s_ref) and _same_fp8(q.cpu(), q_ref)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_block_dequant_matches_torch(out_dtype):
    from awex_b200.ops.fp8 import block_dequant, block_quant

    x = (torch.randn(300, 520, device="cuda") * 0.1).to(torch.bfloat16)
    q, s = block_quant(x)
    y = block_dequant(q, s, out_dtype)
    want = per_block_dequant_from_fp8(q.cpu(), s.cpu(), out_dtype)
    torch.cuda.synchronize()
    assert torch.equal(y.cpu(), want)
    assert (y.float() - x.float()).abs().max().item() < 0.05


@pytest.mark.parametrize("arch,train,infer", [
    ("tiny-qwen3-moe", dict(tp=1, dp=2, ep=2), dict(tp=1, fp8=True)),  # blocks gather rows of de-interleaved Q/K/V
    ("tiny-llama", dict(tp=1), dict(tp=2, fp8=True)),
])
def test_fused_transfer_quantises_like_torch(arch, train, infer):
    """Training bf16 shards -> inference fp8 shards with scales, quantised inside
    the transfer kernel, compared with quantising the destination-layout bf16
    shards in PyTorch."""
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout

    job = SimulatedJob(get_arch(arch), TrainLayout(**train), InferLayout(**infer), dtype=torch.bfloat16, device="cuda")
    job.compile_all()
    assert job.check_coverage() == []
    job.build_gpu_programs()
    job.run_gpu(1)
    torch.cuda.synchronize()
    job.gpu_status()
    assert job.mismatches() == []
