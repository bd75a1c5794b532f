"""Host-side statements of the numeric contracts the kernels are held to."""

import numpy as np
import torch


def _pow2_ceil(s: np.ndarray) -> np.ndarray:
    """Smallest power of two >= s, from the float's bits (what the kernels do)."""
    b = s.astype(np.float32).view(np.uint32).copy()
    bump = (b & 0x007FFFFF) != 0
    b[bump] = (b[bump] & 0x7F800000) + 0x00800000
    return b.view(np.float32)


def test_power_of_two_scale_rounding_on_bits_equals_log2_ceil_exp2_for_every_16_bit_amax():
    """The UE8M0 scale is defined as fp32 ``log2 -> ceil -> exp2``.  For every
    block maximum a bf16 or fp16 tensor can have, that equals bumping the exponent
    when the mantissa is non-zero, which is how the kernels compute it."""
    bf16 = (torch.arange(0, 0x7F81, dtype=torch.int32) << 16).view(torch.float32)
    fp16 = torch.arange(0, 0x7C01, dtype=torch.int32).to(torch.int16).view(torch.float16).float()
    for amax in (bf16, fp16):
        s = (amax.clamp(min=1e-4) / 448.0).clamp(min=1e-10)
        want = s.log2().ceil().exp2().numpy()
        assert np.array_equal(_pow2_ceil(s.numpy()), want)


def test_checksum_sees_a_swap_of_words_that_differ_only_in_the_top_bit():
    """Two 8-byte words that differ only in bit 63 (the sign of a word's last
    element) exchanged at any distance must change the checksum."""
    from awex_b200.ops.checksum import checksum_reference

    for distance in (1, 2, 64, 4096, 1 << 16):
        words = np.arange(1, (1 << 16) + 8, dtype=np.uint64) * np.uint64(0x0123456789ABCDEF)
        words &= np.uint64(0x7FFFFFFFFFFFFFFF)
        i, j = 3, 3 + distance
        words[j] = words[i] | np.uint64(1 << 63)
        a = torch.from_numpy(words.view(np.int64).copy())
        swapped = words.copy()
        swapped[i], swapped[j] = words[j], words[i]
        b = torch.from_numpy(swapped.view(np.int64).copy())
        assert checksum_reference(a) != checksum_reference(b), distance


def test_checksum_sees_single_bit_flips_and_row_swaps():
    from awex_b200.ops.checksum import checksum_reference

    g = torch.Generator().manual_seed(0)
    t = torch.randn(64, 96, generator=g).to(torch.bfloat16)
    base = checksum_reference(t)
    flipped = t.clone()
    flipped.view(torch.int16)[17, 5] ^= 1
    assert checksum_reference(flipped) != base
    swapped = t.clone()
    swapped[[3, 40]] = t[[40, 3]]
    assert checksum_reference(swapped) != base
