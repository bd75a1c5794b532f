"""Block-scaled fp8 (e4m3) quantisation contract and scale-tensor naming.

A quantised weight travels under its own name and its scales under
``<name>_scale_inv`` (`awex/converter/weights_converter.py:25-61` in the
reference).  :func:`per_block_cast_to_fp8` is the plain-PyTorch statement of
the math and the oracle for the CUDA kernels: 128x128 blocks over a
zero-padded copy, ``scale = max(amax, 1e-4) / 448`` in fp32 (optionally rounded
up to a power of two), ``q = fp8(x / scale)`` with a true division.
"""

from __future__ import annotations

from typing import Tuple

import torch

FP8_BLOCK = 128
FP8_E4M3_MAX = 448.0
SCALE_SUFFIX = "_scale_inv"


def normalize_scale_inv_name(name: str) -> Tuple[str, bool]:
    if name.endswith(SCALE_SUFFIX):
        return name[: -len(SCALE_SUFFIX)], True
    return name, False


def append_scale_inv(name: str, has_scale_inv: bool) -> str:
    return name + SCALE_SUFFIX if has_scale_inv else name


def ceil_div(x: int, y: int) -> int:
    return -(-x // y)


def block_scale_shape(rows: int, cols: int) -> Tuple[int, int]:
    return ceil_div(rows, FP8_BLOCK), ceil_div(cols, FP8_BLOCK)


def per_block_cast_to_fp8(x: torch.Tensor, scale_ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(q[m, n] float8_e4m3fn, scale[ceil(m/128), ceil(n/128)] float32)``."""
    assert x.dim() == 2, "block quantisation is defined for 2-D weights"
    m, n = x.shape
    bm, bn = block_scale_shape(m, n)
    padded = x.new_zeros((bm * FP8_BLOCK, bn * FP8_BLOCK))
    padded[:m, :n] = x
    tiles = padded.view(bm, FP8_BLOCK, bn, FP8_BLOCK)
    scale = tiles.abs().float().amax(dim=(1, 3), keepdim=True).clamp(min=1e-4) / FP8_E4M3_MAX
    if scale_ue8m0:
        scale = scale.clamp(min=1e-10).log2().ceil().exp2()
    q = (tiles / scale).to(torch.float8_e4m3fn)
    return q.view_as(padded)[:m, :n].contiguous(), scale.view(bm, bn)


def per_block_dequant_from_fp8(q: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Inverse map used by validation: ``x ~= float(q) * scale`` per block."""
    m, n = q.shape
    s = scale.repeat_interleave(FP8_BLOCK, 0)[:m].repeat_interleave(FP8_BLOCK, 1)[:, :n]
    return (q.float() * s).to(dtype)
