"""Block-scaled fp8 (e4m3, 128x128 blocks, fp32 scales) on the device.

``block_quant`` / ``block_dequant`` launch the stand-alone kernels of
``csrc/fp8_block.cu``.  Inputs that do not meet the TMA alignment rules
(16-byte aligned base, row pitch a multiple of 16 bytes) are quantised by the
fused transfer kernel's element path instead, so there is no PyTorch fallback
on a GPU.  On CPU tensors the plain-PyTorch oracle runs.

The arithmetic is that of the reference's ``per_block_cast_to_fp8``
(`awex/converter/weights_converter.py:42-61`), bit for bit.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from awex_b200.converter.weights_converter import block_scale_shape, per_block_cast_to_fp8, per_block_dequant_from_fp8

_DT = {torch.bfloat16: 1, torch.float16: 2, torch.float32: 3}


def _status(device) -> torch.Tensor:
    return torch.zeros(4, dtype=torch.int32, device=device)


def block_quant(x: torch.Tensor, scale_ue8m0: bool = False, out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(q[m, n] float8_e4m3fn, scale[ceil(m/128), ceil(n/128)] float32)``."""
    assert x.dim() == 2, "block quantisation is defined for 2-D weights"
    if not x.is_cuda:
        return per_block_cast_to_fp8(x, scale_ue8m0)
    from awex_b200.ops import native

    if x.dtype not in _DT:
        raise TypeError(f"unsupported source dtype {x.dtype}")
    if x.stride(1) != 1:
        x = x.contiguous()
    m, n = x.shape
    if out is None:
        q = torch.empty((m, n), dtype=torch.float8_e4m3fn, device=x.device)
        s = torch.empty(block_scale_shape(m, n), dtype=torch.float32, device=x.device)
    else:
        q, s = out
    lib = native.load()
    status = _status(x.device)
    code = lib.awex_launch_fp8_block_quant(
        x.data_ptr(), q.data_ptr(), s.data_ptr(), m, n, x.stride(0), q.stride(0), s.stride(0), _DT[x.dtype], int(scale_ue8m0),
        status.data_ptr(), native.current_stream_ptr(),
    )
    if code == -2:
        _quant_via_transfer_kernel(x, q, s, scale_ue8m0)
        return q, s
    native.check(code, "fp8_block_quant launch")
    block_quant.last_status = status
    return q, s


def _quant_via_transfer_kernel(x, q, s, ue8m0: bool) -> None:
    from awex_b200.converter.rows import ValueOp
    from awex_b200.ops.fused_transfer import TransferProgram
    from awex_b200.transfer.descriptors import TensorAddr, encode_items
    from awex_b200.transfer.lowering import CopyItem

    item = CopyItem("x", 0, (0, 0), tuple(x.shape), 0, "q", (0, 0), x.dtype, torch.float8_e4m3fn,
                    ValueOp("fp8_block", dtype=torch.float8_e4m3fn, ue8m0=ue8m0), scale_name="s", scale_start=(0, 0))
    table, n_tiles, enc = encode_items([item], {("x", 0): TensorAddr.of(x)}, {0: {"q": TensorAddr.of(q), "s": TensorAddr.of(s)}})
    TransferProgram(table, n_tiles, x.device, encoder=enc).launch(1)


def block_dequant(q: torch.Tensor, scale: torch.Tensor, dtype: torch.dtype = torch.bfloat16, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x ~= float(q) * scale`` per 128x128 block."""
    if not q.is_cuda:
        return per_block_dequant_from_fp8(q, scale, dtype)
    from awex_b200.ops import native

    m, n = q.shape
    if out is None:
        out = torch.empty((m, n), dtype=dtype, device=q.device)
    if out.dtype not in _DT:
        raise TypeError(f"unsupported destination dtype {out.dtype}")
    assert q.stride(1) == 1 and out.stride(1) == 1 and scale.stride(1) == 1
    lib = native.load()
    code = lib.awex_launch_fp8_block_dequant(
        q.data_ptr(), scale.data_ptr(), out.data_ptr(), m, n, q.stride(0), scale.stride(0), out.stride(0), _DT[out.dtype],
        native.current_stream_ptr(),
    )
    native.check(code, "fp8_block_dequant launch")
    return out


def quant_scales(amax: torch.Tensor, scale_ue8m0: bool = False) -> torch.Tensor:
    """The scale the kernels derive from each block maximum in ``amax`` (fp32,
    CUDA): ``max(amax, 1e-4) / 448``, optionally rounded up to a power of two."""
    from awex_b200.ops import native

    amax = amax.contiguous().float()
    out = torch.empty_like(amax)
    code = native.load().awex_launch_fp8_scale_table(amax.data_ptr(), out.data_ptr(), amax.numel(), int(scale_ue8m0), native.current_stream_ptr())
    native.check(code, "fp8_scale_table launch")
    return out


def quotient_check(dtype: torch.dtype) -> Tuple[int, int, int]:
    """Run the exhaustive device check of the division-free quotient for a 16-bit
    source type: ``(e4m3 bytes that differ from the true division, fp32 quotients
    that differ, pairs checked)`` over every (value, block maximum, scale kind)."""
    from awex_b200.ops import native

    out = torch.zeros(4, dtype=torch.int64, device="cuda")
    code = native.load().awex_launch_fp8_quotient_check(_DT[dtype], out.data_ptr(), native.current_stream_ptr())
    native.check(code, "fp8_quotient_check launch")
    bad_bytes, bad_quotients, checked, example = (int(v) for v in out.tolist())
    if example:
        e = example & 0xFFFFFFFFFFFFFFFF
        quotient_check.example = dict(amax_bits=hex((e >> 48) & 0xFFFF), value_bits=hex((e >> 32) & 0xFFFF), ue8m0=(e >> 24) & 1,
                                      got=hex((e >> 16) & 0xFF), want=hex((e >> 8) & 0xFF))
    return bad_bytes, bad_quotients, checked
