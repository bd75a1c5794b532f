"""Column-wise L2 normalisation on the device (``csrc/col_normalize.cu``):
``out[r, c] = x[r, c] / max(||x[:, c]||_2, eps)``, i.e.
``torch.nn.functional.normalize(x, dim=0, p=2, eps=eps)`` without its
temporaries.  On CPU tensors the PyTorch function runs.  It produces the head
with unit-norm columns that the reference computes with that PyTorch call while
converting the output layer (`awex/converter/mcore_converter.py:668-675`)."""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

_DT = {torch.bfloat16: 1, torch.float16: 2, torch.float32: 3}
_scratch: Dict[Tuple[int, int], torch.Tensor] = {}


def col_l2_normalize(x: torch.Tensor, out: Optional[torch.Tensor] = None, eps: float = 1e-7) -> torch.Tensor:
    if not x.is_cuda:
        value = torch.nn.functional.normalize(x, dim=0, p=2, eps=eps)
        if out is None:
            return value
        out.copy_(value)
        return out
    from awex_b200.ops import native

    if x.dim() != 2 or x.dtype not in _DT:
        raise TypeError(f"column normalisation takes a 2-D bf16 / fp16 / fp32 tensor, got {tuple(x.shape)} {x.dtype}")
    if x.stride(1) != 1:
        x = x.contiguous()
    rows, cols = x.shape
    if out is None:
        out = torch.empty((rows, cols), dtype=x.dtype, device=x.device)
    if out.shape != x.shape or out.dtype != x.dtype or out.stride(1) != 1:
        raise ValueError("output must be a row-major tensor of the input's shape and dtype")
    lib = native.load()
    need = int(lib.awex_col_normalize_scratch_floats(rows, cols))
    key = (x.device.index or 0, need)
    scratch = _scratch.get(key)
    if scratch is None:  # kept: an update reuses it, so that nothing is allocated per update
        scratch = _scratch[key] = torch.empty(need, dtype=torch.float32, device=x.device)
    code = lib.awex_launch_col_l2_normalize(x.data_ptr(), out.data_ptr(), scratch.data_ptr(), rows, cols, x.stride(0), out.stride(0),
                                            _DT[x.dtype], float(eps), native.current_stream_ptr())
    native.check(code, "col_l2_normalize launch")
    return out
