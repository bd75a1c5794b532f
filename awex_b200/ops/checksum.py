"""Device checksums of many tensors in one launch (``csrc/checksum.cu``) and
the same function in numpy as its oracle.

``checksum = sum_i mix(word_i) * (GOLDEN * (2 i + 1)) mod 2**64`` with
``mix(w) = w ^ (w >> 32)`` over the 8-byte words of each row (last word
zero-padded), ``i = row * words_per_row + j``.
Contiguous tensors are hashed as one long row.

Validation of an update compares these sums with the sums of a file-loaded
copy; the reference compares the tensors themselves, parameter by parameter
(`awex/reader/weights_reader.py:457-587`, `awex/util/tensor_util.py:431-537`).
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from awex_b200.ops import native
from awex_b200.transfer.descriptors import _DT_CODE

SUM_DTYPE = np.dtype(
    [("ptr", "<u8"), ("rows", "<u8"), ("row_bytes", "<u8"), ("stride", "<i8"), ("chunk_begin", "<u8"),
     ("rows_per_chunk", "<u4"), ("chunks_per_row", "<u4"), ("out_index", "<u4"), ("dtype", "<u4"), ("pad", "<u8")]
)
assert SUM_DTYPE.itemsize == 64
GOLDEN = np.uint64(0x9E3779B97F4A7C15)


def _as_rows(t: torch.Tensor) -> Tuple[int, int, int]:
    """(rows, row_bytes, stride_bytes) view of a tensor whose inner dims are
    contiguous; fully contiguous tensors become a single row."""
    es = t.element_size()
    if t.is_contiguous():
        return 1, t.numel() * es, 0
    if t.dim() >= 2 and t[0].is_contiguous():
        return t.shape[0], t[0].numel() * es, t.stride(0) * es
    raise ValueError("checksum needs a tensor whose rows are contiguous")


def checksum_reference(t: torch.Tensor) -> int:
    """numpy statement of the checksum (CPU tensors or copies of GPU ones)."""
    rows, row_bytes, _ = _as_rows(t)
    raw = t.detach().cpu().contiguous().view(torch.uint8).numpy().reshape(rows, row_bytes)
    wpr = -(-row_bytes // 8)
    padded = np.zeros((rows, wpr * 8), dtype=np.uint8)
    padded[:, :row_bytes] = raw
    words = padded.view("<u8").reshape(-1)
    with np.errstate(over="ignore"):
        idx = np.arange(words.size, dtype=np.uint64)
        keys = GOLDEN * (np.uint64(2) * idx + np.uint64(1))
        mixed = words ^ (words >> np.uint64(32))
        return int((mixed * keys).sum(dtype=np.uint64))


class ChecksumPlan:
    """Fixed list of tensors whose checksums are recomputed on demand."""

    def __init__(self, tensors: Sequence[torch.Tensor], device=None):
        self.lib = native.load()
        assert self.lib.awex_sum_desc_size() == SUM_DTYPE.itemsize
        self.device = torch.device(device) if device is not None else tensors[0].device
        self.n = len(tensors)
        CHUNK_WORDS = int(self.lib.awex_sum_chunk_words())  # words one CTA sums per step; fixed by the kernel
        table = np.zeros(self.n, dtype=SUM_DTYPE)
        chunks = 0
        for i, t in enumerate(tensors):
            rows, row_bytes, stride = _as_rows(t)
            wpr = -(-row_bytes // 8)
            if wpr >= CHUNK_WORDS or rows == 1:
                rpc, cpr = 1, max(1, -(-wpr // CHUNK_WORDS))
                n_chunks = rows * cpr
            else:
                rpc, cpr = max(1, CHUNK_WORDS // max(wpr, 1)), 1
                n_chunks = -(-rows // rpc)
            table[i] = (t.data_ptr(), rows, row_bytes, stride, chunks, rpc, cpr, i, _DT_CODE.get(t.dtype, 0), 0)
            chunks += n_chunks if t.numel() else 0
        self.n_chunks = chunks
        self.table = torch.from_numpy(table.view(np.uint8).reshape(-1).copy()).to(self.device)
        self.out = torch.zeros(2, max(self.n, 1), dtype=torch.int64, device=self.device)
        self.launches = 0
        self.nbytes = sum(t.numel() * t.element_size() for t in tensors)

    def launch(self, stream_ptr: Optional[int] = None) -> torch.Tensor:
        """Returns the device tensor ``[2, n]`` (checksums, NaN counts); reading
        it on the host synchronises."""
        stream = native.current_stream_ptr() if stream_ptr is None else stream_ptr
        self.out.zero_()
        code = self.lib.awex_launch_checksum(
            self.table.data_ptr(), self.n, self.n_chunks, self.out[0].data_ptr(), self.out[1].data_ptr(), 0, stream
        )
        native.check(code, "checksum launch")
        self.launches += 1
        return self.out

    def run(self) -> Tuple[List[int], List[int]]:
        out = self.launch().cpu()
        sums = [int(v) & 0xFFFFFFFFFFFFFFFF for v in out[0].tolist()]
        return sums, [int(v) for v in out[1].tolist()]


def tensor_checksums(tensors: Sequence[torch.Tensor]) -> Tuple[List[int], List[int]]:
    if not tensors:
        return [], []
    if tensors[0].is_cuda:
        return ChecksumPlan(tensors).run()
    return [checksum_reference(t) for t in tensors], [int(torch.isnan(t.float()).sum()) if t.is_floating_point() else 0 for t in tensors]
