"""Symbolic row algebra for layout conversion.

Every training-side layout transform the exchange needs (QKV de-interleave,
regrouping per inference TP rank with KV-head duplication, gate/up split,
MLA a-proj packing, gated-QKV and Gated-DeltaNet packs) is a permutation, with
possible duplication, of dim-0 rows of one or a few source tensors.  A
:class:`Rows` object records such a permutation as an ordered list of runs
``(source, first_row, n_rows)`` without touching tensor data.  From it we get

* the converted tensor's shape for metadata, without running the transform;
* a materialised tensor when a caller asks for one (CPU oracle, file backend);
* the address map of the fused transfer kernel, so that no converted
  intermediate ever exists in device memory.

A *source* is ``(param_name, tp_rank)``: ``tp_rank`` names the training
tensor-parallel peer that physically holds the rows, which is how a transform
that the reference implements with an all-gather over the TP group
(`awex/converter/mcore_converter.py:1040-1052`) becomes gather-free here: each
rank simply moves the rows it owns.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Hashable, Iterable, List, Optional, Sequence, Tuple

import torch

Source = Hashable
Run = Tuple[Source, int, int]  # (source, first_row, n_rows)


class Rows:
    __slots__ = ("runs", "_n")

    def __init__(self, runs: Iterable[Run]):
        merged: List[Run] = []
        for src, start, n in runs:
            if n <= 0:
                continue
            if merged and merged[-1][0] == src and merged[-1][1] + merged[-1][2] == start:
                merged[-1] = (src, merged[-1][1], merged[-1][2] + n)
            else:
                merged.append((src, start, n))
        self.runs = merged
        self._n = sum(r[2] for r in merged)

    # ---- constructors ----------------------------------------------------
    @staticmethod
    def full(source: Source, n_rows: int) -> "Rows":
        return Rows([(source, 0, n_rows)])

    @staticmethod
    def cat(parts: Sequence["Rows"]) -> "Rows":
        return Rows(run for p in parts for run in p.runs)

    # ---- queries -----------------------------------------------------------
    def __len__(self) -> int:
        return self._n

    def __repr__(self) -> str:
        return f"Rows(n={self._n}, runs={self.runs[:4]}{'...' if len(self.runs) > 4 else ''})"

    def __eq__(self, other) -> bool:
        return isinstance(other, Rows) and self.runs == other.runs

    def sources(self) -> List[Source]:
        seen: Dict[Source, None] = {}
        for src, _, _ in self.runs:
            seen.setdefault(src)
        return list(seen)

    # ---- algebra -------------------------------------------------------------
    def narrow(self, start: int, length: int) -> "Rows":
        if start < 0 or length < 0 or start + length > self._n:
            raise IndexError(f"narrow({start}, {length}) out of range for {self._n} rows")
        out: List[Run] = []
        pos = 0
        end = start + length
        for src, s, n in self.runs:
            lo, hi = max(pos, start), min(pos + n, end)
            if lo < hi:
                out.append((src, s + (lo - pos), hi - lo))
            pos += n
            if pos >= end:
                break
        return Rows(out)

    def split(self, sizes: Sequence[int]) -> List["Rows"]:
        if sum(sizes) != self._n:
            raise ValueError(f"split sizes {list(sizes)} do not sum to {self._n}")
        out, pos = [], 0
        for size in sizes:
            out.append(self.narrow(pos, size))
            pos += size
        return out

    def chunk(self, n_chunks: int) -> List["Rows"]:
        if n_chunks <= 0 or self._n % n_chunks != 0:
            raise ValueError(f"{self._n} rows cannot be cut into {n_chunks} equal chunks")
        return self.split([self._n // n_chunks] * n_chunks)

    def blocks(self, block_rows: int) -> List["Rows"]:
        return self.chunk(self._n // block_rows) if self._n else []

    # ---- realisation -----------------------------------------------------------
    def gather(self, fetch: Callable[[Source], torch.Tensor]) -> torch.Tensor:
        """Build the described tensor.  A single run comes back as a view of
        its source; several runs are concatenated into a new tensor."""
        pieces = [fetch(src).narrow(0, s, n) for src, s, n in self.runs]
        if len(pieces) == 1:
            return pieces[0]
        return torch.cat(pieces, dim=0)

    def segments(self, start: int = 0, length: Optional[int] = None) -> List[Tuple[int, Source, int, int]]:
        """Runs covering destination rows ``[start, start+length)`` as
        ``(dst_row_relative_to_start, source, src_row, n_rows)``."""
        length = self._n - start if length is None else length
        out, pos, end = [], 0, start + length
        for src, s, n in self.runs:
            lo, hi = max(pos, start), min(pos + n, end)
            if lo < hi:
                out.append((lo - start, src, s + (lo - pos), hi - lo))
            pos += n
            if pos >= end:
                break
        return out


# ---- value transforms applied after the row map ---------------------------------
@dataclass(frozen=True)
class ValueOp:
    """Elementwise (or block-wise) change of values that rides along with a
    transfer.  ``kind``: "none" | "cast" | "add" | "l2norm_dim0" | "fp8_block".
    """

    kind: str = "none"
    dtype: Optional[torch.dtype] = None  # target dtype of a cast / fp8 block quant
    const: float = 0.0  # addend for "add"
    ue8m0: bool = False  # power-of-two scales for "fp8_block"

    def out_dtype(self, src_dtype: torch.dtype) -> torch.dtype:
        if self.kind in ("cast", "fp8_block") and self.dtype is not None:
            return self.dtype
        return src_dtype

    def apply(self, t: torch.Tensor) -> torch.Tensor:
        if self.kind == "none":
            return t
        if self.kind == "cast":
            return t.to(self.dtype)
        if self.kind == "add":
            return t + self.const
        if self.kind == "l2norm_dim0":
            return torch.nn.functional.normalize(t, dim=0, p=2, eps=1e-7)
        raise ValueError(f"value op {self.kind!r} has no single-tensor form")


IDENTITY = ValueOp()


@dataclass
class TensorSpec:
    """One canonical (HF-named) tensor described in terms of training tensors."""

    name: str
    rows: Optional[Rows]  # None for 0-d tensors
    trailing: Tuple[int, ...]  # shape[1:]
    src_dtype: torch.dtype
    value_op: ValueOp = IDENTITY
    # for block-scale tensors: name of the weight whose quantisation produces it
    scale_of: Optional[str] = None

    @property
    def shape(self) -> Tuple[int, ...]:
        if self.rows is None:
            return ()
        return (len(self.rows),) + tuple(self.trailing)

    @property
    def dtype(self) -> torch.dtype:
        return self.value_op.out_dtype(self.src_dtype)

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n
