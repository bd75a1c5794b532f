"""RDMA ("astate") mode, reader side: API surface only
(`awex/reader/astate_reader.py:26-85` in the reference: ``multi_get(step,
pairs)`` in place, then ``complete``)."""

from __future__ import annotations

from awex_b200.reader.weights_reader import WeightsReader
from awex_b200.writer.astate_writer import _import_astate


class AStateWeightsReader(WeightsReader):
    def _initialize(self) -> None:
        _import_astate()
        super()._initialize()
