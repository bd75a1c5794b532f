"""The file backend (checkpoint round trip through the engines' own save / load)
and the RDMA-table backend driven against an in-memory stand-in of the table
library: training TP=2 puts canonical shards, one inference worker gets its
(differently cut) shards in place."""

import sys
import threading
import types

import pytest
import torch

from awex_b200.synthetic.arch import get_arch
from awex_b200.synthetic.harness import SyntheticInferenceEngine, SyntheticTrainEngine
from awex_b200.synthetic.simulate import InferLayout
from awex_b200.synthetic.topology import infer_rank_infos, train_rank_infos


def test_file_backend_round_trip(tmp_path):
    from awex_b200.reader.weights_reader import FileWeightExchangeReader, get_weights_exchange_reader
    from awex_b200.writer.weights_writer import FileWeightExchangeWriter, get_weights_exchange_writer

    arch = get_arch("tiny-llama")
    train = SyntheticTrainEngine(arch, train_rank_infos()[0], "127.0.0.1:1", dtype=torch.float32, comm_backend="file")
    infer = SyntheticInferenceEngine(arch, InferLayout(tp=1), infer_rank_infos()[0], "127.0.0.1:1", dtype=torch.float32, comm_backend="file")
    writer, reader = get_weights_exchange_writer(train), get_weights_exchange_reader(infer)
    assert isinstance(writer, FileWeightExchangeWriter) and isinstance(reader, FileWeightExchangeReader)
    writer.initialize()
    reader.initialize()
    with pytest.raises(ValueError):
        writer.write_weights(step_id=1)
    with pytest.raises(ValueError):
        reader.update_weights(step_id=1)
    assert infer.mismatches() != []  # the engine starts zeroed
    writer.write_weights(step_id=1, path=str(tmp_path))
    reader.update_weights(step_id=1, path=str(tmp_path))
    assert infer.mismatches() == []


# ------------------------------------------------------------------------------------------ RDMA table stand-in
class _Table:
    """What the table library does for one job: put shards by (name, global
    shape, offset), get any box of a name assembled from the shards that cover it."""

    def __init__(self):
        self.shards, self.completed, self.lock = {}, [], threading.Lock()
        self.configs = []
        self.put_done = threading.Event()

    def multi_put(self, step, pairs):
        with self.lock:
            for (name, shape, offset), tensor in pairs:
                self.shards.setdefault((step, name), []).append((tuple(offset), tensor.detach().clone()))
        self.put_done.set()

    def multi_get(self, step, pairs):
        assert self.put_done.wait(60), "no writer has put this step"  # a real table blocks until the data is there
        for (name, shape, offset), out in pairs:
            covered = torch.zeros(out.shape, dtype=torch.bool)
            for src_off, src in self.shards.get((step, name), []):
                lo = [max(a, b) for a, b in zip(offset, src_off)]
                hi = [min(a + n, b + m) for a, n, b, m in zip(offset, out.shape, src_off, src.shape)]
                if any(h <= l for l, h in zip(lo, hi)):
                    continue
                dst_sl = tuple(slice(l - a, h - a) for l, h, a in zip(lo, hi, offset))
                src_sl = tuple(slice(l - b, h - b) for l, h, b in zip(lo, hi, src_off))
                out[dst_sl].copy_(src[src_sl])
                covered[dst_sl] = True
            assert bool(covered.all()), f"{name}: the table does not hold all of box {offset}+{tuple(out.shape)}"

    def complete(self, step):
        with self.lock:
            self.completed.append(step)


def _install_fake_astate(monkeypatch):
    table = _Table()
    astate = types.ModuleType("astate")
    utils = types.ModuleType("astate.utils")
    utils.create_sharded_key = lambda name, global_shape, global_offset: (name, tuple(global_shape), tuple(global_offset))

    class ParallelConfig:
        @staticmethod
        def create_training_config(**kw):
            return ("train", kw)

        @staticmethod
        def create_inference_config(**kw):
            return ("infer", kw)

    def create_remote_table(name, parallel_config=None):
        assert name == "weights_exchange"
        table.configs.append(parallel_config)
        return table

    astate.ParallelConfig, astate.create_remote_table, astate.utils = ParallelConfig, create_remote_table, utils
    monkeypatch.setitem(sys.modules, "astate", astate)
    monkeypatch.setitem(sys.modules, "astate.utils", utils)
    return table


def test_astate_backend_needs_the_library():
    from awex_b200.writer.astate_writer import _import_astate

    assert "astate" not in sys.modules
    with pytest.raises(RuntimeError, match="astate RDMA library"):
        _import_astate()


@pytest.mark.timeout(120)
def test_astate_backend_against_an_in_memory_table(monkeypatch):
    import torch.distributed as dist

    from awex_b200.meta.meta_server import MetaServer
    from awex_b200.reader.astate_reader import AStateWeightsReader
    from awex_b200.reader.weights_reader import get_weights_exchange_reader
    from awex_b200.writer.astate_writer import AStateWeightsWriter
    from awex_b200.writer.weights_writer import get_weights_exchange_writer

    table = _install_fake_astate(monkeypatch)
    monkeypatch.setenv("AWEX_DEVICE_TYPE", "cpu")
    server = MetaServer("127.0.0.1", 0)
    server.start()
    addr = f"127.0.0.1:{server.port}"
    arch = get_arch("tiny-llama")
    try:
        train = SyntheticTrainEngine(arch, train_rank_infos()[0], addr, dtype=torch.float32, comm_backend="astate")
        infer = SyntheticInferenceEngine(arch, InferLayout(tp=1), infer_rank_infos()[0], addr, dtype=torch.float32, comm_backend="astate")
        writer, reader = get_weights_exchange_writer(train), get_weights_exchange_reader(infer)
        assert isinstance(writer, AStateWeightsWriter) and isinstance(reader, AStateWeightsReader)
        writer.initialize()
        reader.initialize()
        errors = []

        def read():
            try:
                reader.update_weights(step_id=1)
            except BaseException as exc:
                errors.append(exc)

        # the reader's first update blocks on the training metadata, the writer's on the inference metadata
        t = threading.Thread(target=read)
        t.start()
        writer.prepare()
        writer.write_weights(step_id=1)
        t.join(timeout=60)
        assert not errors, errors
    finally:
        server.stop()
        assert not dist.is_initialized()
    assert [c[0] for c in table.configs] == ["train", "infer"] or sorted(c[0] for c in table.configs) == ["infer", "train"]
    train_cfg = next(c[1] for c in table.configs if c[0] == "train")
    assert train_cfg["role_size"] == 1 and train_cfg["tp_size"] == 1 and train_cfg["cp_size"] == 1
    assert sorted(table.completed) == [1, 1]
    assert infer.mismatches() == []
    assert infer.schedulers[0].flushes == 1
