"""Failure detection on the host, among CPU ranks: a side that never shows up, a
sender whose manifest is missing, a training rank that leaves between two
updates.  Every wait involved is bounded, so each case ends with an exception
within seconds instead of a hang."""

import os
import time

import pytest
import torch
import torch.multiprocessing as mp


def test_writer_gives_up_when_no_inference_side_appears():
    from awex_b200 import NCCLWeightsWriter
    from awex_b200.meta.meta_server import MetaServer
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticTrainEngine
    from awex_b200.synthetic.topology import train_rank_infos

    server = MetaServer("127.0.0.1", 0)
    server.start()
    try:
        engine = SyntheticTrainEngine(get_arch("tiny-llama"), train_rank_infos()[0], f"127.0.0.1:{server.port}", dtype=torch.float32,
                                      host_wait_timeout_s=0.5)
        writer = NCCLWeightsWriter(engine)
        writer.initialize()
        started = time.time()
        with pytest.raises(TimeoutError, match="infer_conf"):
            writer.write_weights(step_id=1)
        assert time.time() - started < 10
    finally:
        server.stop()


def test_reader_gives_up_when_a_sender_never_publishes_its_manifest():
    from awex_b200.meta.meta_server import MetaServer, MetaServerClient
    from awex_b200.transfer.transports import GlooReceiver, _collect_manifests, manifest_key

    server = MetaServer("127.0.0.1", 0)
    server.start()
    try:
        meta = MetaServerClient("127.0.0.1", server.port)
        meta.put_object(manifest_key(1), {"manifest": {0: [("w", (0,), (4,), "torch.float32", None, None)]}, "ready_pad": None})
        started = time.time()
        with pytest.raises(TimeoutError, match="p2p_manifest_2"):
            _collect_manifests(meta, infer_world=1, train_world=2, my_rank=0, timeout=0.5)  # sender 2 is absent
        assert time.time() - started < 10
        receiver = GlooReceiver(meta, {"w": torch.zeros(4)}, 0, 1, 2, ["w"], wait_timeout_s=0.5)
        assert receiver.group is None
    finally:
        server.stop()


def test_missing_or_doubled_writes_are_refused_before_any_transfer():
    from awex_b200.transfer.transports import CoverageError, _check_coverage

    views = {"w": torch.zeros(8, 4)}
    half = [("w", (0, 0), (4, 4), "torch.float32", None, None)]
    with pytest.raises(CoverageError, match="never written"):
        _check_coverage([half], views, ["w"], strict=True, who="rank 0")
    both = half + [("w", (2, 0), (6, 4), "torch.float32", None, None)]
    with pytest.raises(CoverageError, match="overlaps"):
        _check_coverage([both], views, ["w"], strict=True, who="rank 0")
    _check_coverage([half], views, ["w"], strict=False, who="rank 0")  # debug mode only logs


# ------------------------------------------------------------------------------------------ a rank leaves between steps
def _writer_that_leaves(meta_addr, q):
    from awex_b200 import NCCLWeightsWriter
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticTrainEngine
    from awex_b200.synthetic.topology import train_rank_infos

    os.environ["AWEX_DEVICE_TYPE"] = "cpu"
    engine = SyntheticTrainEngine(get_arch("tiny-llama"), train_rank_infos()[0], meta_addr, dtype=torch.float32, device="cpu",
                                  exchange_timeout_s=5)
    writer = NCCLWeightsWriter(engine)
    writer.initialize()
    writer.write_weights(step_id=1)
    q.put(("writer", "left after step 1"))
    # leaves between steps, nothing in flight


def _reader_that_stays(meta_addr, q):
    from awex_b200 import WeightsReader
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticInferenceEngine
    from awex_b200.synthetic.simulate import InferLayout
    from awex_b200.synthetic.topology import infer_rank_infos

    os.environ["AWEX_DEVICE_TYPE"] = "cpu"
    engine = SyntheticInferenceEngine(get_arch("tiny-llama"), InferLayout(tp=1), infer_rank_infos()[0], meta_addr, dtype=torch.float32,
                                      device="cpu", debug_mode_config={"exchange_timeout_s": 5})
    reader = WeightsReader(engine)
    reader.initialize()
    reader.update_weights(step_id=1)
    ok_first = engine.mismatches(step=0) == []
    started = time.time()
    try:
        reader.update_weights(step_id=2)  # nobody sends
        q.put(("reader", ok_first, "no error", time.time() - started))
    except Exception as exc:
        q.put(("reader", ok_first, type(exc).__name__, time.time() - started))


@pytest.mark.timeout(180)
def test_reader_learns_that_the_sender_left_between_steps():
    from awex_b200.meta.meta_server import MetaServer

    server = MetaServer("127.0.0.1", 0)
    server.start()
    addr = f"127.0.0.1:{server.port}"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_reader_that_stays, args=(addr, q)), ctx.Process(target=_writer_that_leaves, args=(addr, q))]
    for p in procs:
        p.start()
    got = {}
    for _ in procs:
        item = q.get(timeout=150)
        got[item[0]] = item[1:]
    for p in procs:
        p.join(timeout=30)
    server.stop()
    ok_first, outcome, seconds = got["reader"]
    assert ok_first, "the first update must have landed"
    assert outcome != "no error", "an update nobody sends must not be reported as done"
    assert seconds < 60


def test_reader_notices_reallocated_parameters():
    """An engine that replaces a parameter's storage after publishing would be
    written through stale addresses: the worker reader refuses the update."""
    from awex_b200.config import InferenceConfig
    from awex_b200.reader.nccl_reader import WorkerWeightsReader
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.models import build_vllm_model, vllm_model_context
    from awex_b200.synthetic.topology import infer_rank_infos

    arch, ri = get_arch("tiny-llama"), infer_rank_infos(tp=1)[0]
    model = build_vllm_model(arch, ri, torch.float32, "cpu")
    cfg = InferenceConfig(tp_size=1, pp_size=1, dp_size=1, ep_size=1)
    fake_meta = [type("M", (), {"name": n, "shards": [type("S", (), {"world_size": 1})()]})() for n in ("model.norm.weight",)]
    reader = WorkerWeightsReader(model, vllm_model_context(ri, infer_engine_config=cfg),
                                 {"engine_name": "vllm", "infer_engine_config": cfg, "infer_world_size": 1}, [], fake_meta,
                                 engine_rank=0, num_engines=1, meta_server_addr="127.0.0.1:1")
    reader.initialize()
    assert reader.parameters_moved() == []
    name, old = next(iter(model.named_parameters()))
    model._tensors[name] = old.clone()  # what a reload or a re-mapping allocator does
    assert reader.parameters_moved() == [name]


def test_worker_reader_refuses_or_follows_moved_parameters():
    """Without ``parameters_may_move`` an update through stale addresses is refused
    with the way out named; with it the worker cuts its views again from the live
    model and hands them to the transport before it announces the update."""
    from types import SimpleNamespace

    from awex_b200.config import InferenceConfig
    from awex_b200.reader.nccl_reader import NCCLWorkerWeightsReader, WorkerWeightsReader
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.models import build_vllm_model, vllm_model_context
    from awex_b200.synthetic.topology import infer_rank_infos

    arch, ri = get_arch("tiny-llama"), infer_rank_infos(tp=1)[0]
    model = build_vllm_model(arch, ri, torch.float32, "cpu")
    cfg = InferenceConfig(tp_size=1, pp_size=1, dp_size=1, ep_size=1)
    fake_meta = [type("M", (), {"name": n, "shards": [type("S", (), {"world_size": 1})()]})() for n in ("model.norm.weight",)]
    reader = NCCLWorkerWeightsReader(model, vllm_model_context(ri, infer_engine_config=cfg),
                                     {"engine_name": "vllm", "infer_engine_config": cfg, "infer_world_size": 1}, [], fake_meta,
                                     engine_rank=0, num_engines=1, meta_server_addr="127.0.0.1:1")
    WorkerWeightsReader.initialize(reader)  # views only; no transport is connected in this test
    calls = []
    reader.transport = SimpleNamespace(may_move=False, begin=lambda epoch: calls.append(("begin", epoch)),
                                       rebind=lambda views: calls.append(("rebind", dict(views))))
    reader.begin_update(1)
    assert calls == [("begin", 1)]
    moved_name = "norm.weight" if "norm.weight" in model._tensors else next(n for n in model._tensors if n.endswith("norm.weight"))
    model._tensors[moved_name] = model._tensors[moved_name].clone()
    with pytest.raises(RuntimeError, match="parameters_may_move"):
        reader.begin_update(2)
    reader.transport.may_move = True
    reader.begin_update(3)
    (kind, views), last = calls[-2], calls[-1]
    assert kind == "rebind" and last == ("begin", 3)
    assert any(v.data_ptr() == model._tensors[moved_name].data_ptr() for v in views.values())  # the views follow the live model
    assert reader.parameters_moved() == [] and reader.parameters is not None
    # same addresses, new memory behind them: the owner says so and the next update publishes again
    reader.transport.republish_if_moved = lambda force=False: calls.append(("republish", force))
    reader.invalidate_addresses()
    reader.begin_update(4)
    assert [c[0] for c in calls[-3:]] == ["rebind", "republish", "begin"] and calls[-2] == ("republish", True)
    reader.begin_update(5)
    assert calls[-1] == ("begin", 5) and calls[-2][0] == "begin"  # only once
    reader.transport.may_move = False
    reader.invalidate_addresses()
    with pytest.raises(RuntimeError, match="parameters_may_move"):
        reader.begin_update(6)


def test_poison_fill_catches_an_unwritten_tensor_whose_values_are_zero():
    """Zero-fill validation cannot see that nobody wrote a tensor that is all
    zeros (a fresh bias); NaN poison can."""
    import torch

    from awex_b200.reader.nccl_reader import WorkerWeightsReader

    def worker(fill):
        w = object.__new__(WorkerWeightsReader)
        w.parameters = {"w": torch.randn(8, 4), "bias": torch.zeros(8), "q": torch.randn(4, 4).to(torch.float8_e4m3fn), "ids": torch.arange(4)}
        w.required_names = set(w.parameters)
        w.device, w.validation_fill, w._snapshot = torch.device("cpu"), fill, None
        return w

    for fill, bias_passes in (("zero", True), ("poison", False)):
        w = worker(fill)
        truth = {n: t.clone() for n, t in w.parameters.items()}
        assert w.snapshot_and_clear() == 4
        if fill == "poison":
            assert torch.isnan(w.parameters["w"]).all() and torch.isnan(w.parameters["q"].float()).all()
            assert (w.parameters["ids"] == 0).all()  # integers have no NaN: zeroed
        for n in ("w", "q", "ids"):  # the update writes everything but the bias
            w.parameters[n].copy_(truth[n])
        result = w.verify_against_snapshot()
        assert result["w"] and result["q"] and result["ids"]
        assert result["bias"] == bias_passes


def test_failed_validation_logs_differences_against_the_reloaded_checkpoint():
    """Where validation only moves checksums, a parameter that fails gets its
    per-element differences from a second load of the checkpoint: received values
    are set aside, the oracle is loaded again, the differences are logged, and the
    received values are put back.  Only the failed parameters are touched."""
    import torch

    from awex_b200.reader.nccl_reader import WorkerWeightsReader
    from awex_b200.reader.weights_reader import WeightsReader

    oracle = {"a.weight": torch.arange(12, dtype=torch.float32).view(3, 4), "b.weight": torch.ones(5)}
    received = {"a.weight": oracle["a.weight"].clone(), "b.weight": torch.ones(5)}
    received["a.weight"][1, 2] = -7.0
    worker = WorkerWeightsReader.__new__(WorkerWeightsReader)
    worker.parameters = {n: t.clone() for n, t in received.items()}
    loads = []

    class Engine:
        def execute_task_in_model_worker(self, fn, **kwargs):
            return [fn(model=None, model_context={"scheduler": type("S", (), {"awes_weights_reader": worker})()}, **kwargs)]

        def update_weights_from_disk(self, path, load_format=None):
            loads.append((path, load_format))
            for n, t in oracle.items():
                worker.parameters[n].copy_(t)

    reader = WeightsReader.__new__(WeightsReader)
    reader.inference_engine = Engine()
    reader._validation_path = ("/ckpt", None)
    reader._log_detailed_differences(3, ["a.weight"])
    assert loads == [("/ckpt", None)]
    assert torch.equal(worker.parameters["a.weight"], received["a.weight"])  # the received values are back
    assert worker._stash == {}
    # without a checkpoint there is nothing to compare with, and nothing is loaded
    reader._validation_path = (None, None)
    reader._log_detailed_differences(4, ["a.weight"])
    assert len(loads) == 1
    # the worker-side pieces on their own
    assert worker.stash_received(["a.weight", "missing"]) == 1
    worker.parameters["a.weight"].copy_(oracle["a.weight"])
    assert worker.diff_against_stash() == {"a.weight": False}
