"""Co-located memory hand-off between a training process and an inference
process (CPU ranks, gloo): the order of release / resume calls on both engines
around two updates, and the meta-server keys that carry the hand-off."""

import os

import pytest
import torch
import torch.multiprocessing as mp


def _writer(meta_addr, q):
    from awex_b200 import NCCLWeightsWriter
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticTrainEngine
    from awex_b200.synthetic.topology import train_rank_infos

    try:
        os.environ["AWEX_DEVICE_TYPE"] = "cpu"
        calls = []

        class Engine(SyntheticTrainEngine):
            def release_memory_occupation(self, tags=None):
                calls.append(("release", tuple(tags or ())))

            def resume_memory_occupation(self, tags=None):
                calls.append(("resume", tuple(tags or ())))

        engine = Engine(get_arch("tiny-llama"), train_rank_infos()[0], meta_addr, dtype=torch.float32, device="cpu",
                        enable_colocate_mode=True, host_wait_timeout_s=120, exchange_timeout_s=120)
        writer = NCCLWeightsWriter(engine)
        writer.initialize()
        for step in (1, 2):
            writer.write_weights(step_id=step)
            calls.append(("step-done", step))
        q.put(("writer", calls))
    except BaseException as exc:
        q.put(("error", f"writer: {exc!r}"))
        raise


def _reader(meta_addr, q):
    from awex_b200 import WeightsReader
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticInferenceEngine
    from awex_b200.synthetic.simulate import InferLayout
    from awex_b200.synthetic.topology import infer_rank_infos

    try:
        os.environ["AWEX_DEVICE_TYPE"] = "cpu"
        calls = []

        class Engine(SyntheticInferenceEngine):
            def release_memory_occupation(self, tags=None):
                calls.append(("release", tuple(tags or ())))

            def resume_memory_occupation(self, tags=None):
                calls.append(("resume", tuple(tags or ())))

        engine = Engine(get_arch("tiny-llama"), InferLayout(tp=1), infer_rank_infos()[0], meta_addr, dtype=torch.float32, device="cpu",
                        enable_colocate_mode=True, debug_mode_config={"host_wait_timeout_s": 120, "exchange_timeout_s": 120})
        reader = WeightsReader(engine)
        reader.initialize()
        bad = []
        for step in (1, 2):
            reader.update_weights(step_id=step)
            calls.append(("step-done", step))
            bad.append(engine.mismatches(step=0))
        q.put(("reader", (calls, bad)))
    except BaseException as exc:
        q.put(("error", f"reader: {exc!r}"))
        raise


@pytest.mark.timeout(400)
def test_memory_hand_off_order_in_colocated_mode():
    from awex_b200.meta.meta_server import MetaServer, MetaServerClient

    server = MetaServer("127.0.0.1", 0)
    server.start()
    addr = f"127.0.0.1:{server.port}"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_reader, args=(addr, q)), ctx.Process(target=_writer, args=(addr, q))]
    for p in procs:
        p.start()
    got = {}
    for _ in procs:
        kind, payload = q.get(timeout=300)
        assert kind != "error", payload
        got[kind] = payload
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    keys = set(MetaServerClient("127.0.0.1", server.port).list_keys())
    server.stop()
    writer_calls = got["writer"]
    reader_calls, bad = got["reader"]
    assert bad == [[], []]
    # training side, per update: optimizer state out, weights in, (plan + send), weights still resident
    per_step = [c for c in writer_calls if c[0] != "step-done"]
    assert per_step[:3] == [("release", ("optimizer",)), ("resume", ("weights",)), ("resume", ("weights",))]
    assert len(per_step) == 6 and per_step[3:] == per_step[:3]
    # inference side: everything released at start-up, then per update: release, weights back, ..., KV cache back
    assert reader_calls[0] == ("release", ())
    first_update = reader_calls[1: reader_calls.index(("step-done", 1))]
    assert first_update == [("release", ()), ("resume", ("weights",)), ("resume", ("kv_cache",))]
    # the per-update hand-off keys are cleaned up by the training side after each update
    assert "finished_weights_update_engines" not in keys and "all_training_offloaded_optimizers" not in keys
    assert {"infer_conf", "num_infer_engines", "training_params_meta", "infer_params_meta"} <= keys
