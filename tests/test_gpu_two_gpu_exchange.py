"""Trainer and inference engine as two processes on TWO GPUs, through the public
API (`NCCLWeightsWriter` / `WeightsReader`): peer stores over NVLink into a
peer's parameters, flags in a peer's memory, CUDA IPC across devices, and the
host rendezvous that opens every update.  Skipped below two devices.

Failures are made on the host only: a sender that stays away makes the reader's
host wait run out; no kernel is ever left waiting for something that will not
come, and the context is checked to be usable afterwards."""

import os
import time

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ARCH = "tiny-qwen2"


def _needs_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")


def _wait_phase(meta, name, timeout=300):
    meta.get_object(f"test_phase_{name}", timeout=timeout)


def _trainer(meta_addr, q, scenario, env):
    os.environ.update(env)
    from awex_b200 import NCCLWeightsWriter
    from awex_b200.meta.meta_server import MetaServerClient
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticTrainEngine
    from awex_b200.synthetic.topology import train_rank_infos

    try:
        torch.cuda.set_device(0)
        meta = MetaServerClient(*meta_addr.rsplit(":", 1))
        engine = SyntheticTrainEngine(get_arch(ARCH), train_rank_infos()[0], meta_addr, dtype=torch.bfloat16, device="cuda:0",
                                      device_wait_timeout_ms=500)
        writer = NCCLWeightsWriter(engine)
        writer.initialize()
        writer.write_weights(step_id=1)
        engine.regenerate(step=2)
        writer.write_weights(step_id=2)
        info = {}
        if scenario == "skew":
            time.sleep(3.0)  # the inference side announces step 3 three seconds before this side gets there
            engine.regenerate(step=3)
            writer.write_weights(step_id=3)
            _wait_phase(meta, "after_absent_sender")  # step 4: this side stays away
            engine.regenerate(step=5)
            writer.write_weights(step_id=5)
            info["epochs"] = writer.epoch
        elif scenario == "moved":
            for step in (3, 4):
                engine.regenerate(step=step)
                writer.write_weights(step_id=step)
            info["rebuilds"] = getattr(writer.transport, "rebuilds", None)
        info["plane"] = type(writer.transport).__name__
        info["remote"] = getattr(writer.transport, "bytes_remote", None)
        info["status"] = writer.transport.program.status.t.tolist() if hasattr(writer.transport, "program") else [0]
        q.put(("trainer", info))
        writer.close()
    except BaseException as exc:  # surfaced by the parent
        q.put(("trainer-error", repr(exc)))
        raise


def _server(meta_addr, q, scenario, env):
    os.environ.update(env)
    from awex_b200 import WeightsReader
    from awex_b200.meta.meta_server import MetaServerClient
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticInferenceEngine
    from awex_b200.synthetic.simulate import InferLayout
    from awex_b200.synthetic.topology import infer_rank_infos

    try:
        torch.cuda.set_device(1)
        meta = MetaServerClient(*meta_addr.rsplit(":", 1))
        debug = {"parameters_may_move": True} if scenario == "moved" else {}
        engine = SyntheticInferenceEngine(get_arch(ARCH), InferLayout(tp=1), infer_rank_infos()[0], meta_addr, dtype=torch.bfloat16,
                                          device="cuda:1", debug_mode_config=debug, device_wait_timeout_ms=500)
        reader = WeightsReader(engine)
        reader.initialize()
        bad = []
        reader.update_weights(step_id=1)
        bad.append(engine.mismatches(step=0))
        reader.update_weights(step_id=2)
        bad.append(engine.mismatches(step=2))
        worker = engine.schedulers[0].awes_weights_reader
        info = {"plane": type(worker.transport).__name__}
        if scenario == "skew":
            t0 = time.time()
            reader.update_weights(step_id=3)  # waits on the host for the late sender; the 0.5 s device wait must not run out
            info["waited_s"] = time.time() - t0
            bad.append(engine.mismatches(step=3))
            # a sender that never comes: the host wait runs out, the announcement is withdrawn, nothing hangs
            worker.transport.host_wait_timeout_s = 1.0
            t0 = time.time()
            try:
                reader.update_weights(step_id=4)
                info["absent"] = "no error"
            except Exception as exc:  # noqa: BLE001
                info["absent"] = type(exc).__name__
            info["absent_s"] = time.time() - t0
            info["usable"] = float(torch.ones(1024, device="cuda:1").sum().item())
            worker.transport.host_wait_timeout_s = 300.0
            meta.put_object("test_phase_after_absent_sender", 1)
            reader.update_weights(step_id=5)
            bad.append(engine.mismatches(step=5))
            info["epochs"] = worker.epoch
        elif scenario == "moved":
            # the engine re-allocates every weight between updates (sleep / wake-up)
            model = engine.model
            old = dict(model._tensors)
            for name in list(model._tensors):
                model._tensors[name] = torch.zeros_like(old[name])
            for t in old.values():
                t.fill_(7.0)
            reader.update_weights(step_id=3)
            bad.append(engine.mismatches(step=3))
            info["stale_untouched"] = all(bool((t == 7.0).all()) for t in old.values())
            reader.update_weights(step_id=4)
            bad.append(engine.mismatches(step=4))
        info["bad"] = bad
        info["flushes"] = engine.schedulers[0].flushes if hasattr(engine.schedulers[0], "flushes") else None
        q.put(("server", info))
        worker.close()
    except BaseException as exc:
        q.put(("server-error", repr(exc)))
        raise


def _run(scenario, env=None):
    from awex_b200.meta.meta_server import MetaServer

    server = MetaServer("127.0.0.1", 0)
    server.start()
    addr = f"127.0.0.1:{server.port}"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_server, args=(addr, q, scenario, env or {})), ctx.Process(target=_trainer, args=(addr, q, scenario, env or {}))]
    for p in procs:
        p.start()
    got = {}
    try:
        for _ in procs:
            kind, info = q.get(timeout=400)
            assert not kind.endswith("error"), (kind, info)
            got[kind] = info
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    finally:
        for p in procs:  # a child that neither reported nor left is not left behind
            if p.is_alive():
                p.kill()
        server.stop()
    return got


def test_separated_update_across_two_gpus_with_skew_and_an_absent_sender():
    _needs_two_gpus()
    got = _run("skew")
    assert got["trainer"]["plane"] == "PeerStoreSender" and got["server"]["plane"] == "PeerStoreReceiver"
    assert got["trainer"]["remote"] and got["trainer"]["remote"] > 0  # every byte crossed NVLink
    assert got["server"]["bad"] == [[], [], [], []]
    assert got["server"]["waited_s"] >= 2.0  # the reader waited for the late sender on the host
    assert got["server"]["absent"] == "HostHandshakeTimeout" and got["server"]["absent_s"] < 20
    assert got["server"]["usable"] == 1024.0
    # the reader spent an epoch on the abandoned update; the sender followed its announcements
    assert got["server"]["epochs"] == 5 and got["trainer"]["epochs"] == 5
    assert got["trainer"]["status"][0] == 0


def test_a_reader_that_reallocates_its_weights_is_followed_across_gpus():
    _needs_two_gpus()
    got = _run("moved")
    assert got["server"]["bad"] == [[], [], [], []]
    assert got["server"]["stale_untouched"] is True
    assert got["trainer"]["rebuilds"] == 1


def test_message_plane_over_nccl_with_bounded_staging():
    """`AWEX_DATA_PLANE=messages`: packed messages over a NCCL group spanning both
    sides, cut into runs of at most `AWEX_CHUNK_MB`."""
    _needs_two_gpus()
    got = _run("plain", env={"AWEX_DATA_PLANE": "messages", "AWEX_CHUNK_MB": "1", "NCCL_NVLS_ENABLE": "0"})
    assert got["trainer"]["plane"] == "GlooSender" and got["server"]["plane"] == "GlooReceiver"
    assert got["server"]["bad"] == [[], []]
