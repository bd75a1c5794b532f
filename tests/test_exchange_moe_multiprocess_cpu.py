"""Expert-parallel exchange across real processes on CPU: two Megatron-layout
writers (TP=1, DP=2, EP=2: experts split, dense parameters replicated) feed two
inference engines of one worker each (vLLM layout, fused per-expert tensors)
through the public API over gloo, with the least-loaded replica pairing."""

import os

import pytest
import torch
import torch.multiprocessing as mp


def _writer(rank, meta_addr, store_port, q, pairing):
    import torch.distributed as dist

    from awex_b200 import NCCLWeightsWriter
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticTrainEngine
    from awex_b200.synthetic.topology import train_rank_infos

    try:
        os.environ["AWEX_DEVICE_TYPE"] = "cpu"
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{store_port}", rank=rank, world_size=2)
        ri = train_rank_infos(tp=1, dp=2, ep=2)[rank]
        engine = SyntheticTrainEngine(get_arch("tiny-qwen3-moe"), ri, meta_addr, dtype=torch.float32, device="cpu", exchange_timeout_s=120,
                                      **({"replica_pairing": pairing} if pairing else {}))  # "local": engine e shares a GPU with writer e
        writer = NCCLWeightsWriter(engine)
        writer.initialize()
        writer.write_weights(step_id=1)
        engine.regenerate(step=2)
        writer.write_weights(step_id=2)
        from awex_b200.transfer.cpu_exec import entry_nbytes

        per_dst = {d: sum(entry_nbytes(e) for e in es) for d, es in writer.transport.manifest.items()}
        q.put(("writer", rank, writer.transport.bytes_out, (sorted(writer.transport.destinations), per_dst)))
        dist.destroy_process_group()
    except BaseException as exc:
        q.put(("error", f"writer {rank}: {exc!r}", 0, []))
        raise


def _reader(engine_rank, meta_addr, q):
    from awex_b200 import WeightsReader
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticInferenceEngine
    from awex_b200.synthetic.simulate import InferLayout
    from awex_b200.synthetic.topology import infer_rank_infos

    try:
        os.environ["AWEX_DEVICE_TYPE"] = "cpu"
        layout = InferLayout(tp=1, num_engines=2)
        ri = infer_rank_infos(tp=1, engine_rank=engine_rank)[0]
        # the engine has loaded the weights training starts from, so the first update can be validated against
        # what the engine holds: recorded, cleared, received, compared
        engine = SyntheticInferenceEngine(get_arch("tiny-qwen3-moe"), layout, ri, meta_addr, dtype=torch.float32, device="cpu", zero=False,
                                          weights_validation_steps=1, debug_mode_config={"exchange_timeout_s": 120})
        reader = WeightsReader(engine)
        reader.initialize()
        reader.update_weights(step_id=1)
        assert reader.last_validation_failed == [], reader.last_validation_failed[:5]
        bad1 = engine.mismatches(step=0)
        reader.update_weights(step_id=2)
        bad2 = engine.mismatches(step=2)
        worker = engine.schedulers[0].awes_weights_reader
        q.put(("reader", engine_rank, worker.transport.bytes_in, (bad1, bad2, sorted(worker.transport.senders))))
    except BaseException as exc:
        q.put(("error", f"reader {engine_rank}: {exc!r}", 0, []))
        raise


@pytest.mark.timeout(400)
@pytest.mark.parametrize("pairing", [None, "local"])
def test_expert_parallel_writers_to_two_engines_over_gloo(pairing):
    from awex_b200.meta.meta_server import MetaServer
    from awex_b200.utils.common import get_free_port

    server = MetaServer("127.0.0.1", 0)
    server.start()
    addr = f"127.0.0.1:{server.port}"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = get_free_port()
    procs = [ctx.Process(target=_writer, args=(r, addr, port, q, pairing)) for r in range(2)]
    procs += [ctx.Process(target=_reader, args=(e, addr, q)) for e in range(2)]
    for p in procs:
        p.start()
    results = []
    for _ in procs:
        item = q.get(timeout=300)
        assert item[0] != "error", item[1]
        results.append(item)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    server.stop()
    readers = sorted(r for r in results if r[0] == "reader")
    writers = sorted(r for r in results if r[0] == "writer")
    for _, engine_rank, bytes_in, (bad1, bad2, senders) in readers:
        assert bad1 == [] and bad2 == [], (engine_rank, bad1[:3], bad2[:3])
        assert senders == [0, 1]  # experts come from both expert-parallel ranks
    assert readers[0][2] == readers[1][2] and sum(w[2] for w in writers) == 2 * readers[0][2]
    assert all(w[3][0] == [0, 1] for w in writers)  # every writer feeds both engines
    # dense parameters are replicated on both writers: the pairing shares them out evenly
    assert abs(writers[0][2] - writers[1][2]) < 0.1 * writers[0][2]
    if pairing == "local":
        # ... and each engine takes them from the writer it shares a GPU with: only experts cross
        for _, rank, _total, (_dests, per_dst) in writers:
            assert per_dst[rank] > 1.5 * per_dst[1 - rank], per_dst
