"""Whole protocol across real processes on CPU: MetaServer discovery, metadata
exchange, plan, Gloo transport, zero-fill + bitwise validation against a
file-loaded (safetensors) reference.  Tiny Llama, two Megatron-layout writers
(TP=2) resharded to one vLLM-layout reader (TP=1), fp32."""

import os
import tempfile

import pytest
import torch
import torch.multiprocessing as mp

WORLD_TRAIN = 2


def _writer(rank, meta_addr, store_port, ckpt_dir, result_q):
    import torch.distributed as dist

    from awex_b200 import NCCLWeightsWriter
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticTrainEngine
    from awex_b200.synthetic.topology import train_rank_infos

    os.environ["AWEX_DEVICE_TYPE"] = "cpu"
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{store_port}", rank=rank, world_size=WORLD_TRAIN)
    ri = train_rank_infos(tp=WORLD_TRAIN)[rank]
    engine = SyntheticTrainEngine(get_arch("tiny-llama"), ri, meta_addr, dtype=torch.float32, device="cpu", comm_backend="nccl",
                                  tp_group=dist.new_group(list(range(WORLD_TRAIN))), weights_validation_steps=1, dump_weights_list_for_validation=["model.norm.weight"],
                                  dump_weights_dir_for_validation=os.path.join(ckpt_dir, "dumps"))
    writer = NCCLWeightsWriter(engine)
    writer.initialize()
    writer.write_weights(step_id=1, path=ckpt_dir)  # validated step: also saves the file reference
    engine.regenerate(step=2)
    writer.write_weights(step_id=2)
    result_q.put(("writer", rank, len(writer.items), writer.transport.bytes_out))
    dist.destroy_process_group()


def _reader(meta_addr, ckpt_dir, result_q):
    from awex_b200 import WeightsReader
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticInferenceEngine
    from awex_b200.synthetic.simulate import InferLayout
    from awex_b200.synthetic.topology import infer_rank_infos

    os.environ["AWEX_DEVICE_TYPE"] = "cpu"
    layout = InferLayout(tp=1)
    engine = SyntheticInferenceEngine(get_arch("tiny-llama"), layout, infer_rank_infos(tp=1)[0], meta_addr, dtype=torch.float32,
                                      device="cpu", weights_validation_steps=1, debug_mode_config={"raise_on_validation_fail": True},
                                      dump_weights_list_for_validation=["model.norm.weight"],
                                      dump_weights_dir_for_validation=os.path.join(ckpt_dir, "dumps"))
    reader = WeightsReader(engine)
    reader.initialize()
    reader.update_weights(step_id=1, path=ckpt_dir)
    bad1 = engine.mismatches(step=0)
    reader.update_weights(step_id=2)
    bad2 = engine.mismatches(step=2)
    worker = engine.schedulers[0].awes_weights_reader
    result_q.put(("reader", bad1, bad2, reader.last_validation_failed, engine.schedulers[0].flushes, worker.transport.bytes_in))


@pytest.mark.timeout(300)
def test_two_writers_one_reader_over_gloo():
    from awex_b200.meta.meta_server import MetaServer
    from awex_b200.utils.common import get_free_port

    server = MetaServer("127.0.0.1", 0)
    server.start()
    meta_addr = f"127.0.0.1:{server.port}"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    store_port = get_free_port()
    with tempfile.TemporaryDirectory() as ckpt:
        procs = [ctx.Process(target=_writer, args=(r, meta_addr, store_port, ckpt, q)) for r in range(WORLD_TRAIN)]
        procs.append(ctx.Process(target=_reader, args=(meta_addr, ckpt, q)))
        for p in procs:
            p.start()
        results = [q.get(timeout=240) for _ in procs]
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
        # both sides dumped the listed parameter during the validated step: same values
        dumps = sorted(os.listdir(os.path.join(ckpt, "dumps")))
        received = [f for f in dumps if f.startswith("reader_") and f.endswith("_from_commu_1.model.norm.weight.pt")]
        sent = [f for f in dumps if f.endswith("_converted.pt")]
        assert len(received) == 1 and len(sent) == WORLD_TRAIN, dumps
        got = torch.load(os.path.join(ckpt, "dumps", received[0]))
        want = torch.load(os.path.join(ckpt, "dumps", sent[0]))["model.norm.weight"]
        assert torch.equal(got, want)
    server.stop()
    reader = next(r for r in results if r[0] == "reader")
    _, bad1, bad2, failed, flushes, bytes_in = reader
    assert bad1 == [] and bad2 == [] and failed == []
    assert flushes == 2
    assert bytes_in == 6820864  # the whole fp32 model, once
    writers = sorted(r for r in results if r[0] == "writer")
    assert sum(w[3] for w in writers) == 6820864
