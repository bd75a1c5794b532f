"""Training process and inference process on ONE GPU (the co-located
deployment with separate processes): parameters are written through CUDA IPC
mappings by the fused kernel, and because kernels of two processes on one GPU
must never wait for each other, the pair synchronises on the host through the
meta server.  Two updates, bitwise checks, and the transport must report that it
chose the host handshake."""

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _writer(meta_addr, q):
    from awex_b200 import NCCLWeightsWriter
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticTrainEngine
    from awex_b200.synthetic.topology import train_rank_infos

    try:
        torch.cuda.set_device(0)
        engine = SyntheticTrainEngine(get_arch("tiny-qwen2"), train_rank_infos()[0], meta_addr, dtype=torch.bfloat16, device="cuda")
        writer = NCCLWeightsWriter(engine)
        writer.initialize()
        writer.write_weights(step_id=1)
        engine.regenerate(step=2)
        writer.write_weights(step_id=2)
        q.put(("writer", list(writer.transport.host_destinations), writer.transport.program.status.t.tolist()))
        writer.close()
    except BaseException as exc:  # surfaced by the parent
        q.put(("writer-error", repr(exc), None))
        raise


def _reader(meta_addr, q, expandable=False):
    import os

    if expandable:
        # the engine's weights then live in virtual-memory allocations (cuMemCreate), which CUDA IPC refuses:
        # the address book must hand them over as file descriptors instead
        os.environ["PYTORCH_CUDA_ALLOC_CONF"] = "expandable_segments:True"
    from awex_b200 import WeightsReader
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticInferenceEngine
    from awex_b200.synthetic.simulate import InferLayout
    from awex_b200.synthetic.topology import infer_rank_infos

    try:
        torch.cuda.set_device(0)
        engine = SyntheticInferenceEngine(get_arch("tiny-qwen2"), InferLayout(tp=1), infer_rank_infos()[0], meta_addr,
                                          dtype=torch.bfloat16, device="cuda")
        reader = WeightsReader(engine)
        reader.initialize()
        reader.update_weights(step_id=1)
        bad1 = engine.mismatches(step=0)
        reader.update_weights(step_id=2)
        bad2 = engine.mismatches(step=2)
        worker = engine.schedulers[0].awes_weights_reader
        book = worker.meta_server_client.get_object("p2p_addr_0", timeout=30)
        q.put(("reader", list(worker.transport.host_senders), (bad1, bad2, len(book.vmm))))
    except BaseException as exc:
        q.put(("reader-error", repr(exc), None))
        raise


@pytest.mark.parametrize("expandable", [False, True])
def test_two_processes_one_gpu_host_handshake(expandable):
    from awex_b200.meta.meta_server import MetaServer

    server = MetaServer("127.0.0.1", 0)
    server.start()
    addr = f"127.0.0.1:{server.port}"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_reader, args=(addr, q, expandable)), ctx.Process(target=_writer, args=(addr, q))]
    for p in procs:
        p.start()
    got = {}
    try:
        for _ in procs:
            kind, a, b = q.get(timeout=500)
            assert not kind.endswith("error"), (kind, a)
            got[kind] = (a, b)
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    finally:
        for p in procs:  # a child that neither reported nor left is not left behind
            if p.is_alive():
                p.kill()
        server.stop()
    assert got["writer"][0] == [0], "the sender must have recognised a same-GPU destination in another process"
    assert got["reader"][0] == [0]
    assert got["reader"][1][:2] == ([], [])
    # with expandable segments the parameters were handed over as virtual-memory allocations, otherwise as CUDA IPC handles
    assert (got["reader"][1][2] > 0) == expandable
    assert got["writer"][1][0] == 0
