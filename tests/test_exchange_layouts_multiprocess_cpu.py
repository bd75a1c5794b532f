"""More layouts through the public API across real CPU processes (gloo):
pipeline-parallel writers feeding one engine of two workers (whose metadata is
gathered over the instance group), and block-fp8 serving, where the message
transport carries quantised payloads and their scales."""

import os

import pytest
import torch
import torch.multiprocessing as mp


def _layouts(case):
    from awex_b200.synthetic.simulate import InferLayout

    if case == "pp2_to_tp2_chunked":  # the same layout with staging bounded to 0.25 MiB runs on both sides
        return "tiny-llama", dict(tp=1, pp=2), InferLayout(tp=2), torch.float32
    if case == "pp2_to_tp2":
        return "tiny-llama", dict(tp=1, pp=2), InferLayout(tp=2), torch.float32
    if case == "tp1_to_tp2_fp8":
        return "tiny-llama", dict(tp=1), InferLayout(tp=2, fp8=True), torch.bfloat16
    if case == "tp2_to_tp1_fp8":  # quantisation blocks of the fused QKV mix rows of both training ranks: gathered first
        return "tiny-llama", dict(tp=2), InferLayout(tp=1, fp8=True), torch.bfloat16
    if case == "tp1_to_tp2_norm_head":
        return "tiny-llama-norm-head", dict(tp=1), InferLayout(tp=2), torch.float32
    raise ValueError(case)


def _train_world(spec):
    return spec.get("tp", 1) * spec.get("pp", 1) * spec.get("dp", 1)


def _writer(case, rank, meta_addr, store_port, q):
    import torch.distributed as dist

    from awex_b200 import NCCLWeightsWriter
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticTrainEngine
    from awex_b200.synthetic.topology import train_rank_infos

    try:
        os.environ["AWEX_DEVICE_TYPE"] = "cpu"
        if case.endswith("_chunked"):
            os.environ["AWEX_CHUNK_MB"] = "0.25"
        arch, train, _infer, dtype = _layouts(case)
        world = _train_world(train)
        group = None
        if world > 1:
            dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{store_port}", rank=rank, world_size=world)
        ri = train_rank_infos(**train)[rank]
        tp_group = dist.new_group(list(range(world))) if train.get("tp", 1) == world and world > 1 else None
        engine = SyntheticTrainEngine(get_arch(arch), ri, meta_addr, dtype=dtype, device="cpu", process_group=group, tp_group=tp_group,
                                      exchange_timeout_s=120)
        writer = NCCLWeightsWriter(engine)
        writer.initialize()
        writer.write_weights(step_id=1)
        q.put(("writer", rank, writer.transport.bytes_out))
        if world > 1:
            dist.destroy_process_group()
    except BaseException as exc:
        q.put(("error", f"writer {rank}: {exc!r}", 0))
        raise


def _reader(case, worker_rank, meta_addr, store_port, q):
    import torch.distributed as dist

    from awex_b200 import WeightsReader
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticInferenceEngine
    from awex_b200.synthetic.topology import infer_rank_infos

    try:
        os.environ["AWEX_DEVICE_TYPE"] = "cpu"
        if case.endswith("_chunked"):
            os.environ["AWEX_CHUNK_MB"] = "0.25"
        arch, _train, layout, dtype = _layouts(case)
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{store_port}", rank=worker_rank, world_size=layout.tp)
        ri = infer_rank_infos(tp=layout.tp)[worker_rank]
        engine = SyntheticInferenceEngine(get_arch(arch), layout, ri, meta_addr, dtype=dtype, device="cpu", instance_group=dist.group.WORLD,
                                          debug_mode_config={"exchange_timeout_s": 120, "data_plane": "messages"})  # published; the writers follow it
        reader = WeightsReader(engine)
        reader.initialize()
        reader.update_weights(step_id=1)
        bad = engine.mismatches(step=0)
        if case.endswith("_chunked"):
            peak = engine.schedulers[0].awes_weights_reader.transport.peak_staging_bytes
            # runs of at most a quarter MiB, or one larger tensor travelling alone (the embedding slice: 0.5 MiB)
            assert 0 < peak <= 1024 * 256 * 4 // 2 + 1024, peak
        if case.endswith("norm_head"):
            # the head arrives with unit-norm columns (computed by the single training rank over the whole vocabulary)
            from awex_b200.synthetic.models import CanonicalWeights

            a = get_arch(arch)
            full = CanonicalWeights(a, dtype, "cpu").get("lm_head.weight", (a.vocab, a.hidden))
            want = torch.nn.functional.normalize(full, dim=0, p=2, eps=1e-7).chunk(layout.tp, 0)[worker_rank]
            got = dict(engine.model.named_parameters())["lm_head.weight"]
            assert bad == ["lm_head.weight"] and torch.equal(got, want), bad
            bad = []
        q.put(("reader", worker_rank, bad))
        dist.destroy_process_group()
    except BaseException as exc:
        q.put(("error", f"reader {worker_rank}: {exc!r}", 0))
        raise


@pytest.mark.timeout(400)
@pytest.mark.parametrize("case", ["pp2_to_tp2", "pp2_to_tp2_chunked", "tp1_to_tp2_fp8", "tp2_to_tp1_fp8", "tp1_to_tp2_norm_head"])
def test_layout_over_gloo(case):
    from awex_b200.meta.meta_server import MetaServer
    from awex_b200.utils.common import get_free_port

    _arch, train, layout, _dtype = _layouts(case)
    server = MetaServer("127.0.0.1", 0)
    server.start()
    addr = f"127.0.0.1:{server.port}"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    train_port, infer_port = get_free_port(), get_free_port()
    procs = [ctx.Process(target=_writer, args=(case, r, addr, train_port, q)) for r in range(_train_world(train))]
    procs += [ctx.Process(target=_reader, args=(case, w, addr, infer_port, q)) for w in range(layout.tp)]
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
    for kind, rank, payload in results:
        if kind == "reader":
            assert payload == [], (case, rank, payload[:3])
        else:
            assert payload > 0


# ------------------------------------------------------------------------------------------ interleaved pipeline
def _vpp_writer(rank, meta_addr, store_port, q):
    import dataclasses

    import torch.distributed as dist

    from awex_b200 import NCCLWeightsWriter
    from awex_b200.engine.mcore import MegatronEngine
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.models import build_megatron_model
    from awex_b200.synthetic.topology import train_rank_infos

    try:
        os.environ["AWEX_DEVICE_TYPE"] = "cpu"
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{store_port}", rank=rank, world_size=2)
        arch = dataclasses.replace(get_arch("tiny-llama"), num_layers=4)
        ri = train_rank_infos(tp=1, pp=2)[rank]
        chunks = [build_megatron_model(arch, ri, torch.float32, "cpu", virtual_stage=(vp, 2)) for vp in range(2)]
        engine = MegatronEngine({"meta_server_addr": meta_addr, "comm_backend": "nccl", "exchange_timeout_s": 120}, arch.hf_config(), chunks, rank_info=ri)
        writer = NCCLWeightsWriter(engine)
        writer.initialize()
        writer.write_weights(step_id=1)
        q.put(("writer", rank, sorted({it.dst_name.split(".")[2] for it in writer.items if it.dst_name.startswith("model.layers.")})))
        dist.destroy_process_group()
    except BaseException as exc:
        q.put(("error", f"writer {rank}: {exc!r}", 0))
        raise


def _vpp_reader(meta_addr, q):
    import dataclasses

    from awex_b200 import WeightsReader
    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.harness import SyntheticInferenceEngine
    from awex_b200.synthetic.simulate import InferLayout
    from awex_b200.synthetic.topology import infer_rank_infos

    try:
        os.environ["AWEX_DEVICE_TYPE"] = "cpu"
        arch = dataclasses.replace(get_arch("tiny-llama"), num_layers=4)
        engine = SyntheticInferenceEngine(arch, InferLayout(tp=1), infer_rank_infos()[0], meta_addr, dtype=torch.float32, device="cpu",
                                          debug_mode_config={"exchange_timeout_s": 120, "data_plane": "messages"})  # published; the writers follow it
        reader = WeightsReader(engine)
        reader.initialize()
        reader.update_weights(step_id=1)
        q.put(("reader", 0, engine.mismatches(step=0)))
    except BaseException as exc:
        q.put(("error", f"reader: {exc!r}", 0))
        raise


@pytest.mark.timeout(400)
def test_interleaved_pipeline_chunks_are_renumbered_to_global_layers():
    """Two pipeline ranks with two model chunks each (virtual pipeline): chunk
    (pp, vp) holds global layer vp * 2 + pp under the local id 0."""
    from awex_b200.meta.meta_server import MetaServer
    from awex_b200.utils.common import get_free_port

    server = MetaServer("127.0.0.1", 0)
    server.start()
    addr = f"127.0.0.1:{server.port}"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = get_free_port()
    procs = [ctx.Process(target=_vpp_writer, args=(r, addr, port, q)) for r in range(2)] + [ctx.Process(target=_vpp_reader, args=(addr, q))]
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
    layers = {rank: payload for kind, rank, payload in results if kind == "writer"}
    assert layers == {0: ["0", "2"], 1: ["1", "3"]}
    assert [payload for kind, _, payload in results if kind == "reader"] == [[]]
