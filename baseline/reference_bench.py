"""Benchmark arm that runs the UNMODIFIED reference (``baseline/_ref/awex``) in
its NCCL mode on the same layouts, model and metric as ``bench.py``.

What the harness supplies, because the engines the reference plugs into are
not installable here: a stub ``megatron.core`` (type annotation + parallel
state backed by ``torch.distributed``), synthetic Megatron-layout and
vLLM-layout modules (``baseline/synth.py``), and dummy engine objects exposing
exactly the attributes the reference reads.  Everything that moves or converts
a weight is the reference's own code: ``NCCLWeightsWriter.write_weights`` on
training ranks, ``WeightsReader.update_weights`` -> ``NCCLWorkerWeightsReader``
on inference ranks, its planner, converters, ``batch_send_recv`` and MetaServer.

Process model: the launcher's ranks are split like ``bench.py`` does.  The
reference gathers training metadata over the *default* process group, so the
training ranks form their own default group; the workers of each inference
instance form theirs, and exchange worker metadata through the MetaServer.
"""

from __future__ import annotations

import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
STUBS = os.path.join(HERE, "stubs")


def unavailable(why: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def roles(n: int):
    """(train tp, infer tp, train ranks, [infer ranks per engine], label)"""
    if n == 2:
        return 1, 1, [0], [[1]], "tp1->tp1"
    if n == 4:
        return 2, 2, [0, 1], [[2, 3]], "tp2->tp2"
    if n == 8:
        return 4, 2, [0, 1, 2, 3], [[4, 5], [6, 7]], "tp4->2xtp2"
    return None


class _Scheduler:
    def __init__(self, gpu_id, server_args):
        self.gpu_id, self.local_rank, self.server_args, self.flushes = gpu_id, gpu_id, server_args, 0

    def flush_cache(self):
        self.flushes += 1
        return True


class _InferEngine:
    """One vLLM-like worker (this process); metadata of the instance's other
    workers is exchanged through the MetaServer."""

    engine_name = "vllm"

    def __init__(self, config, hf_config, model, ctx, meta, engine_rank, tp_rank, tp_size):
        self.config, self.hf_config, self.model, self.ctx, self.meta = config, hf_config, model, ctx, meta
        self.num_engines, self.engine_rank = config.num_engines, engine_rank
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self._calls = 0

    def execute_task_in_model_worker(self, fn, **kwargs):
        out = fn(model=self.model, model_context=self.ctx, **kwargs)
        if getattr(fn, "__name__", "") != "_get_model_param_info" or self.tp_size == 1:
            return [out]
        self._calls += 1
        base = f"refbench_meta_{self.engine_rank}_{self._calls}"
        self.meta.put_object(f"{base}_{self.tp_rank}", out)
        return [self.meta.get_object(f"{base}_{r}", timeout=600) for r in range(self.tp_size)]

    def release_memory_occupation(self, tags=None):
        pass

    def resume_memory_occupation(self, tags=None):
        pass

    def update_weights_from_disk(self, path, load_format=None):
        raise NotImplementedError


class _TrainEngine:
    engine_name = "mcore"
    comm_backend = "nccl"
    enable_colocate_mode = False
    enable_debug_mode = False

    def __init__(self, model, hf_config, meta_server_addr):
        self.model, self.hf_config, self.meta_server_addr, self.config = model, hf_config, meta_server_addr, {}

    def release_memory_occupation(self, tags=None):
        pass

    def resume_memory_occupation(self, tags=None):
        pass

    def release_grad_memory(self):
        pass


class _ColocatedTrainEngine(_TrainEngine):
    """The training side of the reference's co-located deployment.  The reference
    frees the storage of every converted tensor after it has copied it into its
    IPC groups (`awex/writer/nccl_writer.py:364`, `release_tensors`), and converted
    tensors alias the model's own parameters wherever a conversion is the identity,
    because in its real deployment the weights are offloaded at that point and
    `resume_memory_occupation("weights")` brings them back at the start of the next
    update.  This engine does the cheapest thing that honours that contract: it
    keeps a second copy of every parameter in device memory and restores emptied
    parameters from it (a real engine reloads them from host memory, which is far
    slower; the choice favours the reference's number)."""

    enable_colocate_mode = True

    def __init__(self, model, hf_config, meta_server_addr):
        super().__init__(model, hf_config, meta_server_addr)
        self._backup = {name: p.detach().clone() for name, p in model.named_parameters()}
        # a parameter may be a view at an offset into a larger storage (a row slice of a full tensor)
        self._storage_bytes = {name: p.untyped_storage().size() for name, p in model.named_parameters()}

    def resume_memory_occupation(self, tags=None):
        import torch

        if tags is not None and "weights" not in tags:
            return
        with torch.no_grad():
            for name, p in self.model.named_parameters():
                keep = self._backup[name]
                storage = p.untyped_storage()
                if storage.size() < self._storage_bytes[name]:
                    storage.resize_(self._storage_bytes[name])
                    p.copy_(keep)


def _hf_config(arch):
    from baseline import synth

    return synth.hf_config_for(arch)


def colocated_child(rank, world, store_addr, store_port, meta_addr, arch, steps, warmup, validate):
    """Inference worker of GPU ``rank`` in the co-located arm (a process of its own,
    as in the reference's deployment: `docs/README.md:78`)."""
    sys.path.insert(0, STUBS)
    sys.path.insert(0, REF)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ.setdefault("AWEX_MASTER_ADDR", "127.0.0.1")
    os.environ["LOCAL_RANK"] = str(rank)
    import torch
    import torch.distributed as dist

    from baseline import synth

    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    store = dist.PrefixStore("refbench", dist.TCPStore(store_addr, store_port, 2 * world, is_master=False, wait_for_workers=False))
    try:
        import awex.logging as ref_logging

        ref_logging.setLevel(os.environ.get("AWEX_LOG_LEVEL", "WARNING"))
        from awex.config import InferenceConfig
        from awex.meta.meta_server import MetaServerClient
        from awex.reader.weights_reader import WeightsReader

        dist.init_process_group("nccl", store=dist.PrefixStore("infer_pg0", store), rank=rank, world_size=world)
        hf_config = _hf_config(arch)
        cfg = InferenceConfig(tp_size=world, pp_size=1, dp_size=1, ep_size=1, enable_dp_attention=False, enable_dp_lm_head=False,
                              num_engines=1, engine_rank=0, meta_server_addr=meta_addr, comm_backend="nccl", enable_colocate_mode=True)
        model = synth.vllm_module(arch, world, rank, torch.bfloat16, device, hf_config, zero=True)
        sched = _Scheduler(rank, cfg)
        ctx = dict(scheduler=sched, infer_engine_config=cfg, tp_rank=rank, tp_size=world, pp_rank=0, pp_size=1, dp_rank=0,
                   dp_size=1, ep_rank=0, ep_size=1, attn_tp_rank=rank, attn_tp_size=world, attn_dp_rank=0,
                   world_size=world, global_rank=rank, local_rank=rank)
        engine = _InferEngine(cfg, hf_config, model, ctx, MetaServerClient(*meta_addr.split(":")), 0, rank, world)
        reader = WeightsReader(engine)
        reader.initialize()
        times_ms, wall_ms = [], []
        for s in range(1, warmup + steps + 1):
            _store_barrier(store, f"step{s}", 2 * world)
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            start.record()
            reader.update_weights(step_id=s)
            stop.record()
            torch.cuda.synchronize()
            wall_ms.append((time.perf_counter() - t0) * 1e3)
            times_ms.append(start.elapsed_time(stop))
        valid, bad = True, []
        if validate:
            want = synth.vllm_module(arch, world, rank, torch.bfloat16, device, hf_config)
            for (name, a), (_, b) in zip(model.named_parameters(), want.named_parameters()):
                if not torch.equal(a, b):
                    bad.append((name, "all zero" if not bool(a.any()) else f"{int((a != b).sum())} of {a.numel()} differ"))
            valid = not bad
        local_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
        store.set(f"result_infer{rank}", json.dumps({"ms": times_ms[warmup:], "wall": wall_ms[warmup:], "bytes": local_bytes, "valid": valid,
                                                     "mismatching": bad[:6], "n_mismatching": len(bad)}))
    except BaseException:
        import traceback

        store.set(f"result_infer{rank}", json.dumps({"error": traceback.format_exc()[-1500:]}))
        raise
    finally:
        _store_barrier(store, "exit", 2 * world)
    os._exit(0)


def run_reference_colocated(args):
    """The reference's co-located mode, unmodified, on the layout ``bench.py
    --config colocated`` times: per GPU one training process (this one, a rank of
    the launcher) and one inference process (spawned here), training TP n ->
    inference TP n on the same GPUs.  The writer hands its converted weights over
    by CUDA IPC through the MetaServer; the inference processes move them among
    themselves with NCCL (`awex/writer/nccl_writer.py:341-427`,
    `awex/reader/nccl_reader.py:227-317,432-493`, `awex/transfer/nccl_stream_batch.py`).
    Two attributes that the writer reads and nothing assigns
    (`nccl_writer.py:175,182`) are set on the writer instance after construction;
    nothing under ``baseline/_ref`` is changed."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if rank == 0:
            unavailable(f"--gpus {args.gpus} but WORLD_SIZE={world}")
        return
    if world == 1:
        # Found by reading, not by running: with one inference rank the reference's reader opens with a blocking NCCL
        # receive from its own rank (`nccl_reader.py:138-146`, src = world_size - 1 = 0) before the matching send two
        # statements later is posted; the receive kernel would spin on the GPU forever.
        unavailable("the reference's co-located reader with a single inference rank starts with a blocking NCCL recv from its own "
                    "rank before the matching send is posted (nccl_reader.py:138-155): a GPU hang by reading, so it is not run; "
                    "its separated mode cannot put two ranks of one communicator on one GPU")
        return
    from baseline import synth

    arch = args.model
    if arch not in synth.ARCHS:
        if rank == 0:
            unavailable(f"the reference harness has no synthetic weights for architecture {arch!r}")
        return
    sys.path.insert(0, STUBS)
    sys.path.insert(0, REF)
    os.environ.setdefault("AWEX_MASTER_ADDR", "127.0.0.1")

    import torch
    import torch.distributed as dist
    import torch.multiprocessing as mp

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    agent_store = os.environ.get("TORCHELASTIC_USE_AGENT_STORE", "False") == "True"
    store_addr, store_port = os.environ.get("MASTER_ADDR", "127.0.0.1"), int(os.environ["MASTER_PORT"])
    raw_store = dist.TCPStore(store_addr, store_port, world, is_master=(rank == 0 and not agent_store), wait_for_workers=False)
    store = dist.PrefixStore("refbench", raw_store)
    os.environ.pop("TORCHELASTIC_USE_AGENT_STORE", None)  # see run_reference

    import awex.logging as ref_logging

    ref_logging.setLevel(os.environ.get("AWEX_LOG_LEVEL", "WARNING"))
    from awex.meta.meta_server import MetaServer

    server = None
    if rank == 0:
        from awex.util.common import get_free_port

        server = MetaServer("127.0.0.1", get_free_port())
        server.start()
        store.set("meta_addr", f"127.0.0.1:{server.port}")
    meta_addr = store.get("meta_addr").decode()
    child = mp.get_context("spawn").Process(
        target=colocated_child, args=(rank, world, store_addr, store_port, meta_addr, arch, args.steps, args.warmup, not args.no_validate))
    child.start()
    error = None
    times_ms, wall_ms = [], []
    sampler = None
    try:
        dist.init_process_group("nccl", store=dist.PrefixStore("train_pg", store), rank=rank, world_size=world)
        from awex.writer.nccl_writer import NCCLWeightsWriter

        hf_config = synth.hf_config_for(arch)
        model = synth.megatron_module(arch, world, rank, torch.bfloat16, device)
        writer = NCCLWeightsWriter(_ColocatedTrainEngine(model, hf_config, meta_addr))
        # read by `_init_writer_in_colocate_mode` / `_destroy_weights_exchange_process_group`, assigned nowhere in the reference
        writer.asystem_train_config = {}
        writer.backend = "nccl"
        writer.initialize()
        sys.path.insert(0, os.path.dirname(HERE))
        from awex_b200.utils.gpu import ClockSampler

        for s in range(1, args.warmup + args.steps + 1):
            if s == args.warmup + 1 and rank == 0:
                sampler = ClockSampler([local_rank], period_ms=50)
                sampler.__enter__()
            _store_barrier(store, f"step{s}", 2 * world)
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            start.record()
            writer.write_weights(step_id=s)
            stop.record()
            torch.cuda.synchronize()
            wall_ms.append((time.perf_counter() - t0) * 1e3)
            times_ms.append(start.elapsed_time(stop))
    except BaseException:
        import traceback

        error = traceback.format_exc()[-1500:]
    if sampler is not None:
        sampler.__exit__(None, None, None)
    store.set(f"result_train{rank}", json.dumps({"error": error} if error else {"ms": times_ms[args.warmup:], "wall": wall_ms[args.warmup:]}))
    if error is not None:
        # the other processes wait in barriers and in the reference's own MetaServer waits: end the job
        if rank == 0:
            unavailable("reference co-located mode failed beyond the two unassigned attributes: " + error.replace("\n", " | "))
        child.kill()
        os._exit(0 if rank == 0 else 1)
    _store_barrier(store, "exit", 2 * world)
    child.join(60)
    if rank == 0:
        from awex_b200.bench_distributed import bench_config  # the record's layout only

        results = [json.loads(store.get(f"result_train{r}").decode()) for r in range(world)] + \
                  [json.loads(store.get(f"result_infer{r}").decode()) for r in range(world)]
        failed = [r["error"] for r in results if "error" in r and r["error"]]
        if failed:
            unavailable("reference co-located mode failed beyond the two unassigned attributes: " + failed[0].replace("\n", " | "))
        else:
            per_step = [max(r["ms"][i] for r in results) for i in range(args.steps)]
            per_wall = [max(r["wall"][i] for r in results) for i in range(args.steps)]
            ms, wall = sum(per_step) / len(per_step), sum(per_wall) / len(per_wall)
            total_bytes = sum(r.get("bytes", 0) for r in results)
            print(json.dumps({
                "metric": "weight_sync_seconds_per_update", "value": ms / 1e3, "unit": "s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "per-N layouts (not a scaling series)",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic random-init N(0,0.02) weights from per-name seeds",
                "impl": "reference", "instance_attrs_set": ["asystem_train_config = {}", "backend = 'nccl'"],
                "mismatching_parameters": [r.get("mismatching") for r in results if r.get("n_mismatching")],
                "config": bench_config(arch, total_bytes, f"colocated-tp{world}->tp{world}", "colocated",
                                       all(r.get("valid", True) for r in results)),
                "config_details": {
                    "processes": "one training and one inference process per GPU (CUDA IPC hand-over, NCCL among the inference processes)",
                    "train_engine": "weights restored from a second device copy at the start of every update (the reference frees them after each)",
                    "timing": "CUDA events around NCCLWeightsWriter.write_weights / WeightsReader.update_weights in every process, max over all"},
                "aggregate_GBps": total_bytes / (ms / 1e3) / 1e9, "nvlink_GBps_per_gpu": 0.0,
                "e2e": {"value": wall / 1e3, "unit": "s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                        "what": "wall clock of the blocking reference calls, max over all processes"},
                "gpu_launches": 0, "per_step_ms": per_step, "clocks": sampler.summary() if sampler is not None else None,
            }), flush=True)
    dist.destroy_process_group()
    if server is not None:
        server.stop()
    os._exit(0)


def _store_barrier(store, name, world):
    store.add(name, 1)
    while int(store.add(name, 0)) < world:
        time.sleep(0.002)


def run_reference(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not os.path.isdir(os.path.join(REF, "awex", "transfer")):
        if rank == 0:
            unavailable("baseline/_ref does not contain an importable copy of the reference package")
        return
    layout = roles(world)
    if layout is None or world != args.gpus:
        if rank == 0:
            unavailable(
                "the reference's NCCL mode needs training and inference ranks on different GPUs (one communicator cannot hold "
                "two ranks of one device); its co-located single-GPU mode needs two processes per GPU and reads attributes "
                "the writer never defines (nccl_writer.py:175,182), so N=1 is not runnable unmodified"
            )
        return
    train_tp, infer_tp, train_ranks, engines, label = layout
    if os.environ.get("REFBENCH_DUMP_AFTER_S"):
        import faulthandler

        faulthandler.dump_traceback_later(int(os.environ["REFBENCH_DUMP_AFTER_S"]), exit=True)
    sys.path.insert(0, STUBS)
    sys.path.insert(0, REF)
    os.environ.setdefault("AWEX_MASTER_ADDR", "127.0.0.1")

    import torch
    import torch.distributed as dist

    from baseline import synth

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    agent_store = os.environ.get("TORCHELASTIC_USE_AGENT_STORE", "False") == "True"
    store = dist.TCPStore(os.environ.get("MASTER_ADDR", "127.0.0.1"), int(os.environ["MASTER_PORT"]), world,
                          is_master=(rank == 0 and not agent_store), wait_for_workers=False)
    store = dist.PrefixStore("refbench", store)
    # The launcher marks its store as agent-hosted, which makes every tcp://
    # rendezvous in the process a pure client.  The reference creates its exchange
    # group with such a rendezvous and expects rank 0 to host the store, as it
    # does outside a launcher; drop the marker once our own store is connected.
    os.environ.pop("TORCHELASTIC_USE_AGENT_STORE", None)

    import awex.logging as ref_logging

    ref_logging.setLevel(os.environ.get("AWEX_LOG_LEVEL", "WARNING"))
    from awex.meta.meta_server import MetaServer, MetaServerClient

    server = None
    if rank == 0:
        from awex.util.common import get_free_port

        server = MetaServer("127.0.0.1", get_free_port())
        server.start()
        store.set("meta_addr", f"127.0.0.1:{server.port}")
    meta_addr = store.get("meta_addr").decode()
    arch = args.model
    dtype = torch.bfloat16
    hf_config = synth.hf_config_for(arch)
    is_train = rank in train_ranks
    engine_rank = next((e for e, rs in enumerate(engines) if rank in rs), None)

    if is_train:
        tp_rank = train_ranks.index(rank)
        dist.init_process_group("nccl", store=dist.PrefixStore("train_pg", store), rank=tp_rank, world_size=train_tp)
        from awex.writer.nccl_writer import NCCLWeightsWriter

        model = synth.megatron_module(arch, train_tp, tp_rank, dtype, device)
        actor = NCCLWeightsWriter(_TrainEngine(model, hf_config, meta_addr))
        actor.initialize()
        step_fn = lambda s: actor.write_weights(step_id=s)  # noqa: E731
        local_bytes = 0
    else:
        tp_rank = engines[engine_rank].index(rank)
        # an inference engine's workers have their own default group (the
        # reference asserts that one exists before it builds the exchange group)
        dist.init_process_group("nccl", store=dist.PrefixStore(f"infer_pg{engine_rank}", store), rank=tp_rank,
                                world_size=infer_tp)
        from awex.config import InferenceConfig
        from awex.reader.weights_reader import WeightsReader

        cfg = InferenceConfig(tp_size=infer_tp, pp_size=1, dp_size=1, ep_size=1, enable_dp_attention=False, enable_dp_lm_head=False,
                              num_engines=len(engines), engine_rank=engine_rank, meta_server_addr=meta_addr, comm_backend="nccl")
        model = synth.vllm_module(arch, infer_tp, tp_rank, dtype, device, hf_config, zero=True)
        sched = _Scheduler(local_rank, cfg)
        ctx = dict(scheduler=sched, infer_engine_config=cfg, tp_rank=tp_rank, tp_size=infer_tp, pp_rank=0, pp_size=1, dp_rank=0,
                   dp_size=1, ep_rank=0, ep_size=1, attn_tp_rank=tp_rank, attn_tp_size=infer_tp, attn_dp_rank=0,
                   world_size=infer_tp, global_rank=tp_rank, local_rank=local_rank)
        engine = _InferEngine(cfg, hf_config, model, ctx, MetaServerClient(*meta_addr.split(":")), engine_rank, tp_rank, infer_tp)
        actor = WeightsReader(engine)
        actor.initialize()
        step_fn = lambda s: actor.update_weights(step_id=s)  # noqa: E731
        local_bytes = sum(p.numel() * p.element_size() for p in model.parameters())

    # clock record of the timed region (a sampler of this repository: it only reads nvidia-smi)
    sys.path.insert(0, os.path.dirname(HERE))
    from awex_b200.utils.gpu import ClockSampler

    sampler = None
    times_ms, wall_ms = [], []
    total = args.warmup + args.steps
    for s in range(1, total + 1):
        if s == args.warmup + 1 and rank == 0:
            sampler = ClockSampler([local_rank], period_ms=50)
            sampler.__enter__()
        _store_barrier(store, f"step{s}", world)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        start.record()
        step_fn(s)
        stop.record()
        torch.cuda.synchronize()
        wall_ms.append((time.perf_counter() - t0) * 1e3)
        times_ms.append(start.elapsed_time(stop))
    if sampler is not None:
        sampler.__exit__(None, None, None)
    valid = True
    if not is_train and not args.no_validate:
        want = synth.vllm_module(arch, infer_tp, tp_rank, dtype, device, hf_config)
        valid = all(torch.equal(a, b) for (_, a), (_, b) in zip(model.named_parameters(), want.named_parameters()))
    store.set(f"result{rank}", json.dumps({"ms": times_ms[args.warmup:], "wall": wall_ms[args.warmup:], "bytes": local_bytes,
                                           "valid": valid, "egress": 0}))
    _store_barrier(store, "done", world)
    if rank == 0:
        from awex_b200.bench_distributed import bench_config  # the record's layout only; nothing of the framework runs in this arm

        results = [json.loads(store.get(f"result{r}").decode()) for r in range(world)]
        per_step = [max(r["ms"][i] for r in results) for i in range(args.steps)]
        per_wall = [max(r["wall"][i] for r in results) for i in range(args.steps)]
        ms, wall = sum(per_step) / len(per_step), sum(per_wall) / len(per_wall)
        total_bytes = sum(r["bytes"] for r in results)
        egress = total_bytes / len(train_ranks)
        out = {
            "metric": "weight_sync_seconds_per_update", "value": ms / 1e3, "unit": "s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False,
            "scaling": "per-N layouts (not a scaling series)",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic random-init N(0,0.02) weights from per-name seeds",
            "impl": "reference",
            "config": bench_config(arch, total_bytes, label, "separated", all(r["valid"] for r in results)),
            "config_details": {"timing": "CUDA events around NCCLWeightsWriter.write_weights / WeightsReader.update_weights, max over ranks"},
            "aggregate_GBps": total_bytes / (ms / 1e3) / 1e9, "nvlink_GBps_per_gpu": egress / (ms / 1e3) / 1e9,
            "e2e": {"value": wall / 1e3, "unit": "s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "what": "wall clock of the blocking reference calls, max over ranks"},
            "gpu_launches": 0, "per_step_ms": per_step, "clocks": sampler.summary() if sampler is not None else None,
        }
        print(json.dumps(out), flush=True)
    _store_barrier(store, "exit", world)
    dist.destroy_process_group()
    if server is not None:
        server.stop()
    os._exit(0)
