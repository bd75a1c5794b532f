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
        results = [json.loads(store.get(f"result{r}").decode()) for r in range(world)]
        per_step = [max(r["ms"][i] for r in results) for i in range(args.steps)]
        per_wall = [max(r["wall"][i] for r in results) for i in range(args.steps)]
        ms, wall = sum(per_step) / len(per_step), sum(per_wall) / len(per_wall)
        total_bytes = sum(r["bytes"] for r in results)
        egress = total_bytes / len(train_ranks)
        out = {
            "metric": "weight_sync_seconds_per_update", "value": ms / 1e3, "unit": "s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": (ms / 1e3) / 0.8, "dtype": "bf16", "data": "synthetic random-init N(0,0.02) weights from per-name seeds",
            "impl": "reference",
            "config": {"model": arch, "bytes_per_update": total_bytes, "parallelism": label, "mode": "separated",
                       "validated_bitwise": all(r["valid"] for r in results),
                       "timing": "CUDA events around NCCLWeightsWriter.write_weights / WeightsReader.update_weights, max over ranks"},
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
