"""Serving-engine integrations against fakes: the vLLM server adapter and plugin,
the in-process SGLang / vLLM wrappers, the mbridge loader, the send/recv helper
layer and process handle accounting.  No serving engine is imported."""

import asyncio
import threading
import types

import pytest
import torch

from awex_b200.config import InferenceConfig


# ------------------------------------------------------------------------------------------ fakes
class FakeParallelConfig:
    def __init__(self, tp=2, pp=1, dp=1, ep=False, pcp=1, rank=0, dp_rank=0):
        self.tensor_parallel_size, self.pipeline_parallel_size, self.data_parallel_size = tp, pp, dp
        self.enable_expert_parallel, self.prefill_context_parallel_size = ep, pcp
        self.world_size, self.rank, self.data_parallel_rank = tp * pp * pcp, rank, dp_rank
        self.world_size_across_dp = self.world_size * dp
        self.nnodes, self.node_rank = 1, 0


class FakeClient:
    """Synchronous engine client with ``collective_rpc`` only."""

    def __init__(self, pc=None):
        self.vllm_config = types.SimpleNamespace(parallel_config=pc or FakeParallelConfig())
        self.model_config = types.SimpleNamespace(hf_config=types.SimpleNamespace(architectures=["Qwen3ForCausalLM"]))
        self.calls = []
        self.slept, self.woken = [], []

    def collective_rpc(self, method, timeout=None, args=(), kwargs=None):
        self.calls.append((method, args, kwargs))
        return [f"{method}-w0", f"{method}-w1"]

    def sleep(self, level):
        self.slept.append(level)

    def wake_up(self, tags):
        self.woken.append(tags)


class FakeDPClient(FakeClient):
    """Client that can address its data-parallel cores one by one."""

    def __init__(self, n_cores=3):
        super().__init__(FakeParallelConfig(tp=1, dp=n_cores))
        self.core_engines = [f"core{i}" for i in range(n_cores)]
        self.per_core = []

    async def _call_utility_async(self, utility, method, timeout, args, kwargs, engine=None):
        self.per_core.append((engine, method))
        return [{"core": engine, "shard": 0}, {"core": engine, "shard": 1}]


def _adapter(client, **kw):
    from awex_b200.vllm_awex_adapter import AwexVLLMServerAdapter

    a = AwexVLLMServerAdapter(client, meta_server_addr="127.0.0.1:1", **kw)
    a._initialized = True
    return a


# ------------------------------------------------------------------------------------------ adapter
def test_inference_config_from_vllm_expert_parallel_spans_tp_dp_pcp():
    from awex_b200.vllm_awex_adapter import inference_config_from_vllm

    cfg = inference_config_from_vllm(FakeParallelConfig(tp=2, dp=4, ep=True, pcp=2), num_engines=3, engine_rank=1)
    assert (cfg.tp_size, cfg.dp_size, cfg.ep_size, cfg.num_engines, cfg.engine_rank) == (2, 4, 16, 3, 1)
    assert inference_config_from_vllm(FakeParallelConfig(tp=2, dp=4)).ep_size == 1


def test_adapter_ships_callables_by_name_and_serialises_config():
    from awex_b200.meta.meta_server import MetaServerClient  # any importable callable will do

    client = FakeClient()
    a = _adapter(client)
    out = a.execute_task_in_model_worker(MetaServerClient.barrier, infer_engine_config=a.config, x=1)
    assert out == ["awex_execute-w0", "awex_execute-w1"]
    method, _args, payload = client.calls[-1]
    assert method == "awex_execute"
    assert payload["task_module"] == "awex_b200.meta.meta_server" and payload["task_qualname"] == "MetaServerClient.barrier"
    assert isinstance(payload["task_kwargs"]["infer_engine_config"], dict) and payload["task_kwargs"]["x"] == 1
    a.execute_task_in_model_worker("_update_parameters_in_tp_worker", step_id=3)
    assert client.calls[-1] == ("_update_parameters_in_tp_worker", (), {"step_id": 3})


def test_adapter_meta_collection_fans_out_to_every_dp_core():
    from awex_b200.meta.infer_meta_resolver import collect_worker_param_info

    client = FakeDPClient(3)
    loop = asyncio.new_event_loop()
    t = threading.Thread(target=loop.run_forever, daemon=True)
    t.start()
    try:
        a = _adapter(client, loop=loop)
        merged = a.execute_task_in_model_worker(collect_worker_param_info, engine_name="vllm", infer_engine_config=a.config)
        assert [m["core"] for m in merged] == ["core0", "core0", "core1", "core1", "core2", "core2"]
        assert sorted(e for e, _ in client.per_core) == ["core0", "core1", "core2"]
        # other tasks go through the plain collective call once
        a.execute_task_in_model_worker("_begin_update_in_tp_worker", step_id=1)
        assert client.calls[-1][0] == "_begin_update_in_tp_worker" and len(client.per_core) == 3
    finally:
        loop.call_soon_threadsafe(loop.stop)
        t.join()


def test_adapter_refuses_tasks_before_initialize_and_maps_memory_hooks():
    client = FakeClient()
    a = _adapter(client)
    a._initialized = False
    with pytest.raises(RuntimeError):
        a.execute_task_in_model_worker("x")
    with pytest.raises(RuntimeError):
        a.update_weights(1)
    a.release_memory_occupation()
    a.resume_memory_occupation(["weights"])
    assert client.slept == [1] and client.woken == [["weights"]]
    a.update_weights_from_disk("/ckpt")
    assert client.calls[-1] == ("awex_update_weights_from_disk", ("/ckpt", None), None)


# ------------------------------------------------------------------------------------------ plugin
def test_kwarg_whitelist_drops_unknown_and_reports_missing():
    from awex_b200.vllm_plugin import AWEX_WORKER_METHODS, AWEX_WORKER_SIGNATURES, filter_awex_kwargs, resolve_task

    assert filter_awex_kwargs("_update_parameters_in_tp_worker", {"step_id": 1, "junk": 2}) == {"step_id": 1}
    with pytest.raises(ValueError, match="step_id"):
        filter_awex_kwargs("_update_parameters_in_tp_worker", {"junk": 2})
    assert filter_awex_kwargs("not_listed", {"a": 1}) == {"a": 1}
    assert set(AWEX_WORKER_METHODS) == set(AWEX_WORKER_SIGNATURES)
    for module, qualname in AWEX_WORKER_METHODS.values():
        assert callable(resolve_task(module, qualname))


def test_sanitize_for_ipc_makes_plain_data():
    from awex_b200.vllm_plugin import sanitize_for_ipc

    cfg = InferenceConfig(tp_size=2)
    out = sanitize_for_ipc({"d": torch.bfloat16, "dev": torch.device("cpu"), "t": (1, (2, torch.float32)), "c": cfg})
    assert out["d"] == "bfloat16" and out["dev"] == "cpu" and out["t"] == [1, [2, "float32"]]
    assert isinstance(out["c"], dict) and out["c"]["tp_size"] == 2


class _Group:
    def __init__(self, rank, size):
        self.rank_in_group, self.world_size = rank, size


def _fake_worker(pc):
    class Worker:
        def __init__(self):
            self.model_runner = types.SimpleNamespace(model=torch.nn.Linear(2, 2), vllm_config=types.SimpleNamespace(parallel_config=pc))
            self.local_rank = pc.rank

    return Worker


def echo_task(model, model_context, infer_engine_config=None, step_id=None):
    return {"tp": (model_context["tp_rank"], model_context["tp_size"]), "global_rank": model_context["global_rank"],
            "engine_rank": model_context["engine_rank"], "cfg_tp": model_context["infer_engine_config"].tp_size,
            "dtype": model.weight.dtype, "step_id": step_id, "has_flush": hasattr(model_context["scheduler"], "flush_cache")}


def test_patched_worker_runs_tasks_with_rank_context():
    from awex_b200.vllm_plugin import patch_worker_class

    pc = FakeParallelConfig(tp=2, dp=2, rank=1, dp_rank=1)
    worker_cls = _fake_worker(pc)
    groups = {"tp": lambda: _Group(1, 2), "pp": lambda: _Group(0, 1), "dp": lambda: _Group(1, 2), "ep": lambda: _Group(0, 1)}
    patch_worker_class(worker_cls, groups)
    w = worker_cls()
    ctx = w.awex_get_model_context()
    assert (ctx["tp_rank"], ctx["dp_rank"], ctx["global_rank"], ctx["world_size"], ctx["is_infer"]) == (1, 1, 3, 4, True)
    cfg = InferenceConfig(tp_size=2, dp_size=2, engine_rank=1, num_engines=2, comm_backend="nccl", meta_server_addr="127.0.0.1:1")
    import dataclasses

    out = w.awex_execute(__name__, "echo_task", {"infer_engine_config": dataclasses.asdict(cfg), "step_id": 7})
    assert out == {"tp": [1, 2], "global_rank": 3, "engine_rank": 1, "cfg_tp": 2, "dtype": "float32", "step_id": 7, "has_flush": True}
    assert w.flush_cache() is True
    for name in ("_update_parameters_in_tp_worker", "_get_model_param_info", "awex_update_weights_from_disk"):
        assert callable(getattr(w, name))
    with pytest.raises(ValueError):
        w._update_parameters_in_tp_worker(junk=1)


def test_router_init_and_update_routes():
    fastapi = pytest.importorskip("fastapi")
    from fastapi.testclient import TestClient

    from awex_b200.vllm_plugin import build_router

    made = {}

    class FakeAdapter:
        def __init__(self, client, loop=None, **fields):
            made["fields"], made["client"] = fields, client
            self.steps = []

        def initialize(self):
            made["initialized"] = True

        def update_weights(self, step_id, **kw):
            if step_id < 0:
                raise RuntimeError("bad step")
            self.steps.append((step_id, kw))

    app = fastapi.FastAPI()
    app.include_router(build_router(FakeAdapter))
    app.state.engine_client = "client"
    with TestClient(app) as http:
        r = http.post("/areal_awex_update", json={"step_id": 1})
        assert r.status_code == 400 and not r.json()["success"]
        r = http.post("/areal_awex_init", json={"meta_server_addr": "h:1", "engine_rank": 1, "num_engines": 2, "comm_backend": "nccl"})
        assert r.status_code == 200 and r.json()["success"], r.text
        assert made["initialized"] and made["fields"]["engine_rank"] == 1 and made["fields"]["comm_backend"] == "nccl"
        r = http.post("/areal_awex_update", json={"step_id": 5, "kwargs": {"a": 1}})
        assert r.status_code == 200 and app.state.awex_adapter.steps == [(5, {"a": 1})]
        r = http.post("/areal_awex_update", json={"step_id": -1})
        assert r.status_code == 500 and "bad step" in r.json()["message"]
        assert http.post("/areal_awex_init", json={}).status_code == 422


# ------------------------------------------------------------------------------------------ in-process engines
class FakeSGL:
    def __init__(self):
        self.tokenizer_manager = types.SimpleNamespace(model_config=types.SimpleNamespace(architectures=["Qwen3ForCausalLM"]))
        self.log = []

    def update_weights_from_disk(self, model_path, load_format=None):
        self.log.append(("disk", model_path, load_format))

    def release_memory_occupation(self, tags):
        self.log.append(("release", sorted(tags)))

    def resume_memory_occupation(self, tags):
        self.log.append(("resume", sorted(tags)))

    def execute_task_in_model_worker(self, fn, **kw):
        return [fn(**kw)]


def test_sglang_engine_memory_tags_are_idempotent_and_node_gated():
    from awex_b200.engine.sglang import SGLangEngine

    sgl = FakeSGL()
    eng = SGLangEngine(InferenceConfig(tp_size=1), sgl)
    with pytest.raises(RuntimeError):
        eng.execute_task_in_model_worker(lambda: 1)
    eng._initialized = True  # the reader itself is covered by the exchange tests
    eng.release_memory_occupation("weights")
    eng.release_memory_occupation()  # only kv_cache is still held
    eng.release_memory_occupation()  # nothing left
    eng.resume_memory_occupation(["kv_cache", "weights"])
    eng.resume_memory_occupation()
    assert sgl.log == [("release", ["weights"]), ("release", ["kv_cache"]), ("resume", ["kv_cache", "weights"])]
    assert eng.execute_task_in_model_worker(lambda a: a + 1, a=1) == [2]
    eng.update_weights_from_disk("/ckpt", "auto")
    assert sgl.log[-1] == ("disk", "/ckpt", "auto")
    other = SGLangEngine(InferenceConfig(tp_size=1, nnodes=2, node_rank=1), sgl)
    other._initialized = True
    with pytest.raises(RuntimeError):
        other.execute_task_in_model_worker(lambda: 1)
    # weights that come back from a release may sit in new memory: with parameters_may_move the reader is told
    told = []
    for may_move, expected in ((False, 0), (True, 1)):
        moving = SGLangEngine(InferenceConfig(tp_size=1, debug_mode_config={"parameters_may_move": may_move}), FakeSGL())
        moving._initialized = True
        moving.weights_exchange_reader = types.SimpleNamespace(invalidate_addresses=lambda: told.append(1))
        moving.release_memory_occupation()
        moving.resume_memory_occupation(["kv_cache"])  # the weights are still away
        assert len(told) == 0 if not may_move else True
        before = len(told)
        moving.resume_memory_occupation(["weights"])
        assert len(told) - before == expected


class FakeVLLMHandle:
    def __init__(self, cores=2):
        self.initialized, self.cores, self.calls = False, cores, []
        self._engine = types.SimpleNamespace(offload=lambda: self.calls.append("offload"), onload=lambda tags: self.calls.append(("onload", tags)))

    def initialize(self):
        self.initialized = True

    def call_utility(self, method, args, kwargs, run_on_all):
        self.calls.append((method, args, kwargs, run_on_all))
        one = {"results": [f"{method}-a", f"{method}-b"]}
        return [one] * self.cores if run_on_all else one


def test_vllm_engine_ships_tasks_and_merges_core_results():
    from awex_b200.engine import vllm as vllm_engine

    handle = FakeVLLMHandle()
    eng = vllm_engine.VLLMEngine(InferenceConfig(tp_size=1), handle, hf_config=types.SimpleNamespace())
    with pytest.raises(ValueError):
        vllm_engine.VLLMEngine(InferenceConfig(tp_size=1), handle)
    eng._before_initialize()
    assert handle.initialized
    eng._initialized = True
    assert eng.execute_task_in_model_worker(echo_task, step_id=1) == ["awex_execute-a", "awex_execute-b"] * 2
    method, _a, payload, run_on_all = handle.calls[-1]
    assert (method, run_on_all) == ("awex_execute", True)
    assert payload == {"task_module": __name__, "task_qualname": "echo_task", "task_kwargs": {"step_id": 1}}
    assert eng.execute_task_in_model_worker("ping", run_on_all=False, x=1) == ["ping-a", "ping-b"]
    eng.release_memory_occupation()
    eng.resume_memory_occupation("weights")
    assert handle.calls[-2:] == ["offload", ("onload", ["weights"])]
    vllm_engine.VLLM_TASK_SIGNATURES["strict"] = {"required": ["a"], "optional": ["b"]}
    try:
        assert vllm_engine.adapt_task_kwargs("strict", {"a": 1, "c": 2}) == {"a": 1}
        with pytest.raises(ValueError):
            vllm_engine.adapt_task_kwargs("strict", {"b": 1})
    finally:
        del vllm_engine.VLLM_TASK_SIGNATURES["strict"]


# ------------------------------------------------------------------------------------------ mbridge loader
def test_mbridge_loader_merges_fused_parameters(tmp_path):
    from awex_b200.mbridge_loader import concat_along_matching_dim, load_weights_from_hf_with_mbridge
    from awex_b200.utils.safetensors_io import save_checkpoint

    hf = {"q": torch.randn(4, 8), "k": torch.randn(2, 8), "v": torch.randn(2, 8), "o": torch.randn(8, 4), "head": torch.randn(3, 8)}
    save_checkpoint(str(tmp_path), hf, max_shard_bytes=200)

    class Model(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.qkv = torch.nn.Parameter(torch.zeros(8, 8))
            self.proj = torch.nn.Parameter(torch.zeros(8, 4, dtype=torch.bfloat16))
            self.output_layer = torch.nn.Parameter(torch.zeros(3, 8))

    class Bridge:
        def _weight_name_mapping_mcore_local_to_global(self, model):
            return {"qkv": "g.qkv", "proj": "g.proj", "output_layer": "g.output_layer", "absent": "g.absent"}

        def _weight_name_mapping_mcore_to_hf(self, name):
            return {"g.qkv": ["q", "k", "v"], "g.proj": "o", "g.output_layer": ["head"]}[name]

    m = Model()
    load_weights_from_hf_with_mbridge(Bridge(), [m], str(tmp_path), is_critic=True)
    assert torch.equal(m.qkv.data, torch.cat([hf["q"], hf["k"], hf["v"]]))
    assert torch.equal(m.proj.data, hf["o"].to(torch.bfloat16))
    assert not m.output_layer.data.any()  # critics keep their own head
    load_weights_from_hf_with_mbridge(Bridge(), [m], str(tmp_path))
    assert torch.equal(m.output_layer.data, hf["head"])
    cols = concat_along_matching_dim([torch.ones(2, 3), torch.ones(2, 5)], (2, 8))
    assert cols.shape == (2, 8)
    with pytest.raises(ValueError):
        concat_along_matching_dim([torch.ones(2, 3), torch.ones(2, 3)], (5, 3))


# ------------------------------------------------------------------------------------------ send/recv helpers
def test_rank_map_validation_and_two_phase_colouring():
    import math

    from awex_b200.transfer.nccl_comm import compute_two_phase_partition, interleave_by_peer, ring_peers, validate_rank_mappings

    validate_rank_mappings({0: 1, 1: 0}, {1: 0, 0: 1})
    with pytest.raises(ValueError):
        validate_rank_mappings({0: 1, 1: 0}, {1: 0, 0: 0})
    for world in (2, 4, 6, 8, 12):
        for stage in range(1, world):
            if (world // math.gcd(world, stage)) % 2:
                continue  # odd cycles cannot be two-coloured
            for r in range(world):
                to, frm = ring_peers(r, stage, world)
                assert compute_two_phase_partition(r, stage, world) != compute_two_phase_partition(to, stage, world)
                assert ring_peers(frm, stage, world)[0] == r
    ops = [types.SimpleNamespace(peer=p, i=i) for p, n in ((3, 3), (1, 1), (2, 2)) for i in range(n)]
    assert [(o.peer, o.i) for o in interleave_by_peer(ops)] == [(1, 0), (2, 0), (3, 0), (2, 1), (3, 1), (3, 2)]


def test_watchdog_reports_a_stalled_exchange():
    import time

    from awex_b200.transfer.nccl_comm import ExchangeWatchdog

    seen = []
    with ExchangeWatchdog("stall", lambda: ["op-a"], timeout_s=0.05, sink=seen.append) as dog:
        time.sleep(0.3)
    assert dog.fired and "op-a" in seen[0] and "test_watchdog_reports_a_stalled_exchange" in seen[0]
    with ExchangeWatchdog("quick", timeout_s=5.0, sink=seen.append) as dog:
        pass
    assert not dog.fired and len(seen) == 1


def test_handle_counts():
    from awex_b200.utils.system_util import get_handle_counts

    counts = get_handle_counts()
    assert counts["open_fds"] > 0 and counts["soft_limit"] <= counts["hard_limit"] or counts["hard_limit"] == -1
    assert counts["total_ipc"] == counts["sysv_ipc"] + counts["posix_ipc"]


def test_server_wrapper_separates_its_own_flags():
    from awex_b200.awex_vllm_server import split_own_arguments

    rest, own = split_own_arguments(["--model", "m", "--awex-comm-backend", "nccl", "--tp", "2", "--awex-meta-server-addr=10.0.0.1:80"])
    assert rest == ["--model", "m", "--tp", "2"]
    assert own == {"AWEX_COMM_BACKEND": "nccl", "AWEX_META_SERVER_ADDR": "10.0.0.1:80"}
    with pytest.raises(SystemExit):
        split_own_arguments(["--awex-comm-backend"])


def test_vllm_integration_script_speaks_the_plugin_protocol(monkeypatch, tmp_path):
    """The manual vLLM integration script (needs GPUs and a server to run) builds
    request bodies that the plugin's models accept, picks one training GPU plus
    tp*pp serving GPUs, and starts the server wrapper with flags the wrapper
    understands."""
    import importlib.util
    import os
    from types import SimpleNamespace

    from awex_b200.awex_vllm_server import split_own_arguments
    from awex_b200.vllm_plugin import AwexInitRequest, AwexUpdateRequest

    path = os.path.join(os.path.dirname(__file__), "weights_exchange_vllm_it.py")
    spec = importlib.util.spec_from_file_location("weights_exchange_vllm_it", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    args = SimpleNamespace(host="127.0.0.1", port=8123, tp=2, pp=1, comm_backend="nccl", debug=False, validate=True,
                           dump_weights_list_for_validation=["model.norm.weight"], dump_weights_dir_for_validation=None,
                           gpu_memory_utilization=0.5, startup_timeout=1.0)
    run = module.VLLMWeightsExchange(args)
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "3,4,5,6")
    assert run._devices() == ("3", ["4", "5"])
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "3,4")
    with pytest.raises(SystemExit):
        run._devices()
    posted = []
    run._post = lambda route, payload, timeout: posted.append((route, payload)) or {"success": True}
    run.awex_init("127.0.0.1:9999")
    run.step = 7
    run.awex_update("/ckpt")
    run.awex_update(None)
    (r0, init), (r1, up1), (r2, up2) = posted
    assert (r0, r1, r2) == ("/areal_awex_init", "/areal_awex_update", "/areal_awex_update")
    request = AwexInitRequest(**init)
    assert request.comm_backend == "nccl" and request.weights_validation_steps == 1
    assert request.dump_weights_list_for_validation == ["model.norm.weight"] and request.dump_weights_dir_for_validation == run.workdir
    assert AwexUpdateRequest(**up1).kwargs == {"path": "/ckpt"} and AwexUpdateRequest(**up2).step_id == 7
    # the server's processes discover the plugin of this source tree like an installed one
    import subprocess
    import sys

    probe = ("from importlib.metadata import entry_points; "
             "print([(e.name, e.value) for e in entry_points(group='vllm.general_plugins') if e.name == 'awex_adapter'])")
    found = subprocess.run([sys.executable, "-c", probe], env={**os.environ, "PYTHONPATH": run.plugin_path()}, capture_output=True, text=True)
    assert "awex_b200.vllm_plugin:register_awex_plugin" in found.stdout, found.stderr
    # the server command: our own flags are separated from vLLM's
    started = []
    monkeypatch.setattr(module.subprocess, "Popen", lambda cmd, env: started.append((cmd, env)) or SimpleNamespace(poll=lambda: 1, returncode=1))
    with pytest.raises(RuntimeError, match="exited"):
        run.start_server(str(tmp_path), ["4", "5"], "127.0.0.1:9999")
    cmd, env = started[0]
    assert cmd[1:3] == ["-m", "awex_b200.awex_vllm_server"] and env["CUDA_VISIBLE_DEVICES"] == "4,5"
    assert run.plugin_path() in env["PYTHONPATH"].split(os.pathsep)
    rest, own = split_own_arguments(cmd[3:])
    assert own == {"AWEX_COMM_BACKEND": "nccl", "AWEX_META_SERVER_ADDR": "127.0.0.1:9999"}
    assert "--tensor-parallel-size" in rest and not any(a.startswith("--awex") for a in rest)
    import shutil

    shutil.rmtree(run.workdir)


def test_sglang_integration_script_runs_against_a_stand_in_engine(monkeypatch, tmp_path):
    """``tests/weights_exchange_it.py`` end to end on the CPU with the file
    backend: a stand-in ``sglang`` package whose ``Engine`` keeps what it loads
    from disk, wrapped in :class:`SGLangEngine` by the script; every exchange's
    checkpoint must hold the weights the training side had at that step."""
    import dataclasses
    import importlib.util
    import os
    import sys

    import torch

    from awex_b200.synthetic.arch import get_arch
    from awex_b200.synthetic.models import CanonicalWeights, canonical_state_dict
    from awex_b200.utils.safetensors_io import load_checkpoint

    @dataclasses.dataclass
    class ServerArgs:
        model_path: str = ""
        skip_tokenizer_init: bool = False
        load_format: str = "auto"
        dtype: str = "auto"
        device: str = "cuda"
        mem_fraction_static: float = 0.9
        tp_size: int = 1
        pp_size: int = 1
        dp_size: int = 1
        ep_size: int = 1
        random_seed: int = 0
        log_level: str = "info"

    engines = []

    class Engine:
        def __init__(self, **kwargs):
            self.server_args = ServerArgs(**kwargs)  # refuses what the real dataclass would not know
            self.tokenizer_manager = types.SimpleNamespace(model_config=types.SimpleNamespace(architectures=["LlamaForCausalLM"]))
            self.loaded, self.down = [], False
            engines.append(self)

        def update_weights_from_disk(self, model_path, load_format=None):
            self.loaded.append(load_checkpoint(model_path))

        def release_memory_occupation(self, tags=None):
            pass

        def resume_memory_occupation(self, tags=None):
            pass

        def execute_task_in_model_worker(self, fn, **kwargs):
            return [fn(**kwargs)]

        def shutdown(self):
            self.down = True

    package, srt, server_args = types.ModuleType("sglang"), types.ModuleType("sglang.srt"), types.ModuleType("sglang.srt.server_args")
    package.Engine, package.srt, srt.server_args, server_args.ServerArgs = Engine, srt, server_args, ServerArgs
    for name, module in (("sglang", package), ("sglang.srt", srt), ("sglang.srt.server_args", server_args)):
        monkeypatch.setitem(sys.modules, name, module)
    monkeypatch.setenv("AWEX_DEVICE_TYPE", "cpu")
    monkeypatch.setattr("tempfile.mkdtemp", lambda prefix="": str(tmp_path))
    spec = importlib.util.spec_from_file_location("weights_exchange_it", os.path.join(os.path.dirname(__file__), "weights_exchange_it.py"))
    script = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(script)
    args = types.SimpleNamespace(comm_backend="file", arch="tiny-llama", layers=0, tp=1, steps=2, mem_fraction_static=0.5, debug=False)
    assert script.main(args) == 0
    (engine,) = engines
    assert engine.down and engine.server_args.load_format == "dummy" and engine.server_args.device == "cpu"
    assert not hasattr(engine.server_args, "attention_backend")  # settings the engine's arguments do not know were dropped
    arch = get_arch("tiny-llama")
    assert len(engine.loaded) == 3  # the first exchange and two more, each after an "optimizer step"
    for step, got in zip((0, 2, 3), engine.loaded):
        want = canonical_state_dict(arch, CanonicalWeights(arch, torch.bfloat16, "cpu", 0, step))
        assert set(got) == set(want)
        assert all(torch.equal(got[name], want[name]) for name in want), step
