"""The plugin against the vLLM that is installed (not a fake): the worker
methods land on the real `vllm.v1.worker.worker_base.WorkerBase`, the routes are
added by the real `vllm.entrypoints.openai.api_server.build_app`, and the two
HTTP endpoints drive an adapter.  Runs without a GPU; skipped where vLLM is not
installed.  (Reference: `awex/vllm_plugin.py:174-376,413-506`.)"""

import argparse

import pytest

vllm = pytest.importorskip("vllm")


@pytest.fixture(scope="module")
def patched():
    from awex_b200 import vllm_plugin

    assert vllm_plugin.patch_vllm_worker() is True
    return vllm_plugin


def test_worker_methods_land_on_the_installed_worker_base(patched):
    from vllm.v1.worker.worker_base import WorkerBase

    for name in ("awex_get_model_context", "awex_execute", "awex_update_weights_from_disk", "flush_cache", *patched.AWEX_WORKER_METHODS):
        assert callable(getattr(WorkerBase, name, None)), name

    # a task reaches the worker's model through awex_execute, addressed by module and qualified name
    class Runner:
        model = object()

        def get_model(self):
            return self.model

    worker = WorkerBase.__new__(WorkerBase)
    worker.model_runner = Runner()
    worker.rank, worker.local_rank = 0, 0
    assert WorkerBase.flush_cache(worker) is True  # no cache to flush on this stand-in runner


def test_routes_are_added_by_the_real_build_app_and_drive_the_adapter(patched):
    from fastapi.testclient import TestClient
    from vllm.entrypoints.openai import api_server

    calls = []

    class Adapter:
        def __init__(self, engine_client, loop=None, **fields):
            calls.append(("new", engine_client, fields["meta_server_addr"], fields["comm_backend"], fields["num_engines"]))

        def initialize(self):
            calls.append(("initialize",))

        def update_weights(self, step_id, **kwargs):
            if step_id < 0:
                raise RuntimeError("no such step")
            calls.append(("update", step_id, kwargs))

    assert patched.attach_router_to_vllm(patched.build_router(Adapter)) is True
    # the arguments `build_app` reads, with the server's defaults (its own parser needs a device to build)
    args = argparse.Namespace(allow_credentials=False, allowed_headers=["*"], allowed_methods=["*"], allowed_origins=["*"],
                              api_key=None, disable_fastapi_docs=True, enable_offline_docs=False, enable_request_id_headers=False,
                              middleware=[], root_path=None)
    app = api_server.build_app(args)
    paths = {getattr(r, "path", None) for r in app.routes}
    assert {"/areal_awex_init", "/areal_awex_update"} <= paths
    engine_client = object()
    app.state.engine_client = engine_client
    client = TestClient(app)
    early = client.post("/areal_awex_update", json={"step_id": 1})
    assert early.status_code == 400 and "not initialized" in early.json()["message"]
    made = client.post("/areal_awex_init", json={"meta_server_addr": "127.0.0.1:9", "comm_backend": "nccl", "num_engines": 2})
    assert made.status_code == 200 and made.json()["success"] is True
    done = client.post("/areal_awex_update", json={"step_id": 7, "kwargs": {"path": "/x"}})
    assert done.status_code == 200 and done.json()["success"] is True
    failed = client.post("/areal_awex_update", json={"step_id": -1})
    assert failed.status_code == 500 and "no such step" in failed.json()["message"]
    assert calls == [("new", engine_client, "127.0.0.1:9", "nccl", 2), ("initialize",), ("update", 7, {"path": "/x"})]


def test_a_reload_from_disk_never_uses_the_dummy_loader(patched):
    """A server started with `--load-format dummy` must read the checkpoint when it
    is asked to reload from disk, and a caller's `load_format` wins."""
    from vllm.config import LoadConfig
    from vllm.model_executor.model_loader import get_model_loader

    dummy = LoadConfig(load_format="dummy")
    picked = patched.reload_load_config(dummy)
    assert str(picked.load_format).rsplit(".", 1)[-1].lower() == "auto" and str(dummy.load_format).rsplit(".", 1)[-1].lower() == "dummy"
    assert type(get_model_loader(picked)).__name__ != type(get_model_loader(dummy)).__name__
    auto = LoadConfig(load_format="auto")
    assert patched.reload_load_config(auto) is auto
    assert str(patched.reload_load_config(auto, "safetensors").load_format).rsplit(".", 1)[-1].lower() == "safetensors"
