"""Manual integration run against a real vLLM server (not collected by pytest):

    python tests/weights_exchange_vllm_it.py -b nccl --tp 2 --validate

The main process holds a Megatron-layout training shard (random init, training
TP=1) on the first visible GPU and a MetaServer; a vLLM OpenAI server with this
framework's routes (``python -m awex_b200.awex_vllm_server``) runs as a
subprocess on the next ``--tp`` GPUs with dummy weights of the same
architecture and is driven over HTTP: ``/health``, ``/areal_awex_init``,
``/areal_awex_update``.  One warm-up exchange, then ``--steps`` timed ones; with
``--validate`` the first exchange is checked inside the workers against an HF
checkpoint that the training side writes and the server loads from disk.  The
same flow as `awex/tests/weights_exchange_vllm_it.py` in the reference, with a
synthetic training engine in place of Megatron and a generated ``config.json``
in place of a downloaded model.
"""

from __future__ import annotations

import argparse
import os
import subprocess
import sys
import tempfile
import threading
import time
from typing import List, Optional

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


class VLLMWeightsExchange:
    def __init__(self, args):
        self.args = args
        self.host, self.port = args.host, args.port
        self.server: Optional[subprocess.Popen] = None
        self.meta_server = None
        self.engine = None
        self.writer = None
        self.step = 0
        self.workdir = tempfile.mkdtemp(prefix="awex_vllm_it_")

    # ---- devices: training on the first visible GPU, the server on the next tp ----------------------
    def _devices(self):
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        ids: List[str] = [d for d in visible.split(",") if d] if visible else [str(i) for i in range(self._device_count())]
        need = 1 + self.args.tp * self.args.pp
        if len(ids) < need:
            raise SystemExit(f"{need} GPUs needed (1 training + {need - 1} serving), {len(ids)} visible")
        return ids[0], ids[1:need]

    @staticmethod
    def _device_count() -> int:
        import torch

        return torch.cuda.device_count()

    # ---- server ------------------------------------------------------------------------------------
    def start_meta_server(self) -> str:
        from awex_b200.meta.meta_server import MetaServer

        self.meta_server = MetaServer("127.0.0.1", 0)
        self.meta_server.start()
        return f"127.0.0.1:{self.meta_server.port}"

    def plugin_path(self) -> str:
        """A directory that announces this source tree's vLLM plugin to
        ``importlib.metadata`` (what an installed wheel's entry point does), so
        that worker processes vLLM starts with ``spawn`` register the worker
        methods too."""
        meta = os.path.join(self.workdir, "plugin", "awex_b200_in_tree-0.dist-info")
        os.makedirs(meta, exist_ok=True)
        with open(os.path.join(meta, "METADATA"), "w") as f:
            f.write("Metadata-Version: 2.1\nName: awex-b200-in-tree\nVersion: 0\n")
        with open(os.path.join(meta, "entry_points.txt"), "w") as f:
            f.write("[vllm.general_plugins]\nawex_adapter = awex_b200.vllm_plugin:register_awex_plugin\n")
        return os.path.dirname(meta)

    def start_server(self, model_dir: str, devices: List[str], meta_addr: str) -> None:
        env = os.environ.copy()
        env["CUDA_VISIBLE_DEVICES"] = ",".join(devices)
        env["PYTHONPATH"] = os.pathsep.join([ROOT, self.plugin_path(), env.get("PYTHONPATH", "")])
        cmd = [
            sys.executable, "-m", "awex_b200.awex_vllm_server", "--model", model_dir, "--host", self.host, "--port", str(self.port),
            "--tensor-parallel-size", str(self.args.tp), "--pipeline-parallel-size", str(self.args.pp),
            "--load-format", "dummy", "--skip-tokenizer-init", "--enforce-eager", "--dtype", "bfloat16",
            "--max-model-len", "1024", "--gpu-memory-utilization", str(self.args.gpu_memory_utilization),
            "--awex-comm-backend", self.args.comm_backend, "--awex-meta-server-addr", meta_addr,
        ]
        print("[it] starting", " ".join(cmd), flush=True)
        self.server = subprocess.Popen(cmd, env=env)
        self._wait_for_health(self.args.startup_timeout)

    def _wait_for_health(self, timeout: float) -> None:
        import requests

        deadline = time.time() + timeout
        while time.time() < deadline:
            if self.server.poll() is not None:
                raise RuntimeError(f"vLLM server exited with code {self.server.returncode} before becoming healthy")
            try:
                if requests.get(f"http://{self.host}:{self.port}/health", timeout=5).status_code == 200:
                    return
            except requests.RequestException:
                pass
            time.sleep(1)
        raise RuntimeError(f"vLLM server not healthy after {timeout:.0f}s")

    def _post(self, route: str, payload: dict, timeout: float) -> dict:
        import requests

        resp = requests.post(f"http://{self.host}:{self.port}{route}", json=payload, timeout=timeout)
        if resp.status_code != 200:
            raise RuntimeError(f"{route} failed with {resp.status_code}: {resp.text}")
        return resp.json()

    def awex_init(self, meta_addr: str) -> None:
        payload = {
            "meta_server_addr": meta_addr, "engine_rank": 0, "num_engines": 1, "comm_backend": self.args.comm_backend,
            "enable_debug_mode": self.args.debug, "nnodes": 1, "node_rank": 0,
        }
        if self.args.validate:
            payload.update(weights_validation_steps=1, validate_weights_every_n_steps=1,
                           debug_mode_config={"raise_on_validation_fail": True})
            if self.args.dump_weights_list_for_validation:
                payload["dump_weights_list_for_validation"] = self.args.dump_weights_list_for_validation
                payload["dump_weights_dir_for_validation"] = self.args.dump_weights_dir_for_validation or self.workdir
        self._post("/areal_awex_init", payload, 120)

    def awex_update(self, path: Optional[str]) -> None:
        kwargs = {"path": path} if path else {}
        self._post("/areal_awex_update", {"step_id": self.step, "kwargs": kwargs}, 600)

    # ---- training side --------------------------------------------------------------------------------
    def setup_training(self, arch, meta_addr: str) -> None:
        import torch

        from awex_b200.synthetic.harness import SyntheticTrainEngine
        from awex_b200.synthetic.topology import train_rank_infos
        from awex_b200.writer.weights_writer import get_weights_exchange_writer

        torch.cuda.set_device(0)  # the first visible GPU; the server's devices are hidden from this process's work
        config = {"enable_debug_mode": self.args.debug}
        if self.args.validate:
            config.update(weights_validation_steps=1, validate_weights_every_n_steps=1)
            if self.args.dump_weights_list_for_validation:
                config["dump_weights_list_for_validation"] = self.args.dump_weights_list_for_validation
                config["dump_weights_dir_for_validation"] = self.args.dump_weights_dir_for_validation or self.workdir
        self.engine = SyntheticTrainEngine(arch, train_rank_infos(tp=1)[0], meta_addr, dtype=torch.bfloat16, device="cuda:0",
                                           comm_backend=self.args.comm_backend, **config)
        self.writer = get_weights_exchange_writer(self.engine)
        self.writer.initialize()

    def exchange(self, validated: bool = False) -> float:
        """One update; returns its wall-clock seconds as the caller of both sides sees them."""
        self.step += 1
        path = os.path.join(self.workdir, f"checkpoint_{self.step}") if (self.args.comm_backend == "file" or validated) else None
        started = time.time()
        if self.args.comm_backend == "file":
            self.writer.write_weights(step_id=self.step, path=path)
            self.awex_update(path)
            return time.time() - started
        # The writer runs beside the HTTP call (it waits until the server's workers announce the update).  The
        # server's answer decides: when the update fails there, this side must not go on waiting for it.
        failure: List[BaseException] = []

        def write():
            try:
                self.writer.write_weights(step_id=self.step, **({"path": path} if path else {}))
            except BaseException as exc:  # surfaced after the join
                failure.append(exc)

        thread = threading.Thread(target=write, daemon=True)
        thread.start()
        self.awex_update(path)  # raises when the server reports a failure; the daemon thread ends with the process
        thread.join(timeout=300)
        if thread.is_alive():
            raise RuntimeError("the server finished the update but the writer did not return within 300 s")
        if failure:
            raise failure[0]
        return time.time() - started

    def close(self) -> None:
        if self.writer is not None and hasattr(self.writer, "close"):
            self.writer.close()
        if self.server is not None and self.server.poll() is None:
            self.server.terminate()
            try:
                self.server.wait(timeout=30)
            except subprocess.TimeoutExpired:
                self.server.kill()
        if self.meta_server is not None:
            self.meta_server.stop()


def main(args) -> int:
    from awex_b200.synthetic.arch import get_arch

    arch = get_arch(args.arch)
    if args.layers:
        arch = arch.with_layers(args.layers)
    run = VLLMWeightsExchange(args)
    train_device, serve_devices = run._devices()
    # this process computes on the training GPU only
    os.environ["CUDA_VISIBLE_DEVICES"] = ",".join([train_device] + serve_devices)
    try:
        meta_addr = run.start_meta_server()
        model_dir = arch.write_model_dir(os.path.join(run.workdir, "model"))
        run.start_server(model_dir, serve_devices, meta_addr)
        run.awex_init(meta_addr)
        run.setup_training(arch, meta_addr)
        first = run.exchange(validated=args.validate)
        print(f"[it] first exchange (one-time planning included{', validated' if args.validate else ''}): {first:.3f}s", flush=True)
        times = []
        for _ in range(args.steps):
            run.engine.regenerate(step=run.step + 1)  # an "optimizer step": new values at the same addresses
            times.append(run.exchange())
        if times:
            times.sort()
            print(f"[it] {len(times)} exchanges: median {times[len(times) // 2]:.4f}s min {times[0]:.4f}s max {times[-1]:.4f}s", flush=True)
        print("[it] OK", flush=True)
        return 0
    finally:
        run.close()


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description="Weight exchange between a synthetic Megatron-layout trainer and a vLLM server")
    parser.add_argument("-b", "--comm_backend", default="file", choices=["file", "nccl"], help="weight exchange backend")
    parser.add_argument("--arch", default="llama3-8b", help="architecture preset (awex_b200.synthetic.arch)")
    parser.add_argument("--layers", type=int, default=4, help="number of decoder layers to keep (0: the preset's own)")
    parser.add_argument("--tp", type=int, default=1, help="tensor-parallel size of the vLLM server")
    parser.add_argument("--pp", type=int, default=1, help="pipeline-parallel size of the vLLM server")
    parser.add_argument("--steps", type=int, default=10, help="timed exchanges after the first")
    parser.add_argument("--host", default="127.0.0.1")
    parser.add_argument("--port", type=int, default=8000)
    parser.add_argument("--gpu-memory-utilization", type=float, default=0.5)
    parser.add_argument("--startup-timeout", type=float, default=600.0, help="seconds to wait for the server's /health")
    parser.add_argument("--validate", action="store_true", help="validate the first exchange against a file-loaded reference")
    parser.add_argument("--debug", action="store_true", help="enable_debug_mode on both sides (metadata and plan dumps)")
    parser.add_argument("--dump-weights-list-for-validation", default="", help="comma-separated parameter names to dump during validation")
    parser.add_argument("--dump-weights-dir-for-validation", default="", help="directory for those dumps")
    cli = parser.parse_args()
    cli.dump_weights_list_for_validation = [n.strip() for n in cli.dump_weights_list_for_validation.split(",") if n.strip()]
    cli.dump_weights_dir_for_validation = cli.dump_weights_dir_for_validation or None
    sys.exit(main(cli))
