"""Manual integration run against a real SGLang engine (not collected by pytest):

    python tests/weights_exchange_it.py -b nccl --tp 2

The flow of `awex/tests/weights_exchange_it.py` in the reference: an SGLang
engine with dummy weights on the first ``--tp`` GPUs, wrapped in
:class:`awex_b200.engine.sglang.SGLangEngine`; a training shard (random init,
Megatron layout, training TP=1) on the next GPU; one warm-up exchange, a check of
a handful of parameters read back from the engine's tensor-parallel workers
against the training side's converted parameters, then ``--steps`` further
exchanges.  A synthetic training engine stands in for Megatron and a generated
``config.json`` for a downloaded model.

SGLang must be importable and its ``Engine`` must offer
``execute_task_in_model_worker`` (the fork the reference targets); the script
says so and exits with code 2 otherwise.
"""

from __future__ import annotations

import argparse
import os
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# canonical names to check after the first exchange: (name, dimension along which inference TP cuts it, or None)
CHECKED_PARAMETERS = [
    ("model.embed_tokens.weight", 0),
    ("model.layers.0.self_attn.o_proj.weight", 1),
    ("model.layers.0.mlp.down_proj.weight", 1),
    ("model.layers.0.input_layernorm.weight", None),
    ("model.norm.weight", None),
]


def read_from_worker(**kwargs):
    """Runs inside every SGLang model worker: a slice of one canonical parameter."""
    reader = kwargs["model_context"]["scheduler"].awes_weights_reader
    if reader is None or kwargs["param_name"] not in reader.parameters:
        return None
    return reader.parameters[kwargs["param_name"]][kwargs["slices"]].detach().cpu()


class WeightsExchangeIT:
    def __init__(self, args):
        self.args = args
        self.workdir = tempfile.mkdtemp(prefix="awex_sgl_it_")
        self.executor = ThreadPoolExecutor(max_workers=1)
        self.meta_server = None
        self.sgl = None
        self.inference = None
        self.training = None
        self.writer = None
        self.step = 0

    def initialize(self, arch) -> None:
        import sglang
        import torch

        from awex_b200.config import InferenceConfig
        from awex_b200.engine.sglang import SGLangEngine, extract_sgl_config
        from awex_b200.meta.meta_server import MetaServer
        from awex_b200.synthetic.harness import SyntheticTrainEngine
        from awex_b200.synthetic.topology import train_rank_infos
        from awex_b200.utils import device as device_util
        from awex_b200.writer.weights_writer import get_weights_exchange_writer

        on_gpu = device_util.get_device_type() == "cuda"
        self.meta_server = MetaServer("127.0.0.1", 0)
        self.meta_server.start()
        meta_addr = f"127.0.0.1:{self.meta_server.port}"
        model_dir = arch.write_model_dir(os.path.join(self.workdir, "model"))
        settings = {
            "model_path": model_dir, "skip_tokenizer_init": True, "load_format": "dummy", "dtype": "bfloat16", "device": "cuda" if on_gpu else "cpu",
            "mem_fraction_static": self.args.mem_fraction_static, "tp_size": self.args.tp, "pp_size": 1, "dp_size": 1, "ep_size": 1,
            "random_seed": 47, "log_level": "info", "attention_backend": "torch_native",
        }
        self.sgl = sglang.Engine(**extract_sgl_config(settings))
        if not hasattr(self.sgl, "execute_task_in_model_worker"):
            raise SystemExit("this SGLang build has no Engine.execute_task_in_model_worker (needed to reach the model workers)")
        config = InferenceConfig.from_sgl_engine(self.sgl, comm_backend=self.args.comm_backend, meta_server_addr=meta_addr,
                                                 num_engines=1, engine_rank=0, enable_debug_mode=self.args.debug)
        self.inference = SGLangEngine(config, self.sgl)
        self.inference.initialize()
        # the training shard lives on the GPU after the engine's
        device = f"cuda:{self.args.tp}" if on_gpu else "cpu"
        if on_gpu:
            torch.cuda.set_device(self.args.tp)
        self.training = SyntheticTrainEngine(arch, train_rank_infos(tp=1)[0], meta_addr, dtype=torch.bfloat16, device=device,
                                             comm_backend=self.args.comm_backend, enable_debug_mode=self.args.debug)
        self.writer = get_weights_exchange_writer(self.training)
        self.writer.initialize()

    def exchange(self) -> float:
        self.step += 1
        path = {"path": os.path.join(self.workdir, f"checkpoint_{self.step}")} if self.args.comm_backend == "file" else {}
        started = time.time()
        if path:
            self.writer.write_weights(step_id=self.step, **path)
            self.inference.update_weights(step_id=self.step, **path)
        else:
            pending = self.executor.submit(self.inference.update_weights, step_id=self.step)
            self.writer.write_weights(step_id=self.step)
            pending.result(timeout=600)
        return time.time() - started

    def verify(self, length: int = 4096) -> None:
        """A handful of parameters, read back from every tensor-parallel worker,
        against the training side's converted tensors."""
        import torch

        converted = self.writer.convert_parameters()
        tp = self.args.tp
        for name, cut_dim in CHECKED_PARAMETERS:
            if name not in converted:
                raise RuntimeError(f"{name} is not among the training side's converted parameters")
            want = converted[name].detach().cpu()
            local = list(want.shape)
            if cut_dim is not None:
                local[cut_dim] //= tp
            slices = tuple(slice(0, min(length, n)) for n in local)
            got = self.inference.execute_task_in_model_worker(read_from_worker, param_name=name, slices=slices)
            got = got if isinstance(got, list) else [got] * tp
            for rank in range(tp):
                if got[rank] is None:
                    raise RuntimeError(f"worker {rank} holds no parameter {name}")
                part = want if cut_dim is None else want.narrow(cut_dim, rank * local[cut_dim], local[cut_dim])
                if not torch.equal(got[rank], part[slices]):
                    raise RuntimeError(f"{name}: worker {rank} differs from the training side")
            print(f"[it] verified {name}", flush=True)

    def close(self) -> None:
        if self.writer is not None and hasattr(self.writer, "close"):
            self.writer.close()
        if self.sgl is not None and hasattr(self.sgl, "shutdown"):
            self.sgl.shutdown()
        if self.meta_server is not None:
            self.meta_server.stop()
        self.executor.shutdown(wait=False)


def main(args) -> int:
    try:
        import sglang  # noqa: F401
    except ImportError:
        print("[it] SGLang is not installed: nothing to run", flush=True)
        return 2
    from awex_b200.synthetic.arch import get_arch

    arch = get_arch(args.arch)
    if args.layers:
        arch = arch.with_layers(args.layers)
    run = WeightsExchangeIT(args)
    try:
        run.initialize(arch)
        first = run.exchange()
        print(f"[it] first exchange (one-time planning included): {first:.3f}s", flush=True)
        if args.comm_backend != "file":
            run.verify()
        times = []
        for _ in range(args.steps):
            run.training.regenerate(step=run.step + 1)  # an "optimizer step": new values at the same addresses
            times.append(run.exchange())
        if times:
            times.sort()
            print(f"[it] {len(times)} exchanges: median {times[len(times) // 2]:.4f}s min {times[0]:.4f}s max {times[-1]:.4f}s", flush=True)
        print("[it] OK", flush=True)
        return 0
    finally:
        run.close()


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description="Weight exchange between a synthetic Megatron-layout trainer and an SGLang engine")
    parser.add_argument("-b", "--comm_backend", required=True, choices=["file", "nccl", "astate"], help="weight exchange backend")
    parser.add_argument("--arch", default="llama3-8b", help="architecture preset (awex_b200.synthetic.arch)")
    parser.add_argument("--layers", type=int, default=4, help="number of decoder layers to keep (0: the preset's own)")
    parser.add_argument("--tp", type=int, default=1, help="tensor-parallel size of the SGLang engine")
    parser.add_argument("--steps", type=int, default=10, help="exchanges after the first")
    parser.add_argument("--mem-fraction-static", type=float, default=0.5)
    parser.add_argument("--debug", action="store_true", help="enable_debug_mode on both sides (metadata and plan dumps)")
    parser.add_argument("--device-backend", choices=["auto", "cuda", "cpu"], default="auto", help="device of both sides (auto: CUDA when there is one)")
    cli = parser.parse_args()
    if cli.device_backend != "auto":
        os.environ["AWEX_DEVICE_TYPE"] = cli.device_backend
    sys.exit(main(cli))
