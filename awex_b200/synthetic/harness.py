"""Engines for synthetic jobs that span real processes.

:class:`SyntheticTrainEngine` is what a Megatron host framework would hand the
writer (model shards, HF config, rank coordinates, an HF-checkpoint saver);
:class:`SyntheticInferenceEngine` is a vLLM-like engine whose single worker
lives in the calling process, with a checkpoint loader.  One process per GPU
(or per CPU rank) creates one of them, or both when training and inference
share the device.
"""

from __future__ import annotations

import torch

from awex_b200.engine.mcore import MegatronEngine
from awex_b200.sharding.rank_info import RankInfo
from awex_b200.synthetic.arch import Arch
from awex_b200.synthetic.models import (
    CanonicalWeights, FlatModule, StoredCanonicalWeights, build_megatron_model, build_vllm_model, canonical_state_dict,
)
from awex_b200.synthetic.simulate import InferLayout, LocalInferenceEngine


class SyntheticTrainEngine(MegatronEngine):
    def __init__(self, arch: Arch, rank_info: RankInfo, meta_server_addr: str, dtype=torch.bfloat16, device="cpu",
                 seed: int = 0, process_group=None, comm_backend: str = "nccl", tp_group=None, **config):
        self.arch, self.dtype, self.device, self.seed = arch, dtype, device, seed
        model = build_megatron_model(arch, rank_info, dtype, device, seed)
        cfg = dict(meta_server_addr=meta_server_addr, comm_backend=comm_backend)
        cfg.update(config)
        super().__init__(cfg, arch.hf_config(), model, rank_info=rank_info, process_group=process_group, tp_group=tp_group)

    def save_hf_checkpoint(self, path: str):
        """Rank 0 writes the canonical tensors (regenerated from the seeds the
        shards were cut from)."""
        if self.rank_info.global_rank == 0:
            from awex_b200.utils.safetensors_io import save_checkpoint

            weights = CanonicalWeights(self.arch, self.dtype, self.device, self.seed, getattr(self, "step", 0))
            save_checkpoint(path, canonical_state_dict(self.arch, weights))

    def regenerate(self, step: int) -> None:
        """Overwrite the shards in place with the weights of ``step`` (a stand-in
        for an optimizer step; addresses do not change)."""
        self.step = step  # a checkpoint written from now on holds these weights
        fresh = build_megatron_model(self.arch, self.rank_info, self.dtype, self.device, self.seed, step=step)
        for (_, old), (_, new) in zip(self.model.named_parameters(), fresh.named_parameters()):
            old.copy_(new)


class SyntheticInferenceEngine(LocalInferenceEngine):
    """One worker (this process) of an inference instance."""

    def __init__(self, arch: Arch, layout: InferLayout, rank_info: RankInfo, meta_server_addr: str, dtype=torch.bfloat16,
                 device="cpu", seed: int = 0, zero: bool = True, instance_group=None, **config):
        self.arch, self.dtype, self.device, self.seed, self.layout = arch, dtype, device, seed, layout
        # the other workers of this inference instance live in other processes;
        # metadata collection is gathered over this group so that every process
        # can act as the instance's control process
        self.instance_group = instance_group
        model = build_vllm_model(arch, rank_info, dtype, device, seed, fp8=layout.fp8, zero=zero)
        super().__init__(arch, layout, [rank_info], [model], engine_rank=rank_info.engine_rank,
                         meta_server_addr=meta_server_addr, **config)

    @property
    def model(self) -> FlatModule:
        return self.models[0]

    def execute_task_in_model_worker(self, fn, **kwargs):
        local = super().execute_task_in_model_worker(fn, **kwargs)
        if self.instance_group is None or getattr(fn, "__name__", "") != "collect_worker_param_info":
            return local
        import torch.distributed as dist

        gathered = [None] * dist.get_world_size(self.instance_group)
        dist.all_gather_object(gathered, local[0], group=self.instance_group)
        return gathered

    def update_weights_from_disk(self, path, load_format=None):
        from awex_b200.utils.safetensors_io import load_checkpoint

        stored = StoredCanonicalWeights(self.arch, load_checkpoint(path), self.dtype, self.device)
        fresh = build_vllm_model(self.arch, self.ranks[0], self.dtype, self.device, fp8=self.layout.fp8, weights=stored)
        for (_, old), (_, new) in zip(self.model.named_parameters(), fresh.named_parameters()):
            old.copy_(new)

    def oracle(self, step: int = 0) -> FlatModule:
        return build_vllm_model(self.arch, self.ranks[0], self.dtype, self.device, self.seed, step=step, fp8=self.layout.fp8)

    def mismatches(self, step: int = 0):
        bad = []
        for (name, got), (_, want) in zip(self.model.named_parameters(), self.oracle(step).named_parameters()):
            if not torch.equal(got.view(torch.uint8), want.view(torch.uint8)):
                bad.append(name)
        return bad
