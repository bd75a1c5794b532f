"""Load a Hugging Face checkpoint into Megatron modules through an mbridge
name mapping (`awex/mbridge_loader.py:29-125` in the reference).

``bridge`` is duck-typed: ``_get_actual_hf_path(path)``,
``_weight_name_mapping_mcore_local_to_global(model)`` and
``_weight_name_mapping_mcore_to_hf(global_name)`` are used when present, identity
otherwise.  Several HF tensors that map to one Megatron parameter (fused QKV,
gate+up) are concatenated along the one dimension whose sizes add up to the
target.
"""

from __future__ import annotations

import os
from typing import Callable, Dict, Iterable, List, Optional, Union

import torch

TensorReader = Callable[[str, str], torch.Tensor]


class CheckpointReader:
    """``reader(weights_path, name)`` over a sharded or single-file safetensors
    checkpoint.  The name -> file map is built once per directory and every
    shard file is opened once and stays open until :meth:`close`."""

    def __init__(self):
        self._maps: Dict[str, Dict[str, str]] = {}
        self._open: Dict[str, object] = {}

    def __call__(self, weights_path: str, name: str) -> torch.Tensor:
        from safetensors import safe_open

        from awex_b200.utils.safetensors_io import checkpoint_weight_map

        key = os.path.abspath(weights_path)
        if key not in self._maps:
            self._maps[key] = checkpoint_weight_map(weights_path)
        shard = self._maps[key].get(name)
        if shard is None:
            raise KeyError(f"Weight {name} not found in safetensors under {weights_path}.")
        if shard not in self._open:
            self._open[shard] = safe_open(shard, framework="pt", device="cpu").__enter__()
        return self._open[shard].get_tensor(name)

    def close(self) -> None:
        for handle in self._open.values():
            handle.__exit__(None, None, None)
        self._open.clear()


def coerce_names(names: Union[str, Iterable[str]]) -> List[str]:
    return [names] if isinstance(names, str) else list(names)


def concat_along_matching_dim(tensors: List[torch.Tensor], target_shape) -> torch.Tensor:
    """Concatenate along the first dimension where the parts agree everywhere
    else and their sizes sum to the target's."""
    target_shape = tuple(target_shape)
    if len(tensors) == 1:
        return tensors[0]
    rank = len(target_shape)
    if all(t.ndim == rank for t in tensors):
        first = tensors[0].shape
        for dim in range(rank):
            others_agree = all(t.shape[d] == first[d] for t in tensors for d in range(rank) if d != dim)
            if others_agree and sum(t.shape[dim] for t in tensors) == target_shape[dim]:
                return torch.cat(tensors, dim=dim)
    raise ValueError(f"Cannot concatenate tensors of shapes {[tuple(t.shape) for t in tensors]} to match target shape {target_shape}.")


def load_weights_from_hf_with_mbridge(bridge, models: List[torch.nn.Module], weights_path: str,
                                      reader: Optional[TensorReader] = None, is_critic: bool = False) -> None:
    own_reader = reader is None
    reader = reader or CheckpointReader()
    if hasattr(bridge, "_get_actual_hf_path"):
        weights_path = bridge._get_actual_hf_path(weights_path)
    for model in models:
        state = model.state_dict()
        if hasattr(bridge, "_weight_name_mapping_mcore_local_to_global"):
            local_to_global = bridge._weight_name_mapping_mcore_local_to_global(model)
        else:
            local_to_global = {name: name for name in state}
        for local_name, global_name in local_to_global.items():
            if local_name not in state or (is_critic and "output_layer" in local_name):
                continue
            hf_names = coerce_names(bridge._weight_name_mapping_mcore_to_hf(global_name)) if hasattr(bridge, "_weight_name_mapping_mcore_to_hf") else [global_name]
            target = state[local_name]
            merged = concat_along_matching_dim([reader(weights_path, n) for n in hf_names], target.shape)
            with torch.no_grad():
                target.copy_(merged.to(device=target.device, dtype=target.dtype))
    if own_reader:
        reader.close()
