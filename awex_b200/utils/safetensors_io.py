"""Hugging Face style checkpoint directories: ``model-XXXXX-of-YYYYY.safetensors``
shards plus ``model.safetensors.index.json``.  Used by the ``file`` backend and
as the file-loaded reference of weight validation (the reference writes such
directories from its file-mode writer, `awex/writer/weights_writer.py:374-410`,
and loads them through the engine, `awex/reader/weights_reader.py:380-400`)."""

from __future__ import annotations

import glob
import json
import os
from typing import Dict, Iterable, Mapping, Optional

import torch
from safetensors import safe_open
from safetensors.torch import save_file

INDEX_NAME = "model.safetensors.index.json"


def save_checkpoint(path: str, tensors: Mapping[str, torch.Tensor], max_shard_bytes: int = 4 * 1024**3) -> Dict[str, str]:
    """Write ``tensors`` as one or more shards plus an index.  Returns the
    weight map (tensor name -> shard file)."""
    os.makedirs(path, exist_ok=True)
    shards, current, size = [], {}, 0
    for name, t in tensors.items():
        nbytes = t.numel() * t.element_size()
        if current and size + nbytes > max_shard_bytes:
            shards.append(current)
            current, size = {}, 0
        current[name] = t.detach().cpu().contiguous()
        size += nbytes
    if current:
        shards.append(current)
    weight_map: Dict[str, str] = {}
    total = 0
    for i, shard in enumerate(shards):
        fname = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(shard, os.path.join(path, fname), metadata={"format": "pt"})
        for name, t in shard.items():
            weight_map[name] = fname
            total += t.numel() * t.element_size()
    with open(os.path.join(path, INDEX_NAME), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)
    return weight_map


def checkpoint_weight_map(path: str) -> Dict[str, str]:
    """tensor name -> absolute shard path, from the index or by scanning."""
    index = os.path.join(path, INDEX_NAME)
    if os.path.exists(index):
        with open(index) as f:
            return {name: os.path.join(path, fname) for name, fname in json.load(f)["weight_map"].items()}
    out: Dict[str, str] = {}
    for shard in sorted(glob.glob(os.path.join(path, "*.safetensors"))):
        with safe_open(shard, framework="pt") as f:
            for name in f.keys():
                out[name] = shard
    if not out:
        raise FileNotFoundError(f"no safetensors files under {path}")
    return out


def load_checkpoint(path: str, names: Optional[Iterable[str]] = None, device: str = "cpu") -> Dict[str, torch.Tensor]:
    weight_map = checkpoint_weight_map(path)
    wanted = list(names) if names is not None else list(weight_map)
    by_file: Dict[str, list] = {}
    for name in wanted:
        if name not in weight_map:
            raise KeyError(f"{name} is not in the checkpoint at {path}")
        by_file.setdefault(weight_map[name], []).append(name)
    out: Dict[str, torch.Tensor] = {}
    for shard, shard_names in by_file.items():
        with safe_open(shard, framework="pt", device=device) as f:
            for name in shard_names:
                out[name] = f.get_tensor(name)
    return out
