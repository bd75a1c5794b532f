"""Architecture registry.

Every module of :mod:`awex_b200.models` may define ``CONFIG`` (a dict or a list
of dicts) with ``model_name`` and any of ``sharding_strategy``,
``mcore_converter``, ``sglang_converter``, ``vllm_converter``.  A converter
entry is a class or a zero-argument factory returning a class.  Unknown
architectures use the default strategy and converters
(`awex/models/registry.py:49-172` in the reference).

Unlike the reference, every architecture has one canonical contract on both
inference engines: an architecture that registers only an SGLang-side
converter gets it on vLLM too (wrapped so that ``self_attn.*`` names are
normalised only when that converter keeps QKV fused), and unregistered
architectures use the name-normalising converter on SGLang as well.
"""

from __future__ import annotations

import importlib
import inspect
import pkgutil
from dataclasses import dataclass
from functools import lru_cache
from typing import Any, Callable, Dict, Optional

from awex_b200 import logging
from awex_b200.converter.sglang_converter import SGlangToHFWeightConverter
from awex_b200.converter.vllm_converter import VLLMToHFWeightConverter
from awex_b200.sharding.param_sharding import ShardingStrategy

logger = logging.getLogger(__name__)


@dataclass
class ModelConfig:
    sharding_strategy: Callable[..., ShardingStrategy] = ShardingStrategy
    mcore_converter: Optional[Callable[..., Any]] = None
    sglang_converter: Optional[Callable[..., Any]] = None
    vllm_converter: Optional[Callable[..., Any]] = None


def _field(config, name: str, default=None):
    if isinstance(config, dict):
        return config.get(name, default)
    return getattr(config, name, default)


@lru_cache
def import_model_configs() -> Dict[str, Any]:
    found: Dict[str, Any] = {}
    package = importlib.import_module("awex_b200.models")
    for info in pkgutil.iter_modules(package.__path__, "awex_b200.models."):
        if info.ispkg or info.name.endswith(".registry"):
            continue
        try:
            module = importlib.import_module(info.name)
        except Exception as exc:  # a model file with a missing optional dependency
            logger.warning(f"Ignore import error when loading {info.name}. {exc}")
            continue
        entries = getattr(module, "CONFIG", None)
        if entries is None:
            continue
        for entry in entries if isinstance(entries, list) else [entries]:
            name = entry["model_name"]
            assert name not in found, f"Duplicated model config for {name}"
            found[name] = entry
    return found


class _ModelRegistry:
    def __init__(self, models: Dict[str, Any]):
        self.models = models

    def get_registered_models(self) -> Dict[str, Any]:
        return dict(self.models)

    def get_model_config(self, model_name: str):
        if model_name in self.models:
            return self.models[model_name]
        logger.info(f"Model {model_name} not found, using default strategy.")
        return ModelConfig()


class _LazyRegistry:
    """Defers the package scan until first use so model files can import this
    module."""

    _inner: Optional[_ModelRegistry] = None

    def _get(self) -> _ModelRegistry:
        if self._inner is None:
            self._inner = _ModelRegistry(import_model_configs())
        return self._inner

    def __getattr__(self, item):
        return getattr(self._get(), item)


ModelRegistry = _LazyRegistry()


def get_sharding_strategy(model_name: str):
    return _field(ModelRegistry.get_model_config(model_name), "sharding_strategy", ShardingStrategy) or ShardingStrategy


def _resolve_converter(config_value, default):
    if config_value is None:
        return default
    if inspect.isclass(config_value):
        return config_value
    resolved = config_value()
    if not inspect.isclass(resolved):
        raise TypeError(f"Expected converter class from factory, got {type(resolved)}")
    return resolved


def get_train_weights_converter(engine_name: str, model_name: str, hf_config, rank_info, infer_conf: Dict, tf_config=None):
    if engine_name != "mcore":
        raise NotImplementedError(f"Engine {engine_name} not implemented.")
    from awex_b200.converter.mcore_converter import McoreToHFWeightConverter

    cls = _resolve_converter(_field(ModelRegistry.get_model_config(model_name), "mcore_converter"), McoreToHFWeightConverter)
    if tf_config is None and isinstance(infer_conf, dict):
        tf_config = infer_conf.get("tf_config")
    if tf_config is None:
        raise ValueError("tf_config is required for McoreToHFWeightConverter")
    return cls(hf_config, rank_info, infer_conf, tf_config=tf_config)


@lru_cache(maxsize=None)
def _vllm_flavour_of(sglang_cls):
    """Give an SGLang-side converter vLLM's name normalisation for the pieces
    it keeps in the default ``attention.*`` namespace."""
    if not sglang_cls(None, None, _Probe())._fuse_qkv("self_attn.qkv_proj.weight"):
        return sglang_cls  # publishes self_attn.{q,k,v}_proj: vLLM names already match

    class _VLLMFlavoured(VLLMToHFWeightConverter, sglang_cls):
        pass

    _VLLMFlavoured.__name__ = f"VLLM{sglang_cls.__name__}"
    return _VLLMFlavoured


class _Probe:
    tp_rank = 0
    ep_rank = 0


def get_infer_weights_converter(engine_name: str, model_name: str, hf_config, rank_info, infer_engine_config):
    config = ModelRegistry.get_model_config(model_name)
    if engine_name == "sglang":
        # unregistered architectures get the name-normalising converter on both
        # engines, so "self_attn.qkv_proj" and "attention.query_key_value_proj"
        # spellings meet the training side's default contract alike
        cls = _resolve_converter(_field(config, "sglang_converter"), VLLMToHFWeightConverter)
    elif engine_name == "vllm":
        explicit = _field(config, "vllm_converter")
        sgl = _field(config, "sglang_converter")
        if explicit is not None:
            cls = _resolve_converter(explicit, VLLMToHFWeightConverter)
        elif sgl is not None:
            cls = _vllm_flavour_of(_resolve_converter(sgl, SGlangToHFWeightConverter))
        else:
            cls = VLLMToHFWeightConverter
    else:
        raise NotImplementedError(f"Engine {engine_name} not implemented.")
    return cls(hf_config, infer_engine_config, rank_info)
