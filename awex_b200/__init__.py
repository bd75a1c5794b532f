"""B200-native weight synchronisation between RL training and inference.

Public names match the reference package (`awex/__init__.py:18-28`); they are
resolved lazily so that importing the package does not pull in CUDA code.
"""

from awex_b200.version import __version__  # noqa: F401

_LAZY = {
    "InferenceConfig": ("awex_b200.config", "InferenceConfig"),
    "NCCLWeightsWriter": ("awex_b200.writer.nccl_writer", "NCCLWeightsWriter"),
    "WeightsReader": ("awex_b200.reader.weights_reader", "WeightsReader"),
    "NCCLWorkerWeightsReader": ("awex_b200.reader.nccl_reader", "NCCLWorkerWeightsReader"),
}

__all__ = list(_LAZY)


def __getattr__(name):
    if name in _LAZY:
        import importlib

        module, attr = _LAZY[name]
        return getattr(importlib.import_module(module), attr)
    raise AttributeError(f"module 'awex_b200' has no attribute {name!r}")
