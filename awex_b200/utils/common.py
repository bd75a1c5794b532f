"""Small host-side helpers shared by every layer.

Wire format of MetaServer objects (`awex/util/common.py:93-108` in the
reference): a 4-byte big-endian payload length followed by a pickle.
"""

from __future__ import annotations

import json
import math
import os
import pickle
import socket
import struct
from enum import Enum
from typing import Any, Dict, Iterable, List, Sequence

import torch

from awex_b200 import logging

logger = logging.getLogger(__name__)

_TIED_PAIR = ("lm_head.weight", "model.embed_tokens.weight")


def is_allowed_infer_only_alias(extra_key: str, infer_keys: set, train_keys: set) -> bool:
    """An inference-only key is tolerated only when it is the second name of a
    tied embedding whose other name both sides publish
    (`awex/util/common.py:34-50`)."""
    if extra_key not in _TIED_PAIR:
        return False
    other = _TIED_PAIR[1] if extra_key == _TIED_PAIR[0] else _TIED_PAIR[0]
    return other in infer_keys and other in train_keys


# the reference spells it with a leading underscore
_is_allowed_infer_only_alias = is_allowed_infer_only_alias


def configure_logging(level=None, force: bool = True) -> None:
    """Configure the standard library's root logger with the line format of this
    package's own logger (`awex/util/common.py:53-58`), for host programs that log
    through ``logging``."""
    import logging as std_logging

    std_logging.basicConfig(
        level=std_logging.INFO if level is None else level,
        format="%(asctime)s\t%(levelname)s %(filename)s:%(lineno)s -- %(process)d -- %(message)s",
        force=force,
    )


def ensure_divisibility(numerator: int, denominator: int) -> None:
    if numerator % denominator != 0:
        raise AssertionError(f"{numerator} is not divisible by {denominator}")


def divide(numerator: int, denominator: int) -> int:
    ensure_divisibility(numerator, denominator)
    return numerator // denominator


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def get_ip_address() -> str:
    forced = os.environ.get("AWEX_MASTER_ADDR")
    if forced:
        return forced
    try:
        with socket.socket(socket.AF_INET, socket.SOCK_DGRAM) as probe:
            probe.connect(("8.8.8.8", 80))
            return probe.getsockname()[0]
    except OSError:
        try:
            return socket.gethostbyname(socket.gethostname())
        except OSError:
            return "127.0.0.1"


def get_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("", 0))
        return s.getsockname()[1]


def to_binary(obj: Any) -> bytes:
    body = pickle.dumps(obj)
    return struct.pack("!I", len(body) & 0xFFFFFFFF) + body


def from_binary(blob: bytes) -> Any:
    (size,) = struct.unpack("!I", blob[:4])
    # payloads of 4 GiB or more wrap the length field; the pickle itself is
    # self-delimiting, so trust the remaining bytes in that case
    body = blob[4 : 4 + size] if len(blob) - 4 == size else blob[4:]
    return pickle.loads(body)


def to_dict(obj: Any, ignore_keys: Iterable[str] | None = None) -> Any:
    """Recursively turn dataclasses/slots objects, enums, dtypes and slices into
    JSON-friendly values."""
    skip = set(ignore_keys or ())

    def walk(v):
        if isinstance(v, Enum):
            return v.value
        if isinstance(v, (list, tuple)):
            return [walk(x) for x in v]
        if isinstance(v, (torch.dtype, slice)):
            return str(v)
        if isinstance(v, dict):
            return {k: walk(x) for k, x in v.items() if k not in skip}
        if hasattr(v, "__dict__"):
            return {k: walk(x) for k, x in vars(v).items() if not k.startswith("_") and k not in skip}
        if hasattr(v, "__slots__"):
            return {k: walk(getattr(v, k)) for k in v.__slots__ if not k.startswith("_") and k not in skip}
        return v

    return walk(obj)


def to_json(obj: Any, ignore_keys: Iterable[str] | None = None) -> str:
    return json.dumps(to_dict(obj, ignore_keys), indent=2)


def compute_statistics(stage_history: Dict[str, List[float]], step_id: int, duration: float, stage: str) -> Dict[str, float]:
    """Rolling per-stage timing statistics (`awex/util/common.py:149-168`).

    At step 2 the largest sample is dropped because step 1 contains
    initialisation.  Returns the statistics as a dict as well as logging them.
    """
    history = stage_history.setdefault(stage, [])
    history.append(duration)
    if len(history) > 10000:
        del history[0]
    if step_id == 2 and len(history) > 1:
        history.remove(max(history))
    ordered = sorted(history)
    stage_history[stage] = ordered
    n = len(ordered)
    stats = {
        "avg": sum(ordered) / n,
        "median": ordered[n // 2],
        "min": ordered[0],
        "max": ordered[-1],
    }
    logger.info(
        f"{stage} time statistics for step {step_id}: average time: {stats['avg']:.4f} seconds, "
        f"median time: {stats['median']:.4f} seconds, min time: {stats['min']:.4f} seconds,  "
        f"max time: {stats['max']:.4f} seconds"
    )
    return stats


def check_train_infer_params_meta(
    training_params_meta: Sequence,
    infer_parameters_meta: Sequence,
    raise_exception: bool = False,
    strict_key_match: bool = False,
) -> List[str]:
    """Check the train/infer metadata alignment contract
    (`awex/util/common.py:171-261`): key sets (train ⊆ infer modulo the tied
    embedding alias, or exact in strict mode), global numel/shape/dtype per
    common key, and TP sizes dividing each other.  Returns the list of
    problems; raises ``ValueError`` on the first one when asked to."""
    infer = {m.name: m for m in infer_parameters_meta}
    train = {m.name: m for m in training_params_meta}
    ik, tk = set(infer), set(train)
    missing = tk - ik
    extra = ik - tk
    bad_extra = {k for k in extra if not is_allowed_infer_only_alias(k, ik, tk)}
    problems: List[str] = []

    def report(msg: str) -> None:
        problems.append(msg)
        if raise_exception:
            raise ValueError(msg)
        logger.error(msg)

    if missing or (extra if strict_key_match else bad_extra):
        report(
            "Inconsistent parameters meta keys: "
            f"train={len(train)} infer={len(infer)} missing_on_infer={sorted(missing)} "
            f"extra_on_infer={sorted(extra)} unsupported_extra_on_infer={sorted(bad_extra)} "
            f"strict={strict_key_match}"
        )
    elif extra:
        logger.info(
            f"Infer meta has extra keys not required by training (allowed alias subset), "
            f"count={len(extra)} sample={sorted(extra)[:8]}"
        )
    for name in ik & tk:
        im, tm = infer[name], train[name]
        if im.global_numel != tm.global_numel:
            report(f"Inconsistent number of elements for parameter {name}: {im.global_numel} != {tm.global_numel}")
        if tuple(im.global_shape) != tuple(tm.global_shape):
            report(f"Inconsistent shape for parameter {name}: {im.global_shape} != {tm.global_shape}")
        if im.dtype != tm.dtype:
            report(f"Inconsistent dtype for parameter {name}: {im.dtype} != {tm.dtype}")
        a, b = len(im.replicas[0].shards), len(tm.replicas[0].shards)
        if max(a, b) % min(a, b) != 0:
            report(f"Inference for parameter {name} has wrong tp_size: infer {a} train {b}")
    return problems


def pretty_bytes(n: int) -> str:
    if n <= 0:
        return "0B"
    units = ["B", "KB", "MB", "GB", "TB", "PB"]
    idx = min(int(math.log(n, 1024)), len(units) - 1)
    return f"{round(n / 1024 ** idx, 2)} {units[idx]}"


def stripped_env_vars() -> Dict[str, str]:
    env = {k: v for k, v in os.environ.items() if "secret" not in k.lower()}
    env.pop("LS_COLORS", None)
    return env


class AttrDict(dict):
    """dict whose keys are also attributes."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.__dict__ = self


def simple_hf_config(hf_config) -> AttrDict:
    """Plain, picklable view of a Hugging Face config (values that reference
    inference-engine classes are dropped)."""
    raw = hf_config.to_dict() if hasattr(hf_config, "to_dict") else dict(hf_config)
    return AttrDict(**{k: v for k, v in raw.items() if "sglang" not in str(v)})


def cfg_get(config: Any, key: str, default: Any = None) -> Any:
    """Read ``key`` from a dict, a namespace or ``None``."""
    if config is None:
        return default
    if isinstance(config, dict):
        return config.get(key, default)
    return getattr(config, key, default)
