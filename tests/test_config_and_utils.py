"""Configuration validation, the metadata alignment contract, wire helpers,
timing statistics, tensor packing and diagnostics, the logger, the model
registry and the descriptor validator on seeded-bad tables."""

import dataclasses
import io
from contextlib import redirect_stdout
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from awex_b200.config import InferenceConfig, InferenceConfigValidationError


# ------------------------------------------------------------------------------------------ config
def test_config_reports_every_problem_at_once():
    cfg = InferenceConfig(comm_backend="smoke-signals", weights_exchange_ipc_backend="tape", num_engines=2, engine_rank=5,
                          tp_size=0, nnodes=2, node_rank=2, validate_weights_every_n_steps=0, weights_validation_steps=-1,
                          dump_weights_list_for_validation=["w"], ep_num_redundant_experts=1, enable_eplb=True,
                          device_wait_timeout_ms=0)
    with pytest.raises(InferenceConfigValidationError) as err:
        cfg.validate()
    text = str(err.value)
    for needle in ("comm_backend", "weights_exchange_ipc_backend", "engine_rank", "tp_size", "node_rank",
                   "validate_weights_every_n_steps", "weights_validation_steps", "dump_weights_dir_for_validation",
                   "ep_num_redundant_experts", "enable_eplb", "device_wait_timeout_ms"):
        assert needle in text, needle
    assert text.count("\n  - ") >= 11


def test_config_from_dict_drops_unknown_keys_and_validates():
    cfg = InferenceConfig.from_dict({"tp_size": 2, "comm_backend": "nccl", "not_a_field": 1, "meta_server_addr": "h:1"})
    assert cfg.tp_size == 2 and not hasattr(cfg, "not_a_field")
    with pytest.raises(InferenceConfigValidationError, match="meta_server_addr"):
        InferenceConfig.from_dict({"num_engines": 2, "comm_backend": "nccl"})
    lenient = InferenceConfig.from_dict({"num_engines": 2, "comm_backend": "nccl"}, validate=False)
    assert lenient.num_engines == 2
    assert InferenceConfig(num_engines=2, comm_backend="file").validated().comm_backend == "file"
    for backend in ("file", "nccl", "hccl", "astate"):
        InferenceConfig(comm_backend=backend).validate()
    assert {"tp_size", "meta_server_addr", "enable_colocate_mode", "device_wait_timeout_ms"} <= set(InferenceConfig.field_names())
    assert dataclasses.asdict(InferenceConfig())["weights_exchange_ipc_backend"] == "cuda"


# ------------------------------------------------------------------------------------------ alignment contract
def _meta(name, shape=(4, 4), dtype=torch.float32, shards=1):
    one = SimpleNamespace(shards=[None] * shards)
    numel = int(np.prod(shape))
    return SimpleNamespace(name=name, global_numel=numel, global_shape=tuple(shape), dtype=dtype, replicas=[one])


def test_alignment_contract():
    from awex_b200.utils.common import check_train_infer_params_meta, is_allowed_infer_only_alias

    train = [_meta("model.embed_tokens.weight"), _meta("w")]
    infer = train + [_meta("lm_head.weight")]
    assert check_train_infer_params_meta(train, infer) == []
    assert check_train_infer_params_meta(train, infer, strict_key_match=True)
    with pytest.raises(ValueError, match="Inconsistent parameters meta keys"):
        check_train_infer_params_meta(train + [_meta("only_train")], infer, raise_exception=True)
    assert check_train_infer_params_meta(train, infer + [_meta("stray")])
    assert any("shape" in p for p in check_train_infer_params_meta([_meta("w", (2, 8))], [_meta("w", (4, 4))]))
    assert any("number of elements" in p for p in check_train_infer_params_meta([_meta("w", (2, 4))], [_meta("w", (4, 4))]))
    assert any("dtype" in p for p in check_train_infer_params_meta([_meta("w", dtype=torch.bfloat16)], [_meta("w")]))
    assert any("tp_size" in p for p in check_train_infer_params_meta([_meta("w", shards=3)], [_meta("w", shards=2)]))
    assert is_allowed_infer_only_alias("lm_head.weight", {"lm_head.weight", "model.embed_tokens.weight"}, {"model.embed_tokens.weight"})
    assert not is_allowed_infer_only_alias("lm_head.weight", {"lm_head.weight"}, set())
    assert not is_allowed_infer_only_alias("other", {"other"}, set())


# ------------------------------------------------------------------------------------------ common helpers
def test_wire_format_statistics_and_small_helpers():
    import struct

    from awex_b200.utils import common

    blob = common.to_binary({"a": (1, 2)})
    assert struct.unpack("!I", blob[:4])[0] == len(blob) - 4 and common.from_binary(blob) == {"a": (1, 2)}
    with pytest.raises(Exception):
        common.from_binary(blob[:-1])
    history = {}
    common.compute_statistics(history, 1, 9.0, "send")  # step 1 carries initialisation
    stats = common.compute_statistics(history, 2, 1.0, "send")
    assert stats == {"avg": 1.0, "median": 1.0, "min": 1.0, "max": 1.0}  # the outlier of step 1 was dropped
    stats = common.compute_statistics(history, 3, 3.0, "send")
    assert stats["avg"] == 2.0 and stats["max"] == 3.0
    assert common.divide(8, 4) == 2 and common.ceil_div(9, 4) == 3
    with pytest.raises(AssertionError):
        common.divide(9, 4)
    assert common.pretty_bytes(0) == "0B" and common.pretty_bytes(1536).endswith("KB")
    port = common.get_free_port()
    assert 0 < port < 65536
    hf = common.simple_hf_config(SimpleNamespace(hidden_size=8, to_dict=lambda: {"hidden_size": 8, "rope": {"theta": 1.0}}))
    assert hf.hidden_size == 8 and hf["rope"]["theta"] == 1.0
    assert common.cfg_get({"a": 1}, "a") == 1 and common.cfg_get(SimpleNamespace(a=2), "a") == 2 and common.cfg_get(None, "a", 3) == 3
    nested = common.to_dict({"t": torch.float32, "d": InferenceConfig(tp_size=2), "skip": 1}, ignore_keys=["skip"])
    assert nested["d"]["tp_size"] == 2 and "skip" not in nested and isinstance(common.to_json(nested), str)


def test_master_address_override(monkeypatch):
    from awex_b200.utils import common

    monkeypatch.setenv("AWEX_MASTER_ADDR", "10.1.2.3")
    assert common.get_ip_address() == "10.1.2.3"
    monkeypatch.delenv("AWEX_MASTER_ADDR")
    assert common.get_ip_address().count(".") == 3


# ------------------------------------------------------------------------------------------ tensor utils
def test_group_by_dtype_round_trip_and_limits():
    from awex_b200.utils.tensor_util import (
        group_tensors_by_shape_and_dtype, ipc_deserialize, ipc_serialize, reconstruct_ipc_weights,
        reconstruct_tensors_from_groups, release_tensors,
    )

    tensors = [torch.randn(3, 4), torch.arange(6, dtype=torch.int64), torch.randn(5).to(torch.bfloat16), torch.randn(2, 2)]
    groups, meta = group_tensors_by_shape_and_dtype(tensors)
    assert len(groups) == 3 and all(g.dim() == 1 for g in groups)
    back = reconstruct_tensors_from_groups(groups, meta)
    assert all(torch.equal(a, b) for a, b in zip(tensors, back))
    back[0].zero_()
    assert not groups[meta[0]["group_index"]][: 12].any()  # views, not copies
    small, small_meta = group_tensors_by_shape_and_dtype([torch.ones(4), torch.ones(4), torch.ones(4)], max_tensor_size=20)
    assert len(small) == 3  # 16 bytes each: no two fit in 20
    assert group_tensors_by_shape_and_dtype([]) == ([], [])
    with pytest.raises(ValueError):
        group_tensors_by_shape_and_dtype([torch.ones(2).to_sparse()])
    with pytest.raises(ValueError):
        reconstruct_tensors_from_groups(groups[:1], meta)
    with pytest.raises(ValueError):
        reconstruct_tensors_from_groups(groups, [m for m in meta if m["original_index"] != 1])
    payload = ipc_serialize((groups, meta, ["a", "b", "c", "d"]))
    named = reconstruct_ipc_weights(payload)
    assert list(named) == ["a", "b", "c", "d"] and torch.equal(named["b"], tensors[1])
    assert ipc_deserialize(ipc_serialize({"x": 1})) == {"x": 1}
    victim = torch.ones(8)
    release_tensors(victim)
    assert victim.numel() == 0


def test_nan_scan_and_difference_report():
    from awex_b200.utils.tensor_util import check_and_log_nan_values, compare_and_log_tensor_differences

    clean, dirty = torch.ones(4, 4), torch.ones(4, 4)
    dirty[1, 2] = float("nan")
    out = io.StringIO()
    with redirect_stdout(out):
        assert not check_and_log_nan_values(clean, "clean")
        assert check_and_log_nan_values(dirty, "dirty", "after update")
        assert check_and_log_nan_values({"a": clean, "b": dirty}, "train")
        assert not check_and_log_nan_values(torch.ones(3, dtype=torch.int32), "ints")
        assert compare_and_log_tensor_differences(clean, clean.clone(), "same", exact_match=True)
        assert compare_and_log_tensor_differences(clean, clean + 1e-6, "close")
        assert not compare_and_log_tensor_differences(clean, clean + 1e-6, "close-but-not-equal", exact_match=True)
        other = clean.clone()
        other[3, 0] = 2.0
        assert not compare_and_log_tensor_differences(clean, other, "off")
        assert not compare_and_log_tensor_differences(clean, torch.ones(4, 5), "shape")
        assert not compare_and_log_tensor_differences(clean, clean.double(), "dtype")
    text = out.getvalue()
    assert "NaN values in dirty after update: 1 of 16" in text and "[1, 2]" in text
    assert "Tensor off differs in 1 of 16 elements" in text and "off[3, 0]" in text
    assert "Shape mismatch for shape" in text and "Dtype mismatch for dtype" in text


def test_logger_prints_level_location_and_pid():
    import os

    from awex_b200 import logging

    log = logging.getLogger("awex_b200.tests")
    out = io.StringIO()
    logging.setLevel("INFO")
    try:
        with redirect_stdout(out):
            log.info("hello there")
            log.debug("hidden")
            log.warning("careful")
    finally:
        logging.setLevel(os.environ.get("AWEX_LOG_LEVEL", "WARNING"))
    text = out.getvalue()
    assert "INFO" in text and "hello there" in text and "careful" in text and "hidden" not in text
    assert f"-- {os.getpid()} --" in text and "test_config_and_utils.py:" in text


# ------------------------------------------------------------------------------------------ registry
def test_registry_discovers_models_and_falls_back():
    from awex_b200.models import registry

    names = set(registry.import_model_configs())
    for arch in ("Qwen3ForCausalLM", "Qwen3MoeForCausalLM", "BailingMoeV2ForCausalLM", "Qwen3VLForConditionalGeneration"):
        assert arch in names, (arch, sorted(names))
    assert len(names) >= 13
    # unknown architectures get the default strategy and converters instead of an error
    assert registry.get_sharding_strategy("NeverHeardOfForCausalLM") is not None


# ------------------------------------------------------------------------------------------ descriptor validator
def _good_table():
    from awex_b200.transfer.descriptors import TensorAddr, encode_items
    from awex_b200.transfer.lowering import CopyItem

    src, dst = torch.zeros(64, 256, dtype=torch.bfloat16), torch.zeros(64, 256, dtype=torch.bfloat16)
    items = [CopyItem("w", 0, (0, 0), (32, 256), 0, "w", (0, 0), torch.bfloat16, torch.bfloat16),
             CopyItem("w", 0, (32, 0), (32, 256), 0, "w", (32, 0), torch.bfloat16, torch.bfloat16)]
    table, n_tiles, _ = encode_items(items, {("w", 0): TensorAddr.of(src)}, {0: {"w": TensorAddr.of(dst)}})
    return table, n_tiles, [TensorAddr.of(src).byte_span()], [TensorAddr.of(dst).byte_span()], (src, dst)


def test_descriptor_validator_rejects_seeded_bad_tables():
    from awex_b200.transfer.descriptors import validate_table

    table, n_tiles, src_spans, dst_spans, _keep = _good_table()
    assert validate_table(table, n_tiles, src_spans, dst_spans) == []

    def broken(**changes):
        bad = table.copy()
        for field, value in changes.items():
            bad[field][1] = value
        return validate_table(bad, n_tiles, src_spans, dst_spans)

    assert broken(dst=int(table["dst"][1]) + 10_000_000)            # destination outside every published view
    assert broken(src=int(table["src"][1]) + 10_000_000)            # source outside the local shards
    assert broken(rows=int(table["rows"][1]) * 1000)                # runs past the end
    assert broken(dst=int(table["dst"][0]))                         # two descriptors write the same bytes
    assert broken(tile_begin=int(table["tile_begin"][1]) + 1)       # tile numbering has a hole
    assert broken(op=99)                                            # unknown operation
    assert broken(tile_rows=0)
    assert validate_table(table, n_tiles + 1, src_spans, dst_spans)  # tile count does not match


def test_span_index_agrees_with_a_linear_scan():
    import random

    from awex_b200.transfer.descriptors import _SpanIndex

    rng = random.Random(5)
    spans = []
    for _ in range(200):
        lo = rng.randrange(0, 10_000)
        spans.append((lo, lo + rng.randrange(1, 400)))  # overlapping and nested ranges included
    index = _SpanIndex(spans)
    for _ in range(5000):
        lo = rng.randrange(0, 10_500)
        hi = lo + rng.randrange(1, 300)
        assert index.contains(lo, hi) == any(a <= lo and hi <= b for a, b in spans), (lo, hi)
    assert not _SpanIndex([]).contains(0, 1)


def test_environment_table(monkeypatch):
    from awex_b200.utils import env

    monkeypatch.setenv("AWEX_P2P_HCCL_BUFFER_SIZE", "64")
    monkeypatch.setenv("AWEX_P2P_TRACE", "1")
    monkeypatch.setenv("AWEX_TYPO", "x")
    lines = env.describe_env()
    assert any(line.startswith("AWEX_P2P_HCCL_BUFFER_SIZE=64: no effect") for line in lines)
    assert any(line.startswith("AWEX_TYPO=x: not a variable") for line in lines)
    assert env.flag("AWEX_P2P_TRACE") and not env.flag("AWEX_MEM_DEBUG")
    warned = []
    env.warn_about_ignored(SimpleNamespace(warning=warned.append))
    assert len(warned) == 1 and "AWEX_P2P_HCCL_BUFFER_SIZE" in warned[0]
    # every variable the package reads is in the table
    import os
    import re

    root = os.path.dirname(os.path.dirname(os.path.abspath(env.__file__)))
    used = set()
    for folder, _dirs, files in os.walk(root):
        for name in files:
            if name.endswith(".py"):
                with open(os.path.join(folder, name)) as f:
                    used |= set(re.findall(r'''environ(?:\.get)?[(\[]\s*["'](AWEX_[A-Z0-9_]+)''', f.read()))
    assert used and used - set(env.KNOBS) - {"AWEX_BENCH_VERBOSE"} == set(), used - set(env.KNOBS)


def test_bench_roofline_arithmetic():
    from awex_b200 import bench_distributed as bd

    writer = SimpleNamespace(transport=SimpleNamespace(bytes_remote=7.7e9, bytes_in=8.0e9, bytes_local=0.3e9, bytes_out=8.0e9))
    worker = SimpleNamespace(transport=SimpleNamespace(bytes_in_remote=3.85e9))
    engine = SimpleNamespace(schedulers=[SimpleNamespace(awes_weights_reader=worker)])
    r = bd._roofline(writer, object(), engine, measured_ms=12.5, ctl=None)
    assert r["bound"] == "nvlink_egress" and abs(r["ms"] - 10.0) < 1e-6 and abs(r["fraction_of_roofline"] - 0.8) < 1e-6
    assert abs(r["per_resource_ms"]["nvlink_ingress"] - 5.0) < 1e-6
    local = bd._roofline(SimpleNamespace(transport=SimpleNamespace(bytes_remote=0, bytes_in=8e9, bytes_local=8e9)), None, None, 5.0, None)
    assert local["bound"] == "hbm" and 2.0 < local["ms"] < 3.0
    bare = bd._roofline(SimpleNamespace(transport=object()), None, None, 1.0, None)  # a transport without byte accounting
    assert bare["ms"] == 0.0
    layouts = {cfg: bd.role_table(8, cfg)[4] for cfg in ("separated", "colocated", "moe", "fp8")}
    assert layouts == {"separated": "tp4->2xtp2", "colocated": "colocated-tp8->tp8", "moe": "colocated-ep8->2xtp4ep4", "fp8": "colocated-ep8->tp8-fp8"}
    with pytest.raises(SystemExit):
        bd.role_table(3)


def test_data_plane_choice(monkeypatch):
    from awex_b200.transfer.transports import choose_data_plane

    monkeypatch.delenv("AWEX_DATA_PLANE", raising=False)
    assert choose_data_plane("cuda") == "peer_stores" and choose_data_plane("cpu") == "messages"
    assert choose_data_plane("cuda", "messages") == "messages"  # several machines: messages over NCCL
    with pytest.raises(ValueError, match="CUDA"):
        choose_data_plane("cpu", "peer_stores")
    with pytest.raises(ValueError, match="one of"):
        choose_data_plane("cuda", "rdma")
    monkeypatch.setenv("AWEX_DATA_PLANE", "messages")
    assert choose_data_plane("cuda", "peer_stores") == "messages"  # the environment wins


def test_device_helpers_without_a_gpu(monkeypatch):
    """The device helpers answer for the CPU when it is forced (the reference's
    `awex/util/device.py` surface, CUDA and CPU only)."""
    from awex_b200.utils import device

    monkeypatch.setenv("AWEX_DEVICE_TYPE", "cpu")
    assert device.get_device_type() == "cpu" and device.device_count() == 0 and device.current_device() == 0
    device.set_device(0), device.synchronize(), device.empty_cache()  # no-ops
    assert device.get_device_name() == "cpu" and device.get_torch_device() == torch.device("cpu")
    assert device.memory_stats() == {"allocated": 0, "reserved": 0, "free": 0, "total": 0}
    assert device.current_stream() is None and device.get_dist_backend() == "gloo"
    with device.stream_context(None):
        pass
    with pytest.raises(RuntimeError, match="CUDA"):
        device.get_device_properties()
    assert device.visible_devices_env_names() == ["CUDA_VISIBLE_DEVICES"]
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "3,4")
    assert device.visible_devices_env_value() == "3,4"
    assert device.is_cuda_available() == torch.cuda.is_available()
    monkeypatch.setenv("AWEX_DEVICE_TYPE", "npu")
    with pytest.raises(ValueError, match="not supported"):
        device.get_device_type()


def test_config_from_an_sglang_engine_and_small_helpers(monkeypatch):
    from awex_b200.config import InferenceConfig
    from awex_b200.ops.checksum import checksum_reference, tensor_checksums
    from awex_b200.utils.common import stripped_env_vars

    server_args = SimpleNamespace(tp_size=4, pp_size=1, dp_size=2, ep_size=2, enable_dp_attention=True, unknown_to_us=7, nnodes=None)
    cfg = InferenceConfig.from_sgl_engine(SimpleNamespace(server_args=server_args), comm_backend="nccl", meta_server_addr="10.0.0.1:8080")
    assert (cfg.tp_size, cfg.dp_size, cfg.ep_size, cfg.enable_dp_attention, cfg.comm_backend) == (4, 2, 2, True, "nccl")
    assert not hasattr(cfg, "unknown_to_us")
    monkeypatch.setenv("MY_SECRET_TOKEN", "x")
    monkeypatch.setenv("PLAIN_SETTING", "y")
    env = stripped_env_vars()
    assert "MY_SECRET_TOKEN" not in env and env["PLAIN_SETTING"] == "y" and "LS_COLORS" not in env
    a, b = torch.arange(64, dtype=torch.float32), torch.tensor([1.0, float("nan"), 3.0, float("nan")])
    sums, nans = tensor_checksums([a, b])
    assert sums == [checksum_reference(a), checksum_reference(b)] and nans == [0, 2]
    assert tensor_checksums([]) == ([], [])


def test_small_public_helpers_of_the_reference_surface(monkeypatch, capsys):
    import logging as std_logging

    from awex_b200 import logging as awex_logging
    from awex_b200.engine.core import Engine
    from awex_b200.logging import LogLevel
    from awex_b200.utils import device, gpu
    from awex_b200.utils.common import configure_logging
    from awex_b200.utils.tensor_util import monkey_patch_torch_compile

    assert [int(level) for level in LogLevel] == [awex_logging.DEBUG, awex_logging.INFO, awex_logging.WARNING, awex_logging.ERROR, awex_logging.CRITICAL]
    log = awex_logging.getLogger("levels")
    log.level = LogLevel.ERROR
    assert not log.isEnabledFor(awex_logging.WARNING) and log.isEnabledFor(LogLevel.CRITICAL)

    class Plain(Engine):
        pass

    engine = Plain()
    assert engine.global_step == 0
    engine.set_global_step(7)
    assert engine.global_step == 7

    monkeypatch.setenv("AWEX_DEVICE_TYPE", "cpu")
    assert device.get_stream_class() is None and device.create_stream(0) is None and device.is_npu_available() is False
    monkeypatch.setattr(awex_logging.getLogger("awex_b200.utils.gpu"), "level", awex_logging.INFO)
    gpu.print_gpu_status("before")
    gpu.print_current_gpu_status("before")
    out = capsys.readouterr().out
    assert "GPU status for before" in out and "memory status for [before]" in out
    root = std_logging.getLogger()
    handlers, level = list(root.handlers), root.level
    try:
        configure_logging(level=std_logging.WARNING)
        assert root.level == std_logging.WARNING and "%(process)d" in root.handlers[0].formatter._fmt
    finally:  # the test runner's own handlers come back
        for handler in list(root.handlers):
            root.removeHandler(handler)
        for handler in handlers:
            root.addHandler(handler)
        root.setLevel(level)
    assert monkey_patch_torch_compile() is None
