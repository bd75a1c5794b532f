"""Offline analysis tools on real debug-mode dumps of a simulated job, with
faults seeded afterwards."""

import copy
import json
import os

import pytest
import torch

from awex_b200.synthetic.arch import get_arch
from awex_b200.synthetic.simulate import InferLayout, SimulatedJob, TrainLayout


@pytest.fixture(scope="module")
def job():
    return SimulatedJob(get_arch("tiny-llama"), TrainLayout(tp=2), InferLayout(tp=2), dtype=torch.float32)


def test_meta_dump_analysis_finds_seeded_faults(job, tmp_path):
    from awex_b200.debug import meta_dumps
    from awex_b200.meta.weight_meta import dump_parameters_meta

    train, infer = dump_parameters_meta(job.train_meta), dump_parameters_meta(job.infer_meta)
    t_path, i_path = tmp_path / "train_params_meta_0.json", tmp_path / "infer_params_meta_0.json"
    t_path.write_text(json.dumps(train))
    i_path.write_text(json.dumps(infer))
    assert meta_dumps.main([str(t_path), str(i_path)]) == 0
    clean = meta_dumps.analyze_meta(meta_dumps.load_meta(str(t_path)), meta_dumps.load_meta(str(i_path)))
    assert clean["summary"]["critical_errors"] == 0 and clean["summary"]["common_params"] == len(train)
    broken = copy.deepcopy(infer)
    broken[0]["global_shape"] = [1, 1]
    broken[1]["dtype"] = "torch.float16"
    dropped = broken.pop()
    broken.append({"name": "mystery.weight", "global_shape": [1], "global_numel": 1, "dtype": "torch.float32", "replicas": []})
    report = meta_dumps.analyze_meta(train, broken)
    s = report["summary"]
    assert s["shape_mismatch_count"] == 1 and s["dtype_mismatch_count"] == 1 and s["critical_errors"] >= 3
    assert report["missing_on_infer"] == [dropped["name"]] and report["unsupported_extra_on_infer"] == ["mystery.weight"]
    with pytest.raises(ValueError):
        (tmp_path / "junk.json").write_text("{}")
        meta_dumps.load_meta(str(tmp_path / "junk.json"))


def test_plan_dump_analysis_checks_bounds_coverage_and_mirror(job, tmp_path, monkeypatch):
    from awex_b200.debug import bundle, plan_dumps
    from awex_b200.meta.weight_meta import dump_parameters_meta
    from awex_b200.transfer.transfer_plan import TransferPlanBuilder

    monkeypatch.chdir(tmp_path)
    builder = TransferPlanBuilder(job.infer_world_size, job.train.world, 1, enable_debug_mode=True)
    for rank in range(job.infer_world_size + job.train.world):
        builder.build_local_transfer_plan(job.infer_meta, job.train_meta, rank)
    files = sorted(os.listdir(tmp_path))
    assert sum(f.startswith("local_communication_plan_infer") for f in files) == 2
    report = plan_dumps.analyze_files([str(tmp_path)])
    assert report["problems"] == [] and report["receivers_checked"] == [0, 1] and report["shards_checked"] > 10
    assert plan_dumps.main([str(tmp_path)]) == 0
    # drop one operation from a receiver's plan: its shard is no longer covered, and the sender disagrees
    victim = next(f for f in files if f.startswith("local_communication_plan_infer_0"))
    plan = json.loads((tmp_path / victim).read_text())
    peer = sorted(plan)[0]
    removed = plan[peer].pop()
    (tmp_path / victim).write_text(json.dumps(plan))
    report = plan_dumps.analyze_files([str(tmp_path / victim)] + [str(tmp_path / f) for f in files if f.startswith("local_communication_plan_train")])
    assert any("never written" in p or "receives" in p for p in report["problems"]) or any("disagree" in p for p in report["problems"])
    assert any("disagree" in p for p in report["problems"])
    # an operation that leaves its shard
    removed["recv_offset"] = [10_000] + removed["recv_offset"][1:]
    assert plan_dumps.bounds_problems(removed)
    # the bundle runner needs the metadata dumps beside the plans
    (tmp_path / "train_params_meta_0_1.json").write_text(json.dumps(dump_parameters_meta(job.train_meta)))
    (tmp_path / "infer_params_meta_0_1.json").write_text(json.dumps(dump_parameters_meta(job.infer_meta)))
    whole = bundle.analyze_bundle(str(tmp_path))
    assert whole["meta"]["summary"]["critical_errors"] == 0 and whole["critical_errors"] == len(whole["plans"]["problems"]) > 0


def test_weight_comparison_between_training_and_inference_dumps(job, tmp_path):
    from awex_b200.debug.compare_weights import (
        assemble_from_shards, compare_named_tensors, dump_converted_inference_shards, dump_converted_training_shards,
        load_named_tensors, main,
    )
    from awex_b200.models.registry import get_infer_weights_converter
    from awex_b200.synthetic.models import build_vllm_model, vllm_model_context

    train_shards = {}
    for ri, model in zip(job.train_ranks, job.train_models):
        path = dump_converted_training_shards(str(tmp_path), [model], job._train_converter(ri), ri)
        train_shards[ri.global_rank] = load_named_tensors(path)
    infer_shards = {}
    for ri in job.infer_ranks[0]:
        model = build_vllm_model(job.arch, ri, torch.float32, "cpu")  # an engine that holds the same weights
        conv = get_infer_weights_converter("vllm", job.arch.architecture, job.hf_config, ri, job.engines[0].config)
        path = dump_converted_inference_shards(str(tmp_path), model, conv, vllm_model_context(ri))
        infer_shards[ri.global_rank] = load_named_tensors(path)
    left = assemble_from_shards(job.train_meta, train_shards)
    right = assemble_from_shards(job.infer_meta, infer_shards)
    report = compare_named_tensors(left, right)
    assert report["ok"], report["summary"]
    right["model.norm.weight"] = right["model.norm.weight"] + 1
    right["extra.weight"] = torch.zeros(1)
    del right["lm_head.weight"]
    bad = compare_named_tensors(left, right)
    assert not bad["ok"] and bad["value_mismatch"][0]["name"] == "model.norm.weight"
    assert bad["missing_on_right"] == ["lm_head.weight"] and bad["missing_on_left"] == ["extra.weight"]
    assert compare_named_tensors(left, right, ignore=["norm", "extra", "lm_head"])["ok"]
    torch.save({"w": torch.ones(2)}, tmp_path / "a.pt")
    torch.save({"w": torch.ones(2) + 1e-4}, tmp_path / "b.pt")
    assert main([str(tmp_path / "a.pt"), str(tmp_path / "b.pt")]) == 1
    assert main([str(tmp_path / "a.pt"), str(tmp_path / "b.pt"), "--atol", "1e-3"]) == 0


def test_canonical_names_exist_in_the_checkpoint(job, tmp_path):
    from awex_b200.debug.verify_names import canonical_names_of, checkpoint_equivalents, verify_names
    from awex_b200.models.registry import get_infer_weights_converter
    from awex_b200.synthetic.models import CanonicalWeights, canonical_state_dict, vllm_model_context
    from awex_b200.utils.safetensors_io import checkpoint_weight_map, save_checkpoint

    save_checkpoint(str(tmp_path), canonical_state_dict(job.arch, CanonicalWeights(job.arch, torch.float32, "cpu")))
    ri = job.infer_ranks[0][0]
    conv = get_infer_weights_converter("vllm", job.arch.architecture, job.hf_config, ri, job.engines[0].config)
    names = canonical_names_of(job.infer_models[0][0], conv, vllm_model_context(ri))
    report = verify_names(names, checkpoint_weight_map(str(tmp_path)))
    assert report["ok"] and report["checked"] == len(names), report["missing"][:3]
    assert not verify_names(names + ["model.layers.0.mlp.ghost.weight"], checkpoint_weight_map(str(tmp_path)))["ok"]
    assert checkpoint_equivalents("model.layers.3.mlp.gate_up_proj.weight") == ["model.layers.3.mlp.gate_proj.weight", "model.layers.3.mlp.up_proj.weight"]


def test_plan_study_reports_bytes_and_bounds():
    from awex_b200.debug.plan_study import main, parse_layout, study

    assert parse_layout("tp1,dp4,ep4") == {"tp": 1, "dp": 4, "ep": 4} and parse_layout("tp2,engines2") == {"tp": 2, "engines": 2}
    with pytest.raises(SystemExit):
        parse_layout("tp")
    spread = study("tiny-qwen3-moe", {"tp": 1, "dp": 4, "ep": 4}, {"tp": 2, "ep": 2, "engines": 2}, placement="colocated")
    rr = study("tiny-qwen3-moe", {"tp": 1, "dp": 4, "ep": 4}, {"tp": 2, "ep": 2, "engines": 2}, placement="colocated", pairing="round_robin")
    assert spread["coverage_problems"] == [] and len(spread["senders"]) == 4
    total = lambda rep: sum(x["remote_egress"] + x["local_written"] for x in rep["senders"])  # noqa: E731
    assert total(spread) == total(rr)  # the same bytes, differently shared
    assert max(x["read"] for x in spread["senders"]) < max(x["read"] for x in rr["senders"])
    separated = study("tiny-qwen3-moe", {"tp": 1, "dp": 4, "ep": 4}, {"tp": 2, "ep": 2, "engines": 2}, placement="separated")
    assert all(x["local_written"] == 0 for x in separated["senders"]) and separated["lower_bound_ms"] > 0
    assert sum(separated["ingress_per_inference_rank"]) == total(separated)
    assert main(["--model", "tiny-llama", "--train", "tp2", "--infer", "tp1", "--placement", "separated"]) == 0


def test_plan_study_finds_a_placement_that_keeps_more_bytes_local():
    from awex_b200.debug.plan_study import parse_layout, study

    train, infer = parse_layout("tp1,dp4,ep4"), parse_layout("tp2,ep2,engines2")
    plain = study("tiny-qwen3-moe", train, infer, placement="colocated")
    best = study("tiny-qwen3-moe", train, infer, placement="colocated-best")
    local = lambda report: sum(x["local_written"] for x in report["senders"])  # noqa: E731
    assert sorted(best["gpu_of_inference_rank"].values()) == [0, 1, 2, 3] and best["coverage_problems"] == []
    assert local(best) > local(plain)
    assert best["bound_ms"]["nvlink_egress"] < plain["bound_ms"]["nvlink_egress"]
    # the same bytes move either way
    total = lambda report: sum(x["local_written"] + x["remote_egress"] for x in report["senders"])  # noqa: E731
    assert total(best) == total(plain)
