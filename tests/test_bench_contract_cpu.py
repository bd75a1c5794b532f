"""The benchmark harness end to end on CPU ranks (gloo): one JSON line on
stdout with the keys the contract names, bitwise-validated weights, for the
separated layouts at 2 and 4 processes."""

import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REQUIRED = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
            "dtype", "data", "config", "clocks", "e2e", "gpu_launches"}


def _run(n, extra, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "bench.py"), "--device", "cpu", "--gpus", str(n), "--steps", "2",
           "--warmup", "1"] + extra
    env = dict(os.environ, AWEX_LOG_LEVEL="WARNING")
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=400, cwd=ROOT, env=env)
    assert proc.returncode == 0, proc.stderr[-3000:]
    lines = [line for line in proc.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1, proc.stdout[-2000:]
    return json.loads(lines[0])


@pytest.mark.timeout(900)
@pytest.mark.parametrize("n,extra,label", [
    (2, ["--model", "tiny-llama"], "tp1->tp1"),
    (4, ["--model", "tiny-qwen2"], "tp2->tp2"),
])
def test_bench_prints_one_contract_line(n, extra, label):
    from awex_b200.utils.common import get_free_port

    result = _run(n, extra, get_free_port())
    assert REQUIRED <= set(result), REQUIRED - set(result)
    assert result["n_gpus"] == n and result["steps"] == 2 and result["warmup"] == 1
    assert result["higher_is_better"] is False and result["unit"] == "s" and result["value"] > 0
    assert abs(result["ms_per_step"] - result["value"] * 1e3) < 1e-6
    assert result["config"]["parallelism"] == label and result["config"]["validated_bitwise"] is True
    assert set(result["e2e"]) >= {"value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"} and result["e2e"]["value"] > 0
    assert result["e2e"]["h2d_bytes_per_step"] > 0 and result["e2e"]["d2h_bytes_per_step"] > 0
    assert len(result["per_step_ms"]) == 2 and result["device"].startswith("cpu")


def test_reference_arm_declines_co_located_configurations():
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--config", "colocated"],
                          capture_output=True, text=True, timeout=120, cwd=ROOT)
    assert proc.returncode == 0
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line


def test_role_table_placements():
    """The MoE configuration's two placements: instances on halves of the box, or
    every worker beside the two training ranks that hold its experts."""
    from awex_b200.bench_distributed import role_table

    train, infer, train_ranks, engines, label = role_table(8, "moe")
    assert engines == [[0, 1, 2, 3], [4, 5, 6, 7]] and train_ranks == list(range(8)) and "interleaved" not in label
    _t, _i, _r, engines, label = role_table(8, "moe", "interleaved")
    assert engines == [[0, 2, 4, 6], [1, 3, 5, 7]] and label.endswith("-interleaved")
    assert role_table(4, "moe", "interleaved")[3] == [[0, 2], [1, 3]]
    # other configurations ignore the placement
    assert role_table(8, "separated", "interleaved")[3] == role_table(8, "separated")[3] == [[4, 5], [6, 7]]
    assert role_table(8, "fp8", "interleaved")[3] == [list(range(8))]
