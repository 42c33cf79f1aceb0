"""The benchmark's output contract, checked without a GPU: layout per GPU count, the JSON line and its required
keys, the clock summary parsed from nvidia-smi rows, and the reference arm's answer when the reference is absent."""
import argparse
import io
import json
import os
import sys
from contextlib import redirect_stdout

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
import bench  # noqa: E402


def _args(**over):
    base = dict(gpus=1, steps=2, warmup=3, impl="b200moe", layers=None, microbatches=32, batch=None, seq=8192,
                recompute=None, backend=None, layout=None, kernel_times=None)
    base.update(over)
    return argparse.Namespace(**base)


def test_layout_scales_layers_with_gpus_and_names_the_published_configuration():
    seen = {n: bench.run_config(_args(gpus=n)) for n in (1, 2, 4, 8)}
    assert [seen[n]["pp"] * seen[n]["blocks_per_stage"] for n in (1, 2, 4, 8)] == [8, 8, 16, 32]
    assert seen[8] == {"pp": 4, "fsdp": 2, "ddp": 1, "blocks_per_stage": 8, "batch": 128, "microbatches": 32,
                       "seq": 8192, "experts_per_rank": 4, "rope_theta": 1e4}
    for n, cfg in seen.items():
        assert cfg["pp"] * cfg["fsdp"] * cfg["ddp"] == n
        # weak scaling: sequences per data-parallel rank and blocks per GPU stay fixed
        assert cfg["batch"] // (cfg["fsdp"] * cfg["ddp"]) == 64 and cfg["blocks_per_stage"] == 8
    with pytest.raises(SystemExit):
        bench.run_config(_args(gpus=3))


def test_named_layouts_cover_the_replica_and_the_wide_expert_configurations():
    ddp2 = bench.run_config(_args(gpus=8, layout="ddp2"))
    assert (ddp2["pp"], ddp2["fsdp"], ddp2["ddp"], ddp2["blocks_per_stage"], ddp2["batch"]) == (1, 4, 2, 8, 32)
    assert ddp2["experts_per_rank"] == 2 and ddp2["rope_theta"] == 1e6
    assert ddp2["batch"] % (ddp2["fsdp"] * ddp2["ddp"] * ddp2["microbatches"]) == 0
    pp2 = bench.run_config(_args(gpus=8, layout="pp2"))
    assert (pp2["pp"], pp2["fsdp"], pp2["ddp"], pp2["blocks_per_stage"], pp2["batch"], pp2["microbatches"]) == \
        (2, 4, 1, 16, 64, 16)
    with pytest.raises(SystemExit):
        bench.run_config(_args(gpus=4, layout="pp2"))


def test_a_failing_rank_names_its_exception_once_and_leaves_non_zero(monkeypatch, capsys):
    codes = []
    monkeypatch.setattr(bench.os, "_exit", lambda code: codes.append(code))
    monkeypatch.setenv("MASTER_PORT", "1")
    monkeypatch.setenv("RANK", "3")
    monkeypatch.setenv("WORLD_SIZE", "8")
    marker = os.path.join("/tmp", f"b200moe_bench_failed_1_{os.getppid()}")
    if os.path.exists(marker):
        os.unlink(marker)
    try:
        bench.say_failure("reference", _args(gpus=8, impl="reference"), RuntimeError("out of memory\nmore"))
        bench.say_failure("reference", _args(gpus=8, impl="reference"), RuntimeError("NCCL: peer gone"))
    finally:
        if os.path.exists(marker):
            os.unlink(marker)
    captured = capsys.readouterr()
    lines = [json.loads(l) for l in captured.out.strip().splitlines()]
    assert len(lines) == 1 and lines[0]["unavailable"] == "rank 3: RuntimeError: out of memory"
    assert "RuntimeError: out of memory" in captured.err and "peer gone" in captured.err
    assert codes == [1, 1]
    # a lone reference process ends normally after its line
    monkeypatch.setenv("WORLD_SIZE", "1")
    bench.say_failure("reference", _args(impl="reference"), ValueError("x"))
    os.unlink(marker)
    assert codes[-1] == 0


def test_json_line_has_the_contract_keys_and_consistent_numbers():
    args = _args(gpus=8)
    cfg = bench.run_config(args)
    clocks = {"sm_mhz": 1560.0, "sm_max_mhz": 1965.0, "power_w_max": 990.0, "samples": 70, "reasons": ["sw_power_cap"]}
    out = io.StringIO()
    with redirect_stdout(out):
        bench.report(args, cfg, 14000.0, 14100.0, clocks, 12345, 10.4, 8388608, 4, "b200moe", {"peak_mem_gib": 150.0})
    line = json.loads(out.getvalue().strip())
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches"):
        assert key in line, key
    tokens = 128 * 8192
    assert line["value"] == pytest.approx(tokens / 14.0)             # 32 blocks: no normalisation at N = 8
    assert line["vs_baseline"] == pytest.approx(line["value"] / 75076.0)
    assert line["n_gpus"] == 8 and line["higher_is_better"] is True and line["scaling"] == "weak"
    assert line["dtype"] == "bf16" and "synthetic" in line["data"]
    assert line["config"]["parallelism"] == "pp4·fsdp2·ep2·ddp1" and line["config"]["global_batch"] == 128
    assert "H2D" in line["config"]["loop"] and line["config"]["layout"] == "scaling"
    assert line["e2e"]["value"] == pytest.approx(tokens / 14.1) and line["e2e"]["h2d_bytes_per_step"] == 8388608
    assert line["e2e"]["d2h_bytes_per_step"] == 4 and line["gpu_launches"] == 12345
    assert line["mfu"] == pytest.approx(line["tokens_per_s_raw"] * 84.007714816e9 / (8 * 2.25e15), rel=1e-6)
    # fewer blocks: the value is scaled by FLOPs per token, the raw rate is reported next to it
    args1 = _args(gpus=1)
    out = io.StringIO()
    with redirect_stdout(out):
        bench.report(args1, bench.run_config(args1), 11000.0, None, clocks, 1, 10.4, 0, 4, "b200moe")
    line1 = json.loads(out.getvalue().strip())
    assert "e2e" not in line1
    assert line1["value"] == pytest.approx(line1["tokens_per_s_raw"] * line1["gflops_per_token"] / 84.007714816, rel=1e-6)
    assert line1["value"] < line1["tokens_per_s_raw"]


def test_clock_summary_from_sampled_rows():
    sampler = bench.ClockSampler(0)

    class Done:
        def terminate(self):
            pass

        def wait(self, timeout=None):
            return 0
    sampler.proc = Done()
    sampler.rows = [
        ["0", "1965", "1965", "310.5", "0x0000000000000000", "Not Active", "Not Active", "Not Active", "Not Active"],
        ["0", "1590", "1965", "987.2", "0x0000000000000004", "Not Active", "Not Active", "Not Active", "Active"],
        ["0", "1560", "1965", "991.0", "0x0000000000000004", "Not Active", "Not Active", "Not Active", "Active"],
        ["garbage"],
        ["0", "N/A", "1965", "1.0", "x", "Not Active", "Not Active", "Not Active", "Not Active"],
    ]
    summary = sampler.stop()
    assert summary == {"sm_mhz": 1590.0, "sm_max_mhz": 1965.0, "power_w_max": 991.0, "samples": 3,
                       "reasons": ["sw_power_cap"]}
    assert bench.ClockSampler(0).stop()["reasons"] == ["nvidia-smi unavailable"]


def test_reference_arm_reports_unavailable_when_the_reference_is_not_installed(monkeypatch, tmp_path):
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    out = io.StringIO()
    with redirect_stdout(out):
        bench.bench_reference(_args(impl="reference"))
    line = json.loads(out.getvalue().strip())
    assert line["impl"] == "reference" and "unavailable" in line
