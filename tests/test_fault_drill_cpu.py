"""The launcher-level fault drill on CPU: torchrun starts two gloo ranks, the chaos trigger SIGKILLs rank 1 after
iteration 7 of the first attempt, torchrun restarts the group, the workers resume from the newest committed checkpoint
and the iterations they repeat reproduce the first attempt's losses (reference recovery model: README.md:85,
distributed_parallel_training_pipelined.py:39-64)."""
import os
import re
import subprocess
import sys

import pytest
import yaml

import _workers as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _losses(text):
    found, current = {}, None
    for line in text.splitlines():
        done = re.search(r"finishes iteration (\d+)", line)
        if done:
            current = int(done.group(1))
        loss = re.search(r"Rank 0 Loss from last 1 iterations is (?:tensor\()?([0-9.eE+-]+)", line)
        if loss and current is not None:
            found[current] = float(loss.group(1))
    return found


@pytest.mark.timeout(900)
def test_torchrun_restarts_the_group_after_a_killed_rank_and_the_run_resumes(tmp_path):
    config = W.tiny_config(2, 2, 1, 1, tmp_path, target=10, save=2, batch=4, micro=2)
    config["recovery"] = {"collective_timeout_seconds": 60}
    config["chaos_engineering"] = {"random_kill": {"enabled": True, "chance": 1.0, "after_iteration": 7,
                                                   "first_attempt_only": True, "rank": 1}}
    path = tmp_path / "run.yaml"
    path.write_text(yaml.safe_dump(config))
    env = {k: v for k, v in os.environ.items() if k not in ("MASTER_ADDR", "MASTER_PORT", "RANK", "WORLD_SIZE",
                                                            "LOCAL_RANK")}
    env["GLOO_SOCKET_IFNAME"] = "lo"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr=127.0.0.1", "--nnodes=1",
           "--nproc-per-node=2", "--max-restarts=1", "--monitor-interval=1",
           os.path.join(ROOT, "distributed_parallel_training_pipelined.py"), "--config-path", str(path)]
    drill = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=850)
    text = drill.stdout + drill.stderr
    assert drill.returncode == 0, text[-4000:]
    first, _, second = drill.stdout.partition("loaded checkpoint at")
    assert second, text[-4000:]
    start = int(re.match(r"\s*(\d+) iterations", second).group(1))
    assert start in (2, 4, 6)
    assert "finishes iteration 7" in first and "finishes iteration 8" not in first
    assert "finishes iteration 10" in second
    before, after = _losses(first), _losses(second)
    assert set(range(start + 1, 11)) <= set(after), after
    for iteration in range(start + 1, 8):
        assert after[iteration] == pytest.approx(before[iteration], rel=1e-4, abs=1e-4), (iteration, before, after)
    committed = sorted(int(p.parent.name) for p in (tmp_path / "checkpoint").glob("*/*/COMMITTED"))
    assert committed and committed[-1] == 10, committed
