"""Kill one rank between steps, let torchrun restart the group, resume from the last committed checkpoint: the
reference's recovery model (README.md:85, distributed_parallel_training_pipelined.py:39-64) on two GPUs.

The failure is made on the host: the chaos trigger SIGKILLs rank 1 after iteration 7 of the first attempt, after a
device synchronisation, with no kernel or collective of that rank in flight.  The run uses ``comm.backend: nccl``
with ``NCCL_NVLS_ENABLE=0``: no buffer of either rank is bound to an NVLink multicast object and none of this
framework's peer-memory kernels is involved, so the surviving rank only ever sees a collective that does not
complete, which the launcher ends when it notices the dead worker."""
import os
import re
import subprocess
import sys

import pytest
import yaml

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _config(folder, kill):
    return {
        "general": {"device": "gpu", "n_workers": 2, "gpu_per_node": 2, "info_src": 0,
                    "checkpoint_folder": str(folder)},
        "recovery": {"collective_timeout_seconds": 30, "status_poll_seconds": 0.5},
        "comm": {"backend": "nccl"},
        "data": {"vocab_size": 2048, "mock_data": True, "seed": 0, "validate_batches": True},
        "model": {"num_head": 4, "d_model": 512, "d_ff": 1024, "context_len": 256, "num_layers": 2,
                  "num_expert_per_node": 2, "rope_theta": 10000},
        "train": {"fsdp_parallel_num": 2, "data_parallel_num": 1, "pipeline_parallel_stages": 1,
                  "microbatch_num": 2, "batch_size": 8, "save_interval": 2, "target_iteration": 10,
                  "learning_rate": 1e-3, "optimizer": {"beta1": 0.9, "beta2": 0.999, "lambda": 0.01},
                  "learning_rate_scheduler": {"a_max": 1e-3, "a_min": 1e-4, "t_w": 2, "t_c": 100},
                  "print_loss_interval": 1, "load_checkpoint_path": ""},
        "chaos_engineering": {"random_kill": {"enabled": bool(kill), "chance": 1.0, "after_iteration": 7,
                                              "first_attempt_only": True, "rank": 1}},
        "profile": {"enabled": False},
    }


def _launch(config_path, port, restarts):
    # --standalone: a fresh rendezvous (and a fresh store prefix) for every attempt, so the restarted workers do not
    # pick up the first attempt's NCCL bootstrap address; loopback for the rendezvous and for NCCL's bootstrap
    env = {**os.environ, "NCCL_NVLS_ENABLE": "0", "NCCL_SOCKET_IFNAME": "lo"}
    for key in ("MASTER_ADDR", "MASTER_PORT", "RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(key, None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr=127.0.0.1", "--nnodes=1",
           "--nproc-per-node=2", f"--max-restarts={restarts}", "--monitor-interval=1",
           os.path.join(ROOT, "distributed_parallel_training_pipelined.py"), "--config-path", str(config_path)]
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)


def _losses(text):
    """{iteration: loss} from the trainer's log lines (the last value printed for an iteration wins)."""
    found, current = {}, None
    for line in text.splitlines():
        done = re.search(r"finishes iteration (\d+)", line)
        if done:
            current = int(done.group(1))
        loss = re.search(r"Rank 0 Loss from last 1 iterations is (?:tensor\()?([0-9.eE+-]+)", line)
        if loss and current is not None:
            found[current] = float(loss.group(1))
    return found


def test_kill_one_rank_between_steps_and_resume_from_the_committed_checkpoint(tmp_path, free_port):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    (tmp_path / "run.yaml").write_text(yaml.safe_dump(_config(tmp_path, kill=True)))
    drill = _launch(tmp_path / "run.yaml", free_port, restarts=1)
    text = drill.stdout + drill.stderr
    assert drill.returncode == 0, text[-4000:]
    first, _, second = drill.stdout.partition("loaded checkpoint at")
    assert second, text[-4000:]
    start = int(re.match(r"\s*(\d+) iterations", second).group(1))
    assert start in (2, 4, 6)                                            # the newest step committed before the kill
    assert "finishes iteration 7" in first and "finishes iteration 8" not in first
    assert "finishes iteration 10" in second
    # the restarted group restored weights, optimizer state and the data sampler: the iterations it repeats give
    # the losses the first attempt saw (the weights of a run are not seeded, so only the two attempts compare)
    before, after = _losses(first), _losses(second)
    assert set(range(start + 1, 11)) <= set(after), after
    for iteration in range(start + 1, 8):
        assert after[iteration] == pytest.approx(before[iteration], rel=2e-3, abs=2e-3), (iteration, before, after)
    committed = sorted(int(p.parent.name) for p in (tmp_path / "checkpoint").glob("*/*/COMMITTED"))
    assert committed and committed[-1] == 10, committed
