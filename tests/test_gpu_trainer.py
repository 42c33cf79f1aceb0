"""The torchrun entry point on one GPU: train, commit checkpoints, resume (watchdog, status checks and the
pinned-memory checkpoint staging all run for real here; the multi-rank plumbing is covered by the gloo tests)."""
import os
import subprocess
import sys

import pytest
import yaml

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _config(folder, target):
    return {
        "general": {"device": "gpu", "n_workers": 1, "gpu_per_node": 1, "info_src": 0,
                    "checkpoint_folder": str(folder), "metrics_path": str(folder / "metrics.jsonl")},
        "recovery": {"collective_timeout_seconds": 60, "status_poll_seconds": 0.2},
        "data": {"vocab_size": 2048, "mock_data": True, "seed": 0, "validate_batches": True},
        "model": {"num_head": 4, "d_model": 512, "d_ff": 1024, "context_len": 256, "num_layers": 2,
                  "num_expert_per_node": 4, "rope_theta": 10000},
        "train": {"fsdp_parallel_num": 1, "data_parallel_num": 1, "pipeline_parallel_stages": 1,
                  "microbatch_num": 2, "batch_size": 4, "save_interval": 2, "target_iteration": target,
                  "learning_rate": 1e-3, "optimizer": {"beta1": 0.9, "beta2": 0.999, "lambda": 0.01},
                  "learning_rate_scheduler": {"a_max": 1e-3, "a_min": 1e-4, "t_w": 2, "t_c": 100},
                  "print_loss_interval": 1, "load_checkpoint_path": ""},
        "profile": {"enabled": False},
    }


def _run(config_path, port):
    env = {**os.environ, "RANK": "0", "LOCAL_RANK": "0", "WORLD_SIZE": "1", "LOCAL_WORLD_SIZE": "1",
           "GROUP_RANK": "0", "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)}
    return subprocess.run([sys.executable, os.path.join(ROOT, "distributed_parallel_training_pipelined.py"),
                           "--config-path", str(config_path)], cwd=ROOT, env=env, capture_output=True, text=True,
                          timeout=600)


@pytest.mark.gpu
def test_entry_point_trains_commits_and_resumes_on_one_gpu(tmp_path, free_port):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    path = tmp_path / "run.yaml"
    path.write_text(yaml.safe_dump(_config(tmp_path, 8)))
    first = _run(path, free_port)
    assert first.returncode == 0, first.stdout[-3000:] + first.stderr[-3000:]
    assert "Loss from last 1 iterations" in first.stdout and "tokens/s" in first.stdout
    committed = sorted(int(p.parent.name) for p in (tmp_path / "checkpoint").glob("*/*/COMMITTED"))
    assert committed and committed[-1] == 8, committed
    assert (tmp_path / "metrics.jsonl").exists()
    # a second launch with a larger target finds the newest committed step and continues from it
    path.write_text(yaml.safe_dump(_config(tmp_path, 10)))
    second = _run(path, free_port)
    assert second.returncode == 0, second.stdout[-3000:] + second.stderr[-3000:]
    assert "loaded checkpoint at 8 iterations" in second.stdout
    assert "finishes iteration 10" in second.stdout and "finishes iteration 8" not in second.stdout
