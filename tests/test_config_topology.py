import copy
import os

import numpy as np
import pytest
import yaml

from b200moe import config as cfg
from b200moe.topology import parallel_rank_groups, parallel_sizes

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture
def base():
    with open(os.path.join(ROOT, "configs", "run_config.yaml"), encoding="utf-8") as f:
        return yaml.safe_load(f)


def test_shipped_config_is_valid(base):
    cfg.validate_config(base)


def test_parallel_sizes_legacy_and_errors():
    assert parallel_sizes({"data_parallel_num": 4}) == (4, 1)
    assert parallel_sizes({"fsdp_parallel_num": 2, "data_parallel_num": 3}) == (2, 3)
    for bad in (0, -1, 1.0, True):
        with pytest.raises(ValueError):
            parallel_sizes({"fsdp_parallel_num": bad, "data_parallel_num": 1})


def test_rank_groups_pp4_fsdp2():
    g = parallel_rank_groups({"fsdp_parallel_num": 2, "data_parallel_num": 1, "pipeline_parallel_stages": 4}, 8, 8)
    assert g["fsdp"] == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert g["data"] == g["fsdp"]
    assert g["ddp"] == [[0], [1], [2], [3], [4], [5], [6], [7]]
    assert g["pp"] == [[0, 2, 4, 6], [1, 3, 5, 7]]


def test_rank_groups_fsdp4_ddp2():
    g = parallel_rank_groups({"fsdp_parallel_num": 4, "data_parallel_num": 2, "pipeline_parallel_stages": 1}, 8, 8)
    assert g["fsdp"] == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert g["ddp"] == [[0, 4], [1, 5], [2, 6], [3, 7]]
    assert g["data"] == [list(range(8))]
    assert g["pp"] == [[r] for r in range(8)]


def test_rank_groups_reject_bad_shapes():
    t = {"fsdp_parallel_num": 2, "data_parallel_num": 1, "pipeline_parallel_stages": 4}
    with pytest.raises(ValueError):
        parallel_rank_groups(t, 6, 6)
    with pytest.raises(ValueError):
        parallel_rank_groups({**t, "fsdp_parallel_num": 4, "pipeline_parallel_stages": 2}, 8, 2)


@pytest.mark.parametrize("mutate,match", [
    (lambda c: c["train"].__setitem__("batch_size", 100), "divisible"),
    (lambda c: c["general"].__setitem__("info_src", 8), "info_src"),
    (lambda c: c["model"].__setitem__("d_model", 4100), "divisible"),
    (lambda c: c["model"].__setitem__("context_len", 8190), "context_len"),
    (lambda c: c["train"]["learning_rate_scheduler"].__setitem__("t_w", 30000), "Scheduler"),
    (lambda c: c["general"].__setitem__("n_workers", 16), "one node"),
    (lambda c: c["train"].__setitem__("router_aux_loss_coef", float("nan")), "router_aux_loss_coef"),
    (lambda c: c["train"].__setitem__("activation_recompute", "all"), "activation_recompute"),
    (lambda c: c["data"].__setitem__("vocab_size", 32001), "divisible"),
    (lambda c: c["model"].__setitem__("num_layers", 0), "positive integer"),
    (lambda c: c["train"].__setitem__("fsdp_gather", "always"), "fsdp_gather"),
    (lambda c: c["comm"].__setitem__("backend", "mpi"), "comm.backend"),
])
def test_validation_failures(base, mutate, match):
    bad = copy.deepcopy(base)
    mutate(bad)
    with pytest.raises(ValueError, match=match):
        cfg.validate_config(bad)


def test_gpu_only_mode_rejects_cpu(base):
    base["general"]["device"] = "cpu"
    cfg.validate_config(base)
    with pytest.raises(ValueError, match="device must be gpu"):
        cfg.validate_config(base, allow_cpu=False)


def test_load_config_resolves_relative_paths_and_cli_generates_data(tmp_path, base, capsys):
    base["data"]["train_dataset_path"] = "data/tokens.npy"
    base["general"]["checkpoint_folder"] = "ckpt"
    base["model"]["context_len"] = 64
    path = tmp_path / "run.yaml"
    path.write_text(yaml.safe_dump(base))
    loaded = cfg.load_config(path)
    assert loaded["data"]["train_dataset_path"] == str(tmp_path / "data" / "tokens.npy")
    assert loaded["general"]["checkpoint_folder"] == str(tmp_path / "ckpt")
    assert cfg.main(["--config", str(path), "--generate-data"]) == 0
    tokens = np.load(tmp_path / "data" / "tokens.npy")
    assert tokens.dtype == np.int32 and tokens.size == 4096
    assert "Startup checks passed" in capsys.readouterr().out
    with pytest.raises(FileExistsError):
        cfg.generate_dataset(loaded)
