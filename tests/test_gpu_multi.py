"""Multi-GPU tests of the peer-memory communication layer (one process per GPU)."""
import pytest
import torch
import torch.multiprocessing as mp

import _gpu_workers as W

pytestmark = pytest.mark.gpu


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _run(fn, world, tmp_path, port, *args):
    mp.spawn(fn, args=(world, port, str(tmp_path), *args), nprocs=world, join=True)
    assert all((tmp_path / f"ok_{r}").exists() for r in range(world))


def test_replica_allreduce_kernels(tmp_path, free_port):
    _need(2)
    _run(W.run_allreduce, 2, tmp_path, free_port)


def test_allgather_fused_with_gemm(tmp_path, free_port):
    _need(2)
    _run(W.run_allgather_gemm, 2, tmp_path, free_port)


def test_expert_parallel_dispatch_matches_nccl(tmp_path, free_port):
    _need(2)
    _run(W.run_moe_ep, 2, tmp_path, free_port)


def test_training_steps_fused_vs_nccl_fsdp2(tmp_path, free_port):
    _need(2)
    _run(W.run_train_parity, 2, tmp_path, free_port, 1)


def test_training_steps_when_every_row_goes_to_one_rank(tmp_path, free_port):
    """The worst routing there is: every token of both ranks picks the two first experts, which live on rank 0.  The
    fused exchange must neither overflow nor drop a row, and must agree with the NCCL path."""
    _need(2)
    _run(W.run_train_parity, 2, tmp_path, free_port, 1, 1, True)


def test_training_steps_fused_vs_nccl_pp2_fsdp2(tmp_path, free_port):
    _need(4)
    _run(W.run_train_parity, 4, tmp_path, free_port, 2)


def test_training_steps_fused_vs_nccl_fsdp4_ep4(tmp_path, free_port):
    _need(4)
    _run(W.run_train_parity, 4, tmp_path, free_port, 1)


def test_training_steps_fused_vs_nccl_fsdp2_with_two_replicas(tmp_path, free_port):
    _need(4)
    _run(W.run_train_parity, 4, tmp_path, free_port, 1, 2)


def test_pipeline_peer_link_matches_nccl_link_two_stages(tmp_path, free_port):
    _need(2)
    _run(W.run_pipeline_link, 2, tmp_path, free_port)


def test_pipeline_peer_link_matches_nccl_link_four_stages(tmp_path, free_port):
    _need(4)
    _run(W.run_pipeline_link, 4, tmp_path, free_port)
