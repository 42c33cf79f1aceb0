"""Training worker: topology, model build, checkpoint discovery, the loop.

Launched by ``torchrun … --module distributed_parallel_training_pipelined
--config-path X`` (one process per GPU).  Behaviour follows the reference
worker (distributed_parallel_training_pipelined.py:91-326): same config keys,
same log lines, same checkpoint protocol, same NVTX range names.  Additions:
``general.device: cpu`` runs the same code on gloo; throughput is also timed on
the device (CUDA events, max over ranks) and written with MFU to an optional
JSONL sink; the chaos triggers fire once per iteration when enabled.
"""
from __future__ import annotations

import argparse
import os
import time
from concurrent.futures import Future
from datetime import datetime, timedelta
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import yaml

from .models import TransformerLMPipelined
from .ops.functional import cross_entropy
from .optim import AdamW
from .parallel import FSDPWrapperPipelined, pipelined_train_overlap
from .topology import build_groups, parallel_rank_groups, parallel_sizes
from .utils import checkpoint as ckpt
from .utils.chaos import ChaosEnginnerTrigger, release_leaks
from .utils.data import get_batch, load_dataset
from .utils.metrics import MetricsSink, flops_per_token, mfu
from .utils.profiling import DeviceStepTimer, nvtx_range
from .utils.schedule import learning_rate_schedule_wrapper

_nvtx_range = nvtx_range
_latest_checkpoint = ckpt.latest_checkpoint
_select_checkpoint = ckpt.select_checkpoint
_verify_pending_checkpoints = ckpt.verify_pending_checkpoints

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def resolve_device(config: dict, local_rank: int) -> torch.device:
    if config["general"].get("device") == "gpu" and torch.cuda.is_available():
        torch.cuda.set_device(local_rank)
        return torch.device("cuda", local_rank)
    return torch.device("cpu")


def init_process_group(backend: str, rank: int, world_size: int, timeout, device=None) -> None:
    """``dist.init_process_group`` from the torchrun environment.  After an elastic restart the workers talk to the
    same agent-hosted store as the attempt before, which still holds that attempt's keys (for NCCL: the bootstrap
    address of a process that no longer exists), and a rank that reads before rank 0 has overwritten them connects
    to nobody.  Restarted attempts therefore rendezvous under a key prefix of their own."""
    extra = {"device_id": device} if device is not None else {}
    restart = int(os.environ.get("TORCHELASTIC_RESTART_COUNT", "0") or 0)
    if restart > 0 and os.environ.get("TORCHELASTIC_USE_AGENT_STORE") == "True":
        base = dist.TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]), world_size, is_master=False,
                             timeout=timeout)
        store = dist.PrefixStore(f"/b200moe/attempt_{restart}", base)
        dist.init_process_group(backend, store=store, rank=rank, world_size=world_size, timeout=timeout, **extra)
    else:
        dist.init_process_group(backend, init_method="env://", rank=rank, world_size=world_size, timeout=timeout,
                                **extra)


def build_model(config: dict, mesh, device, fsdp_group, ddp_group, compute_dtype, comm=None):
    """Stage model + sharding wrapper + optimizer from a run configuration."""
    model_cfg, train_cfg, data_cfg = config["model"], config["train"], config["data"]
    moe_dtype = torch.bfloat16 if device.type == "cuda" else compute_dtype
    model = TransformerLMPipelined(
        data_cfg["vocab_size"], model_cfg["context_len"], model_cfg["d_model"], model_cfg["num_layers"],
        model_cfg["num_head"], mesh.stage, mesh.pp, num_expert_per_node=model_cfg["num_expert_per_node"],
        d_ff=model_cfg["d_ff"], theta=model_cfg.get("rope_theta", 10000), dp_group=fsdp_group,
        moe_compute_dtype=moe_dtype)
    model.to(device)
    # ``train.activation_recompute``: ``none`` keeps every activation (the reference's behaviour), ``swiglu``
    # rebuilds the experts' gate/up pre-activations in the backward pass, ``block`` re-runs whole blocks, ``auto``
    # (the default on a GPU) keeps gate/up while the stage's activation budget has room (parallel/memory.py).
    recompute = train_cfg.get("activation_recompute") or ("auto" if device.type == "cuda" else "none")
    if recompute not in ("none", "swiglu", "block", "auto"):
        raise ValueError("train.activation_recompute must be none, swiglu, block or auto")
    model.block_recompute = recompute == "block"
    # ``train.recompute_layers``: how many blocks (from the front of the stage) rebuild their gate/up
    # activations in the backward pass; an int, or one int per pipeline stage (earlier stages keep more
    # microbatches in flight under 1F1B and need it more).  Default: all blocks when ``swiglu``.
    count = train_cfg.get("recompute_layers")
    if isinstance(count, (list, tuple)):
        count = count[mesh.stage]
    if count is None:
        count = len(model.layers)
    for index, layer in enumerate(model.layers):
        layer.ffn.recompute = recompute == "swiglu" and index < count
    backend = (config.get("comm") or {}).get("backend", "fused" if device.type == "cuda" else "nccl")
    wrapped = FSDPWrapperPipelined(
        model, FSDP_communication_group=fsdp_group,
        DDP_communication_group=ddp_group if mesh.ddp > 1 else None, compute_dtype=compute_dtype,
        moe_compute_dtype=moe_dtype, backend=backend if comm is not None else "nccl", comm=comm,
        expert_grad_dtype=_DTYPES[train_cfg.get("expert_grad_dtype", "float32")],
        expert_state_dtype=_DTYPES[train_cfg.get("expert_state_dtype", "float32")],
        gather=os.environ.get("B200MOE_FSDP_GATHER") or train_cfg.get("fsdp_gather", "step"))
    opt_cfg = train_cfg["optimizer"]
    optimizer = AdamW(wrapped.parameters(), lr=train_cfg["learning_rate"],
                      betas=(opt_cfg["beta1"], opt_cfg["beta2"]), weight_decay=opt_cfg["lambda"])
    wrapped.activation_budget = None
    if recompute == "auto" and device.type == "cuda" and "batch_size" in train_cfg and "microbatch_num" in train_cfg:
        from .parallel.memory import stage_activation_budget
        optimizer.materialize_state()
        fsdp, ddp = parallel_sizes(train_cfg)
        local_batch = train_cfg["batch_size"] // (fsdp * ddp)
        tokens = local_batch // train_cfg["microbatch_num"] * model_cfg["context_len"]
        budget = stage_activation_budget(
            tokens_per_microbatch=tokens, d_model=model_cfg["d_model"], d_ff=model_cfg["d_ff"],
            num_heads=model_cfg["num_head"], experts_total=model_cfg["num_expert_per_node"] * fsdp, ep=fsdp,
            blocks=len(model.layers), pp=mesh.pp, stage=mesh.stage, microbatches=train_cfg["microbatch_num"],
            vocab=data_cfg["vocab_size"], device=device,
            margin_bytes=int(float(train_cfg.get("activation_margin_gib", 6.0)) * 2 ** 30),
            # with the exchange fused into the expert GEMMs a call keeps no routing-dependent tensor but gate/up
            routed_row_bytes=0 if (comm is not None and fsdp > 1) else None)
        for layer in model.layers:
            layer.ffn.budget = budget
        wrapped.activation_budget = budget
    return wrapped, optimizer


def train(local_rank: int, cluster_rank: int, world_size: int, config: dict):
    rank = int(os.environ["RANK"])
    general, train_cfg, model_cfg, data_cfg = (config[k] for k in ("general", "train", "model", "data"))
    parallel_rank_groups(train_cfg, world_size, general["gpu_per_node"])
    fsdp_size, ddp_size = parallel_sizes(train_cfg)
    width = fsdp_size * ddp_size
    batch_size, microbatch_num = train_cfg["batch_size"], train_cfg["microbatch_num"]
    if microbatch_num < 1 or batch_size < 1 or batch_size % (width * microbatch_num):
        raise ValueError("batch_size must be positive and divisible by FSDP * DDP * microbatch_num")
    if rank % general["gpu_per_node"] != local_rank:
        raise ValueError("Node-local topology requires contiguous torchrun ranks per node")
    device = resolve_device(config, local_rank)
    timeout = timedelta(seconds=config.get("recovery", {}).get("collective_timeout_seconds", 180))
    if device.type == "cuda":
        init_process_group("nccl", rank, world_size, timeout, device)
        torch.backends.cuda.matmul.allow_tf32 = True
        torch.backends.cudnn.allow_tf32 = True
    else:
        init_process_group("gloo", rank, world_size, timeout)
    compute_dtype = torch.bfloat16 if device.type == "cuda" else torch.float32

    mesh = build_groups(train_cfg, rank, world_size, general["gpu_per_node"], timeout=timeout)
    fsdp_group, ddp_group = mesh.group("fsdp"), mesh.group("ddp")
    data_group, pp_group = mesh.group("data"), mesh.group("pp")
    stage, dp_idx = mesh.stage, mesh.dp_idx
    info_src = general["info_src"]
    resume_dir = ckpt.select_checkpoint(config, rank, info_src)

    comm = None
    comm_cfg = config.get("comm") or {}
    recovery = config.get("recovery", {}) or {}
    if device.type == "cuda" and comm_cfg.get("backend", "fused") == "fused":
        from .comm import make_comm
        # comm.multicast (default off): bind the symmetric buffers to an NVSwitch multicast address, which the NVLS
        # all-reduce needs.  A process must not die while bound, so self-kill fault injection is refused with it.
        # comm.pipeline_link: "peer" (landing rings in peer memory, comm/pp.py) or "nccl" (batched send/recv)
        comm = make_comm(mesh, device, multicast=bool(comm_cfg.get("multicast", False)),
                         wait_seconds=float(recovery.get("device_wait_seconds", 20.0)),
                         pipeline_link=comm_cfg.get("pipeline_link"),
                         pipeline_wait_seconds=float(recovery.get("pipeline_wait_seconds", 120.0)))
    model, optimizer = build_model(config, mesh, device, fsdp_group, ddp_group, compute_dtype, comm)

    run_id = datetime.now().strftime("%Y%m%d%H%M%S%f")
    iteration = 0
    data_rng = np.random.default_rng(data_cfg.get("seed", 42) + dp_idx)
    if resume_dir:
        run_id = Path(resume_dir).parent.name
        iteration = ckpt.load_checkpoint_async_dist(
            os.path.join(resume_dir, ckpt.shard_name(dp_idx, stage)), model, optimizer, data_rng=data_rng)
        if iteration != int(Path(resume_dir).name):
            raise ValueError("Checkpoint shard iteration does not match committed directory")
        print(f"loaded checkpoint at {iteration} iterations, training start time is {run_id}")
    holder = [run_id]
    dist.broadcast_object_list(holder, src=info_src)
    run_id = holder[0]

    sched = train_cfg["learning_rate_scheduler"]
    lr_at = learning_rate_schedule_wrapper(sched["a_max"], sched["a_min"], sched["t_w"], sched["t_c"])
    dist.barrier()
    mock = data_cfg.get("mock_data", False)
    dataset = None if mock else load_dataset(data_cfg["train_dataset_path"], vocab_size=data_cfg["vocab_size"],
                                             validate=data_cfg.get("validate_dataset", False))
    if rank == info_src:
        print(f"training start time {run_id}", flush=True)
    local_batch = batch_size // width
    print(f"Rank {rank} Ready, FSDP={fsdp_size}, DDP={ddp_size}, batch size {batch_size}, "
          f"local batch size {local_batch}", flush=True)

    profile = config.get("profile", {}) or {}
    profiling = profile.get("enabled", False)
    if profiling and int(profile.get("nsight_iterations", 3)) < 1:
        raise ValueError("profile.nsight_iterations must be at least 1")
    target = train_cfg["target_iteration"]
    if profiling:
        target = min(target, int(profile.get("nsight_warmup", 5)) + int(profile.get("nsight_iterations", 3)))
    print_every, save_every = train_cfg["print_loss_interval"], train_cfg["save_interval"]
    ctx_len, d_model, vocab = model_cfg["context_len"], model_cfg["d_model"], data_cfg["vocab_size"]
    aux_coef = train_cfg.get("router_aux_loss_coef", 0.0) if train_cfg.get("use_router_aux_loss", False) else 0.0
    chaos = ChaosEnginnerTrigger(
        config.get("chaos_engineering") if (config.get("chaos_engineering") or {}).get("wired", True) else None,
        multicast_bound=(comm.any_multicast if comm is not None else None))
    sink = MetricsSink(general.get("metrics_path")) if rank == info_src else None
    flops_tok = flops_per_token(d_model, model_cfg["d_ff"], model_cfg["num_head"],
                                model_cfg["num_expert_per_node"] * fsdp_size, vocab,
                                model_cfg["num_layers"] * mesh.pp, ctx_len)
    timer = DeviceStepTimer(device)
    watchdog = None
    if device.type == "cuda":
        from .ops import native as _native
        if _native.has("gemm"):
            from .utils.watchdog import StatusWatchdog, device_status_reader
            watchdog = StatusWatchdog(device_status_reader(device),
                                      interval_s=float(recovery.get("status_poll_seconds", 1.0)),
                                      grace_s=float(recovery.get("status_grace_seconds", 30.0)),
                                      before_exit=(comm.release if comm is not None else None)).start()
            _native.set_nvtx(bool(profiling))
    pp_ranks = dist.get_process_group_ranks(pp_group)
    loss_acc, span_s, span_dev_ms, span_tokens = 0.0, 0.0, 0.0, 0
    pending: list = []

    def device_healthy() -> bool:
        """No kernel of this rank gave up a bounded wait (synchronising read of the status word)."""
        if watchdog is None:
            return True
        from .ops import native
        return watchdog.code == 0 and int(native.status_word(device).item()) == 0

    try:
        while iteration < target:
            if watchdog is not None:
                watchdog.raise_if_failed()
            with nvtx_range(f"train_iteration_{iteration}|rank={rank}|pp={stage}|dp={dp_idx}"):
                x = y = None
                with nvtx_range("batch_preparation"):
                    if rank in (pp_ranks[0], pp_ranks[-1]):
                        x, y = get_batch(dataset, local_batch, ctx_len, device, rng=data_rng, vocab_size=vocab,
                                         validate=data_cfg.get("validate_batches", False), mock_data=mock)
                with nvtx_range("learning_rate_update"):
                    lr = lr_at(iteration)
                    for group in optimizer.param_groups:
                        group["lr"] = lr
                if profiling:
                    with nvtx_range("pre_step_synchronization"):
                        if device.type == "cuda":
                            torch.cuda.synchronize()
                        dist.barrier()
                t0 = time.perf_counter()
                timer.start()
                with nvtx_range("pipeline_step|forward_backward_p2p_dp_sync_optimizer"):
                    loss = pipelined_train_overlap(
                        model, optimizer, x, y, [local_batch, ctx_len, d_model], microbatch_num, stage,
                        cross_entropy, dtype=compute_dtype, device=device, pp_group=pp_group, dp_group=data_group,
                        router_aux_loss_coef=aux_coef)
                reporting = (iteration + 1) % print_every == 0
                if profiling or reporting:
                    with nvtx_range("post_step_synchronization"):
                        span_dev_ms += timer.stop_ms()
                    if device.type == "cuda":
                        from .ops import native
                        if native.has("gemm"):
                            native.check_status()
                span_s += time.perf_counter() - t0
                loss_acc = loss_acc + loss
                span_tokens += batch_size * ctx_len
                iteration += 1
                if reporting:
                    if rank == info_src:
                        print(f"Rank {rank} finishes iteration {iteration}", flush=True)
                        rate = span_tokens / span_s
                        print(f"Iterations {iteration - print_every + 1}-{iteration}: processed {span_tokens:,} "
                              f"tokens in {span_s:.6f} seconds ({rate:,.2f} tokens/s)", flush=True)
                        if sink is not None:
                            sink.write(iteration=iteration, tokens=span_tokens, host_seconds=span_s,
                                       device_ms_last_step=span_dev_ms, tokens_per_s=rate,
                                       mfu=mfu(rate, flops_tok, world_size))
                    if rank == pp_ranks[-1]:
                        print(f"Rank {rank} Loss from last {print_every} iterations is {loss_acc / print_every}",
                              flush=True)
                        loss_acc = 0.0
                    span_s, span_dev_ms, span_tokens = 0.0, 0.0, 0
                ckpt.verify_pending_checkpoints(pending, iteration, rank, info_src, device, healthy=device_healthy)
                if iteration % save_every == 0:
                    with nvtx_range("checkpoint_io"):
                        directory = f"{general['checkpoint_folder']}/checkpoint/{run_id}/{iteration}"
                        try:
                            if not device_healthy():      # never stage a state that a failed wait may have damaged
                                raise RuntimeError("a device-side wait ran out before this checkpoint")
                            os.makedirs(directory, exist_ok=True)
                            future = ckpt.save_checkpoint_async_dist(
                                model, optimizer, iteration, os.path.join(directory, ckpt.shard_name(dp_idx, stage)),
                                data_rng=data_rng)
                        except Exception as error:
                            future = Future()
                            future.set_exception(error)
                        pending.append((iteration, directory, future))
                if len(chaos):
                    chaos.trigger(iteration)
    except BaseException:
        # leaving on an error path: stop the watchdog and let go of the peer-mapped buffers first, with no
        # kernel of this rank in flight, so that the peers never see a mapping vanish under a running kernel
        if watchdog is not None:
            watchdog.stop()
        if comm is not None:
            comm.release()
        raise
    ckpt.verify_pending_checkpoints(pending, iteration, rank, info_src, device, drain=True, healthy=device_healthy)
    release_leaks()
    if watchdog is not None:
        watchdog.stop()
        watchdog.raise_if_failed()
    return iteration


def main(argv=None):
    default = Path(__file__).resolve().parent.parent / "configs" / "run_config.yaml"
    parser = argparse.ArgumentParser(description="Pipeline training/profile worker entrypoint (run under torchrun)")
    parser.add_argument("--config-path", default=str(default))
    args = parser.parse_args(argv)
    with open(args.config_path, encoding="utf-8") as handle:
        config = yaml.safe_load(handle)
    needed = ("LOCAL_RANK", "RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK")
    if any(key not in os.environ for key in needed):
        parser.error("this worker entrypoint must be launched by torchrun")
    world_size = int(os.environ["WORLD_SIZE"])
    if world_size != config["general"]["n_workers"]:
        raise ValueError("torchrun WORLD_SIZE does not match general.n_workers")
    if int(os.environ["LOCAL_WORLD_SIZE"]) != config["general"]["gpu_per_node"]:
        raise ValueError("torchrun LOCAL_WORLD_SIZE does not match general.gpu_per_node")
    try:
        train(int(os.environ["LOCAL_RANK"]), int(os.environ["GROUP_RANK"]), world_size, config)
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
