"""Run configuration: loading, validation and the startup command line.

The schema is the ``run_config.yaml`` of the reference (sections ``general``,
``recovery``, ``data``, ``model``, ``train``, ``profile``, ``experiment``,
``chaos_engineering``; reference implementation/startup.py:14-101 and
distributed_parallel_training_pipelined.py:104-131).  Keys this framework adds
are optional and default to the reference's behaviour:

``model.rope_theta``            RoPE base, default 10000 (reference layers.py:383)
``train.activation_recompute``  ``none`` | ``swiglu`` | ``block`` | ``auto`` (keep gate/up while HBM has room)
``train.router_aux_loss_coef``  passed to the pipeline step (reference validates
                                it in startup.py:57 but never forwards it)
``train.expert_state_dtype``    ``float32`` | ``bfloat16`` AdamW m/v of experts
``train.expert_grad_dtype``     ``float32`` | ``bfloat16`` expert grad accumulators
``comm.backend``                ``fused`` (peer-memory kernels) | ``nccl``
``comm.pipeline_link``          ``peer``: a stage stores its activations and gradients into landing rings of
                                its neighbour (no rendezvous of the two stages) | ``nccl``: batched send/recv
``recovery.pipeline_wait_seconds``  budget of a stage's wait for its neighbour inside the peer link (default 120)
``train.fsdp_gather``           ``step``: the end-of-step kernel pushes every new weight to the peers;
                                ``first_use``: the attention projections are gathered by the first GEMM
                                that uses them (all-gather and GEMM in one kernel)
``recovery.status_poll_seconds``, ``recovery.status_grace_seconds``
                                watchdog on the kernels' status word: poll period (default 1) and how long
                                the training thread may take to react before the process exits for a
                                group restart (default 30)
``general.device``              ``gpu`` or ``cpu`` (cpu runs the gloo plumbing tier)
"""
from __future__ import annotations

import argparse
import math
from pathlib import Path

import numpy as np
import yaml

from .topology import parallel_rank_groups, parallel_sizes

__all__ = [
    "load_config", "validate_config", "validate_router_aux_loss_coef",
    "parallel_sizes", "parallel_rank_groups", "generate_dataset", "main",
]

_PATH_KEYS = (("data", "train_dataset_path"), ("general", "checkpoint_folder"),
              ("train", "load_checkpoint_path"))
_POSITIVE_INTS = {
    "general": ("n_workers", "gpu_per_node"),
    "train": ("data_parallel_num", "pipeline_parallel_stages", "microbatch_num", "batch_size",
              "save_interval", "print_loss_interval", "target_iteration"),
    "model": ("num_head", "d_model", "d_ff", "context_len", "num_layers", "num_expert_per_node"),
    "data": ("vocab_size",),
}


def validate_router_aux_loss_coef(value) -> None:
    """Finite, non-negative real and not a bool (reference startup.py:9-11)."""
    ok = isinstance(value, (int, float)) and not isinstance(value, bool)
    if not ok or not math.isfinite(value) or value < 0:
        raise ValueError("router_aux_loss_coef must be finite and nonnegative")


def load_config(path) -> dict:
    """Load YAML and resolve relative paths against the config file's folder."""
    path = Path(path).resolve()
    with path.open(encoding="utf-8") as handle:
        config = yaml.safe_load(handle)
    for section, key in _PATH_KEYS:
        value = (config.get(section) or {}).get(key)
        if value and not Path(value).is_absolute():
            config[section][key] = str((path.parent / value).resolve())
    return config


def _require_positive_int(section: dict, key: str) -> None:
    if type(section.get(key)) is not int or section[key] < 1:
        raise ValueError(f"{key} must be a positive integer")


def validate_config(config: dict, *, check_data: bool = False, check_cuda: bool = False,
                    allow_cpu: bool = True) -> None:
    """Fail-fast checks of a run configuration (reference startup.py:55-101).

    Differences from the reference, all relaxations: ``general.device: cpu`` is
    accepted when ``allow_cpu`` (the gloo plumbing tier needs it) and the head
    dimension only has to be a multiple of 8 on CPU; on ``gpu`` the attention
    kernel's head-dim/ctx constraints are the reference's.
    """
    general, train, model, data = (config[k] for k in ("general", "train", "model", "data"))
    validate_router_aux_loss_coef(train.get("router_aux_loss_coef", 0.01))
    for name, keys in _POSITIVE_INTS.items():
        for key in keys:
            _require_positive_int(config[name], key)
    fsdp, ddp = parallel_sizes(train)
    width = fsdp * ddp
    if general["device"] not in (("gpu", "cpu") if allow_cpu else ("gpu",)):
        raise ValueError("Training requires CUDA/NCCL; general.device must be gpu")
    if general["n_workers"] != general["gpu_per_node"]:
        raise ValueError("The bundled launchers support one node only")
    parallel_rank_groups(train, general["n_workers"], general["gpu_per_node"])
    if train["batch_size"] % (width * train["microbatch_num"]):
        raise ValueError("batch_size must be divisible by FSDP * DDP * microbatch_num")
    if not 0 <= general["info_src"] < general["n_workers"]:
        raise ValueError("info_src must identify a worker")
    if model["d_model"] % model["num_head"]:
        raise ValueError("d_model must be divisible by num_head")
    if model["num_head"] % 4:
        raise ValueError("num_head must be divisible by 4 (4:1 grouped-query attention)")
    head_dim = model["d_model"] // model["num_head"]
    if head_dim < 16 or head_dim & (head_dim - 1):
        raise ValueError("attention requires a power-of-two head dimension >= 16")
    if model["context_len"] % 16:
        raise ValueError("Use context_len divisible by the attention tile size (16)")
    if model["num_expert_per_node"] * fsdp < 2:
        raise ValueError("Top-2 MoE routing requires at least two experts")
    if any(v % fsdp for v in (data["vocab_size"], model["d_model"], model["d_ff"])):
        raise ValueError("vocab_size, d_model and d_ff must be divisible by fsdp_parallel_num")
    sched = train["learning_rate_scheduler"]
    if not 0 <= sched["t_w"] < sched["t_c"]:
        raise ValueError("Scheduler requires 0 <= t_w < t_c")
    if train.get("activation_recompute", "none") not in ("none", "swiglu", "block", "auto"):
        raise ValueError("train.activation_recompute must be none, swiglu, block or auto")
    for key in ("expert_state_dtype", "expert_grad_dtype"):
        if train.get(key, "float32") not in ("float32", "bfloat16"):
            raise ValueError(f"train.{key} must be float32 or bfloat16")
    if train.get("fsdp_gather", "step") not in ("step", "first_use"):
        raise ValueError("train.fsdp_gather must be step or first_use")
    if (config.get("comm") or {}).get("backend", "fused") not in ("fused", "nccl"):
        raise ValueError("comm.backend must be fused or nccl")
    if (config.get("comm") or {}).get("pipeline_link") not in (None, "peer", "nccl"):
        raise ValueError("comm.pipeline_link must be peer or nccl")
    if check_data:
        from .utils.data import load_dataset
        tokens = load_dataset(data["train_dataset_path"], vocab_size=data["vocab_size"], validate=True)
        if tokens.size <= model["context_len"]:
            raise ValueError("Dataset must contain more tokens than context_len")
    if check_cuda:
        import torch
        if not torch.distributed.is_nccl_available() or torch.cuda.device_count() < general["gpu_per_node"]:
            raise ValueError(f"Requires NCCL and {general['gpu_per_node']} visible CUDA GPUs")
        if not torch.cuda.is_bf16_supported():
            raise ValueError("MoE computation requires a BF16-capable GPU")


def generate_dataset(config: dict) -> Path:
    """Write ``max(4096, 4*ctx)`` random int32 tokens; refuses to overwrite
    (exclusive create, reference startup.py:112-120)."""
    output = Path(config["data"]["train_dataset_path"])
    output.parent.mkdir(parents=True, exist_ok=True)
    rng = np.random.default_rng(config["data"].get("seed", 42))
    count = max(4096, config["model"]["context_len"] * 4)
    tokens = rng.integers(0, config["data"]["vocab_size"], size=count, dtype=np.int32)
    with output.open("xb") as target:
        np.save(target, tokens)
    return output


def main(argv=None) -> int:
    """``python -m implementation.startup --config X [--generate-data] [--check-cuda]``"""
    parser = argparse.ArgumentParser(
        description="Validate configuration or generate synthetic smoke-test tokens")
    parser.add_argument("--config", required=True)
    parser.add_argument("--generate-data", action="store_true")
    parser.add_argument("--check-cuda", action="store_true")
    args = parser.parse_args(argv)
    config = load_config(args.config)
    validate_config(config)
    if args.generate_data:
        print(f"Created synthetic test tokens: {generate_dataset(config)}")
    validate_config(config, check_data=True, check_cuda=args.check_cuda)
    print("Startup checks passed")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
