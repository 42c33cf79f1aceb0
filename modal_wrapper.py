"""Modal launcher: one container with 8 GPUs running torchrun on the worker.

Mirrors the reference launcher's behaviour (modal_wrapper.py:54-156): volumes
for datasets, checkpoints and profiles, rendezvous and NCCL environment, a
torchrun command with a restart budget from ``recovery.max_restarts``, and an
optional Nsight Systems wrapper driven by the ``profile`` section.  ``modal`` is
imported lazily so the command builders can be used and tested without it.
"""
from __future__ import annotations

import os
import shlex
import subprocess
import sys
from pathlib import Path

import yaml

APP_NAME = "b200moe-train"
GPU_SPEC = os.environ.get("B200MOE_MODAL_GPU", "B200:8")
REMOTE_ROOT = "/workspace/b200moe"
VOLUMES = {"/mnt/dataset": "b200moe-datasets", "/mnt/checkpoints": "b200moe-checkpoints",
           "/mnt/profile-data": "b200moe-profiles"}


def nccl_environment(master_addr: str = "127.0.0.1", master_port: int = 29500) -> dict:
    return {"MASTER_ADDR": master_addr, "MASTER_PORT": str(master_port), "NCCL_HOSTID": "b200moe-node-0",
            "NCCL_IB_DISABLE": "1", "NCCL_DEBUG": os.environ.get("NCCL_DEBUG", "WARN")}


def torchrun_command(config: dict, config_path: str, node_rank: int = 0, master_addr: str = "127.0.0.1",
                     master_port: int = 29500, run_id: str = "b200moe") -> list[str]:
    general = config["general"]
    per_node = general["gpu_per_node"]
    nodes = max(1, general["n_workers"] // per_node)
    restarts = int((config.get("recovery") or {}).get("max_restarts", 0))
    return [sys.executable, "-m", "torch.distributed.run", f"--nnodes={nodes}", f"--nproc-per-node={per_node}",
            f"--node-rank={node_rank}", f"--master-addr={master_addr}", f"--master-port={master_port}",
            f"--max-restarts={restarts}", "--monitor-interval=1", "--rdzv-backend=c10d",
            f"--rdzv-endpoint={master_addr}:{master_port}", f"--rdzv-id={run_id}",
            "--module", "distributed_parallel_training_pipelined", "--config-path", config_path]


def nsys_prefix(config: dict, run_id: str) -> list[str]:
    profile = config.get("profile") or {}
    if not profile.get("enabled", False):
        return []
    out_dir = profile.get("output_dir", "/mnt/profile-data")
    trace = profile.get("nsight_trace", "cuda-sw,nvtx,nccl")
    return ["nsys", "profile", f"--trace={trace}", "--sample=none", "--cpuctxsw=none", "--wait=all",
            "--force-overwrite=true", "-o", str(Path(out_dir) / f"{run_id}")]


def launch(config_path: str) -> int:
    with open(config_path, encoding="utf-8") as handle:
        config = yaml.safe_load(handle)
    env = {**os.environ, **nccl_environment()}
    command = nsys_prefix(config, "b200moe") + torchrun_command(config, config_path)
    print("launching:", " ".join(shlex.quote(c) for c in command), flush=True)
    return subprocess.call(command, env=env, cwd=str(Path(__file__).resolve().parent))


def build_app():
    import modal
    image = (modal.Image.from_registry("nvidia/cuda:12.9.1-devel-ubuntu24.04", add_python="3.12")
             .pip_install("torch==2.11.0", "numpy", "pyyaml", "einops")
             .add_local_dir(str(Path(__file__).resolve().parent), REMOTE_ROOT, copy=True)
             .run_commands(f"cd {REMOTE_ROOT} && python -m b200moe.build"))
    app = modal.App(APP_NAME, image=image)
    volumes = {path: modal.Volume.from_name(name, create_if_missing=True) for path, name in VOLUMES.items()}

    @app.function(gpu=GPU_SPEC, volumes=volumes, timeout=24 * 3600)
    def train(config_path: str = f"{REMOTE_ROOT}/configs/run_config.yaml"):
        os.chdir(REMOTE_ROOT)
        code = launch(config_path)
        for volume in volumes.values():
            volume.commit()
        if code:
            raise RuntimeError(f"training exited with code {code}")

    @app.local_entrypoint()
    def main(config_path: str = f"{REMOTE_ROOT}/configs/run_config.yaml"):
        train.remote(config_path)

    return app


if os.environ.get("MODAL_IS_REMOTE") or os.path.basename(sys.argv[0]) == "modal":
    app = build_app()

if __name__ == "__main__":
    raise SystemExit(launch(sys.argv[1] if len(sys.argv) > 1 else str(Path(__file__).parent / "configs" / "run_config.yaml")))
