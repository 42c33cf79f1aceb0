"""Modal launcher: one container per node, eight B200s each, ``torchrun`` on the worker.

Same behaviour and entry-point names as the reference launcher
(modal_wrapper.py:52-156): volumes for datasets, checkpoints and profiles; a
cluster of ``n_workers / gpu_per_node`` containers that rendezvous on the first
container's address (loopback when there is one node: a sandboxed container
cannot reach its own cluster address); one ``NCCL_HOSTID`` per node; a torchrun
command with the restart budget of ``recovery.max_restarts``; and, with
``profile.enabled``, Nsight Systems around torchrun, whose report must exist
afterwards and is committed to the profile volume.

``modal`` is imported only when an app is built, so the command builders can be
used and tested without it.  Without Modal, ``python modal_wrapper.py CONFIG``
runs the same node launch on this machine.
"""
from __future__ import annotations

import contextlib
import json
import os
import shlex
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

import yaml

PROJECT_ROOT = Path(__file__).resolve().parent
APP_NAME = "b200moe-train"
GPU_SPEC = os.environ.get("B200MOE_MODAL_GPU", "B200:8")
NODES = int(os.environ.get("B200MOE_MODAL_NODES", "1"))      # containers of the clustered function
REMOTE_ROOT = "/workspace/b200moe"
VOLUMES = {"/mnt/dataset": "b200moe-datasets", "/mnt/checkpoints": "b200moe-checkpoints",
           "/mnt/profile-data": "b200moe-profiles"}
ENTRY_MODULE = "distributed_parallel_training_pipelined"


# ------------------------------------------------------------------------------------------ command builders
@contextlib.contextmanager
def _environment(**values):
    """Set (or, for ``None``, leave alone) environment variables for the length of a block."""
    saved = {key: os.environ.get(key) for key in values}
    os.environ.update({key: str(value) for key, value in values.items() if value is not None})
    try:
        yield
    finally:
        for key, value in saved.items():
            if value is None:
                os.environ.pop(key, None)
            else:
                os.environ[key] = value


def node_count(world_size: int, gpu_per_node: int) -> int:
    if world_size < 1 or gpu_per_node < 1 or world_size % gpu_per_node:
        raise ValueError("n_workers must be positive and divisible by gpu_per_node")
    return world_size // gpu_per_node


def _endpoint(host: str, port) -> str:
    """``host:port`` for the c10d rendezvous; a bare IPv6 address goes in brackets."""
    return f"[{host}]:{port}" if ":" in host and not host.startswith("[") else f"{host}:{port}"


def _build_torchrun_command(config_path, cluster_rank, world_size, gpu_per_node, max_restarts=3):
    """The reference's builder (modal_wrapper.py:102-130), same arguments: rendezvous address and port come from
    ``MASTER_ADDR`` / ``MASTER_PORT``, the rendezvous id from the cluster part of ``NCCL_HOSTID``."""
    if isinstance(max_restarts, bool) or not isinstance(max_restarts, int) or max_restarts < 0:
        raise ValueError("recovery.max_restarts must be a nonnegative integer")
    nodes = node_count(world_size, gpu_per_node)
    if not 0 <= cluster_rank < nodes:
        raise ValueError("node rank must be in [0, n_workers / gpu_per_node)")
    address = os.environ.get("MASTER_ADDR")
    if nodes > 1 and not address:
        raise ValueError("MASTER_ADDR must be set for multi-node training")
    address = address or "127.0.0.1"
    port = os.environ.get("MASTER_PORT", "29500")
    run_id = os.environ.get("NCCL_HOSTID", "b200moe").rsplit("-node-", 1)[0]
    launcher = [sys.executable, "-m", "torch.distributed.run"]
    layout = [f"--nnodes={nodes}", f"--nproc-per-node={gpu_per_node}", f"--node-rank={cluster_rank}"]
    rendezvous = [f"--master-addr={address}", f"--master-port={port}", f"--max-restarts={max_restarts}",
                  "--monitor-interval=1", "--rdzv-backend=c10d", f"--rdzv-endpoint={_endpoint(address, port)}",
                  f"--rdzv-id={run_id}"]
    return launcher + layout + rendezvous + ["--module", ENTRY_MODULE, "--config-path", str(config_path)]


def torchrun_command(config: dict, config_path: str, node_rank: int = 0, master_addr: str | None = None,
                     master_port: int | None = None, run_id: str | None = None) -> list[str]:
    """``_build_torchrun_command`` from a run configuration, with the rendezvous given as arguments."""
    general = config["general"]
    restarts = (config.get("recovery") or {}).get("max_restarts", 3)
    host_id = None if run_id is None else f"{run_id}-node-{node_rank}"
    with _environment(MASTER_ADDR=master_addr, MASTER_PORT=master_port, NCCL_HOSTID=host_id):
        return _build_torchrun_command(config_path, node_rank, general["n_workers"], general["gpu_per_node"], restarts)


def _build_nsys_command(nsys, output, training_command, profile_config):
    """Nsight Systems around the training command.  Software CUDA tracing by default (a sandboxed container has no
    access to the hardware tracer); no sampling, no context-switch trace; the profiler waits for every child and
    does not kill them, since torchrun's workers outlive the process it started with."""
    trace = (profile_config or {}).get("nsight_trace", "cuda-sw,nvtx")
    options = {"trace": trace, "trace-fork-before-exec": "false", "kill": "none", "cuda-event-trace": "false",
               "cuda-memory-usage": "false", "sample": "none", "cpuctxsw": "none", "wait": "all",
               "force-overwrite": "true", "output": output}
    return [nsys, "profile"] + [f"--{name}={value}" for name, value in options.items()] + list(training_command)


def nsys_prefix(config: dict, run_id: str) -> list[str]:
    """The profiler part alone (empty unless ``profile.enabled``)."""
    profile = config.get("profile") or {}
    if not profile.get("enabled", False):
        return []
    output = str(Path(profile.get("output_dir", "/mnt/profile-data")) / run_id)
    return _build_nsys_command("nsys", output, [], profile)


def nccl_environment(master_addr: str = "127.0.0.1", master_port: int = 29500, cluster_id: str = "b200moe",
                     node_rank: int = 0) -> dict:
    """Rendezvous and NCCL settings of one node: one host id per physical node (inherited by its workers), sockets
    instead of InfiniBand between containers, IPv6 sockets when the cluster address is IPv6."""
    env = {"MASTER_ADDR": master_addr, "MASTER_PORT": str(master_port),
           "NCCL_HOSTID": f"{cluster_id}-node-{node_rank}", "NCCL_IB_DISABLE": "1",
           "NCCL_DEBUG": os.environ.get("NCCL_DEBUG", "WARN")}
    if ":" in master_addr:
        env["NCCL_SOCKET_FAMILY"] = "AF_INET6"
    return env


# ------------------------------------------------------------------------------------------ one node
def run_node(config: dict, node_rank: int = 0, container_ips=None, cluster_id: str = "b200moe",
             runner=subprocess.run, commit_profile=None) -> list[str]:
    """Launch this node's workers and wait for them.  ``container_ips``: addresses of the cluster's containers
    (first one hosts the rendezvous); ``runner`` and ``commit_profile`` are injectable for tests.  Returns the
    command that ran."""
    general = config["general"]
    nodes = node_count(general["n_workers"], general["gpu_per_node"])
    # a single node meets itself on loopback; several nodes meet on the first container's address
    address = container_ips[0] if nodes > 1 and container_ips else "127.0.0.1"
    if nodes > 1 and not container_ips:
        raise ValueError("a multi-node launch needs the addresses of its containers")
    env = {**os.environ, **nccl_environment(address, 29500, cluster_id, node_rank)}
    profile = config.get("profile") or {}
    profiling = bool(profile.get("enabled", False))
    restarts = (config.get("recovery") or {}).get("max_restarts", 3)
    with tempfile.TemporaryDirectory(prefix="b200moe-launch-") as scratch:
        config_path = Path(scratch) / "config.json"
        config_path.write_text(json.dumps(config), encoding="utf-8")      # JSON is YAML: the worker's loader reads it
        with _environment(MASTER_ADDR=env["MASTER_ADDR"], MASTER_PORT=env["MASTER_PORT"],
                          NCCL_HOSTID=env["NCCL_HOSTID"]):
            command = _build_torchrun_command(config_path, node_rank, general["n_workers"], general["gpu_per_node"],
                                              restarts)
        report = None
        if profiling:
            nsys = shutil.which("nsys")
            if nsys is None:
                raise RuntimeError("profile.enabled needs Nsight Systems (`nsys`) in the training image; "
                                   "use an image that has it or switch profile.enabled off")
            out_dir = profile.get("output_dir", "/mnt/profile-data")
            os.makedirs(out_dir, exist_ok=True)
            output = os.path.join(out_dir, f"pipeline-node-{node_rank}")
            command = _build_nsys_command(nsys, output, command, profile)
            report = output + ".nsys-rep"
        print(f"launching {'under Nsight Systems' if profiling else 'training'}: "
              + " ".join(shlex.quote(str(c)) for c in command), flush=True)
        runner(command, check=True, env=env, cwd=str(PROJECT_ROOT))
        if report is not None:
            if not os.path.isfile(report):
                raise RuntimeError(f"Nsight Systems did not write {report}")
            if commit_profile is not None:
                commit_profile()
            print(f"Nsight report: {report}", flush=True)
    return command


def _read_config(config_path) -> dict:
    """The run configuration with its relative paths resolved against the file's folder: the workers read a copy
    written elsewhere."""
    try:
        from b200moe.config import load_config
        return load_config(config_path)
    except ImportError:
        with open(config_path, encoding="utf-8") as handle:
            return yaml.safe_load(handle)


def launch(config_path: str) -> int:
    """Without Modal: run the node launch for ``config_path`` on this machine."""
    config = _read_config(config_path)
    try:
        run_node(config)
    except subprocess.CalledProcessError as error:
        return error.returncode or 1
    return 0


# ------------------------------------------------------------------------------------------ the Modal app
def profile_wrapper(config):
    """Body of the remote function (the reference's ``profile_wrapper``): launch training on this node, under
    Nsight Systems when the configuration asks for it.  Inside a Modal cluster the node rank, the cluster id and
    the containers' addresses come from Modal; elsewhere it is a one-node launch."""
    rank, ips, cluster_id, commit = 0, None, "b200moe", None
    try:
        import modal
        info = modal.experimental.get_cluster_info()
        rank, ips, cluster_id = info.rank, list(info.container_ips), str(info.cluster_id)
        commit = modal.Volume.from_name(VOLUMES["/mnt/profile-data"], create_if_missing=True).commit
    except Exception:       # not inside a Modal cluster
        pass
    return run_node(config, rank, ips, cluster_id, commit_profile=commit)


def main(config_path: str = str(PROJECT_ROOT / "configs" / "run_config.yaml")):
    """Local entry point: read the run configuration here and hand it to the remote function (or, without Modal,
    run it on this machine)."""
    config = _read_config(config_path)
    remote = globals().get("_remote_profile_wrapper")
    if remote is not None:
        return remote.remote(config)
    return profile_wrapper(config)


def build_app():
    import modal
    image = (modal.Image.from_registry("nvidia/cuda:12.9.1-devel-ubuntu24.04", add_python="3.12")
             .pip_install("torch==2.11.0", "numpy", "pyyaml", "einops")
             .add_local_dir(str(PROJECT_ROOT), REMOTE_ROOT, copy=True)
             .run_commands(f"cd {REMOTE_ROOT} && python -m b200moe.build"))
    app = modal.App(APP_NAME, image=image)
    volumes = {path: modal.Volume.from_name(name, create_if_missing=True) for path, name in VOLUMES.items()}
    remote = modal.experimental.clustered(size=NODES)(profile_wrapper)
    remote = app.function(gpu=GPU_SPEC, volumes=volumes, scaledown_window=10, timeout=12 * 3600)(remote)
    globals()["_remote_profile_wrapper"] = remote
    app.local_entrypoint()(main)
    return app


if os.environ.get("MODAL_IS_REMOTE") or os.path.basename(sys.argv[0]) == "modal":
    app = build_app()

if __name__ == "__main__":
    raise SystemExit(launch(sys.argv[1] if len(sys.argv) > 1 else str(PROJECT_ROOT / "configs" / "run_config.yaml")))
