"""Launch a ``vllm serve`` process pinned to one GPU, with NCCL weight transfer enabled so that a trainer can push
new policy weights into it (reference rl/worker_node/start_vllm.py:8-62).

``kill_existing_vllm_server(port)`` first ends a server that a previous run left on the port.  It looks the
processes up one by one (``vllm serve`` with that ``--port`` on their command line, never this process or its
parents) and signals exactly those PIDs: SIGTERM, two seconds of grace, then SIGKILL for the ones still there.
"""
from __future__ import annotations

import json
import logging
import os
import signal
import subprocess
import time

logger = logging.getLogger(__name__)


def _command_lines():
    """``(pid, argv)`` of every process whose command line this user may read."""
    found = []
    for entry in os.listdir("/proc"):
        if not entry.isdigit():
            continue
        try:
            with open(f"/proc/{entry}/cmdline", "rb") as handle:
                argv = [part.decode(errors="replace") for part in handle.read().split(b"\0") if part]
        except OSError:
            continue
        if argv:
            found.append((int(entry), argv))
    return found


def _ancestors(pid: int) -> set:
    seen = set()
    while pid > 1 and pid not in seen:
        seen.add(pid)
        try:
            with open(f"/proc/{pid}/stat", encoding="utf-8", errors="replace") as handle:
                pid = int(handle.read().rsplit(")", 1)[1].split()[1])
        except (OSError, IndexError, ValueError):
            break
    return seen


def find_vllm_servers(port: int, processes=None) -> list[int]:
    """PIDs of ``vllm serve`` processes started with ``--port <port>``."""
    protected = _ancestors(os.getpid())
    pids = []
    for pid, argv in (_command_lines() if processes is None else processes):
        if pid in protected or "serve" not in argv:
            continue
        serve = argv.index("serve")
        if not any(os.path.basename(part) == "vllm" or part.endswith("vllm") for part in argv[:serve]):
            continue
        if any(a == "--port" and b == str(port) for a, b in zip(argv, argv[1:])) or f"--port={port}" in argv:
            pids.append(pid)
    return pids


def kill_existing_vllm_server(port: int, processes=None, send=os.kill, grace_s: float = 2.0, sleep=time.sleep) -> list:
    """End the ``vllm serve`` processes on ``port``; returns the PIDs it signalled."""
    pids = find_vllm_servers(port, processes)
    for pid in pids:
        try:
            send(pid, signal.SIGTERM)
        except ProcessLookupError:
            pass
    if pids:
        sleep(grace_s)
        for pid in find_vllm_servers(port, processes):
            if pid in pids:
                try:
                    send(pid, signal.SIGKILL)
                except ProcessLookupError:
                    pass
    return pids


def build_command(model_id: str, host: str = "localhost", port: int = 8000, seed: int = 0, load_format: str = "auto",
                  gpu_memory_utilization: float = 0.9, dtype: str = "bfloat16", max_model_len: int | None = None,
                  extra: list[str] | None = None) -> list[str]:
    """One engine per GPU (tensor-parallel size 1), prefix caching on, weights replaceable over NCCL."""
    command = ["vllm", "serve", model_id, "--host", host, "--port", str(port), "--dtype", dtype,
               "--enable-prefix-caching", "--gpu-memory-utilization", str(gpu_memory_utilization),
               "--seed", str(seed), "--tensor-parallel-size", "1",
               "--weight-transfer-config", json.dumps({"backend": "nccl"}), "--load-format", load_format]
    if max_model_len:
        command += ["--max-model-len", str(max_model_len)]
    return command + list(extra or [])


def start_server(model_id: str, host: str = "localhost", port: int = 8000, gpu: int = 0, seed: int = 0,
                 load_format: str = "auto", logging_level: str = "INFO", gpu_memory_utilization: float = 0.9,
                 max_model_len: int | None = None, extra: list[str] | None = None, popen=subprocess.Popen):
    """Start the server in its own session (signals to this process do not reach it) and return the process.
    ``VLLM_SERVER_DEV_MODE`` opens the endpoints that weight updates use."""
    env = dict(os.environ, CUDA_VISIBLE_DEVICES=str(gpu), VLLM_SERVER_DEV_MODE="1", VLLM_LOGGING_LEVEL=logging_level)
    command = build_command(model_id, host, port, seed, load_format, gpu_memory_utilization,
                            max_model_len=max_model_len, extra=extra)
    logger.info("starting vLLM server: %s", " ".join(command))
    return popen(command, env=env, start_new_session=True)


if __name__ == "__main__":
    import argparse
    parser = argparse.ArgumentParser()
    parser.add_argument("--model", default="allenai/OLMo-2-0425-1B")
    parser.add_argument("--host", default="localhost")
    parser.add_argument("--gpu", type=int, default=0)
    parser.add_argument("--port", type=int, default=8088)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--load-format", default="auto")
    parser.add_argument("--logging-level", default="INFO")
    args = parser.parse_args()
    kill_existing_vllm_server(args.port)
    process = start_server(args.model, args.host, args.port, args.gpu, args.seed, args.load_format, args.logging_level)
    print("return code:", process.wait())
