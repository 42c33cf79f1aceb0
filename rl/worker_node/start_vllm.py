"""Launch a ``vllm serve`` process pinned to one GPU with NCCL weight transfer
enabled (reference rl/worker_node/start_vllm.py:18-55)."""
from __future__ import annotations

import json
import os
import subprocess


def build_command(model: str, port: int = 8000, dtype: str = "bfloat16", max_model_len: int | None = None,
                  extra: list[str] | None = None) -> list[str]:
    command = ["vllm", "serve", model, "--port", str(port), "--dtype", dtype,
               "--weight-transfer-config", json.dumps({"backend": "nccl"})]
    if max_model_len:
        command += ["--max-model-len", str(max_model_len)]
    return command + list(extra or [])


def start_server(model: str, gpu: int = 0, port: int = 8000, dtype: str = "bfloat16", max_model_len: int | None = None,
                 extra: list[str] | None = None, popen=subprocess.Popen):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES=str(gpu))
    return popen(build_command(model, port, dtype, max_model_len, extra), env=env)


if __name__ == "__main__":
    import argparse
    parser = argparse.ArgumentParser()
    parser.add_argument("--model", required=True)
    parser.add_argument("--gpu", type=int, default=0)
    parser.add_argument("--port", type=int, default=8000)
    args = parser.parse_args()
    raise SystemExit(start_server(args.model, args.gpu, args.port).wait())
