"""Module microbenchmark driven by the ``experiment`` section of run_config.yaml.

``python run_experiment.py --config-path configs/run_config.yaml`` builds the
module returned by ``module_wrapper`` (by default three dense SwiGLU layers of
width 14336), warms it up, times every iteration with CUDA events and prints
latency statistics and allocator peaks as JSON.  Same contract as the
reference tool (run_experiment.py:38-210); the timed module runs this
framework's kernels, so there is no compile step.
"""
import argparse
import json
from pathlib import Path

import torch
import yaml

from b200moe.utils.profiling import cuda_device, make_module_step, profile_callable  # noqa: F401

ITERATIONS = 100
DEFAULT_CONFIG_PATH = Path(__file__).resolve().parent / "configs" / "run_config.yaml"


def load_experiment_config(path):
    with Path(path).open(encoding="utf-8") as source:
        config = yaml.safe_load(source)
    if not isinstance(config, dict) or not isinstance(config.get("experiment"), dict):
        raise ValueError("Configuration must contain an experiment section")
    experiment = config["experiment"]
    for key, minimum in (("warmup", 0), ("iterations", 1)):
        value = experiment.get(key)
        if type(value) is not int or value < minimum:
            raise ValueError(f"experiment.{key} must be an integer >= {minimum}")
    if experiment.get("dtype") not in ("float32", "float16", "bfloat16"):
        raise ValueError("experiment.dtype must be float32, float16, or bfloat16")
    if not isinstance(experiment.get("device"), str):
        raise ValueError("experiment.device must be a CUDA device string")
    if experiment.get("mode") not in ("training", "evaluation"):
        raise ValueError("experiment.mode must be training or evaluation")
    shapes = experiment.get("input_shapes")
    good = isinstance(shapes, list) and shapes and all(
        isinstance(shape, list) and shape and all(type(d) is int and d > 0 for d in shape) for shape in shapes)
    if not good:
        raise ValueError("experiment.input_shapes must be a list of positive integer shapes")
    return config


def module_wrapper(config, device, dtype):
    """Edit this function to profile another module: build the module and its
    inputs here (setup is outside the timed region) and return a step closure."""
    from b200moe.models import ModuleStack
    inputs = [torch.randn(*shape, device=device, dtype=dtype) for shape in config["experiment"]["input_shapes"]]
    if len(inputs) != 1:
        raise ValueError("The ModuleStack wrapper requires exactly one input shape")
    module = ModuleStack(inputs[0].shape[-1], inputs[0].shape[-1], device=device, dtype=dtype)
    return make_module_step(module, inputs, config["experiment"]["mode"])


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--config-path", type=Path, default=DEFAULT_CONFIG_PATH)
    args = parser.parse_args(argv)
    config = load_experiment_config(args.config_path)
    experiment = config["experiment"]
    device = cuda_device(experiment["device"])
    dtype = getattr(torch, experiment["dtype"])
    with torch.cuda.device(device):
        step = module_wrapper(config, device, dtype)
        result = profile_callable(step, device=device, warmup=experiment["warmup"],
                                  iterations=experiment["iterations"])
    result["mode"] = experiment["mode"]
    result["config_path"] = str(Path(args.config_path).resolve())
    result["experiment"] = experiment
    print(json.dumps(result, indent=2))
    return result


if __name__ == "__main__":
    main()
