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


def _is_shape_list(value) -> bool:
    def is_shape(shape):
        return isinstance(shape, list) and len(shape) > 0 and all(type(d) is int and d > 0 for d in shape)
    return isinstance(value, list) and len(value) > 0 and all(is_shape(shape) for shape in value)


# one rule per key of the ``experiment`` section: (key, predicate, message)
_EXPERIMENT_RULES = (
    ("warmup", lambda v: type(v) is int and v >= 0, "experiment.warmup must be an integer >= 0"),
    ("iterations", lambda v: type(v) is int and v >= 1, "experiment.iterations must be an integer >= 1"),
    ("dtype", lambda v: v in ("float32", "float16", "bfloat16"),
     "experiment.dtype must be float32, float16, or bfloat16"),
    ("device", lambda v: isinstance(v, str), "experiment.device must be a CUDA device string"),
    ("mode", lambda v: v in ("training", "evaluation"), "experiment.mode must be training or evaluation"),
    ("input_shapes", _is_shape_list, "experiment.input_shapes must be a list of positive integer shapes"),
)


def load_experiment_config(path):
    """Read the YAML file and check its ``experiment`` section rule by rule (the keys and verdicts of the
    reference tool, run_experiment.py:101-124)."""
    config = yaml.safe_load(Path(path).read_text(encoding="utf-8"))
    section = config.get("experiment") if isinstance(config, dict) else None
    if not isinstance(section, dict):
        raise ValueError("Configuration must contain an experiment section")
    for key, accepts, message in _EXPERIMENT_RULES:
        if not accepts(section.get(key)):
            raise ValueError(message)
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


def run(config_path) -> dict:
    """Profile the module of ``module_wrapper`` as the ``experiment`` section of ``config_path`` says."""
    config = load_experiment_config(config_path)
    section = config["experiment"]
    device = cuda_device(section["device"])
    with torch.cuda.device(device):
        step = module_wrapper(config, device, getattr(torch, section["dtype"]))
        report = profile_callable(step, device=device, warmup=section["warmup"], iterations=section["iterations"])
    report.update(mode=section["mode"], config_path=str(Path(config_path).resolve()), experiment=section)
    return report


def main(argv=None):
    cli = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    cli.add_argument("--config-path", type=Path, default=DEFAULT_CONFIG_PATH)
    report = run(cli.parse_args(argv).config_path)
    print(json.dumps(report, indent=2))
    return report


if __name__ == "__main__":
    main()
