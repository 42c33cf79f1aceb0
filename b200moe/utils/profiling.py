"""NVTX ranges, device-side step timing and the module microbenchmark.

``profile_callable`` follows the reference tool (run_experiment.py:38-98): warm
up, time each call with CUDA events, report latency statistics and allocator
peaks.  ``DeviceStepTimer`` times a region with CUDA events on the launching
stream and reduces the result as the maximum over ranks.
"""
from __future__ import annotations

import statistics
from contextlib import nullcontext

import torch

__all__ = ["nvtx_range", "cuda_device", "profile_callable", "make_module_step", "DeviceStepTimer"]


def nvtx_range(name: str):
    return torch.cuda.nvtx.range(name) if torch.cuda.is_available() else nullcontext()


def cuda_device(device="cuda:0") -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise ValueError("Profiling requires an NVIDIA CUDA device, not CPU.")
    if torch.version.cuda is None or not torch.cuda.is_available():
        raise RuntimeError("An NVIDIA GPU and CUDA-enabled PyTorch are required.")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    if device.index >= torch.cuda.device_count():
        raise ValueError(f"CUDA device index {device.index} is not available.")
    return device


def profile_callable(step, *, device="cuda:0", warmup: int = 10, iterations: int = 100) -> dict:
    if not callable(step):
        raise TypeError("step must be callable")
    if type(warmup) is not int or warmup < 0:
        raise ValueError("warmup must be nonnegative integer")
    if type(iterations) is not int or iterations < 1:
        raise ValueError("iterations must be a positive integer")
    device = cuda_device(device)
    mib = float(1 << 20)
    with torch.cuda.device(device):
        for _ in range(warmup):
            step()
        torch.cuda.synchronize(device)
        begin, end = (torch.cuda.Event(enable_timing=True) for _ in range(2))
        begin.record(); end.record(); end.synchronize()
        base_alloc = torch.cuda.memory_allocated(device)
        base_reserved = torch.cuda.memory_reserved(device)
        torch.cuda.reset_peak_memory_stats(device)
        samples = []
        for _ in range(iterations):
            begin.record()
            result = step()
            end.record()
            end.synchronize()
            samples.append(begin.elapsed_time(end))
            del result
        torch.cuda.synchronize(device)
        peak = torch.cuda.max_memory_allocated(device)
        return {
            "device": str(device),
            "gpu": torch.cuda.get_device_name(device),
            "iterations": iterations,
            "warmup_iterations": warmup,
            "time_ms": {"mean": statistics.mean(samples), "median": statistics.median(samples),
                        "stddev": statistics.pstdev(samples), "min": min(samples),
                        "max": max(samples), "total": sum(samples)},
            "memory_mib": {"baseline_allocated": base_alloc / mib, "peak_allocated": peak / mib,
                           "peak_above_baseline": (peak - base_alloc) / mib,
                           "baseline_reserved": base_reserved / mib,
                           "peak_reserved": torch.cuda.max_memory_reserved(device) / mib},
        }


def make_module_step(module, inputs, mode: str, loss_fn=None):
    """A closure that runs forward (+ backward in ``training`` mode) and clears
    gradients afterwards; no optimizer step (reference run_experiment.py:127-166)."""
    if mode not in ("training", "evaluation"):
        raise ValueError("mode must be training or evaluation")
    training = mode == "training"
    module.train(training)
    leaves = [t for t in inputs if isinstance(t, torch.Tensor) and t.is_leaf]
    for tensor in leaves:
        if tensor.is_floating_point():
            tensor.requires_grad_(training)

    def clear():
        module.zero_grad(set_to_none=True)
        for tensor in leaves:
            tensor.grad = None

    clear()

    def step():
        if not training:
            with torch.no_grad():
                return module(*inputs)
        with torch.enable_grad():
            try:
                output = module(*inputs)
                loss = loss_fn(output) if loss_fn is not None else output.float().mean()
                loss.backward()
                return loss.detach()
            finally:
                clear()

    return step


class DeviceStepTimer:
    """Device-side timing of a region, reduced as max over the ranks of a group.  ``clock="event"`` uses CUDA
    events; ``clock="globaltimer"`` brackets the region with two one-thread kernels of this framework that store
    the GPU's nanosecond ``globaltimer`` (same span, readable by other kernels and comparable across streams)."""

    def __init__(self, device, group=None, clock: str = "event"):
        self.device = torch.device(device)
        self.group = group
        self.cuda = self.device.type == "cuda"
        self.clock = clock if self.cuda else "host"
        if self.cuda:
            self._begin = torch.cuda.Event(enable_timing=True)
            self._end = torch.cuda.Event(enable_timing=True)
        if self.clock == "globaltimer":
            self._stamps = torch.zeros(2, dtype=torch.int64, device=self.device)
        self._t0 = 0.0

    def start(self) -> None:
        import time
        if self.clock == "globaltimer":
            from ..ops import native
            native.device_timestamp(self._stamps, 0)
        elif self.cuda:
            self._begin.record()
        else:
            self._t0 = time.perf_counter()

    def stop_ms(self) -> float:
        import time
        import torch.distributed as dist
        if self.clock == "globaltimer":
            from ..ops import native
            native.device_timestamp(self._stamps, 1)
            begin, end = self._stamps.tolist()      # synchronises with the stream
            elapsed = (end - begin) / 1e6
        elif self.cuda:
            self._end.record()
            self._end.synchronize()
            elapsed = self._begin.elapsed_time(self._end)
        else:
            elapsed = (time.perf_counter() - self._t0) * 1e3
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            value = torch.tensor([elapsed], dtype=torch.float64, device=self.device)
            dist.all_reduce(value, op=dist.ReduceOp.MAX, group=self.group)
            elapsed = float(value.item())
        return elapsed
