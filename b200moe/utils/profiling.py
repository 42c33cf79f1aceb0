"""NVTX ranges, device-side step timing and the module microbenchmark.

``profile_callable`` follows the reference tool (run_experiment.py:38-98): warm
up, time each call with CUDA events, report latency statistics and allocator
peaks.  ``DeviceStepTimer`` times a region with CUDA events on the launching
stream and reduces the result as the maximum over ranks.
"""
from __future__ import annotations

import math
import statistics
from contextlib import nullcontext

import torch

__all__ = ["nvtx_range", "cuda_device", "profile_callable", "make_module_step", "DeviceStepTimer"]


def nvtx_range(name: str):
    return torch.cuda.nvtx.range(name) if torch.cuda.is_available() else nullcontext()


def cuda_device(device="cuda:0") -> torch.device:
    """Resolve a device string to an existing CUDA device (with its index filled in) or say why not."""
    wanted = torch.device(device)
    problems = []
    if wanted.type != "cuda":
        problems.append(ValueError("Profiling requires an NVIDIA CUDA device, not CPU."))
    elif not (torch.version.cuda and torch.cuda.is_available()):
        problems.append(RuntimeError("An NVIDIA GPU and CUDA-enabled PyTorch are required."))
    if problems:
        raise problems[0]
    index = torch.cuda.current_device() if wanted.index is None else wanted.index
    if not 0 <= index < torch.cuda.device_count():
        raise ValueError(f"CUDA device index {index} is not available.")
    return torch.device("cuda", index)


class _LatencySeries:
    """Per-call device times of one closure, taken with a CUDA event pair around each call."""

    def __init__(self):
        self.ms: list[float] = []
        self._pair = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))

    def settle(self):
        """Record the pair once so that the events' own set-up never lands in a sample."""
        first, second = self._pair
        first.record()
        second.record()
        second.synchronize()

    def run(self, fn):
        first, second = self._pair
        first.record()
        out = fn()
        second.record()
        second.synchronize()
        self.ms.append(first.elapsed_time(second))
        return out

    def stats(self) -> dict:
        ms = self.ms
        return {"mean": statistics.fmean(ms), "median": statistics.median(ms), "stddev": statistics.pstdev(ms),
                "min": min(ms), "max": max(ms), "total": math.fsum(ms)}


def _require_count(name: str, value, least: int, message: str) -> None:
    if type(value) is not int or value < least:
        raise ValueError(message)


def profile_callable(step, *, device="cuda:0", warmup: int = 10, iterations: int = 100) -> dict:
    """Latency statistics (ms per call, CUDA events) and allocator peaks (MiB) of ``step()`` after ``warmup``
    untimed calls; the result has the keys of the reference tool (run_experiment.py:38-98)."""
    if not callable(step):
        raise TypeError("step must be callable")
    _require_count("warmup", warmup, 0, "warmup must be nonnegative integer")
    _require_count("iterations", iterations, 1, "iterations must be a positive integer")
    target = cuda_device(device)
    to_mib = 1.0 / (1 << 20)
    with torch.cuda.device(target):
        for _ in range(warmup):
            step()
        torch.cuda.synchronize(target)
        series = _LatencySeries()
        series.settle()
        floor = {"allocated": torch.cuda.memory_allocated(target), "reserved": torch.cuda.memory_reserved(target)}
        torch.cuda.reset_peak_memory_stats(target)
        for _ in range(iterations):
            series.run(step)         # the closure's result is dropped here, before the next call allocates
        torch.cuda.synchronize(target)
        top = {"allocated": torch.cuda.max_memory_allocated(target),
               "reserved": torch.cuda.max_memory_reserved(target)}
    memory = {"baseline_allocated": floor["allocated"] * to_mib, "peak_allocated": top["allocated"] * to_mib,
              "peak_above_baseline": (top["allocated"] - floor["allocated"]) * to_mib,
              "baseline_reserved": floor["reserved"] * to_mib, "peak_reserved": top["reserved"] * to_mib}
    return {"device": str(target), "gpu": torch.cuda.get_device_name(target), "iterations": iterations,
            "warmup_iterations": warmup, "time_ms": series.stats(), "memory_mib": memory}


class _ModuleStep:
    """Callable that runs a module forward (and backward when training) and leaves no gradient behind; there is
    no optimizer step (the contract of the reference's ``make_module_step``, run_experiment.py:127-166)."""

    def __init__(self, module, inputs, training: bool, loss_fn):
        self.module, self.inputs, self.training, self.loss_fn = module, inputs, training, loss_fn
        module.train(training)
        self.leaf_inputs = [t for t in inputs if isinstance(t, torch.Tensor) and t.is_leaf]
        for t in self.leaf_inputs:
            if t.is_floating_point():
                t.requires_grad_(training)
        self.drop_gradients()

    def drop_gradients(self):
        self.module.zero_grad(set_to_none=True)
        for t in self.leaf_inputs:
            t.grad = None

    def __call__(self):
        if not self.training:
            with torch.no_grad():
                return self.module(*self.inputs)
        try:
            with torch.enable_grad():
                out = self.module(*self.inputs)
                value = out.float().mean() if self.loss_fn is None else self.loss_fn(out)
                value.backward()
            return value.detach()
        finally:
            self.drop_gradients()


def make_module_step(module, inputs, mode: str, loss_fn=None):
    if mode not in ("training", "evaluation"):
        raise ValueError("mode must be training or evaluation")
    return _ModuleStep(module, inputs, mode == "training", loss_fn)


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
