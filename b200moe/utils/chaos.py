"""Fault injection on the host side.

The four perturbations of the reference (implementation/chaos_engineer.py:16-81):
a random sleep, a self-SIGKILL, a device-memory leak and a CPU hog.  All of them
act on the host process; none makes a GPU fault, trap or hang.  Unlike the
reference, the trainer calls ``ChaosEnginnerTrigger.trigger()`` once per
iteration (between steps, with no kernel of this rank in flight for the kill),
the leak is capped (``max_total_mb``) and ``release_leaks()`` frees it.
"""
from __future__ import annotations

import logging
import multiprocessing
import os
import random
import signal
import time

import torch

logger = logging.getLogger(__name__)

_leaked: list = []
_leaked_mb = 0


def random_delay(delay_time: float = 5, chance: float = 0.01) -> bool:
    if random.random() >= chance:
        return False
    logger.info("[chaos] random_delay: sleeping %ss", delay_time)
    time.sleep(delay_time)
    return True


def random_kill(chance: float = 0.001) -> bool:
    if random.random() >= chance:
        return False
    logger.warning("[chaos] random_kill: SIGKILL to pid %d", os.getpid())
    if torch.cuda.is_available():
        torch.cuda.synchronize()  # leave no kernel or collective of this rank in flight
    os.kill(os.getpid(), signal.SIGKILL)
    return True


def random_gpu_memory_leak(size_mb: int = 512, chance: float = 0.01, max_total_mb: int = 8192) -> bool:
    global _leaked_mb
    if random.random() >= chance or _leaked_mb + size_mb > max_total_mb:
        return False
    device = "cuda" if torch.cuda.is_available() else "cpu"
    _leaked.append(torch.empty(size_mb * 1024 * 1024 // 4, dtype=torch.float32, device=device))
    _leaked_mb += size_mb
    logger.warning("[chaos] random_gpu_memory_leak: %d MB held in %d tensors", _leaked_mb, len(_leaked))
    return True


def release_leaks() -> int:
    """Free everything ``random_gpu_memory_leak`` holds; returns the MB released."""
    global _leaked_mb
    released, _leaked_mb = _leaked_mb, 0
    _leaked.clear()
    return released


def _cpu_burn(duration: float) -> None:
    deadline = time.time() + duration
    counter = 0
    while time.time() < deadline:
        counter += 1


def random_cpu_hog(num_workers: int = 4, duration: float = 10, chance: float = 0.01) -> bool:
    if random.random() >= chance:
        return False
    pids = []
    for _ in range(num_workers):
        worker = multiprocessing.Process(target=_cpu_burn, args=(duration,), daemon=True)
        worker.start()
        pids.append(worker.pid)
    logger.warning("[chaos] random_cpu_hog: %d busy processes %s for %ss", num_workers, pids, duration)
    return True


# keys of a chaos entry that say WHEN it may fire; everything else is passed to the function
GATES = ("after_iteration", "first_attempt_only", "rank")


def function_register(chaos_function, parameters: dict):
    """Closure around one chaos function.  Optional gates in ``parameters`` (for reproducible fault drills):
    ``after_iteration``: fire only once the loop has reached that iteration; ``first_attempt_only``: not after an
    elastic restart (``TORCHELASTIC_RESTART_COUNT`` > 0); ``rank``: only on that global rank."""
    gates = {k: parameters[k] for k in GATES if k in parameters}
    kwargs = {k: v for k, v in parameters.items() if k not in GATES}

    def trigger(iteration=None):
        if "after_iteration" in gates and (iteration is None or iteration < gates["after_iteration"]):
            return False
        if gates.get("first_attempt_only") and int(os.environ.get("TORCHELASTIC_RESTART_COUNT", "0")) > 0:
            return False
        if "rank" in gates and int(os.environ.get("RANK", "0")) != gates["rank"]:
            return False
        return chaos_function(**kwargs)
    return trigger


CHAOS_FUNCTIONS = {
    "random_delay": random_delay,
    "random_kill": random_kill,
    "random_gpu_memory_leak": random_gpu_memory_leak,
    "random_cpu_hog": random_cpu_hog,
}


class ChaosEnginnerTrigger:
    """Build closures for every enabled entry of ``chaos_engineering`` and fire
    them all on ``trigger()``.  (The class name keeps the reference's spelling.)"""

    def __init__(self, chaos_config: dict | None, multicast_bound=None):
        """``multicast_bound``: optional callable telling whether any buffer of this process is bound to an NVLink
        multicast object.  A process that dies in that state raises NVLink faults on its peers' GPUs, so
        ``random_kill`` is refused while it returns true."""
        self._triggers = []
        for name, parameters in (chaos_config or {}).items():
            if not isinstance(parameters, dict) or not parameters.get("enabled", False):
                continue
            if name not in CHAOS_FUNCTIONS:
                raise ValueError(f"Unknown chaos function: {name}")
            if name == "random_kill" and multicast_bound is not None and multicast_bound():
                raise ValueError("chaos_engineering.random_kill is refused while symmetric buffers are bound to an "
                                 "NVLink multicast object (comm.multicast: true); switch one of them off")
            kwargs = {k: v for k, v in parameters.items() if k != "enabled"}
            self._triggers.append(function_register(CHAOS_FUNCTIONS[name], kwargs))

    def __len__(self) -> int:
        return len(self._triggers)

    def trigger(self, iteration=None) -> int:
        """Fire every enabled function once; ``iteration`` (the number of finished iterations) feeds the
        ``after_iteration`` gate."""
        return sum(1 for fire in self._triggers if fire(iteration))


ChaosEngineerTrigger = ChaosEnginnerTrigger
