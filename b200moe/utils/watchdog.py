"""Watchdog for the kernels' status word.

Every cross-GPU wait and every mbarrier wait inside this framework's kernels is
bounded: when a budget runs out the kernel writes a code into a device status
word and finishes, so the GPU never hangs on a missing peer.  The training
thread, however, may by then sit in a host-side wait (an NCCL send/recv to the
peer that is gone) and never look at the word.  ``StatusWatchdog`` is the piece
that turns the word into a process-level event: a daemon thread copies the word
to pinned host memory on a private stream once per interval; a non-zero code is
recorded for ``raise_if_failed()`` (the loop calls it between steps) and, if the
training thread has not picked it up within a grace period, the process exits
with a distinct code so that ``torchrun --max-restarts`` / the TrainJob's
``RestartJobSet`` policy restarts the whole group from the last committed
checkpoint — the reference's recovery model (README.md:85,
modal_wrapper.py:102-123).
"""
from __future__ import annotations

import os
import threading
import time

__all__ = ["StatusWatchdog", "WATCHDOG_EXIT_CODE", "device_status_reader"]

WATCHDOG_EXIT_CODE = 75      # EX_TEMPFAIL: "try again", which is what a group restart does


def device_status_reader(device=None):
    """Returns ``read() -> int`` that fetches the native status word without touching the training stream."""
    import torch
    from ..ops import native
    word = native.status_word(device)
    stream = torch.cuda.Stream(device=word.device)
    host = torch.zeros(1, dtype=torch.int32).pin_memory()
    done = torch.cuda.Event()

    def read() -> int:
        with torch.cuda.stream(stream):
            host.copy_(word, non_blocking=True)
            done.record(stream)
        done.synchronize()
        return int(host[0])

    return read


class StatusWatchdog:
    def __init__(self, read_status, interval_s: float = 1.0, grace_s: float = 30.0, on_failure=None,
                 exit_process=os._exit, log=print, before_exit=None):
        """``before_exit``: optional callable run (errors ignored) right before the process is ended, e.g. to
        unbind symmetric buffers from their multicast object so that the exit cannot disturb the peers."""
        self._read = read_status
        self._before_exit = before_exit
        self.interval_s, self.grace_s = float(interval_s), float(grace_s)
        self._on_failure = on_failure
        self._exit = exit_process
        self._log = log
        self._stop = threading.Event()
        self._ack = threading.Event()
        self._thread = None
        self.code = 0

    def start(self) -> "StatusWatchdog":
        if self._thread is None:
            self._thread = threading.Thread(target=self._run, name="b200moe-status-watchdog", daemon=True)
            self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5.0)
            self._thread = None

    def raise_if_failed(self) -> None:
        """Called by the training loop between steps."""
        if self.code:
            self._ack.set()
            raise RuntimeError(f"b200moe kernel wait timed out (status code {self.code}); "
                               "exiting so that the launcher restarts the group")

    def _run(self) -> None:
        while not self._stop.wait(self.interval_s):
            try:
                code = int(self._read())
            except Exception as error:      # a dead context also means: restart
                code = -1
                self._log(f"[watchdog] status read failed: {error}", flush=True)
            if not code:
                continue
            self.code = code
            self._log(f"[watchdog] kernel status code {code}: a bounded device wait ran out", flush=True)
            if self._on_failure is not None:
                self._on_failure(code)
            deadline = time.monotonic() + self.grace_s
            while time.monotonic() < deadline and not self._stop.is_set():
                if self._ack.wait(0.05):
                    return                  # the training thread saw it and is unwinding
            if not self._stop.is_set():
                self._log(f"[watchdog] training thread did not react within {self.grace_s:.0f} s; "
                          f"exiting with code {WATCHDOG_EXIT_CODE}", flush=True)
                if self._before_exit is not None:
                    try:
                        self._before_exit()
                    except Exception as error:
                        self._log(f"[watchdog] release before exit failed: {error}", flush=True)
                self._exit(WATCHDOG_EXIT_CODE)
            return
