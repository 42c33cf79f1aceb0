"""Asynchronous sharded checkpoints with an atomic commit protocol.

Layout (kept from the reference, distributed_parallel_training_pipelined.py:27-88,
291-301 and implementation/train_utils.py:151-254)::

    {checkpoint_folder}/checkpoint/{run_id}/{iteration}/shaded_dp_{dp}_pp_{pp}.ckpt
    {checkpoint_folder}/checkpoint/{run_id}/{iteration}/COMMITTED

Each shard is a ``torch.save`` of ``{"model.state_dict", "optimizer.state_dict",
"iteration", "rng"}``.  A save copies device tensors into pinned host buffers on
the current stream, synchronises once, and hands the write to a background
thread that writes ``path.tmp``, fsyncs and renames.  A directory counts only
after every rank reported success and the info rank renamed ``COMMITTED.tmp``
to ``COMMITTED``.  Staging buffers are cached per tensor name and reused by
later saves once the previous write has finished.
"""
from __future__ import annotations

import copy
import os
import random
from concurrent.futures import Future, ThreadPoolExecutor
from pathlib import Path

import torch

__all__ = [
    "shard_name", "latest_checkpoint", "select_checkpoint", "verify_pending_checkpoints",
    "save_checkpoint_async_dist", "load_checkpoint_async_dist", "save_checkpoint", "load_checkpoint",
    "CheckpointStager",
]


def shard_name(dp_idx: int, stage: int) -> str:
    return f"shaded_dp_{dp_idx}_pp_{stage}.ckpt"


def latest_checkpoint(root, dp_size: int, pp_size: int, run: str | None = None):
    """Newest committed step directory that holds every ``dp × pp`` shard file;
    ordered by ``(run name, int(step))``."""
    best, best_key = None, None
    for marker in Path(root).glob(f"{run or '*'}/*/COMMITTED"):
        step_dir = marker.parent
        if not step_dir.name.isdigit():
            continue
        complete = all((step_dir / shard_name(d, p)).is_file()
                       for d in range(dp_size) for p in range(pp_size))
        if not complete:
            continue
        key = (step_dir.parent.name, int(step_dir.name))
        if best_key is None or key > best_key:
            best, best_key = step_dir, key
    return best


def select_checkpoint(config: dict, rank: int, info_src: int, group=None):
    """Decide on ``info_src`` which checkpoint to resume and tell everyone.

    An explicit ``train.load_checkpoint_path`` must be committed; after an elastic
    restart (``TORCHELASTIC_RESTART_COUNT > 0``) it advances to the newest
    committed step of the same run.  Without one, the newest committed step under
    ``checkpoint_folder/checkpoint`` is used.  Errors are re-raised on all ranks.
    """
    import torch.distributed as dist
    from ..topology import parallel_sizes
    decision = [None, None]
    if rank == info_src:
        try:
            train = config["train"]
            fsdp, ddp = parallel_sizes(train)
            pp = train["pipeline_parallel_stages"]
            explicit = train.get("load_checkpoint_path")
            if explicit:
                path = Path(explicit)
                if int(os.environ.get("TORCHELASTIC_RESTART_COUNT", "0")):
                    newer = latest_checkpoint(path.parent.parent, fsdp * ddp, pp, run=path.parent.name)
                    if newer is not None and newer.parent == path.parent:
                        path = newer
                if not (path / "COMMITTED").is_file():
                    raise ValueError(f"Checkpoint is not committed: {path}")
            else:
                root = Path(config["general"]["checkpoint_folder"]) / "checkpoint"
                path = latest_checkpoint(root, fsdp * ddp, pp)
            decision[0] = None if path is None else str(path)
        except Exception as error:  # propagated to every rank below
            decision[1] = str(error)
    if dist.is_available() and dist.is_initialized():
        dist.broadcast_object_list(decision, src=info_src, group=group)
    if decision[1]:
        raise RuntimeError(decision[1])
    return decision[0]


def verify_pending_checkpoints(pending: list, iteration: int, rank: int, info_src: int, device,
                               drain: bool = False, min_age: int = 5, group=None, healthy=None) -> None:
    """Commit saves that are ``min_age`` iterations old (all of them when
    ``drain``): join the writer, agree by ``all_reduce(MIN)`` and let the info
    rank publish the ``COMMITTED`` marker by rename.  ``healthy``: optional
    callable returning a false value when this rank has seen a device-side
    failure (a bounded kernel wait that ran out) since the save; such a rank
    votes against the commit, so a state that may already be damaged is never
    published."""
    import torch.distributed as dist
    while pending and (drain or iteration - pending[0][0] >= min_age):
        saved_iteration, directory, future = pending.pop(0)
        ok = 1
        try:
            future.result()
        except Exception as error:
            ok = 0
            print(f"Rank {rank} checkpoint at iteration {saved_iteration} failed: {error}", flush=True)
        if ok and healthy is not None:
            try:
                fine = bool(healthy())
            except Exception as error:
                fine = False
                print(f"Rank {rank} device status check failed: {error}", flush=True)
            if not fine:
                ok = 0
                print(f"Rank {rank} votes against the checkpoint at iteration {saved_iteration}: a device-side "
                      f"wait ran out since it was staged", flush=True)
        flag = torch.tensor(ok, dtype=torch.int32, device=device)
        if dist.is_available() and dist.is_initialized():
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if rank != info_src:
            continue
        if int(flag.item()) == 1:
            text = f"Checkpoint at iteration {saved_iteration} committed: all ranks saved successfully."
            staging = Path(directory, "COMMITTED.tmp")
            staging.write_text(text + "\n", encoding="utf-8")
            staging.replace(Path(directory, "COMMITTED"))
            print(text, flush=True)
        else:
            print(f"Checkpoint at iteration {saved_iteration} not committed: at least one rank failed.",
                  flush=True)


class CheckpointStager:
    """Pinned host mirrors of device tensors, reused across saves."""

    def __init__(self):
        self._buffers: dict = {}
        self._busy: Future | None = None

    def wait(self) -> None:
        if self._busy is not None:
            try:
                self._busy.result()
            except Exception:
                pass
            self._busy = None

    def stage(self, key, tensor: torch.Tensor) -> torch.Tensor:
        host = self._buffers.get(key)
        if host is None or host.shape != tensor.shape or host.dtype != tensor.dtype:
            host = torch.empty(tensor.shape, dtype=tensor.dtype, device="cpu",
                               pin_memory=tensor.is_cuda)
            self._buffers[key] = host
        host.copy_(tensor.detach(), non_blocking=True)
        return host


_DEFAULT_STAGER = CheckpointStager()


def _stage_optimizer(optimizer, stager: CheckpointStager) -> dict:
    state_dict = optimizer.state_dict()
    staged = {}
    for index, state in state_dict["state"].items():
        staged[index] = {name: stager.stage(("opt", index, name), value) if torch.is_tensor(value) else value
                         for name, value in state.items()}
    return {"state": staged, "param_groups": copy.deepcopy(state_dict["param_groups"])}


def move_model_state(model, stager: CheckpointStager | None = None) -> dict:
    """Host snapshot of ``model.state_dict()`` (reference train_utils.py:151-161): every tensor is copied to
    pinned memory without blocking the host; synchronise the stream before reading the copies.  Without a
    ``stager`` the buffers are fresh, as in the reference; the asynchronous save passes its own and reuses them."""
    stager = CheckpointStager() if stager is None else stager
    return {name: stager.stage(("model", name), tensor) for name, tensor in model.state_dict().items()}


def move_optimizer_state(optimizer, stager: CheckpointStager | None = None) -> dict:
    """Host snapshot of ``optimizer.state_dict()`` (reference train_utils.py:163-180): tensors to pinned memory,
    everything else and the parameter groups copied."""
    return _stage_optimizer(optimizer, CheckpointStager() if stager is None else stager)


def _rng_bundle(data_rng) -> dict:
    return {
        "data": copy.deepcopy(data_rng.bit_generator.state),
        "torch": torch.get_rng_state(),
        "cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None,
        "python": random.getstate(),
    }


def _write_checkpoint(checkpoint: dict, destination) -> None:
    if not isinstance(destination, (str, os.PathLike)):
        torch.save(checkpoint, destination)
        return
    final = os.fspath(destination)
    temporary = final + ".tmp"
    try:
        with open(temporary, "wb") as handle:
            torch.save(checkpoint, handle)
            handle.flush()
            os.fsync(handle.fileno())
        os.replace(temporary, final)
    finally:
        if os.path.exists(temporary):
            os.unlink(temporary)


def save_checkpoint_async_dist(model, optimizer, iteration: int, checkpoint_dir, data_rng=None,
                               stager: CheckpointStager | None = None) -> Future:
    """Stage on the host, then write in the background; returns the ``Future``."""
    stager = stager or _DEFAULT_STAGER
    stager.wait()
    checkpoint = {"model.state_dict": move_model_state(model, stager),
                  "optimizer.state_dict": move_optimizer_state(optimizer, stager),
                  "iteration": iteration}
    if data_rng is not None:
        checkpoint["rng"] = _rng_bundle(data_rng)
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    pool = ThreadPoolExecutor(max_workers=1)
    try:
        future = pool.submit(_write_checkpoint, checkpoint, checkpoint_dir)
    finally:
        pool.shutdown(wait=False)
    stager._busy = future
    return future


def _load_legacy_optimizer(saved_state: dict, optimizer) -> None:
    """Accept the old layout: a bare ``{index: state}`` mapping without groups."""
    params = [p for group in optimizer.param_groups for p in group["params"]]
    values = list(saved_state.values())
    if len(values) != len(params):
        raise ValueError("Checkpoint optimizer state invalid, failed to load")
    groups, base = [], 0
    for group in optimizer.param_groups:
        entry = {k: v for k, v in group.items() if k != "params"}
        entry["params"] = list(range(base, base + len(group["params"])))
        base += len(group["params"])
        groups.append(entry)
    optimizer.load_state_dict({"state": dict(enumerate(values)), "param_groups": groups})


def load_checkpoint_async_dist(src, model, optimizer=None, data_rng=None) -> int:
    """Restore model, optimizer and every RNG stream; returns the iteration."""
    checkpoint = torch.load(src, map_location="cpu", weights_only=False)
    model.load_state_dict(checkpoint["model.state_dict"])
    if optimizer is not None:
        saved = checkpoint["optimizer.state_dict"]
        if "param_groups" in saved:
            optimizer.load_state_dict(saved)
        else:
            _load_legacy_optimizer(saved, optimizer)
    if data_rng is not None:
        rng = checkpoint.get("rng")
        if rng is None:
            raise KeyError("checkpoint has no rng section; cannot restore the data sampler")
        data_rng.bit_generator.state = rng["data"]
        torch.set_rng_state(rng["torch"])
        random.setstate(rng["python"])
        if rng["cuda"] is not None and torch.cuda.is_available():
            torch.cuda.set_rng_state(rng["cuda"])
    return checkpoint["iteration"]


def save_checkpoint(model, optimizer, iteration: int, out) -> None:
    """Synchronous single-file variant (reference train_utils.py:143-148)."""
    torch.save({"model.state_dict": model.state_dict(),
                "optimizer.state_dict": optimizer.state_dict(),
                "iteration": iteration}, out)


def load_checkpoint(src, model, optimizer=None) -> int:
    checkpoint = dict(torch.load(src, weights_only=False))
    model.load_state_dict(checkpoint["model.state_dict"])
    if optimizer is not None:
        optimizer.load_state_dict(checkpoint["optimizer.state_dict"])
    return checkpoint["iteration"]
