"""Module hooks that gather a row-sharded weight before a module runs and put the shard back afterwards.

The reference's sharded-data-parallel wrapper is built from these hooks
(implementation/distributed/ddp_modules.py:23-100): a forward (or backward)
pre-hook all-gathers ``module.weight`` over the sharding group, optionally one
module ahead and asynchronously, and a post-hook restores the shard.  This
framework's wrapper does not use them — it keeps the weights of a step gathered
in one flat buffer and refreshes them in its end-of-step kernel
(``parallel/fsdp.py``) — but they are kept, with the same names and hook
signatures, for code that shards individual modules by hand.

All of them work on any module with a ``weight`` whose rows (dimension 0) are
split evenly over the group, on NCCL and gloo alike.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

__all__ = ["sync_weight_wrapper", "async_weight_wrapper_next", "free_weight", "sync_weight_wrapper_backward",
           "async_weight_wrapper_backward_next", "free_weight_backward", "wait_prefetched_weight",
           "wait_prefetched_weight_backward"]


def _gather_rows(target, dtype, group, works=None):
    """Swap ``target.weight.data`` for the all-gathered weight (kept: ``weight.data_original`` = the shard).  With a
    ``works`` list the gather is asynchronous and its handle is appended there."""
    ranks = dist.get_world_size(group)
    shard = target.weight.data
    full = torch.empty((ranks * shard.shape[0], *shard.shape[1:]), device=shard.device, dtype=dtype)
    work = dist.all_gather_into_tensor(full, shard.to(dtype=dtype).contiguous(), group=group, async_op=works is not None)
    target.weight.data_original = shard
    target.weight.data = full
    if works is not None:
        works.append(work)


def _restore_shard(module):
    module.weight.data = module.weight.data_original
    module.weight.data_original = None


def sync_weight_wrapper(dtype=torch.float32, FSDP_communication_group=None):
    """Forward pre-hook: gather this module's weight now."""
    def sync_weight(module, args):
        _gather_rows(module, dtype, FSDP_communication_group)
    return sync_weight


def async_weight_wrapper_next(next_module, works: list, dtype=torch.float32, FSDP_communication_group=None):
    """Forward pre-hook: start gathering the NEXT module's weight while this one computes."""
    def sync_weight(module, args):
        _gather_rows(next_module, dtype, FSDP_communication_group, works)
    return sync_weight


def free_weight(module, args, output):
    """Forward hook: back to the shard."""
    _restore_shard(module)


def sync_weight_wrapper_backward(dtype=torch.float32, FSDP_communication_group=None):
    """Backward pre-hook (``register_full_backward_pre_hook``): gather this module's weight now."""
    def sync_weight(module, grad_output=None):
        _gather_rows(module, dtype, FSDP_communication_group)
    return sync_weight


def async_weight_wrapper_backward_next(next_module, works: list, dtype=torch.float32, FSDP_communication_group=None):
    """Backward pre-hook: start gathering the weight of the module whose backward pass comes next."""
    def sync_weight(module, grad_output=None):
        _gather_rows(next_module, dtype, FSDP_communication_group, works)
    return sync_weight


def free_weight_backward(module, grad_input, grad_output):
    """Backward hook: back to the shard."""
    _restore_shard(module)


def wait_prefetched_weight(works):
    """Forward pre-hook: wait for the oldest outstanding prefetch (``works``: a deque of handles)."""
    def hook(module, args):
        if works:
            works.popleft().wait()
    return hook


def wait_prefetched_weight_backward(works):
    def hook(module, grad_output=None):
        if works:
            works.popleft().wait()
    return hook
