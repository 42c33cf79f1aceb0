"""Plain data parallel wrapper and the whole-parameter sharded optimizer.

Both exist in the reference as legacy code outside the training path
(implementation/distributed/ddp_modules.py:16-21, 303-362) and are kept for API
parity.  ``DDPWraper`` averages each gradient over the world as soon as autograd
has accumulated it; ``ShardedOptimizer`` gives parameter ``i`` to rank
``i mod world`` and broadcasts updated values from their owners.
"""
from __future__ import annotations

from typing import Any, Type

import torch
import torch.distributed as dist
import torch.nn as nn

__all__ = ["DDPWraper", "ShardedOptimizer", "sync_grad"]


def _world():
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def sync_grad(works: list, FSDP_communication_group=None):
    def hook(param):
        works.append(dist.all_reduce(param.grad.data, op=dist.ReduceOp.AVG, async_op=True,
                                     group=FSDP_communication_group))
    return hook


class DDPWraper(nn.Module):
    def __init__(self, module: nn.Module, src_rank: int = 0):
        super().__init__()
        self.works = []
        self.module = module
        if _world()[1] > 1:
            for p in module.parameters():
                dist.broadcast(p.data, src_rank)
                if p.requires_grad:
                    p.register_post_accumulate_grad_hook(sync_grad(self.works))

    def forward(self, *args, **kwargs):
        return self.module(*args, **kwargs)

    def finish_gradient_synchronization(self):
        for work in self.works:
            work.wait()
        self.works.clear()


class ShardedOptimizer(torch.optim.Optimizer):
    def __init__(self, params, optimizer_cls: Type[torch.optim.Optimizer], **kwargs: Any):
        self.rank, self.world_size = _world()
        self.param_list = []
        mine = []
        for index, p in enumerate(params):
            owner = index % self.world_size
            self.param_list.append((owner, p))
            if owner == self.rank:
                mine.append(p)
        self.param_count = len(self.param_list)
        self.optimizer_this = optimizer_cls(mine, **kwargs)

    def step(self, closure=None, **kwargs):
        self.optimizer_this.step(closure=closure, **kwargs)
        if self.world_size > 1:
            works = [dist.broadcast(p.data, src=owner, async_op=True) for owner, p in self.param_list]
            for work in works:
                work.wait()

    def zero_grad(self, set_to_none: bool = True):
        for _, p in self.param_list:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()

    def add_param_group(self, param_group: dict[str, Any]):
        mine = []
        for p in param_group["params"]:
            owner = self.param_count % self.world_size
            self.param_list.append((owner, p))
            self.param_count += 1
            if owner == self.rank:
                mine.append(p)
        self.optimizer_this.add_param_group({"params": mine})

    def __getattr__(self, name):
        return getattr(self.__dict__["optimizer_this"], name)
