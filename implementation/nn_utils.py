"""The reference's second set of numeric helpers (implementation/nn_utils.py:4-31), with its argument names, on top of
``b200moe.ops.functional``."""
import torch

from b200moe.ops import functional as _Fn


def softmax(x, dim=-1):
    return _Fn.softmax(x, dim_sum=dim)


def log_softmax(x, dim=-1):
    return _Fn.log_softmax(x, dim=dim)


def cross_entropy(inputs, targets):
    return _Fn.cross_entropy(inputs, targets)


def clip_gradient(parameters, max_norm):
    """Scales every gradient in place by ``min(1, max_norm / (norm + 1e-6))``, ``norm`` the global L2 norm."""
    grads = [p.grad for p in parameters if p.grad is not None]
    if not grads:
        return
    norm = torch.sqrt(sum((g.float() ** 2).sum() for g in grads))
    factor = torch.clamp(max_norm / (norm + 1e-6), max=1.0)
    for g in grads:
        g.mul_(factor.to(g.dtype))
