"""Operator seams of the model.

Every hot op of the training step is a function here.  On a CUDA tensor the
function launches the hand-written sm_100a kernel from the in-tree extension
(``b200moe/ops/native.py`` loads it and raises if it is missing on a GPU box);
on a CPU tensor it evaluates the plain PyTorch statement from
``b200moe.ops.functional``, which is the oracle the kernels are tested against
and the compute path of the CPU/gloo plumbing tier.

``set_native(False)`` forces the PyTorch statements on CUDA tensors too; it is an
A/B switch for tests and for the library-kernel baseline measurement, not a
product path.
"""
from __future__ import annotations

import os

import torch

from . import functional as Fn

_FORCE_TORCH = os.environ.get("B200MOE_NATIVE", "1") == "0"
_DISABLED: set[str] = set(filter(None, os.environ.get("B200MOE_DISABLE", "").split(",")))


def set_native(enabled: bool) -> None:
    global _FORCE_TORCH
    _FORCE_TORCH = not enabled


def native_enabled() -> bool:
    return not _FORCE_TORCH


def use_native(t: torch.Tensor, op: str = "") -> bool:
    """True when ``t`` lives on a GPU and native kernels are switched on."""
    if not t.is_cuda or _FORCE_TORCH or op in _DISABLED:
        return False
    from . import native
    return native.has(op)


from .dense import linear, linear_rope, embedding, rmsnorm, add_rmsnorm  # noqa: E402
from .attention import rope_attention  # noqa: E402
from .loss import lm_head_cross_entropy  # noqa: E402
from .moe import router_top2, moe_ffn, DispatchPlan  # noqa: E402

__all__ = [
    "Fn", "set_native", "native_enabled", "use_native", "linear", "linear_rope", "embedding", "rmsnorm", "add_rmsnorm",
    "rope_attention", "lm_head_cross_entropy", "router_top2", "moe_ffn", "DispatchPlan",
]
