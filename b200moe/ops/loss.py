"""LM head fused with the cross-entropy loss.

The reference materialises fp32 logits ``[tokens, vocab]`` and runs max, exp,
sum, log, gather, mean as separate ops (implementation/nnfunctions.py:56-64,
layers.py:415-417).  Here the head GEMM writes bf16 logits once, one kernel
turns them into per-token losses and overwrites them with ``dlogits`` in
place, and the backward pass is two GEMMs on that buffer.  The value returned
is the mean over tokens, like the reference.
"""
from __future__ import annotations

import torch

from . import functional as Fn


def _native():
    from . import native
    return native


class _LMHeadCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, targets):
        native = _native()
        h2d = hidden.reshape(-1, hidden.shape[-1])
        logits = native.gemm_nt(h2d, weight)
        loss_sum = native.cross_entropy_fwd_bwd_(logits, targets.reshape(-1))  # logits <- dlogits/T
        ctx.weight = weight
        ctx.save_for_backward(h2d, logits)
        ctx.shape = hidden.shape
        return loss_sum

    @staticmethod
    def backward(ctx, dloss):
        native = _native()
        h2d, dlogits = ctx.saved_tensors
        weight = ctx.weight
        native.scale_(dlogits, dloss)
        dh = native.gemm_nn(dlogits, weight).view(ctx.shape)
        main_grad = getattr(weight, "main_grad", None)
        dw = None
        if main_grad is not None:
            native.gemm_tn(dlogits, h2d, out=main_grad, accumulate=True)
        else:
            dw = native.gemm_tn(dlogits, h2d, out_dtype=weight.dtype)
        return dh, dw, None


def lm_head_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean next-token loss of ``hidden @ weightᵀ`` against ``targets``."""
    from . import use_native
    from .dense import linear
    if use_native(hidden, "lmhead_ce"):
        return _LMHeadCE.apply(hidden, weight, targets)
    logits = linear(hidden, weight)
    return Fn.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1))
