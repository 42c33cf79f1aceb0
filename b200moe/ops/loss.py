"""LM head fused with the cross-entropy loss, in token chunks.

The reference materialises fp32 logits ``[tokens, vocab]`` and runs max, exp,
sum, log, gather, mean as separate ops (implementation/nnfunctions.py:56-64,
layers.py:415-417).  Here no full logits tensor ever exists.  The tokens are
processed in chunks: the head GEMM writes the bf16 logits of one chunk, one
kernel (row in registers: one read, one write) turns them into the chunk's
loss and, in place, into ``dlogits``, and two more GEMMs consume that buffer at
once: ``dh = dlogits W`` and ``dW += dlogitsᵀ h``.  What is kept for the backward
pass is ``dh`` ``[tokens, d_model]``, a thirty-second of the logits' size.

Because the gradients are formed during the forward pass, the factor that the
caller will back-propagate into the loss has to be known then: ``grad_scale``
(the pipeline step passes ``1 / microbatches``).  The backward pass multiplies
``dh`` by ``dloss / grad_scale``, which is one when the caller keeps its word;
the weight gradient has already been accumulated with ``grad_scale``.  Without
``grad_scale`` (or without a ``main_grad`` buffer on the weight) the logits of
each chunk are rebuilt in the backward pass instead.  The value returned is the
mean over tokens, like the reference.
"""
from __future__ import annotations

import torch

from . import functional as Fn

CHUNK_TOKENS = 4096


def _native():
    from . import native
    return native


def _chunks(total: int, size: int):
    for lo in range(0, total, size):
        yield lo, min(total, lo + size)


class _LMHeadCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, targets, grad_scale):
        native = _native()
        h2d = hidden.reshape(-1, hidden.shape[-1])
        flat_targets = targets.reshape(-1).contiguous()
        tokens = h2d.shape[0]
        main_grad = getattr(weight, "main_grad", None)
        eager = grad_scale is not None and main_grad is not None and ctx.needs_input_grad[0]
        loss = torch.zeros((), dtype=torch.float32, device=hidden.device)
        dh = torch.empty_like(h2d) if eager else None
        for lo, hi in _chunks(tokens, CHUNK_TOKENS):
            logits = native.gemm_nt(h2d[lo:hi], weight)
            native.cross_entropy_scaled_(logits, flat_targets[lo:hi], loss, 1.0 / tokens,
                                         (grad_scale if eager else 1.0) / tokens)
            if eager:
                native.gemm_nn(logits, weight, out=dh[lo:hi])
                native.gemm_tn(logits, h2d[lo:hi], out=main_grad, accumulate=True)
        ctx.weight, ctx.shape, ctx.eager, ctx.grad_scale = weight, hidden.shape, eager, grad_scale
        if eager:
            ctx.save_for_backward(dh)
        else:
            ctx.save_for_backward(h2d, flat_targets)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        native = _native()
        weight = ctx.weight
        if ctx.eager:
            (dh,) = ctx.saved_tensors
            native.scale_(dh, dloss / ctx.grad_scale)
            return dh.view(ctx.shape), None, None, None
        h2d, flat_targets = ctx.saved_tensors
        tokens = h2d.shape[0]
        main_grad = getattr(weight, "main_grad", None)
        dh = torch.empty_like(h2d)
        dw = None
        if main_grad is None and ctx.needs_input_grad[1]:
            dw = torch.zeros(weight.shape, dtype=torch.float32, device=weight.device)
        scratch = torch.zeros((), dtype=torch.float32, device=h2d.device)
        for lo, hi in _chunks(tokens, CHUNK_TOKENS):
            logits = native.gemm_nt(h2d[lo:hi], weight)
            native.cross_entropy_scaled_(logits, flat_targets[lo:hi], scratch, 1.0 / tokens, 1.0 / tokens)
            native.scale_(logits, dloss)
            native.gemm_nn(logits, weight, out=dh[lo:hi])
            native.gemm_tn(logits, h2d[lo:hi], out=main_grad if main_grad is not None else dw, accumulate=True)
        return dh.view(ctx.shape), (dw.to(weight.dtype) if dw is not None else None), None, None


def lm_head_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor,
                          grad_scale: float | None = None) -> torch.Tensor:
    """Mean next-token loss of ``hidden @ weightᵀ`` against ``targets``.  ``grad_scale``: the factor the caller will
    back-propagate into the returned loss, when it is known in advance (see the module text)."""
    from . import use_native
    from .dense import linear
    if use_native(hidden, "lmhead_ce"):
        return _LMHeadCE.apply(hidden, weight, targets, grad_scale)
    logits = linear(hidden, weight)
    return Fn.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1))
