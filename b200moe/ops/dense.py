"""Linear, embedding and RMSNorm ops with explicit backward passes.

Weight gradients follow the "main grad" convention: when the weight tensor
carries a ``main_grad`` attribute (an fp32 buffer owned by the FSDP wrapper)
the backward pass accumulates ``dW`` straight into it from the GEMM epilogue
and returns no gradient to autograd.  Otherwise the gradient is returned and
autograd accumulates it in ``.grad``.

Replaces the reference's ``einsum`` linear (implementation/layers.py:55-69),
``weight[x, :]`` embedding (layers.py:72-82) and fp32 RMSNorm (layers.py:84-97).
"""
from __future__ import annotations

import torch

from . import functional as Fn


def _native():
    from . import native
    return native


def _use_native(t, op):
    from . import use_native
    return use_native(t, op)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, rope=None):
        """``rope``: optional ``(cos, sin, rope_cols, seq)``: the rotary embedding is applied to the leading
        ``rope_cols`` output columns in the GEMM epilogue.  The backward pass then expects the gradient of the
        UNROTATED output (the attention backward kernels deliver exactly that)."""
        ctx.weight = weight
        ctx.save_for_backward(x)
        x2d = x.reshape(-1, x.shape[-1])
        # a weight whose peer rows have not arrived yet carries the call that gathers them and multiplies in one
        # kernel (set by the FSDP wrapper after an optimizer step, consumed by the first use)
        gather = getattr(weight, "pending_gather", None)
        if gather is not None:
            weight.pending_gather = None
            y = gather(x2d if x2d.is_contiguous() else x2d.contiguous())
            if rope is not None:
                cos, sin, cols, seq = rope
                _native().rope_inplace(y, 0, y.shape[0], seq, cols // 128, 128, y.shape[1], cos, sin, 1.0)
        elif rope is not None:
            cos, sin, cols, seq = rope
            y = _native().gemm_nt_rope(x2d, weight, cos, sin, cols, seq)
        elif _use_native(x, "gemm"):
            y = _native().gemm_nt(x2d, weight)
        else:
            w = weight if weight.dtype == x.dtype else weight.to(x.dtype)
            y = x2d @ w.t()
        return y if x.dim() == 2 else y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        weight = ctx.weight
        x2d = x.reshape(-1, x.shape[-1])
        dy2d = dy.reshape(-1, dy.shape[-1])
        if not dy2d.is_contiguous():
            dy2d = dy2d.contiguous()
        native = _use_native(x, "gemm")
        dx = None
        if ctx.needs_input_grad[0]:
            if native:
                dx = _native().gemm_nn(dy2d, weight)
            else:
                w = weight if weight.dtype == dy2d.dtype else weight.to(dy2d.dtype)
                dx = dy2d @ w
            dx = dx.view_as(x)
        dw = None
        main_grad = getattr(weight, "main_grad", None)
        if main_grad is not None:
            if native:
                _native().gemm_tn(dy2d, x2d, out=main_grad, accumulate=True)
            else:
                main_grad.addmm_(dy2d.t().to(main_grad.dtype), x2d.to(main_grad.dtype))
        elif ctx.needs_input_grad[1]:
            if native:
                dw = _native().gemm_tn(dy2d, x2d, out_dtype=weight.dtype)
            else:
                dw = (dy2d.t() @ x2d).to(weight.dtype)
        return dx, dw, None


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``y = x @ weightᵀ`` with ``weight`` of shape ``[d_out, d_in]``; no bias."""
    return _Linear.apply(x, weight)


def linear_rope(x: torch.Tensor, weight: torch.Tensor, cos, sin, rope_cols: int, seq: int) -> torch.Tensor:
    """GPU only: ``x @ weightᵀ`` (``x [tokens, d_in]``, tokens laid out as sequences of ``seq``) with the rotary
    embedding (heads of 128 columns, adjacent pairs) applied to output columns ``[0, rope_cols)`` inside the GEMM.
    Its backward pass takes the gradient with respect to the unrotated product."""
    return _Linear.apply(x, weight, (cos[:seq].contiguous(), sin[:seq].contiguous(), rope_cols, seq))


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        ctx.table = table
        ctx.save_for_backward(ids)
        if _use_native(table, "embedding"):
            return _native().embedding_fwd(ids, table)
        return table[ids]

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        table = ctx.table
        flat_ids = ids.reshape(-1)
        dy2d = dy.reshape(-1, dy.shape[-1])
        main_grad = getattr(table, "main_grad", None)
        if main_grad is not None:
            if _use_native(dy, "embedding"):
                _native().embedding_bwd(flat_ids, dy2d, main_grad)
            else:
                main_grad.index_add_(0, flat_ids, dy2d.to(main_grad.dtype))
            return None, None
        grad = torch.zeros_like(table, dtype=torch.float32)
        grad.index_add_(0, flat_ids, dy2d.float())
        return None, grad.to(table.dtype)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Row gather ``table[ids]``; the backward pass scatter-adds in fp32."""
    return _Embedding.apply(ids, table)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        y, rstd = _native().rmsnorm_fwd(x, weight, eps)
        ctx.save_for_backward(x, weight, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, rstd = ctx.saved_tensors
        dx, dw = _native().rmsnorm_bwd(dy.contiguous(), x, weight, rstd)
        return dx, dw.to(weight.dtype), None


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """``x · rsqrt(mean(x²) + eps) · weight`` evaluated in fp32, cast back."""
    if _use_native(x, "rmsnorm"):
        return _RMSNorm.apply(x, weight, eps)
    return Fn.rmsnorm_ref(x, weight, eps)


class _AddRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, delta, weight, eps):
        summed, y, rstd = _native().add_rmsnorm_fwd(x, delta, weight, eps)
        ctx.save_for_backward(summed, weight, rstd)
        return summed, y

    @staticmethod
    def backward(ctx, dsum, dy):
        summed, weight, rstd = ctx.saved_tensors
        dx, dw = _native().rmsnorm_bwd(dy.contiguous(), summed, weight, rstd, residual_grad=dsum)
        return dx, dx, dw.to(weight.dtype), None


def add_rmsnorm(x: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5):
    """Residual add fused with the following norm: returns ``(x + delta,
    rmsnorm(x + delta))``."""
    if _use_native(x, "rmsnorm"):
        return _AddRMSNorm.apply(x, delta, weight, eps)
    summed = x + delta
    return summed, Fn.rmsnorm_ref(summed, weight, eps)
