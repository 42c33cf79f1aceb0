"""Causal grouped-query attention with rotary embedding folded in.

Replaces ``ROPELayer`` + ``scaled_dot_product_attention(is_causal=True,
enable_gqa=True)`` of the reference (implementation/layers.py:268-333).
Tensors are ``[B, S, H, head_dim]`` (views into the fused QKV projection are
fine); the rotation acts on adjacent element pairs.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import functional as Fn


def _native():
    from . import native
    return native


class _RopeAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cos, sin):
        out, lse, q_rot, k_rot = _native().attention_fwd(q, k, v, cos, sin)
        ctx.save_for_backward(q_rot, k_rot, v, out, lse, cos, sin)
        return out

    @staticmethod
    def backward(ctx, dout):
        q_rot, k_rot, v, out, lse, cos, sin = ctx.saved_tensors
        dq, dk, dv = _native().attention_bwd(dout.contiguous(), q_rot, k_rot, v, out, lse, cos, sin)
        return dq, dk, dv, None, None


class _RopeQK(torch.autograd.Function):
    """Rotate the first ``heads`` heads of every token of a fused projection
    ``[tokens, total_heads * hd]`` in place; the backward pass applies the
    transpose rotation to the gradient."""

    @staticmethod
    def forward(ctx, qkv, seq, total, heads, hd, cos, sin):
        _native().rope_inplace(qkv, 0, qkv.shape[0], seq, heads, hd, total * hd, cos, sin, 1.0)
        ctx.mark_dirty(qkv)
        ctx.meta = (seq, total, heads, hd, cos, sin)
        return qkv

    @staticmethod
    def backward(ctx, dqkv):
        seq, total, heads, hd, cos, sin = ctx.meta
        dqkv = dqkv.contiguous().clone()
        _native().rope_inplace(dqkv, 0, dqkv.shape[0], seq, heads, hd, total * hd, cos, sin, -1.0)
        return dqkv, None, None, None, None, None, None


def rope_qk_(qkv2d, seq, total_heads, heads, head_dim, cos, sin):
    """In-place RoPE on heads ``[0, heads)`` of a ``[tokens, total_heads*head_dim]``
    tensor whose tokens are ``batch`` runs of ``seq`` positions."""
    return _RopeQK.apply(qkv2d, seq, total_heads, heads, head_dim, cos, sin)


def rope_attention(q, k, v, cos, sin):
    """Returns ``[B, S, Hq, head_dim]``.  ``cos``/``sin`` are ``[S_max, hd/2]``
    fp32 tables or ``None`` for no rotation."""
    from . import use_native
    if use_native(q, "attention"):
        return _RopeAttention.apply(q, k, v, cos, sin)
    if q.is_cuda:
        # library attention on the GPU (A/B baseline only)
        qh, kh, vh = (t.transpose(1, 2) for t in (q, k, v))
        if cos is not None:
            seq = qh.shape[-2]
            qh = Fn.apply_rope_ref(qh, cos[:seq], sin[:seq])
            kh = Fn.apply_rope_ref(kh, cos[:seq], sin[:seq])
        out = F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, enable_gqa=True)
        return out.transpose(1, 2)
    return Fn.attention_ref(q, k, v, cos, sin, causal=True)
