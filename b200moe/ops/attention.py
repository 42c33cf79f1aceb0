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


class _FusedQKVAttention(torch.autograd.Function):
    """RoPE + causal GQA attention on the fused QKV projection ``[tokens, (Hq + 2 Hkv) * hd]``.
    Forward rotates q and k in place inside the projection buffer and runs the tcgen05 attention kernel
    on views of it; backward writes dq, dk, dv into one fused gradient buffer and un-rotates it in place,
    so autograd sees a single gradient for the projection output."""

    @staticmethod
    def forward(ctx, qkv, batch, seq, hq, hkv, hd, cos, sin, pre_rotated):
        native = _native()
        total = hq + 2 * hkv
        if cos is not None and not pre_rotated:      # the projection GEMM did not rotate q and k in its epilogue
            native.rope_inplace(qkv, 0, qkv.shape[0], seq, hq + hkv, hd, total * hd, cos, sin, 1.0)
        ctx.mark_dirty(qkv)
        view = qkv.view(batch, seq, total, hd)
        out, lse, _, _ = native.attention_fwd(view[:, :, :hq], view[:, :, hq:hq + hkv], view[:, :, hq + hkv:])
        ctx.save_for_backward(qkv, out, lse)
        ctx.meta = (batch, seq, hq, hkv, hd, cos, sin)
        return qkv, out

    @staticmethod
    def backward(ctx, _dqkv_unused, dout):
        native = _native()
        qkv, out, lse = ctx.saved_tensors
        batch, seq, hq, hkv, hd, cos, sin = ctx.meta
        total = hq + 2 * hkv
        view = qkv.view(batch, seq, total, hd)
        dqkv = torch.empty_like(qkv)
        dview = dqkv.view(batch, seq, total, hd)
        # the backward kernels rotate dq and dk back as they store them
        native.attention_bwd(dout, view[:, :, :hq], view[:, :, hq:hq + hkv], view[:, :, hq + hkv:], out, lse,
                             cos=cos, sin=sin,
                             grads=(dview[:, :, :hq], dview[:, :, hq:hq + hkv], dview[:, :, hq + hkv:]))
        return dqkv, None, None, None, None, None, None, None, None


def fused_qkv_attention(qkv2d, batch, seq, hq, hkv, hd, cos, sin, pre_rotated: bool = False):
    """Returns the attention output ``[B, S, Hq, hd]`` of a fused projection ``[B*S, (Hq+2Hkv)*hd]``.
    ``pre_rotated``: q and k inside ``qkv2d`` already carry the rotation (``ops.linear_rope``)."""
    if cos is not None:
        cos, sin = cos[:seq].contiguous(), sin[:seq].contiguous()
    _, out = _FusedQKVAttention.apply(qkv2d, batch, seq, hq, hkv, hd, cos, sin, pre_rotated)
    return out


def attention_backend() -> str:
    """``native`` (this repository's tcgen05 kernels, the default) or ``library`` (cuDNN through PyTorch, for A/B runs); chosen by the
    environment variable ``B200MOE_ATTENTION``."""
    import os
    return os.environ.get("B200MOE_ATTENTION", "native")


def rope_attention(q, k, v, cos, sin):
    """Returns ``[B, S, Hq, head_dim]``.  ``cos``/``sin`` are ``[S_max, hd/2]``
    fp32 tables or ``None`` for no rotation."""
    from . import use_native
    if use_native(q, "attention") and attention_backend() == "native" and q.shape[-1] == 128 and q.shape[1] % 128 == 0:
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


class _PlainAttention(torch.autograd.Function):
    """Attention without rotation, causal or not, on ``[B, S, H, 128]`` bf16 tensors (tcgen05 kernels)."""

    @staticmethod
    def forward(ctx, q, k, v, causal):
        out, lse, _, _ = _native().attention_fwd(q, k, v, None, None, causal=causal)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal = causal
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = _native().attention_bwd(dout, q, k, v, out, lse, causal=ctx.causal)
        return dq, dk, dv, None


def _native_shape_ok(q, k) -> bool:
    from . import use_native
    return (use_native(q, "attention") and q.dtype == torch.bfloat16 and q.shape[-1] == 128
            and q.shape[1] % 128 == 0 and k.shape[1] == q.shape[1])


def attention(q, k, v, causal: bool = True):
    """Differentiable attention on ``[B, S, H, hd]`` tensors (``Hq`` a multiple of ``Hkv``); no rotation.  Runs the
    tcgen05 kernels for bf16, head_dim 128, ``S % 128 == 0`` on a GPU and the PyTorch formula otherwise."""
    if _native_shape_ok(q, k):
        return _PlainAttention.apply(q, k, v, bool(causal))
    return Fn.attention_ref(q, k, v, causal=causal)


def flash_attention_forward(q, k, v, causal: bool = False):
    """Forward-only multi-head attention on contiguous ``[B, H, S, head_dim]`` tensors, non-causal by default: the
    entry point of the reference's hand-written kernel (implementation/kernels/flash_attention.cu:390-448, fp16,
    ``mma.sync``/``wmma``, 32 queries per CTA).  Here every (batch, head) pair is a batch entry of the tcgen05
    forward kernel with one head — ``[B, H, S, 128]`` is read in place as ``[B·H, S, 1, 128]`` — so no transposed
    copy is made.  fp16 inputs are computed in bf16 and returned as fp16; shapes the kernel does not cover
    (head_dim ≠ 128, ``S % 128 ≠ 0``, CPU) take the PyTorch formula, like the reference's scalar fallback kernel."""
    B, H, S, hd = q.shape
    want = q.dtype
    if q.is_cuda and want in (torch.float16, torch.bfloat16):
        q, k, v = (t.to(torch.bfloat16).contiguous().view(B * H, S, 1, hd) for t in (q, k, v))
        if _native_shape_ok(q, k):
            with torch.no_grad():
                out, _, _, _ = _native().attention_fwd(q, k, v, None, None, causal=causal)
            return out.view(B, H, S, hd).to(want)
        q, k, v = (t.view(B, H, S, hd) for t in (q, k, v))
    with torch.no_grad():
        return F.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=causal).to(want)
