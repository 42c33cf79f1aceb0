"""Attention entry points under the reference's names (implementation/kernels/attention.py).

The reference has a tiled PyTorch flash attention (``FlashAttentionFunc``, :11-57), a Triton forward kernel with a
compiled PyTorch backward (``FlashAttentionTritonFunc`` + ``attention_forward`` + ``attention_pytorch``, :60-190),
all on ``[batch, sequence, head_dim]`` tensors with the queries as FIRST argument.  Here the same names run this
framework's attention op: the tcgen05 forward and backward kernels for bf16, head_dim 128 and ``S % 128 == 0`` on a
GPU, the PyTorch formula otherwise.  There is no Triton in this build: ``attention_forward[grid](...)`` keeps the call
shape of a Triton launch and fills ``O`` and ``L`` with the same kernels.
"""
import math

import torch

from b200moe.ops.attention import attention, flash_attention_forward  # noqa: F401


def _attend(q, k, v, causal):
    """``[B, S, hd]`` single-head attention, differentiable."""
    return attention(q.unsqueeze(2), k.unsqueeze(2), v.unsqueeze(2), causal=bool(causal)).squeeze(2)


class FlashAttentionFunc:
    """``FlashAttentionFunc.apply(q, k, v, is_causal=False)``: the first argument holds the queries, as in the
    reference's ``forward(ctx, q, k, v, is_causal)``.  (The reference's PyTorch variant accepts ``is_causal`` and
    ignores it, :13-37; this one applies the mask.)  Differentiation goes through the attention op itself."""

    @staticmethod
    def apply(q, k, v, is_causal=False):
        return _attend(q, k, v, is_causal)

    def __call__(self, *args, **kwargs):          # the reference's layer writes ``FlashAttentionTritonFunc().apply``
        return self.apply(*args, **kwargs)


FlashAttentionTritonFunc = FlashAttentionFunc


def _scores(q, k, l, mask):
    """Probabilities rebuilt from the saved log-sum-exp: ``exp(q kᵀ/√d − L)`` with masked entries at zero."""
    s = torch.einsum("...qd,...kd->...qk", q.float(), k.float()) / math.sqrt(k.shape[-1])
    if mask is not None:
        s = s.masked_fill(mask.to(torch.bool).logical_not(), float("-inf"))
    return torch.exp(s - l.float().unsqueeze(-1))


def attention_pytorch(q, k, v, o, do, l, mask):
    """Backward pass of attention from the saved output and log-sum-exp, in plain PyTorch (the reference compiles
    the same formula for its Triton function's backward, :100-110).  ``mask``: 1 where a query may see a key, or
    ``None``.  Returns ``(dq, dk, dv, None)`` in the inputs' dtype."""
    scale = 1.0 / math.sqrt(k.shape[-1])
    p = _scores(q, k, l, mask)
    do32 = do.float()
    delta = (o.float() * do32).sum(dim=-1, keepdim=True)
    dv = torch.einsum("...qk,...qv->...kv", p, do32)
    ds = p * (torch.einsum("...qv,...kv->...qk", do32, v.float()) - delta)
    dq = torch.einsum("...qk,...kd->...qd", ds, k.float()) * scale
    dk = torch.einsum("...qk,...qd->...kd", ds, q.float()) * scale
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None


class _ForwardLauncher:
    """Stands where the reference has a ``@triton.jit`` kernel: ``attention_forward[grid](Q, K, V, O, L, <14 strides>,
    n_queries, n_keys, scale, D, q_tile, k_tile, is_causal)`` writes the attention output into ``O`` and the
    log-sum-exp of the scaled scores into ``L``.  Grid, strides and tile sizes are accepted and not needed: the
    tensors carry their own layout and the kernel picks its tiles."""

    def __getitem__(self, grid):
        return self

    def __call__(self, Q, K, V, O, L, *layout, is_causal=False, **named):
        # positional tail of the reference's launch: 14 strides, n_queries, n_keys, scale, D, q_tile, k_tile, is_causal
        if len(layout) > 20:
            is_causal = bool(layout[20])
        is_causal = bool(named.get("is_causal", is_causal))
        scale = named.get("scale", layout[16] if len(layout) > 16 else 1.0 / math.sqrt(K.shape[-1]))
        q4, k4, v4 = (t.unsqueeze(2) for t in (Q, K, V))
        native_ok = (Q.is_cuda and Q.dtype == torch.bfloat16 and Q.shape[-1] == 128 and Q.shape[-2] % 128 == 0
                     and K.shape[-2] == Q.shape[-2] and abs(scale * math.sqrt(K.shape[-1]) - 1.0) < 1e-6)
        if native_ok:
            from b200moe.ops import native, use_native
            if use_native(q4, "attention"):
                with torch.no_grad():
                    out, lse, _, _ = native.attention_fwd(q4.contiguous(), k4.contiguous(), v4.contiguous(), None,
                                                          None, causal=is_causal)
                O.copy_(out.squeeze(2))
                L.copy_(lse.squeeze(1))
                return
        with torch.no_grad():
            s = torch.einsum("...qd,...kd->...qk", Q.float(), K.float()) * scale
            if is_causal:
                nq, nk = Q.shape[-2], K.shape[-2]
                allowed = torch.arange(nq, device=Q.device)[:, None] >= torch.arange(nk, device=Q.device)[None, :]
                s = s.masked_fill(~allowed, float("-inf"))
            lse = torch.logsumexp(s, dim=-1)
            O.copy_(torch.einsum("...qk,...kv->...qv", torch.exp(s - lse.unsqueeze(-1)), V.float()))
            L.copy_(lse)


attention_forward = _ForwardLauncher()
