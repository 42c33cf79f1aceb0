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


def _native_ok(q, k, scale=None) -> bool:
    """bf16, head_dim 128, equal lengths that are multiples of 128, on a GPU, scale 1/√d: the tcgen05 kernels."""
    if not (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and q.shape[-2] % 128 == 0
            and k.shape[-2] == q.shape[-2] and q.dim() == 3):
        return False
    if scale is not None and abs(scale * math.sqrt(k.shape[-1]) - 1.0) > 1e-6:
        return False
    from b200moe.ops import use_native
    return use_native(q, "attention")


def _visible(q, k, causal):
    """Boolean ``[Sq, Sk]`` mask of the keys a query may see, or ``None``."""
    if not causal:
        return None
    return torch.arange(q.shape[-2], device=q.device)[:, None] >= torch.arange(k.shape[-2], device=q.device)[None, :]


def _forward_values(q, k, v, causal, scale=None):
    """Attention output and log-sum-exp of the scaled scores for ``[B, S, hd]`` tensors, no graph."""
    with torch.no_grad():
        if _native_ok(q, k, scale):
            from b200moe.ops import native
            out, lse, _, _ = native.attention_fwd(q.unsqueeze(2).contiguous(), k.unsqueeze(2).contiguous(),
                                                  v.unsqueeze(2).contiguous(), None, None, causal=bool(causal))
            return out.squeeze(2), lse.squeeze(1)
        scale = 1.0 / math.sqrt(k.shape[-1]) if scale is None else scale
        s = torch.einsum("...qd,...kd->...qk", q.float(), k.float()) * scale
        visible = _visible(q, k, causal)
        if visible is not None:
            s = s.masked_fill(~visible, float("-inf"))
        lse = torch.logsumexp(s, dim=-1)
        out = torch.einsum("...qk,...kv->...qv", torch.exp(s - lse.unsqueeze(-1)), v.float())
        return out.to(v.dtype), lse


class FlashAttentionFunc(torch.autograd.Function):
    """``FlashAttentionFunc.apply(q, k, v, is_causal=False)`` on ``[B, S, hd]`` tensors: the first argument holds the
    queries, as in the reference's ``forward(ctx, q, k, v, is_causal)``.  (The reference's PyTorch variant accepts
    ``is_causal`` and ignores it, :13-37; this one applies the mask.)  Saves q, k, v, the output and the
    log-sum-exp; the backward pass runs the flash backward kernels where the forward ran the flash kernel, else
    ``attention_pytorch``."""

    @staticmethod
    def forward(ctx, q, k, v, is_causal=False):
        out, lse = _forward_values(q, k, v, is_causal)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.is_causal = bool(is_causal)
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, l = ctx.saved_tensors
        if _native_ok(q, k):
            from b200moe.ops import native
            four = [t.unsqueeze(2).contiguous() for t in (do.to(torch.bfloat16), q, k, v, o)]
            dq, dk, dv = native.attention_bwd(*four, l.unsqueeze(1).contiguous(), causal=ctx.is_causal)
            return dq.squeeze(2), dk.squeeze(2), dv.squeeze(2), None
        visible = _visible(q, k, ctx.is_causal)
        return attention_pytorch(q, k, v, o, do, l, None if visible is None else visible.unsqueeze(0))


class FlashAttentionTritonFunc(FlashAttentionFunc):
    """Same function under the name of the reference's Triton variant (:60-98), which honours ``is_causal``."""


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
    """Stands where the reference has a ``@triton.jit`` kernel: ``attention_forward[grid](Q_ptr, K_ptr, V_ptr, O_ptr,
    L_ptr, <14 strides>, N_QUERIES, N_KEYS, scale, D, Q_TILE_SIZE, K_TILE_SIZE, is_causal)``, positionally or by those
    names, writes the attention output into ``O_ptr`` and the log-sum-exp of the scaled scores into ``L_ptr`` (both
    tensors, as in a Triton launch).  Grid, strides and tile sizes are accepted and not needed: the tensors carry
    their own layout and the kernel picks its tiles."""

    PARAMETERS = ("Q_ptr", "K_ptr", "V_ptr", "O_ptr", "L_ptr",
                  "stride_qb", "stride_qq", "stride_qd", "stride_kb", "stride_kk", "stride_kd",
                  "stride_vb", "stride_vk", "stride_vd", "stride_ob", "stride_oq", "stride_od",
                  "stride_lb", "stride_lq", "N_QUERIES", "N_KEYS", "scale", "D", "Q_TILE_SIZE", "K_TILE_SIZE",
                  "is_causal")

    def __getitem__(self, grid):
        return self

    def __call__(self, *args, **named):
        unknown = set(named) - set(self.PARAMETERS)
        if unknown or len(args) > len(self.PARAMETERS):
            raise TypeError(f"attention_forward: unexpected arguments {sorted(unknown) or len(args)}")
        given = dict(zip(self.PARAMETERS, args))
        given.update(named)
        Q, K, V, O, L = (given[name] for name in self.PARAMETERS[:5])
        out, lse = _forward_values(Q, K, V, bool(given.get("is_causal", False)), given.get("scale"))
        O.copy_(out)
        L.copy_(lse)


attention_forward = _ForwardLauncher()
