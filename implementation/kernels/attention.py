"""Attention entry points under the reference's names (implementation/kernels/
attention.py): autograd functions taking ``(k, q, v)`` and an ``is_causal`` flag."""
import torch

from b200moe.ops.functional import attention_ref


class FlashAttentionFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, k, q, v, is_causal=False):
        ctx.causal = is_causal
        ctx.save_for_backward(k, q, v)
        return _attend(k, q, v, is_causal)

    @staticmethod
    def backward(ctx, dout):
        k, q, v = (t.detach().requires_grad_(True) for t in ctx.saved_tensors)
        with torch.enable_grad():
            out = _attend(k, q, v, ctx.causal)
        dk, dq, dv = torch.autograd.grad(out, (k, q, v), dout)
        return dk, dq, dv, None


def _attend(k, q, v, causal):
    """``[B, S, hd]`` single-head attention."""
    out = attention_ref(q.unsqueeze(2), k.unsqueeze(2), v.unsqueeze(2), causal=causal)
    return out.squeeze(2)


FlashAttentionTritonFunc = FlashAttentionFunc
