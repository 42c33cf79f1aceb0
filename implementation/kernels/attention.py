"""Attention entry points under the reference's names (implementation/kernels/
attention.py): autograd functions taking ``(k, q, v)`` and an ``is_causal`` flag."""
from b200moe.ops.attention import attention, flash_attention_forward  # noqa: F401


class FlashAttentionFunc:
    """``FlashAttentionFunc.apply(k, q, v, is_causal)`` like the reference's autograd function; differentiation goes
    through the attention op itself (flash backward kernels on a GPU)."""

    @staticmethod
    def apply(k, q, v, is_causal=False):
        return _attend(k, q, v, is_causal)


def _attend(k, q, v, causal):
    """``[B, S, hd]`` single-head attention; on a GPU with bf16, head_dim 128 and ``S % 128 == 0`` this is the
    tcgen05 flash kernel pair (forward and backward), otherwise the PyTorch formula."""
    out = attention(q.unsqueeze(2), k.unsqueeze(2), v.unsqueeze(2), causal=causal)
    return out.squeeze(2)


FlashAttentionTritonFunc = FlashAttentionFunc
