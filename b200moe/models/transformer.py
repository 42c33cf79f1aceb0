"""Stage model of the pipelined decoder and the non-pipelined variant."""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from .. import ops
from .layers import EmbeddingLayer, LinearLayer, RMSNormLayer, ROPELayer, TransformerLayer

__all__ = ["TransformerLMPipelined", "TransformerLM", "default_d_ff"]


def default_d_ff(d_model: int) -> int:
    return math.ceil(d_model * (8 / 3) / 64) * 64


class _BlockCheckpoint(torch.autograd.Function):
    """Run one block without keeping its activations and run it again in the
    backward pass (``train.activation_recompute: block``)."""

    @staticmethod
    def forward(ctx, block, x):
        ctx.block = block
        ctx.save_for_backward(x)
        with torch.no_grad():
            return block(x)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        x = x.detach().requires_grad_(True)
        with torch.enable_grad():
            y = ctx.block(x)
        torch.autograd.backward(y, dy)
        return None, x.grad


class TransformerLMPipelined(nn.Module):
    """One pipeline stage: stage 0 owns the embedding, every stage owns
    ``num_layers`` blocks sharing one rotary table, the last stage owns the final
    norm and the untied LM head (reference layers.py:381-418).  ``num_layers`` is
    the count per stage."""

    def __init__(self, vocab_size, context_length, d_model, num_layers, num_heads, stage_this, stage_total,
                 num_expert_per_node=1, d_ff=None, theta=10000, dp_group=None,
                 moe_compute_dtype=torch.bfloat16):
        super().__init__()
        d_ff = default_d_ff(d_model) if d_ff is None else d_ff
        self.stage_this, self.stage_total = stage_this, stage_total
        self.vocab_size, self.context_length, self.num_layers = vocab_size, context_length, num_layers
        self.d_model = d_model
        self.token_embeddings = EmbeddingLayer(vocab_size, d_model) if stage_this == 0 else None
        rope = ROPELayer(theta, d_model // num_heads, context_length)
        self.layers = nn.Sequential(*[
            TransformerLayer(d_model, num_heads, d_ff, num_expert_per_node=num_expert_per_node, RoPELayer=rope,
                             dp_group=dp_group, moe_compute_dtype=moe_compute_dtype)
            for _ in range(num_layers)])
        last = stage_this == stage_total - 1
        self.ln_final = RMSNormLayer(d_model) if last else None
        self.lm_head = LinearLayer(d_model, vocab_size) if last else None
        self.block_recompute = False
        self.activation_dtype = None  # set by the FSDP wrapper (bf16 on GPU)

    @property
    def is_first(self):
        return self.stage_this == 0

    @property
    def is_last(self):
        return self.stage_this == self.stage_total - 1

    def hidden(self, x, return_aux_loss=False):
        """Embedding (stage 0) and the blocks; returns hidden states."""
        if self.is_first:
            x = self.token_embeddings(x)
            if self.activation_dtype is not None:
                x = x.to(self.activation_dtype)
        aux = x.new_zeros((), dtype=torch.float32) if return_aux_loss else None
        for layer in self.layers:
            if return_aux_loss:
                x, layer_aux = layer(x, return_aux_loss=True)
                aux = aux + layer_aux
            elif self.block_recompute and torch.is_grad_enabled():
                x = _BlockCheckpoint.apply(layer, x)
            else:
                x = layer(x)
        return (x, aux) if return_aux_loss else x

    def forward(self, x, return_aux_loss=False):
        out = self.hidden(x, return_aux_loss)
        x, aux = out if return_aux_loss else (out, None)
        if self.is_last:
            x = self.lm_head(self.ln_final(x))
        return (x, aux) if return_aux_loss else x

    def loss(self, x, targets, return_aux_loss=False, grad_scale=None):
        """Last stage only: mean next-token loss with the head fused into the
        loss kernel; the logits are never returned.  ``grad_scale``: the factor
        the caller will back-propagate into the loss, if it knows it already
        (lets the head form its gradients chunk by chunk in the forward pass)."""
        out = self.hidden(x, return_aux_loss)
        x, aux = out if return_aux_loss else (out, None)
        weight = self.lm_head.compute_weight if self.lm_head.compute_weight is not None else self.lm_head.weight
        value = ops.lm_head_cross_entropy(self.ln_final(x), weight, targets, grad_scale)
        return (value, aux) if return_aux_loss else value


class TransformerLM(TransformerLMPipelined):
    """Whole model on one rank (reference layers.py:359-379)."""

    def __init__(self, vocab_size, context_length, d_model, num_layers, num_heads, num_expert_per_node=1,
                 d_ff=None, theta=10000, dp_group=None, moe_compute_dtype=torch.bfloat16):
        super().__init__(vocab_size, context_length, d_model, num_layers, num_heads, 0, 1,
                         num_expert_per_node=num_expert_per_node, d_ff=d_ff, theta=theta, dp_group=dp_group,
                         moe_compute_dtype=moe_compute_dtype)
