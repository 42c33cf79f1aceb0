"""Plain PyTorch statements of every op.

These are the numerical contract (reference implementation/nnfunctions.py and
implementation/layers.py) written with differentiable torch operations.  They
run the CPU/gloo plumbing tier and serve as the fp32 oracle that the sm_100a
kernels are tested against; the GPU training path does not call them.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

__all__ = [
    "softmax", "silu", "cross_entropy", "gradient_clipping", "gradient_clippling", "sample_output",
    "dot_product_att", "rmsnorm_ref", "rope_tables", "apply_rope_ref", "attention_ref",
    "router_top2_ref", "swiglu_ref", "grouped_mm_ref", "log_softmax", "clip_gradient",
]


def softmax(x: torch.Tensor, dim_sum: int = -1, mask: torch.Tensor | None = None) -> torch.Tensor:
    """Max-subtracted softmax; an optional 0/1 mask multiplies the exponentials
    (reference nnfunctions.py:37-43)."""
    shifted = torch.exp(x - x.amax(dim=dim_sum, keepdim=True))
    if mask is not None:
        shifted = shifted * mask.to(shifted.dtype)
    return shifted / shifted.sum(dim=dim_sum, keepdim=True)


def log_softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    shifted = x - x.amax(dim=dim, keepdim=True)
    return shifted - torch.log(torch.exp(shifted).sum(dim=dim, keepdim=True))


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean token negative log-likelihood computed in fp32 (reference
    nnfunctions.py:56-64)."""
    logits = logits.float()
    logits = logits - logits.amax(dim=-1, keepdim=True)
    lse = torch.log(torch.exp(logits).sum(-1))
    picked = logits.gather(-1, targets.unsqueeze(-1)).squeeze(-1)
    return (lse - picked).mean()


def gradient_clipping(params, max_l2: float, eps: float = 1e-6) -> torch.Tensor:
    """Scale every ``.grad`` by ``max_l2 / (norm + eps)`` when the global L2 norm
    exceeds ``max_l2`` (reference nnfunctions.py:9-17); returns the norm."""
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return torch.zeros(())
    norm = torch.sqrt(sum(torch.sum(g.float() ** 2) for g in grads))
    if norm > max_l2:
        scale = max_l2 / (norm + eps)
        for g in grads:
            g.mul_(scale.to(g.dtype))
    return norm


gradient_clippling = gradient_clipping  # the reference's spelling
clip_gradient = gradient_clipping


def sample_output(logits: torch.Tensor, t: float = 1.0, p: float = 0.0) -> torch.Tensor:
    """Temperature + nucleus sampling over ``[batch, vocab]`` logits: the most
    likely token always stays, further tokens stay while the running mass is
    below ``p`` (reference nnfunctions.py:66-81)."""
    prob = softmax(logits / t, dim_sum=-1)
    values, indices = torch.sort(prob, dim=-1, descending=True)
    running = torch.cumsum(values, dim=-1)
    keep = (running < p).to(values.dtype)
    keep[:, 0] = 1.0
    choice = torch.multinomial(values * keep, num_samples=1)
    return torch.gather(indices, -1, choice)


def dot_product_att(k, q, v, mask=None):
    """Naive attention with the reference's argument order (k, q, v)."""
    scores = torch.einsum("...ik,...jk->...ij", q, k) / math.sqrt(k.shape[-1])
    return torch.einsum("...ki,...ij->...kj", softmax(scores, -1, mask), v)


def rmsnorm_ref(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    xf = x.float()
    normed = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (normed * weight.float()).to(x.dtype)


def rope_tables(theta: float, head_dim: int, max_seq_len: int, device=None):
    """``cos, sin`` of shape ``[seq, head_dim/2]``.  Pair ``i`` (elements ``2i``
    and ``2i+1``, adjacent) turns by ``pos · theta^(-2i/head_dim)`` (reference
    layers.py:275-279 with ``i`` counted from 1: ``theta^((2-2i)/d)``)."""
    half = torch.arange(0, head_dim // 2, dtype=torch.float32, device=device)
    inv_freq = theta ** (-2.0 * half / head_dim)
    angles = torch.arange(max_seq_len, dtype=torch.float32, device=device)[:, None] * inv_freq[None, :]
    return torch.cos(angles), torch.sin(angles)


def apply_rope_ref(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate adjacent pairs of the last dim; ``x`` is ``[..., seq, head_dim]``
    and the tables are ``[seq, head_dim/2]``.  ``(a, b) -> (a·cos − b·sin,
    a·sin + b·cos)`` in fp32."""
    pairs = x.float().unflatten(-1, (-1, 2))
    a, b = pairs[..., 0], pairs[..., 1]
    rotated = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1)
    return rotated.flatten(-2).to(x.dtype)


def attention_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cos=None, sin=None,
                  causal: bool = True) -> torch.Tensor:
    """GQA attention on ``[B, S, H, hd]`` tensors with optional RoPE on q and k;
    returns ``[B, S, Hq, hd]``."""
    qh, kh, vh = (t.transpose(1, 2) for t in (q, k, v))
    if cos is not None:
        seq = qh.shape[-2]
        qh = apply_rope_ref(qh, cos[:seq], sin[:seq])
        kh = apply_rope_ref(kh, cos[:seq], sin[:seq])
    ratio = qh.shape[1] // kh.shape[1]
    if ratio > 1:
        kh = kh.repeat_interleave(ratio, dim=1)
        vh = vh.repeat_interleave(ratio, dim=1)
    out = F.scaled_dot_product_attention(qh, kh, vh, is_causal=causal)
    return out.transpose(1, 2)


def router_top2_ref(logits: torch.Tensor, k: int = 2):
    """Softmax over experts, top-k, renormalise the kept probabilities
    (reference layers.py:126-127,142).  Returns ``(weights fp32 [T,k], idx [T,k])``."""
    probs = softmax(logits.float(), dim_sum=-1)
    top, idx = probs.topk(k, dim=-1)
    return top / top.sum(dim=-1, keepdim=True), idx


def swiglu_ref(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return (silu(gate.float()) * up.float()).to(gate.dtype)


def grouped_mm_ref(x: torch.Tensor, w: torch.Tensor, offs: torch.Tensor) -> torch.Tensor:
    """``out[rows of group e] = x[rows of group e] @ w[e].T`` with ``offs`` the
    cumulative row ends; rows past ``offs[-1]`` are zero.  Loop form for tests."""
    out = x.new_zeros(x.shape[0], w.shape[1])
    start = 0
    for e, end in enumerate(offs.tolist()):
        if end > start:
            out[start:end] = x[start:end] @ w[e].to(x.dtype).T
        start = end
    return out
