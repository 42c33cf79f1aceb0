"""Model layers.

Module and parameter names match the reference (implementation/layers.py) so a
checkpoint's ``model.state_dict`` keys are the same:
``token_embeddings.weight``, ``layers.{i}.ln1.weight``,
``layers.{i}.attn.{k,q,v,output}_proj.weight``, ``layers.{i}.ln2.weight``,
``layers.{i}.ffn.experts.{w1,w2,w3}``, ``layers.{i}.ffn.router.weight``,
``ln_final.weight``, ``lm_head.weight``.

Parameters of ``LinearLayer``/``EmbeddingLayer``/``RMSNormLayer`` are fp32 master
copies.  The FSDP wrapper attaches to each sharded layer a ``compute_weight``
(the full bf16 weight it keeps gathered) and, on attention, a fused
``qkv_weight`` view, which the forward pass prefers over ``weight``.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from .. import ops
from ..ops import functional as Fn

__all__ = [
    "LinearLayer", "EmbeddingLayer", "RMSNormLayer", "ROPELayer", "MultiHeadLayerLL",
    "GroupedPositionWiseFFLayer", "PositionWiseFFLayer", "MoELayerMulti", "TransformerLayer",
    "TensorExchange", "Attention_Simple", "Attention_Flash",
]


class TensorExchange(torch.autograd.Function):
    """Variable-size row exchange over the expert group, differentiable.

    ``sent_splits`` holds one row count per *global expert*; rows are grouped by
    destination rank.  Returns the received rows and the received per-expert
    counts (reference layers.py:14-52)."""

    @staticmethod
    def forward(ctx, sent_tensors, sent_splits, dp_group=None):
        import torch.distributed as dist
        world = dist.get_world_size(dp_group)
        per_rank = len(sent_splits) // world
        send = torch.tensor(sent_splits, dtype=torch.int64, device=sent_tensors.device)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=dp_group)
        recv_list = [int(v) for v in recv.cpu().tolist()]
        send_rank = [sum(sent_splits[i:i + per_rank]) for i in range(0, len(sent_splits), per_rank)]
        recv_rank = [sum(recv_list[i:i + per_rank]) for i in range(0, len(recv_list), per_rank)]
        out = sent_tensors.new_empty((sum(recv_rank), *sent_tensors.shape[1:]))
        dist.all_to_all_single(out, sent_tensors.contiguous(), output_split_sizes=recv_rank,
                               input_split_sizes=send_rank, group=dp_group)
        ctx.meta = (send_rank, recv_rank, dp_group)
        return out, recv_list

    @staticmethod
    def backward(ctx, d_recv, *_):
        import torch.distributed as dist
        send_rank, recv_rank, group = ctx.meta
        d_sent = d_recv.new_empty((sum(send_rank), *d_recv.shape[1:]))
        dist.all_to_all_single(d_sent, d_recv.contiguous(), output_split_sizes=send_rank,
                               input_split_sizes=recv_rank, group=group)
        return d_sent, None, None


def _trunc_normal(shape, std, device=None, dtype=None):
    tensor = torch.empty(shape, device=device, dtype=torch.float32)
    nn.init.trunc_normal_(tensor, 0.0, std, -3 * std, 3 * std)
    return tensor.to(dtype) if dtype is not None else tensor


class LinearLayer(nn.Module):
    """``y = x Wᵀ`` with ``W [d_out, d_in]``, fp32 master, truncated-normal init
    ``σ = sqrt(2/(d_in+d_out))`` cut at ±3σ, no bias (reference layers.py:55-69)."""

    def __init__(self, d_in, d_out, device=None, dtype=None):
        super().__init__()
        self.d_in, self.d_out = d_in, d_out
        self.weight = nn.Parameter(_trunc_normal((d_out, d_in), math.sqrt(2 / (d_in + d_out)), device))
        self.compute_weight = None

    def forward(self, x):
        weight = self.compute_weight if self.compute_weight is not None else self.weight
        return ops.linear(x, weight)


class EmbeddingLayer(nn.Module):
    """Row lookup; ``N(0,1)`` truncated at ±3 (reference layers.py:72-82)."""

    def __init__(self, num_embeddings, embedding_dim, device=None, dtype=None):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.weight = nn.Parameter(_trunc_normal((num_embeddings, embedding_dim), 1.0, device))
        self.compute_weight = None

    def forward(self, x):
        weight = self.compute_weight if self.compute_weight is not None else self.weight
        return ops.embedding(x, weight)


class RMSNormLayer(nn.Module):
    """fp32 RMS normalisation with a learned gain initialised to one
    (reference layers.py:84-97)."""

    def __init__(self, d_model, eps: float = 1e-5, device=None, dtype=None):
        super().__init__()
        self.d_model, self.eps = d_model, eps
        self.weight = nn.Parameter(torch.ones(d_model, device=device))

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.eps)


class ROPELayer(nn.Module):
    """Rotary tables for adjacent-pair rotation (reference layers.py:268-287).
    Buffers are non-persistent, so they never appear in a checkpoint."""

    def __init__(self, theta: float, d_k: int, max_seq_len: int, device=None):
        super().__init__()
        self.theta, self.d_k, self.max_seq_len = theta, d_k, max_seq_len
        cos, sin = Fn.rope_tables(theta, d_k, max_seq_len, device)
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    def forward(self, x, token_positions):
        """``x [..., seq, d_k]``; gathers table rows by position."""
        return Fn.apply_rope_ref(x, self.cos[token_positions], self.sin[token_positions])


class MultiHeadLayerLL(nn.Module):
    """Causal 4:1 grouped-query attention with RoPE on q and k (reference
    layers.py:290-333).  Attribute order k, q, v, output is the reference's and
    fixes the FSDP module order."""

    def __init__(self, d_model, num_heads, device=None, dtype=None, use_rope=True, RoPE=None):
        super().__init__()
        if d_model % num_heads:
            raise ValueError(f"d_model ({d_model}) must be divisible by num_heads ({num_heads})")
        if num_heads % 4:
            raise ValueError(f"num_heads ({num_heads}) must be divisible by 4 for 4:1 grouped-query attention")
        self.d_model, self.num_heads = d_model, num_heads
        self.num_kv_heads = num_heads // 4
        self.head_dim = d_model // num_heads
        kv_dim = self.num_kv_heads * self.head_dim
        self.k_proj = LinearLayer(d_model, kv_dim, device=device)
        self.q_proj = LinearLayer(d_model, d_model, device=device)
        self.v_proj = LinearLayer(d_model, kv_dim, device=device)
        self.output_proj = LinearLayer(d_model, d_model, device=device)
        self.use_rope = use_rope
        self.RoPE = (RoPE if RoPE is not None else ROPELayer(10000, self.head_dim, 100000)) if use_rope else None
        self.qkv_weight = None  # fused [q; k; v] view, set by the FSDP wrapper

    def forward(self, x, token_positions=None, mask=None):
        batch, seq = x.shape[0], x.shape[1]
        hq, hkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        fused_rope = False
        if self.qkv_weight is not None:
            from ..ops.attention import attention_backend, fused_qkv_attention
            x2d = x.reshape(batch * seq, -1)
            if (token_positions is None and mask is None and ops.use_native(x2d, "attention")
                    and attention_backend() == "native" and hd == 128 and seq % 128 == 0):
                # RoPE rides in the projection GEMM's epilogue (forward) and in the attention backward kernels'
                # epilogues (its transpose), so q and k are never re-read just to be rotated
                cos, sin = (self.RoPE.cos, self.RoPE.sin) if self.use_rope else (None, None)
                if self.use_rope:
                    qkv = ops.linear_rope(x2d, self.qkv_weight, cos, sin, (hq + hkv) * hd, seq)
                else:
                    qkv = ops.linear(x2d, self.qkv_weight)
                out = fused_qkv_attention(qkv, batch, seq, hq, hkv, hd, cos, sin, pre_rotated=self.use_rope)
                return self.output_proj(out.reshape(batch, seq, hq * hd))
            qkv = ops.linear(x2d, self.qkv_weight)
            if self.use_rope and token_positions is None and mask is None and ops.use_native(qkv, "rope"):
                from ..ops.attention import rope_qk_
                qkv = rope_qk_(qkv, seq, hq + 2 * hkv, hq + hkv, hd, self.RoPE.cos, self.RoPE.sin)
                fused_rope = True
            qkv = qkv.view(batch, seq, hq + 2 * hkv, hd)
            q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hkv], qkv[:, :, hq + hkv:]
        else:
            q = self.q_proj(x).view(batch, seq, hq, hd)
            k = self.k_proj(x).view(batch, seq, hkv, hd)
            v = self.v_proj(x).view(batch, seq, hkv, hd)
        cos = sin = None
        if self.use_rope and not fused_rope:
            cos, sin = self.RoPE.cos, self.RoPE.sin
            if token_positions is not None:
                cos, sin = cos[token_positions], sin[token_positions]
        if mask is not None:
            out = self._masked(q, k, v, cos, sin, mask)
        else:
            out = ops.rope_attention(q, k, v, cos, sin)
        return self.output_proj(out.reshape(batch, seq, hq * hd))

    def _masked(self, q, k, v, cos, sin, mask):
        """Explicit-mask path (non-causal semantics chosen by the caller)."""
        import torch.nn.functional as F
        qh, kh, vh = (t.transpose(1, 2) for t in (q, k, v))
        if cos is not None:
            qh = Fn.apply_rope_ref(qh, cos[:qh.shape[-2]], sin[:qh.shape[-2]])
            kh = Fn.apply_rope_ref(kh, cos[:kh.shape[-2]], sin[:kh.shape[-2]])
        ratio = qh.shape[1] // kh.shape[1]
        kh, vh = kh.repeat_interleave(ratio, 1), vh.repeat_interleave(ratio, 1)
        return F.scaled_dot_product_attention(qh, kh, vh, attn_mask=mask).transpose(1, 2)


class GroupedPositionWiseFFLayer(nn.Module):
    """SwiGLU experts held as three stacked tensors in the compute dtype
    (reference layers.py:215-246)."""

    def __init__(self, num_experts, d_model, d_ff, device=None, dtype=None):
        super().__init__()
        self.num_experts, self.d_model, self.dff = num_experts, d_model, d_ff
        std = math.sqrt(2 / (d_model + d_ff))
        self.w1 = nn.Parameter(_trunc_normal((num_experts, d_ff, d_model), std, device, dtype))
        self.w2 = nn.Parameter(_trunc_normal((num_experts, d_model, d_ff), std, device, dtype))
        self.w3 = nn.Parameter(_trunc_normal((num_experts, d_ff, d_model), std, device, dtype))

    def forward(self, x, offsets, recompute: bool = False):
        from ..ops.moe import grouped_swiglu
        return grouped_swiglu(x, self.w1, self.w2, self.w3, offsets, recompute)


class PositionWiseFFLayer(nn.Module):
    """Dense SwiGLU feed-forward (reference layers.py:249-265)."""

    def __init__(self, d_model, d_ff, device=None, dtype=None):
        super().__init__()
        self.d_model, self.dff = d_model, d_ff
        self.w1 = LinearLayer(d_model, d_ff, device=device)
        self.w2 = LinearLayer(d_ff, d_model, device=device)
        self.w3 = LinearLayer(d_model, d_ff, device=device)

    def forward(self, x):
        gate, up = self.w1(x), self.w3(x)
        return self.w2(Fn.swiglu_ref(gate, up))


class MoELayerMulti(nn.Module):
    """Top-2 routed experts partitioned over ``dp_group`` (reference
    layers.py:100-213).  ``compute dtype`` defaults to bf16; fp32 is accepted so
    the CPU tier can be compared bit-tight against an fp32 oracle."""

    def __init__(self, d_model, d_ff, k=2, num_expert_per_node=4, device=None, dtype=torch.bfloat16,
                 dp_group=None):
        super().__init__()
        import torch.distributed as dist
        self.dp_group = dp_group
        self.world_size = 1 if dp_group is None else dist.get_world_size(dp_group)
        if num_expert_per_node < 1 or not 1 <= k <= self.world_size * num_expert_per_node:
            raise ValueError("Require positive expert count and 1 <= k <= total experts")
        if k != 2:
            raise ValueError("The fused router implements top-2 routing")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Grouped MoE requires torch.bfloat16 compute dtype (float32 on CPU)")
        self.dtype, self.k, self.num_expert_per_node = dtype, k, num_expert_per_node
        self.experts = GroupedPositionWiseFFLayer(num_expert_per_node, d_model, d_ff, device=device, dtype=dtype)
        self.router = LinearLayer(d_model, self.world_size * num_expert_per_node, device=device)
        self.recompute = False
        self.budget = None  # parallel.memory.ActivationBudget of the stage (set by the trainer), or None
        self.comm = None  # peer-memory communication layer, set by the FSDP wrapper (fused backend)

    def forward(self, x, return_aux_loss=False):
        shape, in_dtype = x.shape, x.dtype
        flat = x.reshape(-1, shape[-1]).to(self.dtype)
        experts_total = self.world_size * self.num_expert_per_node
        ep_ctx = None
        if self.comm is not None and self.world_size > 1 and flat.is_cuda:
            ep_ctx = self.comm.ep_context(flat.shape[0], flat.shape[1], experts_total, self.experts.dff)
        if ep_ctx is not None and ops.use_native(flat, "moe"):
            # exchange fused with the expert GEMMs: the router reads the staged copy of the input that the other
            # ranks pull their rows from
            from ..ops.moe_fused import moe_ffn_pull
            seen = {}

            def route(staged):
                seen["logits"] = self.router(staged)
                return ops.router_top2(seen["logits"])

            out, weights, idx = moe_ffn_pull(flat, route, self.experts.w1, self.experts.w2, self.experts.w3, ep_ctx,
                                             recompute=self.recompute, key=id(self), budget=self.budget)
            logits = seen["logits"]
        else:
            logits = self.router(flat)
            weights, idx = ops.router_top2(logits)
            out = ops.moe_ffn(flat, weights, idx, self.experts.w1, self.experts.w2, self.experts.w3,
                              group=self.dp_group if self.world_size > 1 else None,
                              recompute=self.recompute, budget=self.budget)
        out = out.view(shape).to(in_dtype)
        if return_aux_loss:
            from ..ops.moe import aux_loss_from
            aux = aux_loss_from(logits, idx, experts_total, self.k, self.dp_group if self.world_size > 1 else None)
            return out, aux
        return out


    # ---- the reference's two-step form of the same computation (layers.py:140-213) ------------------------------
    # ``forward`` above does not go through these: it hands routing, exchange and experts to one op.  They are kept,
    # with the reference's arguments and return values, for code that drives the steps itself, and they double as a
    # plain-PyTorch statement of what the fused path computes (tests compare the two).
    def _dispatch_tokens(self, x, logits, probs, expert_idx, return_aux_loss):
        """Sort the ``tokens × k`` assignments by global expert, send every row to the rank that owns its expert and
        order what arrives by local expert.  ``x [tokens, d]``, ``probs``/``expert_idx [tokens, k]``.  Returns
        ``(expert_input, cumulative_rows_per_local_expert int32, expert_split_sizes, recv_splits, assignment_order,
        renormalised probs, aux_loss)``."""
        probs = probs / probs.sum(dim=-1, keepdim=True)
        experts_total = self.world_size * self.num_expert_per_node
        group = self.dp_group if self.world_size > 1 else None
        aux_loss = None
        if return_aux_loss:
            from ..ops.moe import aux_loss_from
            aux_loss = aux_loss_from(logits, expert_idx, experts_total, self.k, group)
        flat_idx = expert_idx.reshape(-1)
        assignment_order = torch.argsort(flat_idx, stable=True)          # grouped by expert, token order inside
        split_sizes = torch.bincount(flat_idx, minlength=experts_total).tolist()
        sent = x[assignment_order // self.k]
        if self.world_size == 1:
            received, recv_splits = sent, split_sizes
        else:
            received, recv_splits = TensorExchange.apply(sent, split_sizes, self.dp_group)
        # arrivals are ordered (source rank, local expert); the grouped GEMM wants (local expert, source rank)
        chunks = torch.split(received, recv_splits, dim=0)
        per_expert = [chunks[e::self.num_expert_per_node] for e in range(self.num_expert_per_node)]
        expert_input = torch.cat([c for group_ in per_expert for c in group_], dim=0)
        expert_split_sizes = [c.shape[0] for group_ in per_expert for c in group_]
        rows = torch.tensor([sum(c.shape[0] for c in group_) for group_ in per_expert], device=x.device,
                            dtype=torch.int32)
        return (expert_input, rows.cumsum(dim=0, dtype=torch.int32), expert_split_sizes, recv_splits,
                assignment_order, probs, aux_loss)

    def _combine_tokens(self, expert_outputs, expert_split_sizes, recv_splits, assignment_order, probs, batch_size,
                        context_len, input_dtype):
        """Inverse of ``_dispatch_tokens`` for the experts' outputs: back to (source rank, local expert) order, home
        over the exchange, into assignment order, weighted sum of each token's ``k`` rows."""
        pieces = torch.split(expert_outputs, expert_split_sizes)
        by_rank = [pieces[e * self.world_size + r] for r in range(self.world_size)
                   for e in range(self.num_expert_per_node)]
        sent = torch.cat(by_rank, dim=0)
        if self.world_size == 1:
            returned = sent
        else:
            returned, _ = TensorExchange.apply(sent, recv_splits, self.dp_group)
        rows = torch.empty_like(returned)
        rows[assignment_order] = returned
        mixed = (rows.view(-1, self.k, rows.shape[-1]) * probs.unsqueeze(-1)).sum(dim=1)
        return mixed.view(batch_size, context_len, -1).to(input_dtype)


class TransformerLayer(nn.Module):
    """Pre-norm block: ``x += attn(ln1(x)); x += moe(ln2(x))`` (reference
    layers.py:336-356)."""

    def __init__(self, d_model, num_heads, d_ff, num_expert_per_node=1, RoPELayer=None, dp_group=None,
                 moe_compute_dtype=torch.bfloat16):
        super().__init__()
        self.d_model, self.num_heads, self.d_ff = d_model, num_heads, d_ff
        self.ln1 = RMSNormLayer(d_model)
        self.attn = MultiHeadLayerLL(d_model, num_heads, RoPE=RoPELayer)
        self.ln2 = RMSNormLayer(d_model)
        self.ffn = MoELayerMulti(d_model, d_ff, num_expert_per_node=num_expert_per_node, dp_group=dp_group,
                                 dtype=moe_compute_dtype)

    def forward(self, x, return_aux_loss=False):
        attn_out = self.attn(self.ln1(x))
        x, normed = ops.add_rmsnorm(x, attn_out, self.ln2.weight, self.ln2.eps)
        if return_aux_loss:
            out, aux = self.ffn(normed, return_aux_loss=True)
            return x + out, aux
        return x + self.ffn(normed)


class Attention_Simple(nn.Module):
    """Thin wrapper kept for API parity (reference layers.py:421-428)."""

    def forward(self, k, q, v, mask):
        import torch.nn.functional as F
        return F.scaled_dot_product_attention(q, k, v, attn_mask=mask)


class Attention_Flash(nn.Module):
    """Non-causal flash attention on ``[B, S, hd]`` inputs, called as the reference calls it (layers.py:430-437):
    ``forward(k, q, v, mask)`` hands ``(k, q, v)`` to a function whose first argument holds the queries, so the
    tensor named ``k`` plays the queries and ``mask`` is not used.  Kept that way so that results match."""

    def forward(self, k, q, v, mask=None):
        from ..ops.attention import attention
        squeeze = k.dim() == 3
        queries, keys, values = ((t.unsqueeze(2) if squeeze else t.transpose(1, 2)) for t in (k, q, v))
        out = attention(queries, keys, values, causal=False)
        return out.squeeze(2) if squeeze else out.transpose(1, 2)
