"""Mixture-of-experts ops: router, dispatch plan, grouped SwiGLU experts, combine.

Semantics follow the reference (implementation/layers.py:100-246): softmax over
all experts, top-2, renormalised weights, no token dropping, slots ordered by
``(expert, token·k + j)``, experts laid out expert-major on the owning rank with
the contribution of source rank 0 first.  What differs is the mechanism:

* the plan is computed on the device (counting sort), with no per-expert
  ``nonzero`` loop and no host round trip when the expert group has one rank;
* every expert's row segment is padded to ``ALIGN`` rows (zero rows), so all
  GEMM tiles are whole and belong to one expert;
* expert weight gradients accumulate into ``main_grad`` buffers from the
  weight-gradient GEMM itself.

On CUDA the whole block runs as ``native.moe_*`` kernels (``_MoEFused``); the
code in this file that uses ``torch.distributed`` collectives is the CPU/gloo
tier and the NCCL A/B baseline.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import functional as Fn

ALIGN = 128


def _native():
    from . import native
    return native


def _use_native(t, op):
    from . import use_native
    return use_native(t, op)


# ----------------------------------------------------------------------------- router
class _RouterTop2(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits):
        weights, idx, probs = _native().router_top2_fwd(logits)
        ctx.save_for_backward(probs, idx, weights)
        ctx.mark_non_differentiable(idx)
        return weights, idx

    @staticmethod
    def backward(ctx, dweights, _didx):
        probs, idx, weights = ctx.saved_tensors
        return _native().router_top2_bwd(dweights.contiguous(), probs, idx, weights)


def router_top2(logits: torch.Tensor):
    """``(weights fp32 [T,2], idx int64 [T,2])``: softmax over experts, top-2,
    weights renormalised to sum to one."""
    if _use_native(logits, "router"):
        return _RouterTop2.apply(logits)
    return Fn.router_top2_ref(logits, 2)


# ----------------------------------------------------------------------------- plan
@dataclass
class DispatchPlan:
    """Where every ``(token, j)`` slot goes.

    ``order``        slot ids sorted by ``(expert, slot)``                       [T·k]
    ``recv_to_row``  landing row (padded expert-major) of each received row     [R]
    ``offs``         cumulative padded segment ends per local expert, int32     [E_local]
    ``rows``         number of rows of the padded buffer (a Python int)
    ``send_splits`` / ``recv_splits``  per-rank row counts (host lists) when the
                     expert group has more than one rank, else ``None``
    ``counts``       global slot count per expert (device)                      [E_total]
    """
    order: torch.Tensor
    recv_to_row: torch.Tensor
    offs: torch.Tensor
    rows: int
    send_splits: list | None
    recv_splits: list | None
    counts: torch.Tensor


def _exclusive_cumsum(t: torch.Tensor, dim: int = 0) -> torch.Tensor:
    return torch.cumsum(t, dim) - t


def build_plan(idx: torch.Tensor, num_experts_total: int, group=None, align: int = ALIGN) -> DispatchPlan:
    """Device-side counting sort of the slots plus the landing layout."""
    ep = 1 if group is None else dist.get_world_size(group)
    e_local = num_experts_total // ep
    flat = idx.reshape(-1)
    n = flat.numel()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts_total)
    send_splits = recv_splits = None
    if ep == 1:
        recv_counts = counts.view(1, e_local)
        n_recv = n
    else:
        recv_flat = torch.empty_like(counts)
        dist.all_to_all_single(recv_flat, counts, group=group)
        recv_counts = recv_flat.view(ep, e_local)
        both = torch.stack((counts.view(ep, e_local).sum(1), recv_counts.sum(1))).cpu()
        send_splits, recv_splits = both[0].tolist(), both[1].tolist()
        n_recv = int(sum(recv_splits))
    per_expert = recv_counts.sum(0)
    padded = (per_expert + align - 1) // align * align
    ends = torch.cumsum(padded, 0)
    base = (ends - padded).unsqueeze(0) + _exclusive_cumsum(recv_counts, 0)      # [ep, e_local]
    flat_counts = recv_counts.reshape(-1)
    seg_start = _exclusive_cumsum(flat_counts, 0)
    seg_of_row = torch.repeat_interleave(torch.arange(flat_counts.numel(), device=idx.device),
                                         flat_counts, output_size=n_recv)
    recv_to_row = base.reshape(-1)[seg_of_row] + (torch.arange(n_recv, device=idx.device) - seg_start[seg_of_row])
    rows = (n_recv + e_local * (align - 1) + align - 1) // align * align
    return DispatchPlan(order, recv_to_row, ends.to(torch.int32), rows, send_splits, recv_splits, counts)


class _AllToAllRows(torch.autograd.Function):
    """Uneven row all-to-all; the backward pass is the reverse exchange
    (reference ``TensorExchange``, layers.py:14-52)."""

    @staticmethod
    def forward(ctx, rows, send_splits, recv_splits, group):
        ctx.meta = (send_splits, recv_splits, group)
        out = rows.new_empty((sum(recv_splits), *rows.shape[1:]))
        dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_splits,
                               input_split_sizes=send_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, dout):
        send_splits, recv_splits, group = ctx.meta
        dsent = dout.new_empty((sum(send_splits), *dout.shape[1:]))
        dist.all_to_all_single(dsent, dout.contiguous(), output_split_sizes=send_splits,
                               input_split_sizes=recv_splits, group=group)
        return dsent, None, None, None


# ----------------------------------------------------------------------------- experts
def _gmm_nt(x, w, offs):
    """rows of group e times ``w[e]ᵀ``; ``w`` is ``[E, N, K]``."""
    if hasattr(F, "grouped_mm") and x.dtype in (torch.bfloat16, torch.float32):
        try:
            return F.grouped_mm(x, w.to(x.dtype).transpose(-1, -2), offs=offs)
        except (RuntimeError, NotImplementedError):
            pass
    return Fn.grouped_mm_ref(x, w, offs)


def _gmm_nn(dy, w, offs):
    """rows of group e times ``w[e]``; ``w`` is ``[E, N, K]``, result ``[R, K]``."""
    if hasattr(F, "grouped_mm") and dy.dtype in (torch.bfloat16, torch.float32):
        try:
            return F.grouped_mm(dy, w.to(dy.dtype), offs=offs)
        except (RuntimeError, NotImplementedError):
            pass
    return Fn.grouped_mm_ref(dy, w.transpose(-1, -2), offs)


def _gmm_tn(dy, x, offs, num_experts):
    """``out[e] = dy[rows e]ᵀ @ x[rows e]`` -> ``[E, N, K]`` (fp32)."""
    if hasattr(F, "grouped_mm") and dy.dtype in (torch.bfloat16, torch.float32):
        try:
            return F.grouped_mm(dy.t(), x, offs=offs).float()
        except (RuntimeError, NotImplementedError):
            pass
    out = torch.zeros(num_experts, dy.shape[1], x.shape[1], dtype=torch.float32, device=dy.device)
    start = 0
    for e, end in enumerate(offs.tolist()):
        if end > start:
            out[e] = dy[start:end].float().t() @ x[start:end].float()
        start = end
    return out


def _accumulate(param, grad_fp32):
    main_grad = getattr(param, "main_grad", None)
    if main_grad is not None:
        main_grad.add_(grad_fp32.to(main_grad.dtype))
        return None
    return grad_fp32.to(param.dtype)


class _GroupedSwiGLU(torch.autograd.Function):
    """``y = (silu(x W1ᵀ) · (x W3ᵀ)) W2ᵀ`` per expert segment (reference
    ``GroupedPositionWiseFFLayer``, layers.py:215-246) with a hand-written
    backward pass.  ``recompute`` drops the gate/up activations and rebuilds
    them in the backward pass."""

    @staticmethod
    def forward(ctx, x, w1, w2, w3, offs, recompute):
        gate = _gmm_nt(x, w1, offs)
        up = _gmm_nt(x, w3, offs)
        hidden = Fn.swiglu_ref(gate, up)
        y = _gmm_nt(hidden, w2, offs)
        ctx.params = (w1, w2, w3)
        ctx.recompute = recompute
        if recompute:
            ctx.save_for_backward(x, offs)
        else:
            ctx.save_for_backward(x, offs, gate, up)
        return y

    @staticmethod
    def backward(ctx, dy):
        w1, w2, w3 = ctx.params
        if ctx.recompute:
            x, offs = ctx.saved_tensors
            gate, up = _gmm_nt(x, w1, offs), _gmm_nt(x, w3, offs)
        else:
            x, offs, gate, up = ctx.saved_tensors
        dy = dy.contiguous()
        num_experts = w1.shape[0]
        hidden = Fn.swiglu_ref(gate, up)
        dhidden = _gmm_nn(dy, w2, offs).float()
        gf, uf = gate.float(), up.float()
        sig = torch.sigmoid(gf)
        dgate = (dhidden * uf * sig * (1.0 + gf * (1.0 - sig))).to(x.dtype)
        dup = (dhidden * gf * sig).to(x.dtype)
        dx = _gmm_nn(dgate, w1, offs) + _gmm_nn(dup, w3, offs)
        dw2 = _accumulate(w2, _gmm_tn(dy, hidden, offs, num_experts))
        dw1 = _accumulate(w1, _gmm_tn(dgate, x, offs, num_experts))
        dw3 = _accumulate(w3, _gmm_tn(dup, x, offs, num_experts))
        return dx, dw1, dw2, dw3, None, None


def grouped_swiglu(x, w1, w2, w3, offs, recompute: bool = False):
    return _GroupedSwiGLU.apply(x, w1, w2, w3, offs, recompute)


# ----------------------------------------------------------------------------- full block
def aux_loss_from(logits, idx, num_experts_total: int, k: int, group=None):
    """Switch-style balance loss ``E · Σ_e f_e · P_e`` with the assignment counts
    summed over the expert group (reference layers.py:144-151)."""
    ep = 1 if group is None else dist.get_world_size(group)
    counts = torch.bincount(idx.reshape(-1), minlength=num_experts_total).float()
    if ep > 1:
        dist.all_reduce(counts, group=group)
    assignments = counts.sum().clamp_min(1)
    mean_probs = logits.float().softmax(-1).sum(0) * (ep * k / assignments)
    return num_experts_total * (counts / assignments * mean_probs).sum()


def moe_ffn(x: torch.Tensor, weights: torch.Tensor, idx: torch.Tensor, w1, w2, w3, *,
            group=None, recompute: bool = False, budget=None) -> torch.Tensor:
    """Dispatch ``x [T, D]`` to its top-2 experts, run them, combine with the
    renormalised weights.  ``w1, w3: [E_local, d_ff, D]``, ``w2: [E_local, D, d_ff]``."""
    tokens, k = idx.shape
    ep = 1 if group is None else dist.get_world_size(group)
    if _use_native(x, "moe") and ep == 1:
        from .moe_fused import moe_ffn_fused
        return moe_ffn_fused(x, weights, idx, w1, w2, w3, recompute=recompute, budget=budget)
    plan = build_plan(idx, w1.shape[0] * ep, group)
    sent = x[plan.order // k]
    received = sent if ep == 1 else _AllToAllRows.apply(sent, plan.send_splits, plan.recv_splits, group)
    x_perm = x.new_zeros(plan.rows, x.shape[1]).index_copy(0, plan.recv_to_row, received)
    y_perm = grouped_swiglu(x_perm, w1, w2, w3, plan.offs, recompute)
    back = y_perm[plan.recv_to_row]
    if ep > 1:
        back = _AllToAllRows.apply(back, plan.recv_splits, plan.send_splits, group)
    slots = back.new_zeros(tokens * k, x.shape[1]).index_copy(0, plan.order, back)
    out = (slots.view(tokens, k, -1).float() * weights.unsqueeze(-1).float()).sum(1)
    return out.to(x.dtype)
