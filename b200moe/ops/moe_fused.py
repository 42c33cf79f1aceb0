"""The MoE block as native kernels with a hand-written backward pass.

One rank (``_MoEFused``): plan (device counting sort) → gather rows into the
padded expert-major buffer → grouped gate/up GEMM with the SwiGLU epilogue →
grouped down GEMM → weighted combine; backward: the duals in reverse, with the
three weight-gradient GEMMs accumulating into the experts' ``main_grad``
buffers.  An expert group of several ranks (``_MoEPull``): the row exchange is
part of the expert GEMMs (``b200moe.comm.ep``).  In both, no step involves the
host: tile counts, segment offsets and the tile→expert table stay on the device
and the persistent GEMMs read them there.

Replaces the reference's ``_dispatch_tokens`` / ``GroupedPositionWiseFFLayer`` /
``_combine_tokens`` (implementation/layers.py:139-246) including its per-expert
``nonzero`` loop and ``.cpu()`` split exchange.
"""
from __future__ import annotations

import torch

from . import native

ALIGN = 256       # expert segments are padded to 256 rows (whole 256x256 GEMM tiles)


def capacity_rows(slots: int, num_experts: int) -> int:
    """Worst-case rows of the padded expert-major buffer."""
    return (slots + num_experts * (ALIGN - 1) + ALIGN - 1) // ALIGN * ALIGN


def _wgrad(dy, x, param, offs, num_experts):
    main = getattr(param, "main_grad", None)
    if main is not None:
        native.gemm_tn(dy, x, out=main, accumulate=True, expert_offsets=offs, num_experts=num_experts)
        return None
    return native.gemm_tn(dy, x, out_dtype=param.dtype, expert_offsets=offs, num_experts=num_experts)


class _MoEFused(torch.autograd.Function):
    """The block when the expert group is this rank alone."""

    @staticmethod
    def forward(ctx, x, weights, idx, w1, w2, w3, recompute, budget):
        tokens, dim = x.shape
        experts = w1.shape[0]
        x = x.contiguous()
        weights = weights.float().contiguous()
        cap = capacity_rows(tokens * 2, experts)
        slot_row, row_slot, offs, tile_expert, meta, _ = native.moe_plan(idx, experts, cap)
        x_perm = native.moe_gather(x, row_slot, meta, cap)
        tiles = meta[0:1]
        # what this call keeps for its backward pass: the permuted input and the expert outputs always, the
        # gate/up pre-activations while the stage's activation budget has room for them
        ledger = None
        if budget is not None and any(ctx.needs_input_grad):
            ledger = (cap * dim * 4, cap * w1.shape[1] * 4)
            kept = budget.enter(*ledger)
            recompute = recompute or not kept
            ledger += (not recompute,)
        h, gate, up = native.gemm_swiglu(x_perm, w1, w3, tile_expert, tiles, save_gate_up=not recompute, align256=True)
        y_perm = native.gemm_nt(h, w2, tile_expert=tile_expert, num_m_tiles=tiles, num_experts=experts, align256=True)
        out = native.moe_combine(y_perm, slot_row, weights, tokens)
        ctx.params = (w1, w2, w3)
        ctx.meta_py = (tokens, dim, experts, cap, recompute)
        ctx.budget, ctx.ledger = budget, ledger
        saved = [x_perm, y_perm, weights, offs, tile_expert, meta, slot_row, row_slot]
        if not recompute:
            saved += [gate, up]
        ctx.save_for_backward(*saved)
        return out

    @staticmethod
    def backward(ctx, dout):
        w1, w2, w3 = ctx.params
        tokens, dim, experts, cap, recompute = ctx.meta_py
        saved = list(ctx.saved_tensors)
        x_perm, y_perm, weights, offs, tile_expert, meta, slot_row, row_slot = saved[:8]
        tiles, live_rows = meta[0:1], meta[1:2]
        dout = dout.contiguous()
        ffn = w1.shape[1]
        if recompute:
            _, gate, up = native.gemm_swiglu(x_perm, w1, w3, tile_expert, tiles, save_gate_up=True, align256=True)
        else:
            gate, up = saved[8:10]
        dweights = torch.zeros(tokens, 2, dtype=torch.float32, device=dout.device)
        dy_perm = native.moe_gather(dout, row_slot, meta, cap, scale=weights.view(-1), y_perm=y_perm,
                                    dweights=dweights.view(-1))
        dh = native.gemm_nn(dy_perm, w2, tile_expert=tile_expert, num_m_tiles=tiles, num_experts=experts, align256=True)
        dgu, h = native.swiglu_bwd(dh, gate, up, live_rows=live_rows)
        del dh, gate, up
        dx_perm = native.gemm_nn(dgu, w1, w2=w3, tile_expert=tile_expert, num_m_tiles=tiles, num_experts=experts,
                                 align256=True)
        dw2 = _wgrad(dy_perm, h, w2, offs, experts)
        dw1 = _wgrad(dgu[:, :ffn], x_perm, w1, offs, experts)
        dw3 = _wgrad(dgu[:, ffn:], x_perm, w3, offs, experts)
        dx = native.moe_combine(dx_perm, slot_row, None, tokens)
        if ctx.ledger is not None:
            ctx.budget.leave(*ctx.ledger)
        return dx, dweights, None, dw1, dw2, dw3, None, None


def moe_ffn_fused(x, weights, idx, w1, w2, w3, recompute: bool = False, budget=None):
    """The block on one rank.  ``budget`` (``parallel.memory.ActivationBudget``): when given, the call keeps its
    gate/up pre-activations only while the budget has room and rebuilds them in the backward pass otherwise."""
    return _MoEFused.apply(x, weights, idx, w1, w2, w3, recompute, budget)


# ----------------------------------------------------------------------------- expert-parallel path (comm/ep.py)
class _StageIn(torch.autograd.Function):
    """Copy the block input into a pool slot that the other ranks of the expert group can read.  The router and
    the MoE op both consume the slot tensor, so this node's backward runs after theirs and gives the slot back."""

    @staticmethod
    def forward(ctx, x, epc, slot):
        ctx.epc, ctx.slot = epc, slot
        staged = epc.slot_tensor(slot)
        staged.copy_(x)
        return staged.view_as(x)

    @staticmethod
    def backward(ctx, dx):
        ctx.epc.release(ctx.slot)
        return dx, None, None


class _MoEPull(torch.autograd.Function):
    """The MoE block on ``comm.ep.EPPull``: plan -> gather+gate/up+SwiGLU (one kernel) -> down projection with the
    weighted return in its epilogue -> combine.  Backward: gather+dh (one kernel), gather x again and rebuild the
    gate/up rows that were not kept (one kernel), SwiGLU backward, dx with the return in its epilogue, the three
    weight-gradient GEMMs, combine."""

    @staticmethod
    def forward(ctx, x, weights, idx, w1, w2, w3, recompute, epc, key, budget, slot):
        from ..comm import ep as E
        g = epc.g
        tokens, dim = x.shape
        ffn = w1.shape[1]
        weights = weights.float().contiguous()
        offs, seg_live_end, tile_expert, meta, seq = epc.plan(idx, weights, key)
        wants_grad = any(ctx.needs_input_grad)
        cap_saved, ledger = 0, None
        if wants_grad and not recompute:
            cap_saved = epc.expected_rows(key)
            if budget is not None:
                ledger = (0, cap_saved * ffn * 4)
                kept = budget.enter(*ledger)
                ledger += (kept,)
                if not kept:
                    cap_saved = 0
        dev = x.device
        gate = torch.empty(cap_saved, ffn, dtype=torch.bfloat16, device=dev) if cap_saved else None
        up = torch.empty(cap_saved, ffn, dtype=torch.bfloat16, device=dev) if cap_saved else None
        row_src = torch.empty(epc.cap, dtype=torch.int32, device=dev)
        row_tag = torch.empty(epc.cap, dtype=torch.int32, device=dev)
        row_w = torch.empty(epc.cap, dtype=torch.float32, device=dev)
        x_ws, h = epc.ws("x", dim), epc.ws("h", ffn)
        epc.gather_gemm(0, x_ws, w1, w3, 2 * ffn, dim, tile_expert, meta, seg_live_end, 0, epc.pool[slot].table(), 1,
                        epc.land_src.tensor, epc.land_tag.tensor, epc.land_w.tensor, (row_src, row_tag, row_w),
                        E.SIG_META, seq, 1, h, gate, up, None, None, cap_saved)
        ret_seq = g.next_seq(E.SIG_RET_F)
        native.gemm_nt_push(h, w2, tile_expert, meta[0:1], epc.e_local, epc.ret_f.table(), row_tag, row_src, row_w,
                            g.sig.table(), E.SIG_RET_F, ret_seq, g.rank, epc.ep, epc.tickets[4:])
        out, _ = epc.combine(epc.ret_f, E.SIG_RET_F, ret_seq, with_scalars=False)
        ctx.params = (w1, w2, w3)
        ctx.meta_py = (tokens, dim, ffn, epc, slot, cap_saved)
        ctx.budget, ctx.ledger = budget, ledger
        saved = [offs, seg_live_end, tile_expert, meta, row_src, row_tag, row_w]
        if cap_saved:
            saved += [gate, up]
        ctx.save_for_backward(*saved)
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..comm import ep as E
        w1, w2, w3 = ctx.params
        tokens, dim, ffn, epc, slot, cap_saved = ctx.meta_py
        saved = list(ctx.saved_tensors)
        offs, seg_live_end, tile_expert, meta, row_src, row_tag, row_w = saved[:7]
        gate, up = saved[7:9] if cap_saved else (None, None)
        g = epc.g
        experts = epc.e_local
        tiles = meta[0:1]
        epc.dout.tensor.view(tokens, dim).copy_(dout)
        dy_ws, x_ws, dh, dgu = epc.ws("dy", dim), epc.ws("x", dim), epc.ws("h", ffn), epc.ws("dgu", 2 * ffn)
        gate_ws, up_ws = epc.ws("gate", ffn), epc.ws("up", ffn)
        # dh = dy_perm W2, the rows of dy fetched from the peers' staged output gradients by the same kernel
        bseq = g.next_seq(E.SIG_BDATA)
        epc.gather_gemm(1, dy_ws, w2, None, ffn, dim, tile_expert, meta, seg_live_end, 0, epc.dout.table(), 1,
                        row_src, row_tag, None, None, E.SIG_BDATA, bseq, 2, dh, None, None, None, None, 0)
        # x rows again (for the weight gradients), gate/up rebuilt for the rows that were not kept
        epc.gather_gemm(0, x_ws, w1, w3, 2 * ffn, dim, tile_expert, meta, seg_live_end, cap_saved // 128,
                        epc.pool[slot].table(), 1, row_src, row_tag, None, None, 0, 0, 0, None, None, None, gate_ws,
                        up_ws, cap_saved)
        native.ep_swiglu_bwd(dh, gate, up, gate_ws, up_ws, cap_saved, dgu, meta, row_tag, row_src, row_w,
                             epc.dw_ret.table(), epc.ep)
        ret_seq = g.next_seq(E.SIG_RET_B)
        native.gemm_nn_push(dgu, w1, w3, tile_expert, tiles, experts, epc.ret_b.table(), row_tag, row_src, None,
                            g.sig.table(), E.SIG_RET_B, ret_seq, g.rank, epc.ep, epc.tickets[5:])
        dw2 = _wgrad(dy_ws, dh, w2, offs, experts)
        dw1 = _wgrad(dgu[:, :ffn], x_ws, w1, offs, experts)
        dw3 = _wgrad(dgu[:, ffn:], x_ws, w3, offs, experts)
        dx, dweights = epc.combine(epc.ret_b, E.SIG_RET_B, ret_seq, with_scalars=True)
        if ctx.ledger is not None:
            ctx.budget.leave(*ctx.ledger)
        return dx, dweights, None, dw1, dw2, dw3, None, None, None, None, None


def moe_ffn_pull(x, weights_of, w1, w2, w3, epc, recompute: bool = False, key=None, budget=None):
    """MoE block over the expert group of ``epc`` (``comm.ep.EPPull``).  ``weights_of(staged)`` computes the router's
    ``(weights, idx)`` from the staged copy of ``x`` (so that the router keeps the pool slot, not a second copy of
    the activations, for its backward pass)."""
    slot = epc.acquire()
    staged = _StageIn.apply(x.contiguous(), epc, slot)
    weights, idx = weights_of(staged)
    out = _MoEPull.apply(staged, weights, idx, w1, w2, w3, recompute, epc, key if key is not None else id(w1), budget,
                         slot)
    if not (torch.is_grad_enabled() and (x.requires_grad or weights.requires_grad)):
        epc.release(slot)          # no backward pass will come for this call
    return out, weights, idx
