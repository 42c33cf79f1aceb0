"""The MoE block as native kernels with a hand-written backward pass.

Forward:  plan (device counting sort) → gather rows into the padded
expert-major buffer → grouped gate/up GEMM with the SwiGLU epilogue → grouped
down GEMM → weighted combine.  Backward: the duals in reverse, with the three
weight-gradient GEMMs accumulating into the experts' ``main_grad`` buffers.
No step involves the host: tile counts, segment offsets and the tile→expert
table stay on the device and the persistent GEMMs read them there.

Replaces the reference's ``_dispatch_tokens`` / ``GroupedPositionWiseFFLayer`` /
``_combine_tokens`` (implementation/layers.py:139-246) including its per-expert
``nonzero`` loop and ``.cpu()`` split exchange.  With an expert-parallel context
(``ep_ctx``) the gather and combine steps move rows between GPUs through peer
memory (``b200moe.comm``).
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
    @staticmethod
    def forward(ctx, x, weights, idx, w1, w2, w3, recompute, ep_ctx, key, budget):
        tokens, dim = x.shape
        experts = w1.shape[0]
        x = x.contiguous()
        weights = weights.float().contiguous()
        if ep_ctx is None:
            cap = capacity_rows(tokens * 2, experts)
            slot_row, row_slot, offs, tile_expert, meta, _ = native.moe_plan(idx, experts, cap)
            x_perm = native.moe_gather(x, row_slot, meta, cap)
            route = None
        else:
            route = ep_ctx.dispatch(x, idx, key)
            cap, offs, tile_expert, meta, x_perm = route.cap, route.offs, route.tile_expert, route.meta, route.x_perm
            slot_row = row_slot = None
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
        if ep_ctx is None:
            out = native.moe_combine(y_perm, slot_row, weights, tokens)
        else:
            out = ep_ctx.combine(route, y_perm, weights, tokens)
        ctx.params = (w1, w2, w3)
        ctx.meta_py = (tokens, dim, experts, cap, recompute, ep_ctx, route)
        ctx.budget, ctx.ledger = budget, ledger
        saved = [x_perm, y_perm, weights, offs, tile_expert, meta]
        if ep_ctx is None:
            saved += [slot_row, row_slot]
        if not recompute:
            saved += [gate, up]
        ctx.save_for_backward(*saved)
        return out

    @staticmethod
    def backward(ctx, dout):
        w1, w2, w3 = ctx.params
        tokens, dim, experts, cap, recompute, ep_ctx, route = ctx.meta_py
        saved = list(ctx.saved_tensors)
        x_perm, y_perm, weights, offs, tile_expert, meta = saved[:6]
        rest = saved[6:]
        if ep_ctx is None:
            slot_row, row_slot = rest[:2]
            rest = rest[2:]
        tiles, live_rows = meta[0:1], meta[1:2]
        dout = dout.contiguous()
        ffn = w1.shape[1]
        if recompute:
            _, gate, up = native.gemm_swiglu(x_perm, w1, w3, tile_expert, tiles, save_gate_up=True, align256=True)
        else:
            gate, up = rest
        if ep_ctx is None:
            dweights = torch.zeros(tokens, 2, dtype=torch.float32, device=dout.device)
            dy_perm = native.moe_gather(dout, row_slot, meta, cap, scale=weights.view(-1), y_perm=y_perm,
                                        dweights=dweights.view(-1))
        else:
            dy_perm = ep_ctx.combine_backward(route, dout, y_perm, weights)
        dh = native.gemm_nn(dy_perm, w2, tile_expert=tile_expert, num_m_tiles=tiles, num_experts=experts, align256=True)
        dgu, h = native.swiglu_bwd(dh, gate, up, live_rows=live_rows)
        del dh, gate, up
        dx_perm = native.gemm_nn(dgu, w1, w2=w3, tile_expert=tile_expert, num_m_tiles=tiles, num_experts=experts,
                                 align256=True)
        dw2 = _wgrad(dy_perm, h, w2, offs, experts)
        dw1 = _wgrad(dgu[:, :ffn], x_perm, w1, offs, experts)
        dw3 = _wgrad(dgu[:, ffn:], x_perm, w3, offs, experts)
        if ep_ctx is None:
            dx = native.moe_combine(dx_perm, slot_row, None, tokens)
        else:
            dx, dweights = ep_ctx.dispatch_backward(route, dx_perm, tokens)
        if ctx.ledger is not None:
            ctx.budget.leave(*ctx.ledger)
        return dx, dweights, None, dw1, dw2, dw3, None, None, None, None


def moe_ffn_fused(x, weights, idx, w1, w2, w3, ep_ctx=None, recompute: bool = False, key=None, budget=None):
    """``key`` names the calling layer; the expert-parallel context keeps one
    capacity hint per key.  ``budget`` (``parallel.memory.ActivationBudget``): when given, the call keeps its
    gate/up pre-activations only while the budget has room and rebuilds them in the backward pass otherwise."""
    return _MoEFused.apply(x, weights, idx, w1, w2, w3, recompute, ep_ctx, key if key is not None else id(w1), budget)
