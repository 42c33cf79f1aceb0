"""Activation-memory budget of one pipeline stage.

Under 1F1B a stage keeps ``min(pp − stage, m)`` microbatches alive, so the early
stages of a deep pipeline are the ones that run out of HBM.  The reference keeps
every activation (it was measured on 288 GB parts); on 180 GB the gate/up
pre-activations of the experts — the largest saved tensors, and the only ones
whose size follows the routing — are kept only while they fit.

``ActivationBudget`` is plain host arithmetic.  The trainer builds one per rank
after the model, its gradient buffers and the optimizer moments exist, from the
free HBM it then sees minus what the stage will certainly need (the fixed-size
activations of every live microbatch, transient workspaces, a margin).  Every
MoE call asks before it saves the optional tensors and gives the bytes back in
its backward pass; a call that is refused rebuilds gate/up in the backward pass
instead.  A router that sends most rows to one rank therefore costs time on that
rank, never the process.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

__all__ = ["ActivationBudget", "stage_activation_budget", "fixed_bytes_per_block"]


class ActivationBudget:
    def __init__(self, total_bytes: int, max_live_calls: int = 0, routed_bytes_per_call: int = 0,
                 fixed_bytes_per_call: int = 0, floor_bytes: int = 0, probe=None, cold_floor_bytes: int = 0,
                 cold_calls: int = 0):
        """``probe``: optional callable returning the bytes the device can still hand out right now (free HBM plus
        what the allocator holds unused).  The plan above is arithmetic; the probe is the cross-check against what
        really happened: the optional tensors of a call are kept only if, after them, the device still has room for
        the fixed-size activations of the calls to come (``fixed_bytes_per_call`` each) plus ``floor_bytes``.  During
        the first ``cold_calls`` calls ``cold_floor_bytes`` more are held back: the expert workspaces and the
        backward pass's transients do not exist yet and are about to be allocated."""
        self.total = int(total_bytes)
        self.max_live_calls = int(max_live_calls)
        # bytes of routing-dependent tensors a call saves whatever happens (its share of a balanced split)
        self.routed_bytes_per_call = int(routed_bytes_per_call)
        self.fixed_bytes_per_call = int(fixed_bytes_per_call)
        self.floor_bytes = int(floor_bytes)
        self.cold_floor_bytes, self.cold_calls = int(cold_floor_bytes), int(cold_calls)
        self.probe = probe
        self.used = 0
        self.live_calls = 0
        self.granted = 0
        self.refused = 0

    def reset(self) -> None:
        """Start of a step: nothing of the previous step is alive any more."""
        self.used = 0
        self.live_calls = 0

    def enter(self, routed_bytes: int, optional_bytes: int) -> bool:
        """A call that must keep ``routed_bytes`` and would like to keep ``optional_bytes`` more.  Returns whether
        the optional part fits beside what the calls still to come will need."""
        self.live_calls += 1
        still_to_come = max(0, self.max_live_calls - self.live_calls)
        reserve = still_to_come * self.routed_bytes_per_call
        keep = self.used + routed_bytes + optional_bytes + reserve <= self.total
        if keep and self.probe is not None:
            ahead = still_to_come * (self.fixed_bytes_per_call + self.routed_bytes_per_call) + self.floor_bytes
            if self.granted + self.refused < self.cold_calls:
                ahead += self.cold_floor_bytes
            keep = self.probe() - routed_bytes - optional_bytes >= ahead
        self.used += routed_bytes + (optional_bytes if keep else 0)
        if keep:
            self.granted += 1
        else:
            self.refused += 1
        return keep

    def leave(self, routed_bytes: int, optional_bytes: int, kept: bool) -> None:
        self.live_calls = max(0, self.live_calls - 1)
        self.used = max(0, self.used - routed_bytes - (optional_bytes if kept else 0))

    def summary(self) -> dict:
        return {"budget_gib": round(self.total / 2 ** 30, 2), "kept": self.granted, "recomputed": self.refused}


def fixed_bytes_per_block(tokens: int, d_model: int, num_heads: int, experts_total: int, itemsize: int = 2) -> int:
    """Saved activations of one block for one microbatch whose size does not depend on the routing: block input,
    fused q/k/v projection, attention output and its log-sum-exp, the two normalised copies, the residual sum,
    router probabilities, the returned expert rows."""
    kv = d_model // 4
    per_token = (d_model            # block input (saved by the first norm)
                 + d_model          # normalised input of the attention projections
                 + d_model + 2 * kv  # fused q/k/v
                 + d_model          # attention output (input of the output projection)
                 + d_model          # residual sum after attention
                 + d_model          # normalised input of the MoE block
                 + d_model)         # block output kept by the next block's norm
    small = tokens * (num_heads * 4 + experts_total * 4 * 2 + 64)
    return tokens * per_token * itemsize + small


@dataclass
class _StageShape:
    tokens: int
    d_model: int
    d_ff: int
    num_heads: int
    experts_total: int
    ep: int
    blocks: int
    in_flight: int
    vocab: int
    last_stage: bool


def _workspace_bytes(s: _StageShape) -> int:
    """Transient buffers of the largest backward pass: rebuilt gate/up, dh, dgate|dup and h at the worst-case row
    count a rank can receive, the landing areas, and the logits of the head on the last stage."""
    worst_rows = s.tokens * 2 * s.ep
    expert_side = worst_rows * s.d_ff * 2 * 7        # gate, up, dh, dgu (2), h, slack for allocator rounding
    landing = worst_rows * s.d_model * 2 * 4
    head = s.tokens * s.vocab * 2 * 2 if s.last_stage else 0
    return expert_side + landing + head


def stage_activation_budget(*, tokens_per_microbatch: int, d_model: int, d_ff: int, num_heads: int,
                            experts_total: int, ep: int, blocks: int, pp: int, stage: int, microbatches: int,
                            vocab: int, device=None, free_bytes: int | None = None, margin_bytes: int = 6 << 30,
                            routed_row_bytes: int | None = None) -> ActivationBudget:
    """Budget for the routing-dependent saved tensors of this stage.  ``free_bytes``: HBM still free once weights,
    gradient buffers and optimizer moments are allocated (read from the device when not given).
    ``routed_row_bytes``: bytes a call keeps per received row whatever happens (default: the permuted input and the
    expert output rows)."""
    in_flight = max(1, min(pp - stage, microbatches))
    shape = _StageShape(tokens_per_microbatch, d_model, d_ff, num_heads, experts_total, ep, blocks, in_flight, vocab,
                        stage == pp - 1)
    free_bytes_given = free_bytes
    if free_bytes is None:
        free, _total = torch.cuda.mem_get_info(device)
        cached = torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)
        free_bytes = free + cached
    fixed = in_flight * blocks * fixed_bytes_per_block(tokens_per_microbatch, d_model, num_heads, experts_total)
    fixed += in_flight * tokens_per_microbatch * d_model * 2 * 2          # stage input and output of each microbatch
    total = int(free_bytes) - fixed - _workspace_bytes(shape) - int(margin_bytes)
    if routed_row_bytes is None:
        routed_row_bytes = d_model * 2 * 2
    balanced_rows = tokens_per_microbatch * 2
    probe = None
    if free_bytes_given is None:
        def probe():
            free_now, _ = torch.cuda.mem_get_info(device)
            return free_now + torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)
    per_block = fixed_bytes_per_block(tokens_per_microbatch, d_model, num_heads, experts_total)
    return ActivationBudget(max(total, 0), max_live_calls=in_flight * blocks,
                            routed_bytes_per_call=balanced_rows * routed_row_bytes, fixed_bytes_per_call=per_block,
                            floor_bytes=int(margin_bytes), probe=probe, cold_floor_bytes=_workspace_bytes(shape),
                            cold_calls=2 * in_flight * blocks)
