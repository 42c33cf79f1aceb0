"""Expert-parallel exchange fused with the expert GEMMs (the kernels of ``csrc/moe_ep.cu`` and the ``EPI_PUSH``
epilogue of ``csrc/gemm.cu``).

``EPPull`` owns, for one problem size, the symmetric buffers the ranks of the expert group read and write in each
other's memory, and the local workspaces of the expert side:

===================  ========================  ==============================================================
buffer               where                     written by / read by
===================  ========================  ==============================================================
token pool slots     symmetric ``[T, D]``      own forward (copy of the block input) / every owner's gather
``dout``             symmetric ``[T, D]``      own backward (copy of the output gradient) / owners' gather
row tables           symmetric ``[cap]`` x3    the sources' plan kernels / own gather warps
``ret_f``, ``ret_b``  symmetric ``[2T, D]``     owners' GEMM epilogues (peer stores) / own combine kernel
``dw_ret``           symmetric ``[2T]`` fp32   owners' SwiGLU-backward kernel / own combine kernel
workspaces           local                     expert-major operands and intermediates, shared by all layers
===================  ========================  ==============================================================

Nothing on the expert side that depends on the routing is kept between forward and backward except the gate/up
pre-activations (optional: the first ``cap_saved`` rows, chosen on the host from the stage's activation budget and
an asynchronous read-back of the previous call's row count) and three small per-row tables.  The backward pass
gathers ``x`` again (it is cheaper than keeping the permuted copy) and rebuilds gate/up for the rows beyond
``cap_saved``.  No step reads a device value on the host, and no routing pattern can overflow a saved buffer.

Replaces the reference's ``_dispatch_tokens`` / ``TensorExchange`` / ``_combine_tokens``
(implementation/layers.py:14-52, 139-213).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..ops import native

MAX_RANKS = 8
_U64x8 = ctypes.c_ulonglong * MAX_RANKS
ALIGN = 256

# signal slots of this protocol (disjoint from the ones in comm/__init__.py)
SIG_COUNTS, SIG_META, SIG_RET_F, SIG_BDATA, SIG_RET_B = 16, 17, 18, 19, 20


def _i(v):
    return ctypes.c_int(int(v))


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _align(rows: int) -> int:
    return (rows + ALIGN - 1) // ALIGN * ALIGN


class _Shared:
    """A buffer every rank of the group can address: symmetric memory, or a plain tensor when the group is this
    rank alone."""

    def __init__(self, numel, dtype, device, group, zero=True):
        if group is None:
            self.tensor = torch.zeros(numel, dtype=dtype, device=device) if zero else \
                torch.empty(numel, dtype=dtype, device=device)
            self.handle, self.mc_ptr = None, 0
            self.ptrs = _U64x8(*([self.tensor.data_ptr()] + [0] * (MAX_RANKS - 1)))
        else:
            from . import SymmBuffer
            inner = SymmBuffer(numel, dtype, device, group, zero=zero)
            self.tensor, self.handle, self.mc_ptr, self.ptrs = inner.tensor, inner.handle, inner.mc_ptr, inner.ptrs

    def table(self):
        return self.ptrs


class _Solo:
    """Stand-in for ``GroupComm`` when the expert group is a single rank (one-GPU runs and tests)."""

    def __init__(self, device):
        self.group, self.world, self.rank, self.device = None, 1, 0, device
        self.sig = _Shared(32 * MAX_RANKS, torch.int32, device, None)
        self.seq = [0] * 32

    def next_seq(self, slot):
        self.seq[slot] += 1
        return self.seq[slot]

    def my_sig(self):
        return ctypes.c_void_p(self.sig.tensor.data_ptr())


@dataclass
class Routing:
    """What one forward call leaves for its backward pass."""
    slot: int
    offs: torch.Tensor
    seg_live_end: torch.Tensor
    tile_expert: torch.Tensor
    meta: torch.Tensor
    row_src: torch.Tensor
    row_tag: torch.Tensor
    row_w: torch.Tensor
    cap_saved: int
    gate: torch.Tensor | None
    up: torch.Tensor | None


class EPPull:
    """Dispatch, expert GEMMs and return of one MoE block, forward and backward."""

    def __init__(self, group_comm, status, device, tokens: int, dim: int, ffn: int, experts_total: int,
                 max_skew: float | None = None):
        g = group_comm if group_comm is not None else _Solo(device)
        self.g, self.status, self.device = g, status, device
        self.tokens, self.dim, self.ffn, self.experts_total = tokens, dim, ffn, experts_total
        self.ep = g.world
        self.e_local = experts_total // self.ep
        self.slots = tokens * 2
        worst = _align(self.slots * self.ep + self.e_local * (ALIGN - 1))
        # ``max_skew``: bound of the rows one rank accepts, as a multiple of a balanced split.  None = the worst
        # case (every slot of every rank routed here), which no routing can exceed; a smaller bound saves workspace
        # on wide groups, and a call that exceeds it is refused by the plan kernel (status 102), never clipped.
        self.cap = worst if not max_skew else min(worst, _align(int(self.slots * max_skew) + self.e_local * (ALIGN - 1)))
        grp = g.group
        i32, f32, bf16 = torch.int32, torch.float32, torch.bfloat16
        self.counts_all = _Shared(MAX_RANKS * 32, i32, device, grp)
        self.land_src = _Shared(self.cap, i32, device, grp)
        self.land_tag = _Shared(self.cap, i32, device, grp)
        self.land_w = _Shared(self.cap, f32, device, grp)
        self.dout = _Shared(tokens * dim, bf16, device, grp, zero=False)
        self.ret_f = _Shared(self.slots * dim, bf16, device, grp, zero=False)
        self.ret_b = _Shared(self.slots * dim, bf16, device, grp, zero=False)
        self.dw_ret = _Shared(self.slots, f32, device, grp)
        self.pool: list[_Shared] = []
        self.free: list[int] = []
        self.tile_ready = torch.zeros(self.cap // 128, dtype=i32, device=device)
        self.tickets = torch.zeros(8, dtype=i32, device=device)
        self._ws: dict = {}
        self._hints: dict = {}
        self.null = _U64x8(*([0] * MAX_RANKS))
        self._sync()

    def _sync(self):
        torch.cuda.synchronize(self.device)
        if self.g.group is not None:
            dist.barrier(group=self.g.group)

    def buffers(self):
        return [self.counts_all, self.land_src, self.land_tag, self.land_w, self.dout, self.ret_f, self.ret_b,
                self.dw_ret, *self.pool]

    # -- token pool ------------------------------------------------------------------------------
    def acquire(self) -> int:
        """A free pool slot; the pool grows (collectively: every rank of the group makes the same calls in the
        same order) when all are taken."""
        if not self.free:
            self.pool.append(_Shared(self.tokens * self.dim, torch.bfloat16, self.device, self.g.group, zero=False))
            self._sync()
            self.free.append(len(self.pool) - 1)
        return self.free.pop()

    def release(self, slot: int) -> None:
        self.free.append(slot)

    def new_step(self) -> None:
        """Start of a training step: no call of the previous step is alive, so every slot is free again (a step that
        ended in an exception never ran the backward passes that give slots back).  Same order on every rank."""
        self.free = list(range(len(self.pool) - 1, -1, -1))

    def slot_tensor(self, slot: int) -> torch.Tensor:
        return self.pool[slot].tensor.view(self.tokens, self.dim)

    # -- workspaces --------------------------------------------------------------------------------
    def ws(self, name: str, cols: int) -> torch.Tensor:
        """Expert-major workspace ``[cap, cols]`` bf16, allocated at first use and shared by all layers (a layer's
        forward or backward pass is done with it before the next one starts on the same stream)."""
        buf = self._ws.get(name)
        if buf is None:
            buf = torch.empty(self.cap, cols, dtype=torch.bfloat16, device=self.device)
            self._ws[name] = buf
        return buf

    # -- row-count read-back (never waited for) ---------------------------------------------------------
    def _record_rows(self, key, meta):
        hint = self._hints.get(key)
        if hint is None:
            hint = (torch.zeros(4, dtype=torch.int32, pin_memory=True), torch.cuda.Event())
            self._hints[key] = hint
        hint[0].copy_(meta, non_blocking=True)
        hint[1].record()

    def expected_rows(self, key) -> int:
        """Rows the layer ``key`` needed at its previous call if that read-back has arrived, else a balanced share
        with a quarter of head room.  A guide for what to keep, never a limit."""
        hint = self._hints.get(key)
        # multiples of 2048 rows: a handful of distinct tensor sizes, which the caching allocator can reuse
        if hint is not None and hint[1].query() and int(hint[0][3]) > 0:
            return min(self.cap, (int(int(hint[0][3]) * 1.1) + 2047) // 2048 * 2048)
        return min(self.cap, (int(self.slots * 1.25) + 2047) // 2048 * 2048)

    def worst_load(self) -> float:
        worst = 0
        for hint in self._hints.values():
            if hint[1].query():
                worst = max(worst, int(hint[0][3]))
        return worst / self.slots

    # -- kernels ------------------------------------------------------------------------------------
    def plan(self, idx, weights, key=None):
        g, dev = self.g, self.device
        i32 = dict(dtype=torch.int32, device=dev)
        offs, seg_live_end = torch.empty(self.e_local, **i32), torch.empty(self.e_local, **i32)
        tile_expert = torch.empty(self.cap // 128, **i32)
        meta = torch.zeros(4, **i32)
        seq = g.next_seq(SIG_COUNTS)
        g.seq[SIG_META] = seq
        native._call("b2_ep_plan2", _ptr(idx.contiguous()), _ptr(weights), _i(self.slots), _i(self.experts_total),
                     _i(self.ep), _i(g.rank), _i(seq), _i(self.cap), self.counts_all.table(), self.land_src.table(),
                     self.land_tag.table(), self.land_w.table(), g.sig.table(), _i(SIG_COUNTS), _i(SIG_META),
                     _ptr(offs), _ptr(seg_live_end), _ptr(tile_expert), _ptr(meta), _ptr(self.status), _stream())
        self._record_rows(key, meta)
        return offs, seg_live_end, tile_expert, meta, seq

    def gather_gemm(self, mode, a_buf, w, w_b, N, K, tile_expert, meta, seg_live_end, tile_begin, src_table, shift,
                    row_src, row_tag, row_w, save, sig_slot, seq, handshake, d, gate_lo, up_lo, gate_hi, up_hi,
                    split_row):
        g = self.g
        save_src, save_tag, save_w = save if save is not None else (None, None, None)
        # (return code -20: the device cannot keep one CTA per SM resident, which the cooperative launch needs)
        native._call(
            "b2_ep_gather_gemm",
            _i(mode), _ptr(a_buf), _ptr(w), _ptr(w_b), _i(self.cap), _i(N), _i(K), _i(self.e_local),
            _ptr(tile_expert), _ptr(meta), _ptr(seg_live_end), _i(tile_begin), src_table, _i(shift), _ptr(row_src),
            _ptr(row_tag), _ptr(row_w), _ptr(save_src), _ptr(save_tag), _ptr(save_w), _ptr(self.tile_ready),
            _ptr(self.tickets[mode:]), g.sig.table(), _i(self.ep), _i(g.rank), _i(sig_slot), _i(seq), _i(handshake),
            _ptr(d), _ptr(gate_lo), _ptr(up_lo), _ptr(gate_hi), _ptr(up_hi), _i(split_row), _ptr(self.status),
            _stream(), tag=("gate/up" if mode == 0 else "dh") + (" (re-gather, rebuild)" if gate_hi is not None else ""))

    def combine(self, ret, sig_slot, seq, with_scalars: bool):
        out = torch.empty(self.tokens, self.dim, dtype=torch.bfloat16, device=self.device)
        scalars = torch.empty(self.tokens, 2, dtype=torch.float32, device=self.device) if with_scalars else None
        native._call("b2_ep_combine", _ptr(ret.tensor), _ptr(self.dw_ret.tensor), _ptr(out), _ptr(scalars),
                     _i(self.tokens), _i(self.dim), self.g.my_sig(), _i(sig_slot), _i(self.ep), _i(seq),
                     _ptr(self.status), _stream())
        return out, scalars
