"""Peer-memory communication layer (NVLink 5 / NVSwitch).

``torch.distributed`` (NCCL) stays the plumbing: bootstrap, object broadcast,
barriers, pipeline send/recv and the symmetric-memory rendezvous.  On top of it
this module allocates symmetric buffers (``torch.distributed._symmetric_memory``:
the same allocation mapped into every rank of a group, optionally bound to an
NVSwitch multicast address) and drives the kernels of ``csrc/comm.cu`` that read
and write those buffers through peer pointers:

* ``Comm.ep_context`` → ``comm.ep.EPPull``: the expert-parallel exchange fused
  with the expert GEMMs (replaces the reference's ``TensorExchange``
  all-to-alls and their ``.cpu()`` split sync, implementation/layers.py:14-52,
  139-213);
* ``Comm.fused_update``: FSDP reduce-scatter + AdamW + weight all-gather in one
  kernel (replaces per-parameter ``reduce_scatter_tensor`` + eager AdamW + the
  per-microbatch all-gathers, implementation/distributed/ddp_modules.py:24-100,
  219-292);
* ``Comm.allreduce_avg``: replica all-reduce, one-shot / two-shot / NVLS chosen
  by message size (replaces ddp_modules.py:274-287);
* ``Comm.pp_link`` → ``comm.pp.PeerLink``: the pipeline's stage-to-stage transfers
  as peer stores into landing rings (replaces the blocking batched send/recv of
  pipeline/pipelined_train_overlap.py:40-75).

Sequence numbers: every synchronising phase owns a signal slot and a counter
that all ranks of the group advance in the same order.
"""
from __future__ import annotations

import ctypes
import torch
import torch.distributed as dist

from ..ops import native

MAX_RANKS = 8
_U64x8 = ctypes.c_ulonglong * MAX_RANKS

# signal slots (the expert exchange of comm/ep.py uses 16..20)
SIG_FSDP = 8      # +1
SIG_AR = 12       # +1
SIG_AG_GEMM = 14
NUM_SLOTS = 32


class SymmBuffer:
    """One symmetric allocation: the local tensor plus every rank's address."""

    def __init__(self, numel: int, dtype, device, group, zero: bool = True):
        import torch.distributed._symmetric_memory as symm_mem
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        if zero:
            self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, group)
        ptrs = list(self.handle.buffer_ptrs)
        self.world = len(ptrs)
        self.rank = self.handle.rank
        self.ptrs = _U64x8(*(ptrs + [0] * (MAX_RANKS - len(ptrs))))
        mc = 0
        try:
            if self.handle.has_multicast_support:
                mc = int(self.handle.multicast_ptr)
        except Exception:
            mc = 0
        self.mc_ptr = mc

    def table(self):
        return self.ptrs


def _null_table():
    return _U64x8(*([0] * MAX_RANKS))


def _i(v):
    return ctypes.c_int(int(v))


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class GroupComm:
    """Signal pad, block counter and sequence numbers of one process group."""

    def __init__(self, group, device):
        self.group = group
        self.device = device
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.sig = SymmBuffer(NUM_SLOTS * MAX_RANKS, torch.int32, device, group)
        self.counter = torch.zeros(8, dtype=torch.int32, device=device)
        self.seq = [0] * NUM_SLOTS
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def next_seq(self, slot: int) -> int:
        self.seq[slot] += 1
        return self.seq[slot]

    def my_sig(self):
        return ctypes.c_void_p(self.sig.tensor.data_ptr())


class Comm:
    def __init__(self, mesh, device, multicast: bool = False, wait_seconds: float | None = None,
                 pipeline_link: str | None = None, pipeline_wait_seconds: float = 120.0):
        """``pipeline_link``: ``"peer"`` moves the pipeline's activations and gradients with this library's
        peer-store kernels (``pp_link``), ``"nccl"`` with batched NCCL send/recv (the default);
        ``B200MOE_PIPELINE_LINK`` overrides it.  ``pipeline_wait_seconds``: budget of a pipeline wait
        (they span whole stage steps, so it is longer than ``wait_seconds``).  ``multicast``: let the
        symmetric-memory rendezvous bind buffers to an NVSwitch multicast address (only the NVLS all-reduce uses it).  Off by default: a process that dies while bound raises NVLink faults on the
        other ranks' GPUs, and nothing else here needs the binding.  ``wait_seconds``: budget of every cross-GPU
        wait inside the kernels (``native.set_wait_seconds``)."""
        import os
        native.require()
        self.multicast = bool(multicast)
        if not self.multicast:
            # read by the symmetric-memory allocator at its first rendezvous in this process
            os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
        seconds = os.environ.get("B200MOE_WAIT_SECONDS") or wait_seconds
        if seconds is not None:
            native.set_wait_seconds(float(seconds))
        self.mesh = mesh
        self.device = device
        self.status = native.status_word(device)
        self.fsdp = GroupComm(mesh.group("fsdp"), device) if mesh.fsdp > 1 else None
        self.ddp = GroupComm(mesh.group("ddp"), device) if mesh.ddp > 1 else None
        skew = os.environ.get("B200MOE_EP_MAX_SKEW")
        self.ep_max_skew = float(skew) if skew else None
        chosen = os.environ.get("B200MOE_PIPELINE_LINK") or pipeline_link or "nccl"
        if chosen not in ("peer", "nccl"):
            raise ValueError(f"pipeline_link must be 'peer' or 'nccl', got {chosen!r}")
        self.pipeline_link = chosen
        self.pipeline_wait_seconds = float(os.environ.get("B200MOE_PIPELINE_WAIT_SECONDS") or pipeline_wait_seconds)
        self._pp = {}
        self._symm = {}
        self._ep = {}
        self._ar_stage = {}
        self._ag_state = {}
        self._entries = {}

    # -- lifetime ------------------------------------------------------------------------
    def buffers(self):
        """Every symmetric buffer this object owns."""
        found = list(self._symm.values()) + list(self._ar_stage.values())
        for g in (self.fsdp, self.ddp):
            if g is not None:
                found.append(g.sig)
        for ctx in self._ep.values():
            found.extend(ctx.buffers())
        for link in self._pp.values():
            if link is not None:
                found.extend(link.buffers())
        return found

    def any_multicast(self) -> bool:
        """True while any symmetric buffer of this process is bound to a multicast address."""
        return any(getattr(b, "mc_ptr", 0) for b in self.buffers())

    def release(self) -> None:
        """Let go of every symmetric buffer (call between steps, before the process leaves on an error path, so
        that peers never see a mapping disappear under a kernel).  The object is unusable afterwards."""
        try:
            torch.cuda.synchronize(self.device)
        except Exception:
            pass
        for b in self.buffers():
            b.mc_ptr = 0
            b.handle = None
            b.tensor = None
        self._symm.clear()
        self._ar_stage.clear()
        self._ep.clear()
        self._pp.clear()
        self.fsdp = self.ddp = None

    def new_step(self) -> None:
        """Called by the sharding wrapper at the start of every training step."""
        for ctx in self._ep.values():
            ctx.new_step()

    # -- allocation ----------------------------------------------------------------------
    def alloc_flat(self, numel: int, dtype):
        """Symmetric, zero-filled flat buffer over the FSDP group (plain memory
        when the group has one rank)."""
        if self.fsdp is None:
            return torch.zeros(numel, dtype=dtype, device=self.device)
        padded = (numel + 255) // 256 * 256
        buf = SymmBuffer(padded, dtype, self.device, self.fsdp.group)
        view = buf.tensor[:numel]
        self._symm[view.data_ptr()] = buf
        return view

    def _buffer_of(self, tensor) -> SymmBuffer:
        return self._symm[tensor.data_ptr()]

    # -- FSDP ----------------------------------------------------------------------------
    def _entry_table(self, flat):
        key = id(flat)
        if key not in self._entries:
            rows = [[e["full_off"], e["shard_off"], e["shard_numel"], int(bool(e.get("lazy")))] for e in flat.entries]
            self._entries[key] = torch.tensor(rows, dtype=torch.int64, device=self.device)
        return self._entries[key]

    def _fsdp_launch(self, flat, mode, lr=0.0, beta1=0.0, beta2=0.0, eps=0.0, wd=0.0, a_t=0.0, push_all=False):
        g = self.fsdp
        entries = self._entry_table(flat)
        if flat.m is None:
            flat.m = torch.zeros_like(flat.master)
            flat.v = torch.zeros_like(flat.master)
        seq = g.next_seq(SIG_FSDP)
        native._call("b2_fsdp_step", self._buffer_of(flat.full_g).table(), self._buffer_of(flat.full_w).table(),
                     g.sig.table(), _ptr(entries), _i(len(flat.entries)), _i(g.rank), _i(g.world), _i(seq),
                     _i(SIG_FSDP), _ptr(flat.master), _ptr(flat.m), _ptr(flat.v), _ptr(flat.shard_grad),
                     ctypes.c_float(lr), ctypes.c_float(beta1), ctypes.c_float(beta2), ctypes.c_float(eps),
                     ctypes.c_float(wd), ctypes.c_float(a_t), _i(mode), _i(push_all), _ptr(g.counter),
                     _ptr(self.status), _stream())

    def allgather_cast(self, flat):
        """bf16 cast of every master shard pushed to every rank (also the entries that are normally gathered
        by their first consumer)."""
        self._fsdp_launch(flat, 3, push_all=True)

    def reduce_scatter_avg(self, flat):
        self._fsdp_launch(flat, 0)

    def fused_update(self, flat, reduce: bool, lr, beta1, beta2, eps, wd, a_t):
        """AdamW on the owned shards and push of the new bf16 weights to every rank;
        with ``reduce`` the gradient reduce-scatter happens in the same kernel."""
        self._fsdp_launch(flat, 1 if reduce else 2, lr, beta1, beta2, eps, wd, a_t)

    # -- all-gather fused with the consuming GEMM ---------------------------------------------
    def _locate(self, tensor):
        """Symmetric buffer that contains ``tensor`` and the byte offset of the tensor inside it."""
        addr = tensor.data_ptr()
        for buf in self._symm.values():
            base = buf.tensor.data_ptr()
            if base <= addr < base + buf.tensor.numel() * buf.tensor.element_size():
                return buf, addr - base
        raise KeyError("tensor does not live in a symmetric buffer of this Comm")

    def allgather_gemm(self, x, w, segments=None):
        """``x [M,K] @ w [N,K]ᵀ`` for a weight that is row-sharded over the FSDP group: ``w`` is this rank's
        full-size copy inside a symmetric flat buffer (``alloc_flat``) in which only the own rows
        ``[rank·N/n, (rank+1)·N/n)`` need to be current (``segments``: row counts of stacked parts that are
        sharded one by one, e.g. the q, k and v rows of a fused projection).  One kernel pulls the other rows from the peers and
        multiplies; afterwards all of ``w`` is current on this rank.  A rank must not rewrite its rows before the
        group has synchronised again (the end-of-step kernel does).  Takes the place of the reference's
        per-module ``all_gather_into_tensor`` + einsum (implementation/distributed/ddp_modules.py:24-49)."""
        g = self.fsdp
        if g is None:
            return native.gemm_nt(x, w)
        N, K = w.shape
        segments = [N] if segments is None else [int(v) for v in segments]
        if not w.is_contiguous() or sum(segments) != N or any(v % g.world for v in segments):
            raise ValueError("weight must be contiguous, its parts divisible by the group size")
        buf, off = self._locate(w)
        ptrs = _U64x8(*[(buf.ptrs[r] + off) if r < g.world else 0 for r in range(MAX_RANKS)])
        key = ("ag", w.data_ptr(), N, K)
        state = self._ag_state.get(key)
        if state is None:
            state = {"flags": torch.zeros((N + 255) // 256, dtype=torch.int32, device=self.device), "epoch": 0}
            self._ag_state[key] = state
        state["epoch"] += 1
        seq = g.next_seq(SIG_AG_GEMM)
        y = native.ag_gemm_nt(x, ptrs, N, segments, g.world, g.rank, g.sig.table(), SIG_AG_GEMM, seq,
                              state["flags"], state["epoch"])
        if y is None:      # no cooperative launch on this device: gather with NCCL, multiply
            state["epoch"] -= 1
            begin = 0
            for rows in segments:
                shard = rows // g.world
                part = w[begin:begin + rows]
                dist.all_gather_into_tensor(part, part[g.rank * shard:(g.rank + 1) * shard].clone(), group=g.group)
                begin += rows
            return native.gemm_nt(x, w)
        return y

    # -- replica all-reduce -----------------------------------------------------------------
    ONE_SHOT_MAX = 1 << 18      # floats: below 1 MiB latency dominates, every rank reads everything
    NVLS_MIN = 1 << 22          # floats: from 16 MiB the in-switch reduction wins

    def allreduce_avg(self, tensor, group=None, kind: str | None = None):
        """In-place average of an fp32 tensor over the replica group, staged through a
        symmetric buffer in chunks."""
        g = self.ddp if group is None or group is self.mesh.group("ddp") else None
        if g is None:
            dist.all_reduce(tensor, op=dist.ReduceOp.AVG, group=group)
            return tensor
        if tensor.dtype != torch.float32:
            work = tensor.float()
            self.allreduce_avg(work, group, kind)
            tensor.copy_(work)
            return tensor
        flat = tensor.reshape(-1)
        stage = self._ar_stage.get("f32")
        if stage is None:
            stage = SymmBuffer(1 << 26, torch.float32, self.device, g.group)     # 256 MiB
            self._ar_stage["f32"] = stage
        cap = stage.tensor.numel()
        for lo in range(0, flat.numel(), cap):
            n = min(cap, flat.numel() - lo)
            padded = (n + 3) // 4 * 4
            stage.tensor[:n].copy_(flat[lo:lo + n])
            if padded != n:
                stage.tensor[n:padded].zero_()
            chosen = kind or ("oneshot" if padded <= self.ONE_SHOT_MAX else
                              ("nvls" if stage.mc_ptr and padded >= self.NVLS_MIN else "twoshot"))
            seq = g.next_seq(SIG_AR)
            out = flat[lo:lo + n] if (chosen == "oneshot" and padded == n) else None
            scratch = out if out is not None else (torch.empty(padded, dtype=torch.float32, device=self.device)
                                                   if chosen == "oneshot" else None)
            native._call("b2_comm_allreduce", stage.table(), g.sig.table(), ctypes.c_void_p(stage.mc_ptr),
                         _ptr(scratch), _i({"oneshot": 0, "twoshot": 1, "nvls": 2}[chosen]), _i(g.rank), _i(g.world),
                         _i(seq), _i(SIG_AR), ctypes.c_longlong(padded), ctypes.c_float(1.0 / g.world),
                         _ptr(g.counter[1:]), _ptr(self.status), _stream())
            if chosen == "oneshot":
                if out is None:
                    flat[lo:lo + n].copy_(scratch[:n])
            else:
                flat[lo:lo + n].copy_(stage.tensor[:n])
        return tensor

    # -- pipeline ---------------------------------------------------------------------------
    def pp_link(self, group, stage: int, spec, dtype):
        """The peer-memory link of this stage for microbatches of shape ``spec`` (collective over ``group`` at
        first use), or ``None`` when the pipeline is to use NCCL: ``pipeline_link="nccl"``, a payload that is not
        a whole number of 16-byte units, or stages that do not all sit on this host (peer memory is an NVLink
        domain)."""
        if self.pipeline_link != "peer" or group is None or dtype is None:
            return None
        key = (id(group), tuple(spec), dtype)
        if key not in self._pp:
            from .pp import PeerLink
            import math
            import socket
            stages = dist.get_world_size(group)
            hosts = [None] * stages
            dist.all_gather_object(hosts, socket.gethostname(), group=group)
            usable = (stages <= MAX_RANKS and len(set(hosts)) == 1 and dist.get_rank(group) == stage
                      and (math.prod(spec) * dtype.itemsize) % 16 == 0)
            votes = [None] * stages
            dist.all_gather_object(votes, bool(usable), group=group)
            self._pp[key] = PeerLink.over_group(group, self.device, self.status, spec, dtype,
                                                self.pipeline_wait_seconds) if all(votes) else None
        return self._pp[key]

    # -- expert parallel --------------------------------------------------------------------
    def ep_context(self, tokens: int, dim: int, experts_total: int, ffn: int):
        """The expert-exchange state (``comm.ep.EPPull``) for one problem size, created at first use."""
        key = (tokens, dim, experts_total, ffn)
        ctx = self._ep.get(key)
        if ctx is None:
            from .ep import EPPull
            # a wide group's worst case (every slot of every rank on one rank) is far from anything a trained
            # router does: beyond four ranks the accepted skew is bounded unless configured otherwise
            skew = self.ep_max_skew if self.ep_max_skew else (None if self.fsdp.world <= 4 else 4.0)
            ctx = EPPull(self.fsdp, self.status, self.device, tokens, dim, ffn, experts_total, max_skew=skew)
            self._ep[key] = ctx
        return ctx


def make_comm(mesh, device, multicast: bool = False, wait_seconds: float | None = None,
              pipeline_link: str | None = None, pipeline_wait_seconds: float = 120.0) -> Comm:
    return Comm(mesh, device, multicast=multicast, wait_seconds=wait_seconds, pipeline_link=pipeline_link,
                pipeline_wait_seconds=pipeline_wait_seconds)
