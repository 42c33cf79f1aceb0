"""Pipeline links over peer memory.

A ``PeerLink`` carries the activations a stage sends downstream and the gradients
it sends upstream without NCCL: the sender copies the payload straight into a
landing slot of the receiver (peer stores over NVLink, ``csrc/pp_link.cu``) and
publishes a message number; the receiver makes its stream wait for that number
and then reads the slot in place.  Unlike the batched ``isend``/``irecv`` pair of
the reference scheduler (pipeline/pipelined_train_overlap.py:40-75), a send does
not wait for the neighbour to reach its matching receive, so a stage that is
ahead stays ahead: the stages are coupled by data only, not by the rendezvous of
their transfers.  A send waits only when the receiver's ring is full.

Protocol (per direction, for the life of the link): messages are numbered from 1;
message ``n`` uses slot ``(n − 1) mod R``; the receiver acknowledges messages in
order, after the backward pass of the microbatch that used them, with the count
of backward passes done so far.  Under 1F1B a stage holds at most ``pp − stage``
activations, so an activation ring of ``pp`` slots never makes a sender wait; the
gradient ring has two slots (a gradient is consumed by the backward pass that
follows its arrival).

``PeerLink`` itself is bookkeeping; the three device operations (send, wait,
acknowledge) sit behind a transport object.  ``DeviceTransport`` launches the
kernels; tests substitute a host transport to run the real scheduler on CPU
ranks and check the numbering and the ring discipline.
"""
from __future__ import annotations

import ctypes
import math

import torch
import torch.distributed as dist

from ..ops import native

__all__ = ["PeerLink", "DeviceTransport", "GRAD_SLOTS"]

GRAD_SLOTS = 2
_ACT_FLAGS, _GRAD_FLAGS, _ACK_ACT, _ACK_GRAD, _FLAG_WORDS = 0, 16, 32, 33, 64


class DeviceTransport:
    """Symmetric buffers over the pipeline group and the kernel launches on them."""

    def __init__(self, group, device, status, slot_bytes: int, slots: int, wait_seconds: float):
        from . import SymmBuffer
        self.device, self.status = device, status
        self.slot_bytes = slot_bytes
        self.data = SymmBuffer(slot_bytes * slots, torch.uint8, device, group, zero=False)
        self.flags = SymmBuffer(_FLAG_WORDS, torch.int32, device, group)
        self.ticket = torch.zeros(1, dtype=torch.int32, device=device)
        self.wait_ns = int(float(wait_seconds) * 1e9)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def buffers(self):
        return [self.data, self.flags]

    def slot(self, index: int, spec, dtype) -> torch.Tensor:
        numel = math.prod(spec)
        begin = index * self.slot_bytes
        return self.data.tensor[begin:begin + numel * dtype.itemsize].view(dtype).view(spec)

    def send(self, payload, peer: int, slot: int, flag: int, ack_word: int, seq: int, need_ack: int) -> None:
        nbytes = payload.numel() * payload.element_size()
        native._call("b2_pp_send", ctypes.c_void_p(payload.data_ptr()),
                     ctypes.c_void_p(self.data.ptrs[peer] + slot * self.slot_bytes), ctypes.c_longlong(nbytes),
                     ctypes.c_void_p(self.flags.ptrs[peer] + 4 * flag),
                     ctypes.c_void_p(self.flags.tensor.data_ptr() + 4 * ack_word), ctypes.c_int(seq),
                     ctypes.c_int(need_ack), ctypes.c_longlong(self.wait_ns), ctypes.c_void_p(self.ticket.data_ptr()),
                     ctypes.c_void_p(self.status.data_ptr()), native._stream())

    def wait(self, flag: int, seq: int) -> None:
        native._call("b2_pp_wait", ctypes.c_void_p(self.flags.tensor.data_ptr() + 4 * flag), ctypes.c_int(seq),
                     ctypes.c_longlong(self.wait_ns), ctypes.c_void_p(self.status.data_ptr()), native._stream())

    def ack(self, upstream, downstream, value: int) -> None:
        up = 0 if upstream is None else self.flags.ptrs[upstream] + 4 * _ACK_ACT
        down = 0 if downstream is None else self.flags.ptrs[downstream] + 4 * _ACK_GRAD
        native._call("b2_pp_ack", ctypes.c_void_p(up), ctypes.c_void_p(down), ctypes.c_int(value), native._stream())


class PeerLink:
    """The transfers of one pipeline stage; same ``exchange`` call as the NCCL link of ``parallel.pipeline``."""

    def __init__(self, stage: int, stages: int, spec, dtype, transport, act_slots: int | None = None):
        if not 0 <= stage < stages:
            raise ValueError("stage out of range")
        self.stage, self.stages = stage, stages
        self.spec, self.dtype = list(spec), dtype
        self.act_slots = stages if act_slots is None else int(act_slots)
        # stage 1 takes in ``stages − 1`` activations before its first backward pass hands one back: a smaller ring
        # would stop the schedule for good
        if not max(1, stages - 1) <= self.act_slots <= _GRAD_FLAGS:
            raise ValueError(f"activation ring of {self.act_slots} slots ({max(1, stages - 1)}..{_GRAD_FLAGS})")
        self.transport = transport
        self.sent_act = self.sent_grad = self.got_act = self.got_grad = self.done = 0

    @staticmethod
    def slot_bytes(spec, dtype) -> int:
        return (math.prod(spec) * dtype.itemsize + 255) // 256 * 256

    @classmethod
    def over_group(cls, group, device, status, spec, dtype, wait_seconds: float = 120.0):
        """Link of this rank inside the pipeline group ``group`` (collective: every stage calls it)."""
        stages, stage = dist.get_world_size(group), dist.get_rank(group)
        if stages > 8:
            raise ValueError("peer links span at most 8 stages")
        transport = DeviceTransport(group, device, status, cls.slot_bytes(spec, dtype), stages + GRAD_SLOTS,
                                    wait_seconds)
        return cls(stage, stages, spec, dtype, transport)

    def buffers(self):
        return self.transport.buffers()

    # -- one direction at a time ---------------------------------------------------------------
    def _send(self, tensor, downstream: bool) -> None:
        payload = tensor.detach().contiguous()
        if payload.dtype != self.dtype or payload.numel() != math.prod(self.spec):
            raise ValueError(f"payload {tuple(payload.shape)} {payload.dtype} does not match the link "
                             f"({self.spec}, {self.dtype})")
        if downstream:                      # an activation for stage + 1
            self.sent_act += 1
            n, ring = self.sent_act, self.act_slots
            slot = (n - 1) % ring
            self.transport.send(payload, self.stage + 1, slot, _ACT_FLAGS + slot, _ACK_ACT, n, n - ring)
        else:                               # a gradient for stage − 1
            self.sent_grad += 1
            n, ring = self.sent_grad, GRAD_SLOTS
            slot = (n - 1) % ring
            self.transport.send(payload, self.stage - 1, self.act_slots + slot, _GRAD_FLAGS + slot, _ACK_GRAD, n,
                                n - ring)

    def _receive(self, downstream: bool):
        if downstream:                      # a gradient from stage + 1
            self.got_grad += 1
            slot = (self.got_grad - 1) % GRAD_SLOTS
            self.transport.wait(_GRAD_FLAGS + slot, self.got_grad)
            return self.transport.slot(self.act_slots + slot, self.spec, self.dtype)
        self.got_act += 1                   # an activation from stage − 1
        slot = (self.got_act - 1) % self.act_slots
        self.transport.wait(_ACT_FLAGS + slot, self.got_act)
        return self.transport.slot(slot, self.spec, self.dtype)

    # -- the scheduler's interface ----------------------------------------------------------------
    def exchange(self, send_tensor=None, receive=False, downstream=True):
        if send_tensor is not None:
            self._send(send_tensor, downstream)
        return self._receive(downstream) if receive else None

    def consumed(self) -> None:
        """The backward pass of one more microbatch is on the stream: its activation slot (from upstream) and its
        gradient slot (from downstream) may be reused once the stream gets here."""
        self.done += 1
        upstream = self.stage - 1 if self.stage > 0 else None
        downstream = self.stage + 1 if self.stage < self.stages - 1 else None
        if upstream is not None or downstream is not None:
            self.transport.ack(upstream, downstream, self.done)
