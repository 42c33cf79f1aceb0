"""1F1B pipeline step: microbatch schedule, stage-to-stage transfers, gradient
reduction and the optimizer update.

Same entry point and semantics as the reference scheduler
(pipeline/pipelined_train_overlap.py:26-119): ``warmup = min(pp − stage − 1, m)``
forwards, then forward/backward pairs, then the remaining backwards; each
neighbour exchange is one batched send+recv; the loss of a microbatch is divided
by the microbatch count; the value returned is the mean loss on the last stage
and ``0.0`` elsewhere (or a metrics dict).

Differences in mechanism: the host never blocks on a transfer, so it runs ahead
of the device.  There are two kinds of link between stages.  The NCCL link is the
reference's batched ``isend``/``irecv`` (``work.wait()`` orders the compute stream
after the exchange; a send completes when the neighbour has reached its matching
receive, which keeps the stages in lock step).  The peer link
(``comm.pp.PeerLink``, chosen by the wrapper's ``Comm``) stores the payload into
a landing ring of the neighbour and publishes a message number: a send never
waits for the neighbour unless its ring is full, a receive is a bounded wait on
the stream followed by reads of the slot in place, and a slot is handed back
after the backward pass of its microbatch (``consumed``).
On the last stage the loss comes from the chunked LM-head/cross-entropy op when
the model offers ``loss()`` and the caller passed this framework's
``cross_entropy``; after ``optimizer.step()`` the wrapper refreshes its gathered
weights (``after_optimizer_step``) or runs its fused reduce-scatter/AdamW/
all-gather kernel (``fused_optimizer_step``).
"""
from __future__ import annotations

import collections
import os
import time

import torch
import torch.distributed as dist

from ..config import validate_router_aux_loss_coef
from ..ops import functional as Fn

__all__ = ["pipelined_train_overlap", "pipelined_train", "backward_with_router_loss", "router_loss_metrics"]


def backward_with_router_loss(output, grad, auxiliary, coefficient, split_num):
    if auxiliary is None:
        output.backward(grad)
    else:
        torch.autograd.backward((output, auxiliary), (grad, auxiliary.new_tensor(coefficient / split_num)))


def router_loss_metrics(task_loss, auxiliary, coefficient, pp_group, dp_group):
    metrics = torch.stack((torch.as_tensor(task_loss, device=auxiliary.device).float(), auxiliary))
    if pp_group is not None and dist.get_world_size(pp_group) > 1:
        dist.all_reduce(metrics, group=pp_group)
    if dp_group is not None and dist.get_world_size(dp_group) > 1:
        dist.all_reduce(metrics, group=dp_group)
        metrics /= dist.get_world_size(dp_group)
    return {"task_loss": metrics[0], "router_aux_loss": metrics[1],
            "total_loss": metrics[0] + coefficient * metrics[1]}


class _Link:
    """Batched send/recv with one neighbour stage; the compute stream waits for it."""

    def __init__(self, ranks, stage, pp_group, spec, dtype, device):
        self.ranks, self.stage, self.group = ranks, stage, pp_group
        self.spec, self.dtype, self.device = spec, dtype, device
        self.pending = []

    def exchange(self, send_tensor=None, receive=False, downstream=True):
        peer = self.ranks[self.stage + (1 if downstream else -1)]
        received = torch.empty(self.spec, dtype=self.dtype, device=self.device) if receive else None
        ops = []
        if send_tensor is not None:
            payload = send_tensor.detach().contiguous()
            ops.append(dist.P2POp(dist.isend, payload, peer, group=self.group))
        if receive:
            ops.append(dist.P2POp(dist.irecv, received, peer, group=self.group))
        for work in dist.batch_isend_irecv(ops):
            work.wait()
        return received

    def consumed(self):
        """Nothing to hand back: every received tensor is its own allocation."""


def _make_link(model, ranks, stage, pp_group, spec, dtype, device):
    """The peer-memory link when the wrapper's communication layer offers one for this group, else NCCL."""
    comm = getattr(model, "comm", None)
    offer = getattr(comm, "pp_link", None)
    if offer is not None and pp_group is not None and len(ranks) > 1:
        link = offer(pp_group, stage, spec, dtype)
        if link is not None:
            return link
    return _Link(ranks, stage, pp_group, spec, dtype, device)


def _uses_fused_loss(model, loss_fn):
    target = getattr(model, "module", model)
    return hasattr(target, "loss") and loss_fn in (Fn.cross_entropy, None)


def pipelined_train_overlap(model, optimizer, x, x_label, x_spec: list[int], split_num, pipeline_stage_this,
                            loss_fn, dtype=None, device=None, pp_group=None, dp_group=None,
                            router_aux_loss_coef=0.0, return_metrics=False):
    validate_router_aux_loss_coef(router_aux_loss_coef)
    if split_num <= 0:
        raise ValueError("split_num must be positive")
    if x_spec[0] % split_num != 0:
        raise ValueError(f"batch size {x_spec[0]} must be divisible by split_num {split_num}")
    stages = 1 if pp_group is None else dist.get_world_size(pp_group)
    if not 0 <= pipeline_stage_this < stages:
        raise ValueError("pipeline_stage_this must identify a stage in pp_group")
    first, last = pipeline_stage_this == 0, pipeline_stage_this == stages - 1
    ranks = dist.get_process_group_ranks(pp_group) if pp_group is not None else []
    mb_size = x_spec[0] // split_num
    link = _make_link(model, ranks, pipeline_stage_this, pp_group, [mb_size, *x_spec[1:]], dtype, device)
    data_chunks = torch.split(x, mb_size) if first else None
    label_chunks = torch.split(x_label, mb_size) if last else None
    fused_loss = last and _uses_fused_loss(model, loss_fn)
    in_flight = collections.deque()
    aux_total = torch.zeros((), device=device, dtype=torch.float32)
    loss_total = torch.zeros((), device=device, dtype=torch.float32) if last else 0.0
    optimizer.zero_grad(set_to_none=True)
    model.clear_grad_accumulators()
    forward_count = 0

    timing = os.environ.get("B200MOE_PIPELINE_TIMING") == "1" and torch.cuda.is_available()
    spans, host = [], {"fwd": 0.0, "bwd": 0.0, "xchg": 0.0}

    def timed(kind, fn, *args):
        """Optional instrumentation: device time of each forward/backward (CUDA events) and host time spent
        issuing it; printed per rank at the end of the step."""
        if not timing:
            return fn(*args)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        begin.record()
        out = fn(*args)
        end.record()
        host[kind] += time.perf_counter() - t0
        spans.append((kind, begin, end))
        return out

    def forward_microbatch(x_in):
        nonlocal forward_count
        if not first:
            x_in.requires_grad_(True)
        aux = None
        if fused_loss:
            # the loss of a microbatch is back-propagated with the factor 1/split_num (backward_microbatch below)
            scale = {"grad_scale": 1.0 / split_num} if torch.is_grad_enabled() else {}
            out = model.loss(x_in, label_chunks[forward_count], return_aux_loss=True, **scale) \
                if router_aux_loss_coef else model.loss(x_in, label_chunks[forward_count], **scale)
        else:
            out = model(x_in, return_aux_loss=True) if router_aux_loss_coef else model(x_in)
        if router_aux_loss_coef:
            out, aux = out
        in_flight.append((x_in, out, aux, forward_count))
        forward_count += 1
        return out

    def backward_microbatch(grad):
        nonlocal loss_total
        x_in, out, aux, index = in_flight.popleft()
        if aux is not None:
            aux_total.add_(aux.detach() / split_num)
        if last:
            loss = out if fused_loss else loss_fn(out, label_chunks[index])
            loss_total = loss_total + loss.detach().float() / split_num
            backward_with_router_loss(loss / split_num, None, aux, router_aux_loss_coef, split_num)
        else:
            backward_with_router_loss(out, grad, aux, router_aux_loss_coef, split_num)
        model.accumulate_full_gradients()
        link.consumed()
        return None if first else x_in.grad

    warmup = min(stages - pipeline_stage_this - 1, split_num)
    steady = split_num - warmup
    step_t0 = time.perf_counter()
    for i in range(warmup):
        x_in = data_chunks[i] if first else link.exchange(receive=True, downstream=False)
        link.exchange(send_tensor=timed("fwd", forward_microbatch, x_in))
    if steady:
        x_in = data_chunks[warmup] if first else link.exchange(receive=True, downstream=False)
    for i in range(steady):
        out = timed("fwd", forward_microbatch, x_in)
        grad = None if last else link.exchange(send_tensor=out, receive=True)
        input_grad = timed("bwd", backward_microbatch, grad)
        more = i + 1 < steady
        if not first:
            x_in = link.exchange(send_tensor=input_grad, receive=more, downstream=False)
        elif more:
            x_in = data_chunks[warmup + i + 1]
    for _ in range(steady, split_num):
        input_grad = timed("bwd", backward_microbatch, link.exchange(receive=True))
        if not first:
            link.exchange(send_tensor=input_grad, downstream=False)

    fused_step = getattr(model, "fused_optimizer_step", None)
    if fused_step is None or not fused_step(optimizer):
        model.reduce_accumulated_gradients()
        optimizer.step()
        refresh = getattr(model, "after_optimizer_step", None)
        if refresh is not None:
            refresh()
    if timing:
        torch.cuda.synchronize()
        total = {"fwd": 0.0, "bwd": 0.0}
        for kind, begin, end in spans:
            total[kind] += begin.elapsed_time(end)
        print(f"[pipeline timing] rank {dist.get_rank() if dist.is_initialized() else 0} stage {pipeline_stage_this}: "
              f"device fwd {total['fwd']:.0f} ms, bwd {total['bwd']:.0f} ms over {split_num} microbatches; "
              f"host issue fwd {host['fwd'] * 1e3:.0f} ms, bwd {host['bwd'] * 1e3:.0f} ms; "
              f"step wall {(time.perf_counter() - step_t0) * 1e3:.0f} ms", flush=True)
    if return_metrics:
        return router_loss_metrics(loss_total, aux_total, router_aux_loss_coef, pp_group, dp_group)
    return loss_total


def pipelined_train(model, optimizer, x, x_label, x_spec: list[int], split_num, pipeline_stage_this, loss_fn,
                    dtype=None, device=None, pp_group=None, dp_group=None):
    """Older entry point (reference pipeline/pipelined_train.py:7-114): the same
    1F1B schedule without the router auxiliary loss.  Like the original it
    rewrites ``x_spec[0]`` to the microbatch size."""
    result = pipelined_train_overlap(model, optimizer, x, x_label, list(x_spec), split_num, pipeline_stage_this,
                                     loss_fn, dtype=dtype, device=device, pp_group=pp_group, dp_group=dp_group)
    x_spec[0] = x_spec[0] // split_num
    return result
