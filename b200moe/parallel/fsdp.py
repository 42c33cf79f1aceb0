"""Sharded data parallelism for one pipeline stage, with optional replicas.

Public surface is the reference's ``FSDPWrapperPipelined`` (implementation/
distributed/ddp_modules.py:103-297): construction broadcasts from shard rank 0,
keeps row block ``[idx·rows/n, (idx+1)·rows/n)`` of every ``LinearLayer`` /
``EmbeddingLayer`` weight as the fp32 master parameter, keeps RMSNorm gains
replicated, and offers ``clear_grad_accumulators``, ``accumulate_full_gradients``,
``reduce_accumulated_gradients`` to the pipeline step.  Checkpoint keys and
shapes are unchanged (row shards under ``module.…``).

The mechanism is different.  The reference re-gathers every weight for every
microbatch in forward and backward through module hooks (≈2560 all-gathers per
step) and keeps full fp32 gradient copies per parameter.  Here:

* one flat bf16 buffer holds all *full* compute weights of the stage and stays
  gathered for the whole step (dense weights of a stage are < 1.3 GB in bf16;
  HBM is 180 GB).  It is refreshed once per step, after the optimizer update.
  q, k, v sit next to each other so attention runs one fused QKV GEMM;
* one flat fp32 buffer holds the full gradients; weight-gradient GEMMs
  accumulate into it directly (``main_grad``), so ``accumulate_full_gradients``
  has nothing left to do;
* one flat fp32 master / gradient-shard / moment set backs all shards, so the
  optimizer update is one launch.
* with ``backend="fused"`` the flat buffers live in symmetric memory and the
  end-of-step reduce-scatter, AdamW update and re-gather run as one peer-memory
  kernel (``b200moe.comm``); ``backend="nccl"`` uses ``torch.distributed``
  collectives and is also what the CPU/gloo tier runs.
* expert weights are broadcast over the replica group at start and their
  gradients are averaged over it every step (the reference leaves replicas of
  experts unsynchronised, kubernetes/chart/README.md:25-27).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.layers import (EmbeddingLayer, GroupedPositionWiseFFLayer, LinearLayer, MultiHeadLayerLL,
                             RMSNormLayer)

__all__ = ["FSDPWrapperPipelined", "FlatShards"]


def _group_size(group) -> int:
    if not (dist.is_available() and dist.is_initialized()):
        return 1
    return dist.get_world_size(group)


def _group_rank(group) -> int:
    if not (dist.is_available() and dist.is_initialized()):
        return 0
    return dist.get_rank(group)


class FlatShards:
    """Flat storage behind the sharded parameters of one stage."""

    def __init__(self, entries, world: int, index: int, compute_dtype, device, allocator=None):
        self.entries = entries
        self.world, self.index = world, index
        shard_total = sum(e["shard_numel"] for e in entries)
        full_total = sum(e["full_numel"] for e in entries)
        alloc = allocator or (lambda n, dtype: torch.zeros(n, dtype=dtype, device=device))
        self.master = torch.zeros(shard_total, dtype=torch.float32, device=device)
        self.full_w = alloc(full_total, compute_dtype)
        self.full_g = alloc(full_total, torch.float32)
        self.shard_grad = self.full_g if world == 1 else torch.zeros(shard_total, dtype=torch.float32, device=device)
        self.m = self.v = None
        self._by_param = {}
        for e in entries:
            self._by_param[id(e["param"])] = e

    def moment_views(self, p):
        if self.m is None:
            self.m = torch.zeros_like(self.master)
            self.v = torch.zeros_like(self.master)
        e = self._by_param[id(p)]
        lo, hi = e["shard_off"], e["shard_off"] + e["shard_numel"]
        return self.m[lo:hi].view(e["shard_shape"]), self.v[lo:hi].view(e["shard_shape"])

    def shard_view(self, buf, e):
        return buf[e["shard_off"]:e["shard_off"] + e["shard_numel"]].view(e["shard_shape"])

    def full_view(self, buf, e):
        return buf[e["full_off"]:e["full_off"] + e["full_numel"]].view(e["full_shape"])


class FSDPWrapperPipelined(nn.Module):
    def __init__(self, module: nn.Module, FSDP_communication_group=None, DDP_communication_group=None,
                 compute_dtype: torch.dtype = torch.float32, moe_compute_dtype: torch.dtype = torch.bfloat16,
                 *, prefetch_weights: bool = True, backend: str = "nccl", expert_grad_dtype=torch.float32,
                 expert_state_dtype=torch.float32, comm=None, gather: str = "step"):
        super().__init__()
        self.module = module
        self.compute_dtype = compute_dtype
        self.FSDP_communication_group = FSDP_communication_group
        self.DDP_communication_group = DDP_communication_group
        self.group_size = _group_size(FSDP_communication_group)
        self.shard_index = _group_rank(FSDP_communication_group)
        self.ddp_size = 1 if DDP_communication_group is None else _group_size(DDP_communication_group)
        self.backend = backend
        self.comm = comm
        if gather not in ("step", "first_use"):
            raise ValueError("gather must be 'step' or 'first_use'")
        self.gather = gather
        self.sharded_params, self.replicated_params, self.expert_params = [], [], []
        device = next(module.parameters()).device
        distributed = dist.is_available() and dist.is_initialized()
        fsdp_src = dist.get_global_rank(FSDP_communication_group, 0) if distributed and FSDP_communication_group is not None else 0

        ordered = self._ordered_modules(module)
        entries, shard_off, full_off = [], 0, 0
        for name, sub in ordered:
            weight = sub.weight
            if distributed and self.group_size > 1:
                dist.broadcast(weight.data, fsdp_src, group=FSDP_communication_group)
            rows = weight.shape[0]
            if rows % self.group_size:
                raise AssertionError(
                    f"Cannot shard parameter with shape {tuple(weight.shape)} over {self.group_size} ranks")
            shard_rows = rows // self.group_size
            shard_shape = (shard_rows, *weight.shape[1:])
            entry = {"name": name, "module": sub, "param": weight, "full_shape": tuple(weight.shape),
                     "shard_shape": shard_shape, "full_numel": weight.numel(),
                     "shard_numel": weight.numel() // self.group_size, "shard_off": shard_off,
                     "full_off": full_off}
            shard_off += entry["shard_numel"]
            full_off += entry["full_numel"]
            entries.append(entry)
        allocator = comm.alloc_flat if (comm is not None and backend == "fused") else None
        self.flat = FlatShards(entries, self.group_size, self.shard_index, compute_dtype, device, allocator)
        for e in entries:
            weight = e["param"]
            lo = self.shard_index * e["shard_shape"][0]
            shard = self.flat.shard_view(self.flat.master, e)
            shard.copy_(weight.data[lo:lo + e["shard_shape"][0]])
            weight.data = shard
            weight._flat = self.flat
            compute = self.flat.full_view(self.flat.full_w, e)
            compute.requires_grad_(True)
            compute.main_grad = self.flat.full_view(self.flat.full_g, e)
            e["module"].compute_weight = compute
            self.sharded_params.append(weight)
        self._fuse_qkv(module)

        for sub in module.modules():
            if isinstance(sub, RMSNormLayer):
                if distributed and self.group_size > 1:
                    dist.broadcast(sub.weight.data, fsdp_src, group=FSDP_communication_group)
                self.replicated_params.append(sub.weight)
            elif isinstance(sub, GroupedPositionWiseFFLayer):
                for p in (sub.w1, sub.w2, sub.w3):
                    p.main_grad = torch.zeros(p.shape, dtype=expert_grad_dtype, device=p.device)
                    p._state_dtype = expert_state_dtype
                    self.expert_params.append(p)

        if DDP_communication_group is not None and self.ddp_size > 1:
            ddp_src = dist.get_global_rank(DDP_communication_group, 0)
            dist.broadcast(self.flat.master, ddp_src, group=DDP_communication_group)
            for p in self.replicated_params + self.expert_params:
                dist.broadcast(p.data, ddp_src, group=DDP_communication_group)

        if hasattr(module, "activation_dtype"):
            module.activation_dtype = compute_dtype
        self.fused = backend == "fused" and comm is not None and device.type == "cuda"
        self._pending_reduce = False
        self._weights_fresh = False
        if self.fused:
            from ..models.layers import MoELayerMulti
            for sub in module.modules():
                if isinstance(sub, MoELayerMulti):
                    sub.comm = comm
        if device.type == "cuda":
            self.flat.fused_update = self._fused_update
        self._lazy = []
        if self.fused and self.group_size > 1 and gather == "first_use":
            self._mark_lazy(module)
        self._gain_flat = None
        self._seen_versions = None
        self.materialize()

    # -- construction helpers ------------------------------------------------------------
    @staticmethod
    def _ordered_modules(module):
        """Sharded modules in ``named_modules`` order, except that q, k, v of one
        attention layer are made adjacent (q, k, v) for the fused projection."""
        found = [(n, m) for n, m in module.named_modules() if isinstance(m, (LinearLayer, EmbeddingLayer))]
        rank = {}
        for name, sub in module.named_modules():
            if isinstance(sub, MultiHeadLayerLL):
                rank[id(sub.q_proj)], rank[id(sub.k_proj)], rank[id(sub.v_proj)] = 0, 1, 2
        out, i = [], 0
        while i < len(found):
            if id(found[i][1]) in rank:
                trio = found[i:i + 3]
                if len(trio) == 3 and all(id(m) in rank for _, m in trio):
                    out.extend(sorted(trio, key=lambda nm: rank[id(nm[1])]))
                    i += 3
                    continue
            out.append(found[i])
            i += 1
        return out

    def _fuse_qkv(self, module):
        by_module = {id(e["module"]): e for e in self.flat.entries}
        for sub in module.modules():
            if not isinstance(sub, MultiHeadLayerLL):
                continue
            eq, ek, ev = (by_module[id(m)] for m in (sub.q_proj, sub.k_proj, sub.v_proj))
            if not (eq["full_off"] + eq["full_numel"] == ek["full_off"]
                    and ek["full_off"] + ek["full_numel"] == ev["full_off"]):
                continue
            lo, hi = eq["full_off"], ev["full_off"] + ev["full_numel"]
            rows = eq["full_shape"][0] + ek["full_shape"][0] + ev["full_shape"][0]
            fused = self.flat.full_w[lo:hi].view(rows, eq["full_shape"][1])
            fused.requires_grad_(True)
            fused.main_grad = self.flat.full_g[lo:hi].view(rows, eq["full_shape"][1])
            sub.qkv_weight = fused

    def _mark_lazy(self, module):
        """``gather="first_use"``: the attention projections are not pushed to the peers by the end-of-step
        kernel; the first GEMM that uses them after an optimizer step pulls the peers' rows itself
        (``Comm.allgather_gemm``), so their all-gather runs under tensor-core work of the next step."""
        by_module = {id(e["module"]): e for e in self.flat.entries}
        for sub in module.modules():
            if not isinstance(sub, MultiHeadLayerLL):
                continue
            trio = [by_module[id(m)] for m in (sub.q_proj, sub.k_proj, sub.v_proj)]
            if sub.qkv_weight is not None:
                for e in trio:
                    e["lazy"] = True
                self._lazy.append((sub.qkv_weight, [e["full_shape"][0] for e in trio]))
            out = by_module[id(sub.output_proj)]
            out["lazy"] = True
            self._lazy.append((sub.output_proj.compute_weight, [out["full_shape"][0]]))

    def _arm_lazy(self):
        import functools
        for weight, segments in self._lazy:
            weight.pending_gather = functools.partial(self.comm.allgather_gemm, w=weight, segments=segments)

    def _disarm_lazy(self):
        for weight, _ in self._lazy:
            weight.pending_gather = None

    # -- weights -------------------------------------------------------------------------
    @torch.no_grad()
    def materialize(self):
        """Refresh the gathered compute weights from the fp32 master shards."""
        flat = self.flat
        if getattr(self, "fused", False) and self.group_size > 1:
            self.comm.allgather_cast(flat)
            self._disarm_lazy()
        else:
            for e in flat.entries:
                full = flat.full_view(flat.full_w, e)
                shard = flat.shard_view(flat.master, e).to(self.compute_dtype)
                if self.group_size == 1:
                    full.copy_(shard)
                else:
                    dist.all_gather_into_tensor(full, shard.contiguous(), group=self.FSDP_communication_group)
        self._seen_versions = self._versions()

    def _versions(self):
        return self.flat.master._version

    def _fused_update(self, lr, beta1, beta2, eps, decay, a_t) -> bool:
        """Optimizer hook for the flat shards.  One rank: AdamW and the bf16 cast of
        the new weights in one kernel.  Several ranks, fused backend: reduce-scatter,
        AdamW and the weight all-gather in one peer-memory kernel."""
        from ..ops import native, use_native
        flat = self.flat
        if not use_native(flat.master, "adamw"):
            return False
        if flat.m is None:
            flat.m, flat.v = torch.zeros_like(flat.master), torch.zeros_like(flat.master)
        if self.group_size == 1:
            native.adamw_(flat.master, flat.shard_grad, flat.m, flat.v, lr, beta1, beta2, eps, decay, a_t,
                          p_bf16=flat.full_w if flat.full_w.dtype == torch.bfloat16 else None)
            self._weights_fresh = flat.full_w.dtype == torch.bfloat16
            return True
        if not self.fused:
            return False
        self.comm.fused_update(flat, self._pending_reduce, lr, beta1, beta2, eps, decay, a_t)
        self._pending_reduce = False
        self._weights_fresh = True
        self._arm_lazy()
        return True

    def after_optimizer_step(self):
        if self._weights_fresh:
            self._weights_fresh = False
            self._seen_versions = self._versions()
            return
        self.materialize()

    def forward(self, x, **kwargs):
        if self._seen_versions != self._versions():
            self.materialize()
        return self.module.forward(x, **kwargs)

    def loss(self, x, targets, **kwargs):
        if self._seen_versions != self._versions():
            self.materialize()
        return self.module.loss(x, targets, **kwargs)

    def load_state_dict(self, state_dict, strict: bool = True, assign: bool = False):
        result = super().load_state_dict(state_dict, strict=strict, assign=False)
        self.materialize()
        return result

    # -- gradients -----------------------------------------------------------------------
    @torch.no_grad()
    def clear_grad_accumulators(self):
        budget = getattr(self, "activation_budget", None)
        if budget is not None:
            budget.reset()      # start of a step: no activation of the previous one is alive
        if self.comm is not None and getattr(self, "fused", False):
            self.comm.new_step()
        self.flat.full_g.zero_()
        for p in self.sharded_params + self.replicated_params:
            p.grad = None
        for p in self.expert_params:
            p.main_grad.zero_()
            p.grad = None

    def accumulate_full_gradients(self):
        """Nothing to do: weight-gradient GEMMs add into the flat fp32 buffer."""

    @torch.no_grad()
    def reduce_accumulated_gradients(self):
        flat = self.flat
        fsdp_group, ddp_group = self.FSDP_communication_group, self.DDP_communication_group
        if self.group_size > 1:
            if self.fused and self.ddp_size == 1:
                self._pending_reduce = True          # folded into the optimizer kernel
            elif self.fused:
                self.comm.reduce_scatter_avg(flat)
            else:
                works = []
                for e in flat.entries:
                    works.append(dist.reduce_scatter_tensor(
                        flat.shard_view(flat.shard_grad, e), flat.full_view(flat.full_g, e),
                        op=dist.ReduceOp.AVG, group=fsdp_group, async_op=True))
                for w in works:
                    w.wait()
        gains = [p for p in self.replicated_params if p.grad is not None]
        if gains and (self.group_size > 1 or self.ddp_size > 1):
            packed = torch.cat([p.grad.reshape(-1).float() for p in gains])
            if self.group_size > 1:
                dist.all_reduce(packed, op=dist.ReduceOp.AVG, group=fsdp_group)
            if self.ddp_size > 1:
                dist.all_reduce(packed, op=dist.ReduceOp.AVG, group=ddp_group)
            offset = 0
            for p in gains:
                p.grad.copy_(packed[offset:offset + p.numel()].view_as(p.grad))
                offset += p.numel()
        if self.ddp_size > 1:
            if self.fused:
                self.comm.allreduce_avg(flat.shard_grad, ddp_group)
                for p in self.expert_params:
                    self.comm.allreduce_avg(p.main_grad, ddp_group)
            else:
                dist.all_reduce(flat.shard_grad, op=dist.ReduceOp.AVG, group=ddp_group)
                for p in self.expert_params:
                    dist.all_reduce(p.main_grad, op=dist.ReduceOp.AVG, group=ddp_group)
        for e in flat.entries:
            e["param"].grad = flat.shard_view(flat.shard_grad, e)

    def finish_gradient_synchronization(self):
        """Kept for API parity; all reductions above complete before returning."""
