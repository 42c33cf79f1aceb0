"""AdamW with the reference's update rule and state layout.

Per parameter (reference implementation/optimizer.py:6-40)::

    p ← p · (1 − lr·λ)
    m ← β1·m + (1−β1)·g
    v ← β2·v + (1−β2)·g²
    p ← p − a_t · m / (√v + ε),   a_t = lr · √(1−β2ᵗ) / (1−β1ᵗ)

Group keys are ``lr, beta1, beta2, t, epsilon, lambda_``; ``t`` starts at 1 and
is incremented once per ``step``; state keys are ``"m"`` and ``"v"``.

Differences in mechanism: the arithmetic runs in fp32 whatever the storage
types; a parameter may carry ``main_grad`` (its gradient accumulator, possibly
of another dtype) which is used instead of ``.grad``; parameters that are views
of one flat buffer (``p._flat``) are updated with one launch over the whole
buffer; on CUDA the update is one fused kernel per tensor or flat buffer
instead of six elementwise launches.  Moment dtype: ``state_dtype`` argument,
or per parameter ``p._state_dtype``, default fp32.
"""
from __future__ import annotations

import math

import torch

__all__ = ["AdamW", "adamw_update_"]


def adamw_update_(p, g, m, v, lr, beta1, beta2, eps, weight_decay, a_t, grad_scale: float = 1.0):
    """One AdamW update on tensors of equal shape; fp32 arithmetic."""
    from ..ops import use_native
    if use_native(p, "adamw"):
        from ..ops import native
        native.adamw_(p, g, m, v, lr, beta1, beta2, eps, weight_decay, a_t, grad_scale)
        return
    gf = g.float()
    if grad_scale != 1.0:
        gf = gf * grad_scale
    if p.dtype == torch.float32 and m.dtype == torch.float32 and v.dtype == torch.float32:
        p.mul_(1 - lr * weight_decay)
        m.mul_(beta1).add_(gf, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
        p.addcdiv_(m, v.sqrt().add_(eps), value=-a_t)
        return
    pf = p.float() * (1 - lr * weight_decay)
    mf = m.float() * beta1 + gf * (1 - beta1)
    vf = v.float() * beta2 + gf * gf * (1 - beta2)
    pf = pf - a_t * mf / (vf.sqrt() + eps)
    p.copy_(pf)
    m.copy_(mf)
    v.copy_(vf)


class AdamW(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.1, state_dtype=None):
        defaults = {"lr": lr, "beta1": betas[0], "beta2": betas[1], "t": 1, "epsilon": eps,
                    "lambda_": weight_decay}
        super().__init__(params, defaults)
        self.state_dtype = state_dtype

    def _moments(self, p):
        state = self.state[p]
        if "m" not in state:
            dtype = getattr(p, "_state_dtype", None) or self.state_dtype or torch.float32
            flat = getattr(p, "_flat", None)
            if flat is not None:
                state["m"], state["v"] = flat.moment_views(p)
            else:
                state["m"] = torch.zeros_like(p, dtype=dtype)
                state["v"] = torch.zeros_like(p, dtype=dtype)
        return state["m"], state["v"]

    def materialize_state(self) -> int:
        """Allocate the moments of every parameter now instead of at the first ``step`` (they are zeros either
        way), so that whoever plans the remaining device memory sees them.  Returns the bytes they take."""
        total = 0
        for group in self.param_groups:
            for p in group["params"]:
                m, v = self._moments(p)
                total += m.numel() * m.element_size() + v.numel() * v.element_size()
        return total

    @staticmethod
    def _grad_of(p):
        main = getattr(p, "main_grad", None)
        if main is not None and getattr(p, "_use_main_grad", True):
            return main
        return p.grad

    @torch.no_grad()
    def step(self, closure=None, **kwargs):
        for group in self.param_groups:
            lr, beta1, beta2 = group["lr"], group["beta1"], group["beta2"]
            t, eps, decay = group["t"], group["epsilon"], group["lambda_"]
            a_t = lr * math.sqrt(1 - beta2 ** t) / (1 - beta1 ** t)
            done_flats = set()
            for p in group["params"]:
                grad = self._grad_of(p)
                if grad is None:
                    continue
                m, v = self._moments(p)
                flat = getattr(p, "_flat", None)
                if flat is not None:
                    if id(flat) not in done_flats:
                        done_flats.add(id(flat))
                        fused = getattr(flat, "fused_update", None)
                        if fused is None or not fused(lr, beta1, beta2, eps, decay, a_t):
                            adamw_update_(flat.master, flat.shard_grad, flat.m, flat.v,
                                          lr, beta1, beta2, eps, decay, a_t)
                    continue
                adamw_update_(p.data, grad, m, v, lr, beta1, beta2, eps, decay, a_t,
                              grad_scale=getattr(p, "_grad_scale", 1.0))
            group["t"] = t + 1

    def load_state_dict(self, state_dict):
        """Loaded moments are copied into the flat buffers of flat parameters so
        the fused update keeps addressing one contiguous range."""
        super().load_state_dict(state_dict)
        for group in self.param_groups:
            for p in group["params"]:
                flat = getattr(p, "_flat", None)
                state = self.state.get(p)
                if flat is None or not state or "m" not in state:
                    continue
                m_view, v_view = flat.moment_views(p)
                if state["m"].data_ptr() != m_view.data_ptr():
                    m_view.copy_(state["m"])
                    v_view.copy_(state["v"])
                    state["m"], state["v"] = m_view, v_view
