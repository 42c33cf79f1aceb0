"""PyTorch statements of the ops against independent formulations."""
import math

import pytest
import torch
import torch.nn.functional as F

from b200moe import ops
from b200moe.ops import functional as Fn
from b200moe.ops.moe import build_plan, grouped_swiglu
from b200moe.optim import AdamW
from b200moe.utils.schedule import learning_rate_schedule_wrapper


def test_softmax_silu_cross_entropy_match_torch():
    x = torch.randn(5, 11)
    assert torch.allclose(Fn.softmax(x, -1), torch.softmax(x, -1), atol=1e-6)
    assert torch.allclose(Fn.log_softmax(x), torch.log_softmax(x, -1), atol=1e-6)
    assert torch.allclose(Fn.silu(x), F.silu(x), atol=1e-6)
    t = torch.randint(0, 11, (5,))
    assert torch.allclose(Fn.cross_entropy(x, t), F.cross_entropy(x, t), atol=1e-6)
    mask = (torch.rand(5, 11) > 0.3).float()
    mask[:, 0] = 1
    want = torch.softmax(x.masked_fill(mask == 0, float("-inf")), -1)
    assert torch.allclose(Fn.softmax(x, -1, mask), want, atol=1e-6)


def test_rmsnorm_and_fused_add():
    x, d, w = torch.randn(3, 7, 16), torch.randn(3, 7, 16), torch.rand(16) + 0.5
    want = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w
    assert torch.allclose(ops.rmsnorm(x, w), want, atol=1e-5)
    s, y = ops.add_rmsnorm(x, d, w)
    assert torch.allclose(s, x + d) and torch.allclose(y, Fn.rmsnorm_ref(x + d, w), atol=1e-6)


def test_rope_is_pairwise_rotation_with_reference_frequencies():
    hd, seq, theta = 8, 6, 10000.0
    cos, sin = Fn.rope_tables(theta, hd, seq)
    x = torch.randn(2, 3, seq, hd)
    out = Fn.apply_rope_ref(x, cos, sin)
    for pos in range(seq):
        for i in range(hd // 2):
            angle = pos * theta ** ((2 - 2 * (i + 1)) / hd)
            a, b = x[..., pos, 2 * i], x[..., pos, 2 * i + 1]
            assert torch.allclose(out[..., pos, 2 * i], a * math.cos(angle) - b * math.sin(angle), atol=1e-5)
            assert torch.allclose(out[..., pos, 2 * i + 1], a * math.sin(angle) + b * math.cos(angle), atol=1e-5)
    assert torch.allclose(out.norm(dim=-1), x.norm(dim=-1), atol=1e-5)


def test_attention_is_causal_gqa():
    B, S, Hq, Hkv, hd = 2, 12, 8, 2, 16
    q, k, v = torch.randn(B, S, Hq, hd), torch.randn(B, S, Hkv, hd), torch.randn(B, S, Hkv, hd)
    out = ops.rope_attention(q, k, v, None, None)
    scores = torch.einsum("bshd,bthd->bhst", q, k.repeat_interleave(4, 2)) / math.sqrt(hd)
    scores = scores.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
    want = torch.einsum("bhst,bthd->bshd", scores.softmax(-1), v.repeat_interleave(4, 2))
    assert torch.allclose(out, want, atol=1e-5)


def test_router_top2_renormalises():
    logits = torch.randn(64, 8)
    w, idx = ops.router_top2(logits)
    p = logits.softmax(-1)
    top, ti = p.topk(2, -1)
    assert torch.equal(idx, ti)
    assert torch.allclose(w, top / top.sum(-1, keepdim=True), atol=1e-6)
    assert torch.allclose(w.sum(-1), torch.ones(64), atol=1e-6)


@pytest.mark.parametrize("pattern", ["random", "one_expert", "empty_experts"])
def test_plan_layout_and_padding(pattern):
    T, E = 50, 4
    if pattern == "random":
        idx = torch.stack([torch.randperm(E)[:2] for _ in range(T)])
    elif pattern == "one_expert":
        idx = torch.tensor([[2, 0]] * T)
    else:
        idx = torch.tensor([[1, 3]] * T)
    plan = build_plan(idx, E, None, align=16)
    flat = idx.reshape(-1)
    assert torch.equal(flat[plan.order], flat.sort(stable=True).values)
    ends = plan.offs.tolist()
    assert all(e % 16 == 0 for e in ends) and ends[-1] <= plan.rows
    start = 0
    sorted_experts = flat[plan.order]
    for e, end in enumerate(ends):
        rows = plan.recv_to_row[sorted_experts == e]
        n = int((flat == e).sum())
        assert rows.numel() == n
        if n:
            assert torch.equal(rows, torch.arange(start, start + n))
        assert end - start >= n and end - start < n + 16
        start = end


def test_grouped_swiglu_backward_matches_autograd():
    torch.manual_seed(0)
    E, D, Fd, rows = 3, 8, 12, 48
    offs = torch.tensor([16, 16, 48], dtype=torch.int32)
    x = torch.randn(rows, D, requires_grad=True)
    w1, w2, w3 = (torch.randn(E, Fd, D, requires_grad=True), torch.randn(E, D, Fd, requires_grad=True),
                  torch.randn(E, Fd, D, requires_grad=True))
    dy = torch.randn(rows, D)
    for recompute in (False, True):
        for t in (x, w1, w2, w3):
            t.grad = None
        grouped_swiglu(x, w1, w2, w3, offs, recompute).backward(dy)
        got = [t.grad.clone() for t in (x, w1, w2, w3)]
        for t in (x, w1, w2, w3):
            t.grad = None
        y, start = torch.zeros(rows, D), 0
        parts = []
        for e, end in enumerate(offs.tolist()):
            xe = x[start:end]
            parts.append((F.silu(xe @ w1[e].T) * (xe @ w3[e].T)) @ w2[e].T)
            start = end
        torch.cat(parts).backward(dy)
        for g, t in zip(got, (x, w1, w2, w3)):
            assert torch.allclose(g, t.grad, atol=1e-4, rtol=1e-4)


def test_linear_accumulates_into_main_grad():
    w = torch.randn(6, 4, requires_grad=True)
    w.main_grad = torch.zeros(6, 4)
    x = torch.randn(5, 4, requires_grad=True)
    dy = torch.randn(5, 6)
    for _ in range(2):
        ops.linear(x, w).backward(dy)
    assert w.grad is None
    assert torch.allclose(w.main_grad, 2 * dy.T @ x.detach(), atol=1e-5)
    assert torch.allclose(x.grad, 2 * dy @ w.detach(), atol=1e-5)


def test_lm_head_cross_entropy_equals_two_step():
    h, w = torch.randn(2, 5, 8, requires_grad=True), torch.randn(20, 8, requires_grad=True)
    t = torch.randint(0, 20, (2, 5))
    a = ops.lm_head_cross_entropy(h, w, t)
    b = F.cross_entropy((h @ w.T).reshape(-1, 20), t.reshape(-1))
    assert torch.allclose(a, b, atol=1e-6)


def test_lr_schedule_shape():
    f = learning_rate_schedule_wrapper(1.0, 0.1, 10, 110)
    assert f(0) == 0 and f(5) == 0.5 and abs(f(10) - 1.0) < 1e-12
    assert abs(f(60) - 0.55) < 1e-12 and abs(f(110) - 0.1) < 1e-12 and f(500) == 0.1


@pytest.mark.parametrize("state_dtype", [torch.float32, torch.bfloat16])
def test_adamw_matches_closed_form(state_dtype):
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(7, 3))
    ref = p.detach().clone()
    opt = AdamW([p], lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1, state_dtype=state_dtype)
    m = torch.zeros_like(ref)
    v = torch.zeros_like(ref)
    for t in range(1, 4):
        g = torch.randn(7, 3)
        p.grad = g.clone()
        opt.step()
        ref = ref * (1 - 1e-2 * 0.1)
        m = 0.9 * m + 0.1 * g
        v = 0.99 * v + 0.01 * g * g
        ref = ref - 1e-2 * math.sqrt(1 - 0.99 ** t) / (1 - 0.9 ** t) * m / (v.sqrt() + 1e-8)
        if state_dtype == torch.bfloat16:
            m, v = m.bfloat16().float(), v.bfloat16().float()
    tol = 1e-6 if state_dtype == torch.float32 else 2e-3
    assert torch.allclose(p.detach(), ref, atol=tol)
    assert opt.param_groups[0]["t"] == 4
    sd = opt.state_dict()
    assert set(sd["state"][0]) == {"m", "v"}
    assert {"lr", "beta1", "beta2", "t", "epsilon", "lambda_"} <= set(sd["param_groups"][0])


def test_gradient_clipping_and_sampler():
    ps = [torch.nn.Parameter(torch.ones(4)), torch.nn.Parameter(torch.ones(3))]
    for p in ps:
        p.grad = torch.full_like(p, 2.0)
    norm = Fn.gradient_clipping(ps, 1.0)
    assert abs(float(norm) - math.sqrt(28)) < 1e-5
    total = math.sqrt(sum(float((p.grad ** 2).sum()) for p in ps))
    assert abs(total - 1.0) < 1e-4
    logits = torch.tensor([[0.0, 10.0, 0.0]])
    assert int(Fn.sample_output(logits, t=1.0, p=0.0)) == 1


def test_linear_consumes_a_pending_gather_once():
    """A weight may carry the call that gathers its peer rows and multiplies (all-gather fused with the GEMM);
    the first ``linear`` after an optimizer step uses it, later ones and the backward pass use the weight."""
    import torch
    from b200moe import ops
    torch.manual_seed(0)
    x = torch.randn(6, 8, requires_grad=True)
    w = torch.randn(5, 8, requires_grad=True)
    calls = []

    def gather(x2d):
        calls.append(tuple(x2d.shape))
        return x2d.detach() @ w.detach().t()

    w.pending_gather = gather
    y = ops.linear(x, w)
    assert calls == [(6, 8)] and w.pending_gather is None
    assert torch.allclose(y, x @ w.t(), atol=1e-6)
    y.sum().backward()
    assert torch.allclose(x.grad, torch.ones(6, 5) @ w.detach(), atol=1e-6)
    assert torch.allclose(w.grad, torch.ones(6, 5).t() @ x.detach(), atol=1e-6)
    ops.linear(x, w)
    assert calls == [(6, 8)]


def test_fsdp_first_use_gather_needs_the_fused_backend():
    """On CPU (no peer-memory backend) ``gather="first_use"`` marks nothing lazy and training is unchanged."""
    import torch
    from b200moe.models import TransformerLMPipelined
    from b200moe.parallel import FSDPWrapperPipelined
    torch.manual_seed(0)
    model = TransformerLMPipelined(64, 32, 32, 1, 4, 0, 1, num_expert_per_node=2, d_ff=64)
    wrapped = FSDPWrapperPipelined(model, None, None, compute_dtype=torch.float32, gather="first_use")
    assert wrapped._lazy == [] and not any(e.get("lazy") for e in wrapped.flat.entries)
    with pytest.raises(ValueError):
        FSDPWrapperPipelined(model, None, None, gather="sometimes")
