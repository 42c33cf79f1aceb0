"""sm_100a kernels against plain PyTorch fp32 statements of the same ops."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def native():
    from b200moe.ops import native as n
    n.require()
    return n


@pytest.fixture(params=[0, 2, 3], ids=["tiles_auto", "tiles_256_one_cta", "tiles_cta_pair"])
def tile_mode(request, native):
    """GEMM CTA tile: automatic choice, forced single-CTA 256x256, forced CTA pairs (cta_group::2)."""
    native.set_gemm_tile_mode(request.param)
    yield request.param
    native.set_gemm_tile_mode(0)


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 1024, 4096), (1024, 6144, 1024),
                                   (200, 384, 192), (128, 32000, 512)])
def test_gemm_nt(native, tile_mode, M, N, K):
    x, w = _rand(M, K), _rand(N, K, scale=0.05)
    got = native.gemm_nt(x, w)
    want = x.float() @ w.float().t()
    assert _rel(got, want) < 6e-3
    native.check_status()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 1024, 512), (384, 4096, 2048), (256, 320, 128)])
def test_gemm_nn(native, tile_mode, M, N, K):
    dy, w = _rand(M, K), _rand(K, N, scale=0.05)
    got = native.gemm_nn(dy, w)
    assert _rel(got, dy.float() @ w.float()) < 6e-3
    native.check_status()


@pytest.mark.parametrize("R,M,N", [(128, 128, 256), (512, 256, 512), (4096, 1024, 384), (1024, 6144, 1024)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_tn_accumulates(native, tile_mode, R, M, N, dtype):
    dy, x = _rand(R, M, scale=0.1), _rand(R, N, scale=0.1)
    base = torch.randn(M, N, device="cuda").to(dtype)
    out = base.clone()
    native.gemm_tn(dy, x, out=out, accumulate=True)
    want = base.float() + dy.float().t() @ x.float()
    assert _rel(out, want) < (2e-3 if dtype == torch.float32 else 8e-3)
    fresh = native.gemm_tn(dy, x, out_dtype=torch.float32)
    assert _rel(fresh, dy.float().t() @ x.float()) < 2e-3
    native.check_status()


def _segments(counts, pad=128):
    padded = [(c + pad - 1) // pad * pad for c in counts]
    offs, tiles, row = [], [], 0
    for e, p in enumerate(padded):
        tiles += [e] * (p // 128)
        row += p
        offs.append(row)
    dev = dict(device="cuda", dtype=torch.int32)
    return (torch.tensor(offs, **dev), torch.tensor(tiles, **dev), torch.tensor([len(tiles), row, 0, 0], **dev), row)


@pytest.mark.parametrize("pad", [128, 256])
@pytest.mark.parametrize("counts", [[128, 256], [100, 0, 300, 17], [0, 0, 640, 0], [384] * 4])
def test_grouped_expert_gemms(native, tile_mode, counts, pad):
    """``pad`` = 256: expert segments are whole 256-row tiles, which makes the 256-row tile kinds legal."""
    torch.manual_seed(0)
    E, D, Fd = len(counts), 256, 512
    offs, tile_expert, meta, rows = _segments(counts, pad)
    align = pad == 256
    cap = rows + 256                                  # rows past the live count must be ignored
    x = torch.zeros(cap, D, device="cuda", dtype=torch.bfloat16)
    start = 0
    for e, c in enumerate(counts):
        x[start:start + c] = _rand(c, D)
        start = int(offs[e])
    x[rows:] = float("nan")
    w1, w3, w2 = _rand(E, Fd, D, scale=0.05), _rand(E, Fd, D, scale=0.05), _rand(E, D, Fd, scale=0.05)
    h, gate, up = native.gemm_swiglu(x, w1, w3, tile_expert, meta[0:1], align256=align)
    y = native.gemm_nt(h, w2, tile_expert=tile_expert, num_m_tiles=meta[0:1], num_experts=E, align256=align)
    start = 0
    for e in range(E):
        end = int(offs[e])
        if end > start:
            xe = x[start:end].float()
            g, u = xe @ w1[e].float().t(), xe @ w3[e].float().t()
            he = torch.nn.functional.silu(g) * u
            assert _rel(gate[start:end], g) < 6e-3 and _rel(up[start:end], u) < 6e-3
            assert _rel(h[start:end], he) < 8e-3
            assert _rel(y[start:end], h[start:end].float() @ w2[e].float().t()) < 6e-3
        start = end
    # data gradients: dh = dy W2 ; dx = dg W1 + du W3 in one pass
    dy = torch.zeros(cap, D, device="cuda", dtype=torch.bfloat16)
    dy[:rows] = _rand(rows, D)
    dh = native.gemm_nn(dy, w2, tile_expert=tile_expert, num_m_tiles=meta[0:1], num_experts=E, align256=align)
    dgu = torch.zeros(cap, 2 * Fd, device="cuda", dtype=torch.bfloat16)
    dgu[:rows] = _rand(rows, 2 * Fd, scale=0.1)
    dx = native.gemm_nn(dgu, w1, w2=w3, tile_expert=tile_expert, num_m_tiles=meta[0:1], num_experts=E,
                        align256=align)
    acc = torch.randn(E, Fd, D, device="cuda")
    dw1 = acc.clone()
    native.gemm_tn(dgu[:, :Fd], x, out=dw1, accumulate=True, expert_offsets=offs, num_experts=E)
    dw_new = native.gemm_tn(dy, h, out_dtype=torch.float32, expert_offsets=offs, num_experts=E)
    start = 0
    for e in range(E):
        end = int(offs[e])
        if end > start:
            assert _rel(dh[start:end], dy[start:end].float() @ w2[e].float()) < 6e-3
            want = dgu[start:end, :Fd].float() @ w1[e].float() + dgu[start:end, Fd:].float() @ w3[e].float()
            assert _rel(dx[start:end], want) < 6e-3
            assert _rel(dw1[e], acc[e] + dgu[start:end, :Fd].float().t() @ x[start:end].float()) < 3e-3
            assert _rel(dw_new[e], dy[start:end].float().t() @ h[start:end].float()) < 3e-3
        else:
            assert torch.equal(dw1[e], acc[e]) and float(dw_new[e].abs().max()) == 0.0
        start = end
    native.check_status()


def test_rmsnorm_forward_backward(native):
    from b200moe import ops
    from b200moe.ops import functional as Fn
    for D in (128, 4096):
        x = _rand(300, D).requires_grad_(True)
        d = _rand(300, D).requires_grad_(True)
        w = (torch.rand(D, device="cuda") + 0.5).requires_grad_(True)
        y = ops.rmsnorm(x, w)
        xr, wr = x.detach().float().requires_grad_(True), w.detach().clone().requires_grad_(True)
        yr = Fn.rmsnorm_ref(xr, wr)
        assert _rel(y, yr) < 5e-3
        dy = _rand(300, D)
        y.backward(dy)
        yr.backward(dy.float())
        assert _rel(x.grad, xr.grad) < 8e-3 and _rel(w.grad, wr.grad) < 8e-3
        x.grad = w.grad = None
        s, y2 = ops.add_rmsnorm(x, d, w)
        (s.float().sum() * 0.5 + (y2.float() * dy.float()).sum()).backward()
        xs = (x.detach().float() + d.detach().float()).bfloat16().float().requires_grad_(True)
        wr2 = w.detach().clone().requires_grad_(True)
        (xs.sum() * 0.5 + (Fn.rmsnorm_ref(xs, wr2) * dy.float()).sum()).backward()
        assert _rel(s, xs) < 1e-6 and _rel(x.grad, xs.grad) < 8e-3 and _rel(d.grad, xs.grad) < 8e-3
        assert _rel(w.grad, wr2.grad) < 8e-3


def test_router_linear_and_top2(native):
    from b200moe import ops
    from b200moe.ops import functional as Fn
    T, D, E = 1000, 512, 8
    x = _rand(T, D).requires_grad_(True)
    w = _rand(E, D, scale=0.05).requires_grad_(True)
    logits = ops.linear(x, w)
    assert logits.dtype == torch.float32
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    lr = xr @ wr.t()
    assert _rel(logits, lr) < 1e-3
    weights, idx = ops.router_top2(logits)
    wref, iref = Fn.router_top2_ref(lr, 2)
    assert torch.equal(idx, iref) and _rel(weights, wref) < 1e-4
    dw = torch.randn(T, 2, device="cuda")
    weights.backward(dw)
    wref.backward(dw)
    assert _rel(x.grad, xr.grad) < 1e-2 and _rel(w.grad, wr.grad) < 1e-2


def test_cross_entropy_and_lm_head(native):
    from b200moe import ops
    T, D, V = 512, 256, 32000
    h = _rand(2, T // 2, D).requires_grad_(True)
    w = _rand(V, D, scale=0.05).requires_grad_(True)
    t = torch.randint(0, V, (2, T // 2), device="cuda")
    loss = ops.lm_head_cross_entropy(h, w, t)
    hr, wr = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy((hr @ wr.t()).reshape(-1, V), t.reshape(-1))
    assert abs(float(loss) - float(ref)) < 2e-2
    (loss * 0.5).backward()
    (ref * 0.5).backward()
    assert _rel(h.grad, hr.grad) < 3e-2 and _rel(w.grad, wr.grad) < 3e-2


def test_lm_head_forms_its_gradients_in_the_forward_pass_when_the_loss_factor_is_known(native):
    """Three token chunks (one ragged); the weight gradient lands in ``main_grad`` with the announced factor."""
    from b200moe import ops
    T, D, V = 2 * 4096 + 640, 128, 4096
    h = _rand(T, D).requires_grad_(True)
    w = _rand(V, D, scale=0.05)
    w.main_grad = torch.zeros(V, D, device="cuda")
    t = torch.randint(0, V, (T,), device="cuda")
    hr, wr = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(hr @ wr.t(), t)
    (ref * 0.25).backward()
    for announced in (0.25, None):
        w.main_grad.zero_()
        h.grad = None
        loss = ops.lm_head_cross_entropy(h, w, t, grad_scale=announced)
        assert abs(float(loss) - float(ref)) < 2e-2
        (loss * 0.25).backward()
        assert _rel(h.grad, hr.grad) < 3e-2, announced
        assert _rel(w.main_grad, wr.grad) < 3e-2, announced


def test_embedding_rope_adamw(native):
    from b200moe import ops
    from b200moe.ops import functional as Fn
    from b200moe.ops.attention import rope_qk_
    from b200moe.optim import AdamW
    table = _rand(1000, 128)
    table.main_grad = torch.zeros(1000, 128, device="cuda")
    table.requires_grad_(True)
    ids = torch.randint(0, 1000, (4, 33), device="cuda")
    out = ops.embedding(ids, table)
    assert torch.equal(out, table.detach()[ids])
    dy = _rand(4, 33, 128)
    out.backward(dy)
    want = torch.zeros(1000, 128, device="cuda").index_add_(0, ids.reshape(-1), dy.reshape(-1, 128).float())
    assert _rel(table.main_grad, want) < 1e-5
    # rope
    B, S, H, hd = 2, 64, 6, 128
    cos, sin = Fn.rope_tables(10000.0, hd, 128, device="cuda")
    qkv = _rand(B, S, H, hd).requires_grad_(True)
    rotated = rope_qk_((qkv * 1.0).view(B * S, H * hd), S, H, 4, hd, cos, sin).view(B, S, H, hd)
    ref_in = qkv.detach().float().requires_grad_(True)
    ref = torch.cat((Fn.apply_rope_ref(ref_in[:, :, :4].transpose(1, 2), cos[:S], sin[:S]).transpose(1, 2),
                     ref_in[:, :, 4:]), dim=2)
    assert _rel(rotated, ref) < 5e-3
    g = _rand(B, S, H, hd)
    rotated.backward(g)
    ref.backward(g.float())
    assert _rel(qkv.grad, ref_in.grad) < 5e-3
    # adamw: bf16 parameter with fp32 gradient accumulator and bf16 moments, and plain fp32
    for p_dt, g_dt, s_dt in [(torch.bfloat16, torch.float32, torch.bfloat16), (torch.float32, torch.float32, torch.float32),
                             (torch.bfloat16, torch.bfloat16, torch.float32)]:
        p = torch.nn.Parameter(torch.randn(4097, device="cuda").to(p_dt))
        cpu = torch.nn.Parameter(p.detach().cpu().clone())
        p.main_grad = torch.randn(4097, device="cuda").to(g_dt)
        cpu.main_grad = p.main_grad.cpu().clone()
        o1, o2 = AdamW([p], lr=1e-2, state_dtype=s_dt), AdamW([cpu], lr=1e-2, state_dtype=s_dt)
        for _ in range(3):
            o1.step()
            o2.step()
        assert _rel(p.detach().cpu(), cpu.detach()) < (1e-6 if p_dt == torch.float32 else 4e-3)


@pytest.mark.parametrize("T,E", [(257, 4), (1024, 8), (64, 8)])
def test_moe_plan_gather_combine(native, T, E):
    idx = torch.stack([torch.randperm(E, device="cuda")[:2] for _ in range(T)])
    if T == 64:
        idx[:] = torch.tensor([5, 2], device="cuda")          # everything on two experts
    from b200moe.ops.moe_fused import capacity_rows
    cap = capacity_rows(T * 2, E)
    slot_row, row_slot, offs, tile_expert, meta, counts = native.moe_plan(idx, E, cap)
    flat = idx.reshape(-1)
    assert torch.equal(counts.long(), torch.bincount(flat, minlength=E))
    ends = offs.tolist()
    assert int(meta[1]) == ends[-1] and int(meta[0]) == ends[-1] // 128 and int(meta[2]) == 0
    start = 0
    for e, end in enumerate(ends):
        slots_e = torch.nonzero(flat == e).flatten()
        assert torch.equal(slot_row[slots_e].long(), torch.arange(start, start + slots_e.numel(), device="cuda"))
        assert torch.equal(row_slot[start:start + slots_e.numel()].long(), slots_e)
        assert bool((row_slot[start + slots_e.numel():end] == -1).all())
        assert bool((tile_expert[start // 128:end // 128] == e).all())
        start = end
    x = _rand(T, 256)
    xp = native.moe_gather(x, row_slot, meta, cap)
    live = int(meta[1])
    want = torch.where(row_slot[:live, None] >= 0, x[(row_slot[:live].clamp_min(0) // 2).long()], torch.zeros_like(x[:1]))
    assert torch.equal(xp[:live], want)
    w = torch.rand(T, 2, device="cuda")
    out = native.moe_combine(xp, slot_row, w, T)
    assert _rel(out, x.float() * w.sum(1, keepdim=True)) < 5e-3


@pytest.mark.parametrize("recompute", [False, True])
def test_moe_block_matches_torch_path(native, recompute):
    from b200moe import ops
    from b200moe.ops.moe import moe_ffn
    torch.manual_seed(1)
    T, D, Fd, E = 640, 256, 512, 4
    x = _rand(T, D)
    logits = torch.randn(T, E, device="cuda")
    w1, w3, w2 = _rand(E, Fd, D, scale=0.06), _rand(E, Fd, D, scale=0.06), _rand(E, D, Fd, scale=0.06)
    dout = _rand(T, D)
    results = []
    for use_native in (True, False):
        ops.set_native(use_native)
        try:
            xs = x.clone().requires_grad_(True)
            lg = logits.clone().requires_grad_(True)
            params = [p.clone().requires_grad_(True) for p in (w1, w2, w3)]
            weights, idx = ops.router_top2(lg)
            out = moe_ffn(xs, weights, idx, *params, recompute=recompute)
            out.backward(dout)
            results.append([out.detach(), xs.grad, lg.grad] + [p.grad for p in params])
        finally:
            ops.set_native(True)
    for got, want in zip(*results):
        assert _rel(got, want) < 2e-2
    native.check_status()


@pytest.mark.parametrize("keep_rows,recompute", [(None, False), (512, False), (None, True)])
def test_moe_block_with_fused_exchange_on_a_single_rank_group(native, tile_mode, keep_rows, recompute):
    """The gather+GEMM kernels, the return in the GEMM epilogue and the combine kernel with every pointer local
    (expert group of one rank), against the PyTorch statements of the block."""
    from b200moe import ops
    from b200moe.comm.ep import EPPull
    from b200moe.ops.moe import moe_ffn
    from b200moe.ops.moe_fused import moe_ffn_pull
    torch.manual_seed(3)
    T, D, Fd, E = 1000 if keep_rows is None else 1024, 256, 512, 4
    T = 1024
    x = _rand(T, D)
    logits = torch.randn(T, E, device="cuda")
    logits[:, 1] += 1.0
    w1, w3, w2 = _rand(E, Fd, D, scale=0.06), _rand(E, Fd, D, scale=0.06), _rand(E, D, Fd, scale=0.06)
    dout = _rand(T, D)
    epc = EPPull(None, native.status_word(), torch.device("cuda", torch.cuda.current_device()), T, D, Fd, E)
    if keep_rows is not None:
        epc.expected_rows = lambda key: keep_rows
    results = []
    for fused in (True, False, True):
        xs = x.clone().requires_grad_(True)
        lg = logits.clone().requires_grad_(True)
        params = [p.clone().requires_grad_(True) for p in (w1, w2, w3)]
        if fused:
            out, _, _ = moe_ffn_pull(xs, lambda staged: ops.router_top2(lg), *params, epc, recompute=recompute)
        else:
            ops.set_native(False)
            try:
                weights, idx = ops.router_top2(lg)
                out = moe_ffn(xs, weights, idx, *params)
            finally:
                ops.set_native(True)
        out.backward(dout)
        results.append([out.detach(), xs.grad, lg.grad] + [p.grad for p in params])
    for got, want, again in zip(*results):
        assert _rel(got, want) < 2e-2
        assert _rel(again, want) < 2e-2
    assert len(epc.free) == len(epc.pool) == 1
    native.check_status()


def test_tiny_model_native_vs_torch_path(native):
    from b200moe import ops
    from b200moe.models import TransformerLMPipelined
    from b200moe.ops.functional import cross_entropy
    from b200moe.optim import AdamW
    from b200moe.parallel import FSDPWrapperPipelined, pipelined_train_overlap
    losses = []
    for use_native in (True, False):
        ops.set_native(use_native)
        try:
            torch.manual_seed(3)
            model = TransformerLMPipelined(2048, 256, 512, 2, 4, 0, 1, num_expert_per_node=4, d_ff=1024).cuda()
            wrapped = FSDPWrapperPipelined(model, None, None, compute_dtype=torch.bfloat16)
            opt = AdamW(wrapped.parameters(), lr=1e-3, weight_decay=0.01)
            ids = torch.randint(0, 2048, (4, 257), device="cuda")
            run = []
            for _ in range(4):
                run.append(float(pipelined_train_overlap(wrapped, opt, ids[:, :-1], ids[:, 1:], [4, 256, 512], 2, 0,
                                                         cross_entropy, dtype=torch.bfloat16, device=ids.device)))
            losses.append(run)
        finally:
            ops.set_native(True)
    assert losses[0][-1] < losses[0][0]
    assert losses[0] == pytest.approx(losses[1], abs=5e-2)
    native.check_status()
    assert native.launch_count() > 0


@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 128, 4, 1), (2, 512, 8, 2), (1, 1024, 4, 4)])
def test_attention_forward_backward(native, B, S, Hq, Hkv):
    from b200moe.ops import functional as Fn
    torch.manual_seed(2)
    hd, total = 128, Hq + 2 * Hkv
    qkv = _rand(B, S, total, hd)
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    out, lse, _, _ = native.attention_fwd(q, k, v)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = Fn.attention_ref(qf, kf, vf, None, None, causal=True)
    assert _rel(out, ref) < 1e-2
    scores = torch.einsum("bshd,bthd->bhst", qf, kf.repeat_interleave(Hq // Hkv, 2)) / math.sqrt(hd)
    scores = scores.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device="cuda"), 1), float("-inf"))
    assert _rel(lse, torch.logsumexp(scores, -1)) < 1e-3
    dout = _rand(B, S, Hq, hd)
    dq, dk, dv = native.attention_bwd(dout, q, k, v, out, lse)
    ref.backward(dout.float())
    assert _rel(dq, qf.grad) < 2e-2 and _rel(dk, kf.grad) < 2e-2 and _rel(dv, vf.grad) < 2e-2
    native.check_status()


def test_attention_at_the_training_shape_against_fp32_one_kv_group_at_a_time(native):
    """Sequence 8192 with 32 query and 8 key/value heads: the fp32 statement is evaluated per key/value head (four
    query heads, a 4 x 8192 x 8192 score block) so that it fits beside the kernels' tensors."""
    torch.manual_seed(4)
    B, S, Hq, Hkv, hd = 1, 8192, 32, 8, 128
    ratio, total = Hq // Hkv, Hq + 2 * Hkv
    qkv = _rand(B, S, total, hd)
    q, k, v = qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    dout = _rand(B, S, Hq, hd)
    out, lse, _, _ = native.attention_fwd(q, k, v)
    dq, dk, dv = native.attention_bwd(dout, q, k, v, out, lse)
    native.check_status()
    mask = torch.triu(torch.ones(S, S, dtype=torch.bool, device="cuda"), 1)
    for g in range(Hkv):
        heads = slice(g * ratio, (g + 1) * ratio)
        qf = q[0, :, heads].detach().float().transpose(0, 1).requires_grad_(True)       # [4, S, hd]
        kf = k[0, :, g].detach().float().requires_grad_(True)                           # [S, hd]
        vf = v[0, :, g].detach().float().requires_grad_(True)
        scores = (qf @ kf.t()) / math.sqrt(hd)
        scores = scores.masked_fill(mask, float("-inf"))
        ref = torch.softmax(scores, -1) @ vf                                             # [4, S, hd]
        ref.backward(dout[0, :, heads].float().transpose(0, 1))
        assert _rel(out[0, :, heads].transpose(0, 1), ref) < 1e-2, g
        assert _rel(lse[0, heads], torch.logsumexp(scores.detach(), -1)) < 1e-3, g
        assert _rel(dq[0, :, heads].transpose(0, 1), qf.grad) < 2e-2, g
        assert _rel(dk[0, :, g], kf.grad) < 2e-2 and _rel(dv[0, :, g], vf.grad) < 2e-2, g
        del scores, ref, qf, kf, vf


@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 256, 2, 2), (2, 512, 4, 1)])
def test_attention_non_causal(native, B, S, Hq, Hkv):
    """Every query sees every key (the form of the reference's own flash kernel): forward and backward."""
    from b200moe.ops import functional as Fn
    from b200moe.ops.attention import attention
    torch.manual_seed(4)
    hd = 128
    q, k, v = (_rand(B, S, h, hd).requires_grad_(True) for h in (Hq, Hkv, Hkv))
    out = attention(q, k, v, causal=False)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = Fn.attention_ref(qf, kf, vf, None, None, causal=False)
    assert _rel(out, ref) < 1e-2
    dout = _rand(B, S, Hq, hd)
    out.backward(dout)
    ref.backward(dout.float())
    assert _rel(q.grad, qf.grad) < 2e-2 and _rel(k.grad, kf.grad) < 2e-2 and _rel(v.grad, vf.grad) < 2e-2
    native.check_status()


def test_flash_attention_forward_entry(native):
    """``[B, H, S, 128]`` forward-only entry point, fp16 in and out, against an fp32 softmax(QK^T)V."""
    from b200moe.ops.attention import flash_attention_forward
    torch.manual_seed(5)
    B, H, S, hd = 2, 3, 384, 128
    q, k, v = (torch.randn(B, H, S, hd, device="cuda").half() for _ in range(3))
    before = native.launch_count()
    out = flash_attention_forward(q, k, v)
    assert native.launch_count() > before and out.dtype == torch.float16 and out.shape == (B, H, S, hd)
    ref = torch.softmax(q.float() @ k.float().transpose(-1, -2) / math.sqrt(hd), -1) @ v.float()
    assert _rel(out, ref) < 2e-2
    causal = flash_attention_forward(q, k, v, causal=True)
    mask = torch.triu(torch.ones(S, S, dtype=torch.bool, device="cuda"), 1)
    ref = torch.softmax((q.float() @ k.float().transpose(-1, -2) / math.sqrt(hd)).masked_fill(mask, float("-inf")), -1) @ v.float()
    assert _rel(causal, ref) < 2e-2
    native.check_status()


@pytest.mark.parametrize("causal", [False, True])
def test_reference_named_attention_functions_run_the_flash_kernels(native, causal):
    """``FlashAttentionTritonFunc.apply(q, k, v, is_causal)`` and the ``attention_forward[grid](...)`` launch of the
    reference's module, on bf16 ``[B, S, 128]`` tensors: forward and backward against an fp32 formula."""
    from implementation.kernels.attention import FlashAttentionTritonFunc, attention_forward
    torch.manual_seed(9)
    B, S, hd = 3, 256, 128
    q, k, v = (_rand(B, S, hd).requires_grad_(True) for _ in range(3))
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    scores = qf @ kf.transpose(-1, -2) / math.sqrt(hd)
    if causal:
        scores = scores.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device="cuda"), 1), float("-inf"))
    ref = torch.softmax(scores, -1) @ vf
    before = native.launch_count()
    out = FlashAttentionTritonFunc.apply(q, k, v, causal)
    assert native.launch_count() > before and out.shape == (B, S, hd) and out.dtype == torch.bfloat16
    assert _rel(out, ref) < 2e-2
    dout = _rand(B, S, hd)
    before = native.launch_count()
    out.backward(dout)
    assert native.launch_count() > before
    ref.backward(dout.float())
    assert _rel(q.grad, qf.grad) < 3e-2 and _rel(k.grad, kf.grad) < 3e-2 and _rel(v.grad, vf.grad) < 3e-2
    filled, lse = torch.empty(B, S, hd, device="cuda", dtype=torch.bfloat16), torch.empty(B, S, device="cuda")
    attention_forward[(S // 16, B)](q.detach(), k.detach(), v.detach(), filled, lse, *([0] * 14), S, S,
                                    1 / math.sqrt(hd), hd, 16, 16, causal)
    assert _rel(filled, ref) < 2e-2 and _rel(lse, torch.logsumexp(scores.detach(), -1)) < 1e-3
    native.check_status()


def test_fused_qkv_attention_with_rope(native):
    from b200moe.ops import functional as Fn
    from b200moe.ops.attention import fused_qkv_attention
    B, S, Hq, Hkv, hd = 2, 256, 8, 2, 128
    total = Hq + 2 * Hkv
    cos, sin = Fn.rope_tables(10000.0, hd, S, device="cuda")
    base = _rand(B * S, total * hd).requires_grad_(True)
    out = fused_qkv_attention(base * 1.0, B, S, Hq, Hkv, hd, cos, sin)
    ref_in = base.detach().float().requires_grad_(True)
    view = ref_in.view(B, S, total, hd)
    ref = Fn.attention_ref(view[:, :, :Hq], view[:, :, Hq:Hq + Hkv], view[:, :, Hq + Hkv:], cos, sin, causal=True)
    assert _rel(out, ref) < 1e-2
    g = _rand(B, S, Hq, hd)
    out.backward(g)
    ref.backward(g.float())
    assert _rel(base.grad, ref_in.grad) < 2e-2
    native.check_status()


@pytest.mark.parametrize("tile", [0, 3], ids=["tiles_auto", "tiles_cta_pair"])
def test_projection_with_rope_in_the_gemm_epilogue_then_attention(native, tile):
    """q/k/v projection whose epilogue rotates q and k, attention on the rotated tensors, and a backward pass whose
    attention kernels hand back gradients of the unrotated projection: against the fp32 statements end to end."""
    from b200moe import ops
    from b200moe.ops import functional as Fn
    from b200moe.ops.attention import fused_qkv_attention
    native.set_gemm_tile_mode(tile)
    try:
        B, S, Hq, Hkv, hd, D = 2, 256, 8, 2, 128, 512
        total = Hq + 2 * Hkv
        cos, sin = Fn.rope_tables(10000.0, hd, 2 * S, device="cuda")       # a table longer than the sequence
        x = _rand(B * S, D).requires_grad_(True)
        w = _rand(total * hd, D, scale=0.05).requires_grad_(True)
        qkv = ops.linear_rope(x, w, cos, sin, (Hq + Hkv) * hd, S)
        xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
        plain = (xr @ wr.t()).view(B, S, total, hd)
        rotated = torch.cat([Fn.apply_rope_ref(plain[:, :, :Hq + Hkv].transpose(1, 2), cos[:S], sin[:S]).transpose(1, 2),
                             plain[:, :, Hq + Hkv:]], dim=2)
        assert _rel(qkv.view(B, S, total, hd), rotated) < 1e-2
        out = fused_qkv_attention(qkv, B, S, Hq, Hkv, hd, cos, sin, pre_rotated=True)
        ref = Fn.attention_ref(plain[:, :, :Hq], plain[:, :, Hq:Hq + Hkv], plain[:, :, Hq + Hkv:], cos[:S], sin[:S],
                               causal=True)
        assert _rel(out, ref) < 1.5e-2
        g = _rand(B, S, Hq, hd)
        out.backward(g)
        ref.backward(g.float())
        assert _rel(x.grad, xr.grad) < 3e-2 and _rel(w.grad, wr.grad) < 3e-2
        native.check_status()
    finally:
        native.set_gemm_tile_mode(0)


@pytest.mark.parametrize("M,K,world,segments", [(1000, 512, 2, [1536]), (300, 256, 2, [1984]),
                                                (2048, 1024, 4, [2048]), (700, 512, 2, [1024, 256, 256]),
                                                (513, 256, 4, [1024, 512, 512, 96 * 4])])
def test_allgather_gemm_emulated_ranks(native, M, K, world, segments):
    """The all-gather + GEMM kernel of every rank of a group, run one after the other on this GPU: each "rank" has
    its own full-size copy of W in which only its own rows are valid (the rest is NaN), the "peers" are the other
    copies, and the peers' ready signals are written by the host so that no launch waits for another one.
    ``segments``: stacked parts of W sharded one by one (a fused q/k/v projection has three)."""
    import ctypes
    torch.manual_seed(11)
    N = sum(segments)
    owner = torch.empty(N, dtype=torch.long)
    begin = 0
    for rows in segments:
        owner[begin:begin + rows] = torch.arange(rows) // (rows // world)
        begin += rows
    owner = owner.cuda()
    x = _rand(M, K)

    def fresh():
        full = _rand(N, K)
        parts = []
        for r in range(world):
            c = torch.full((N, K), float("nan"), dtype=torch.bfloat16, device="cuda")
            c[owner == r] = full[owner == r]
            parts.append(c)
        return full, parts

    W, filled = fresh()
    copies = [c.clone() for c in filled]
    table = ctypes.c_ulonglong * 8
    w_ptrs = table(*([c.data_ptr() for c in copies] + [0] * (8 - world)))
    pads = [torch.zeros(32 * 8, dtype=torch.int32, device="cuda") for _ in range(world)]
    sig_ptrs = table(*([s.data_ptr() for s in pads] + [0] * (8 - world)))
    slot = 14
    flags = [torch.zeros((N + 255) // 256, dtype=torch.int32, device="cuda") for _ in range(world)]
    for epoch in (1, 2):
        if epoch == 2:      # a second step: rows change, every copy is stale again outside its own rows
            W, filled = fresh()
        ref = x.float() @ W.float().t()
        for r in range(world):
            # what the ranks hold when rank r runs: their own rows only (nobody else has gathered yet)
            for q in range(world):
                copies[q].copy_(filled[q])
            pads[r].view(32, 8)[slot].fill_(epoch)      # "every peer has announced its rows"
            y = native.ag_gemm_nt(x, w_ptrs, N, segments, world, r, sig_ptrs, slot, epoch, flags[r], epoch)
            assert y is not None, "cooperative launch unavailable"
            native.check_status()
            assert _rel(y, ref) < 1e-2
            assert torch.equal(copies[r], W), "gathered weight differs from the sharded original"


def test_device_timestamp_and_step_timer(native):
    """``globaltimer`` stamps bracket the same span as CUDA events; NVTX wrapping of launches does not change results."""
    from b200moe.utils.profiling import DeviceStepTimer
    a, b = _rand(4096, 4096), _rand(4096, 4096)
    native.gemm_nt(a, b)
    torch.cuda.synchronize()
    by_event, by_clock = DeviceStepTimer("cuda"), DeviceStepTimer("cuda", clock="globaltimer")
    by_event.start()
    by_clock.start()
    for _ in range(20):
        native.gemm_nt(a, b)
    t_clock = by_clock.stop_ms()
    t_event = by_event.stop_ms()
    assert t_clock > 0 and abs(t_clock - t_event) < 0.25 * t_event + 0.05, (t_clock, t_event)
    native.set_nvtx(True)
    try:
        with_ranges = native.gemm_nt(a, b)
    finally:
        native.set_nvtx(False)
    assert torch.equal(with_ranges, native.gemm_nt(a, b))
    native.check_status()

