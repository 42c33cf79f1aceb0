"""Launch one kernel a few times on a small case, for profiler captures.

``python benchmarks/profile_case.py --case gemm_nt`` allocates only what that
case needs (operands larger than L2, well under a few GB), runs two warm-up
launches and three measured ones and prints the CUDA-event time.  Cases:
gemm_nt, gemm_nn, gemm_tn, gemm_pair (gemm_nt on CTA pairs), ag_gemm (the all-gather + GEMM kernel as rank 0 of
two emulated ranks: the "peer" is a second buffer on this GPU and its ready signal is written by the host, so no
launch waits for another), swiglu, moe_down, wgrad, rmsnorm, rmsnorm_bwd, cross_entropy, adamw, swiglu_bwd,
attention_fwd, attention_bwd, sdpa, and the communication kernels with every peer pointer on this GPU: fsdp_step and
allreduce (rank 0 of two emulated ranks, the peer's flags preset by the host), ep_gateup (gather + gate/up GEMM +
SwiGLU over a one-rank expert group), ep_down (down projection with the return in its epilogue), ep_dh (gather of
the output gradient + dh GEMM) and ep_swiglu_bwd; gemm_rope (q/k/v projection with RoPE in its epilogue), router
(skinny GEMM + softmax/top-2), embedding.
"""
import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from b200moe.ops import native  # noqa: E402


def rnd(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def build(case):
    T, D, Fd, E = 16384, 4096, 14336, 2
    if case == "gemm_nt":
        x, w = rnd(T, D), rnd(6144, D, scale=0.02)
        return lambda: native.gemm_nt(x, w), 2 * T * 6144 * D
    if case == "gemm_pair":
        x, w = rnd(T, D), rnd(6144, D, scale=0.02)
        native.set_gemm_tile_mode(3)
        return lambda: native.gemm_nt(x, w), 2 * T * 6144 * D
    if case == "ag_gemm":
        import ctypes
        N, world = 6144, 2
        x = rnd(T, D)
        copies = [rnd(N, D, scale=0.02) for _ in range(world)]
        pads = [torch.zeros(32 * 8, dtype=torch.int32, device="cuda") for _ in range(world)]
        pads[0].fill_(1 << 20)                      # every peer "announced" its rows for all launches to come
        table = ctypes.c_ulonglong * 8
        w_ptrs = table(*([c.data_ptr() for c in copies] + [0] * 6))
        sig_ptrs = table(*([s.data_ptr() for s in pads] + [0] * 6))
        flags = torch.zeros((N + 255) // 256, dtype=torch.int32, device="cuda")
        state = {"epoch": 0}

        def launch():
            state["epoch"] += 1
            return native.ag_gemm_nt(x, w_ptrs, N, [N], world, 0, sig_ptrs, 14, state["epoch"], flags, state["epoch"])
        return launch, 2 * T * N * D
    if case == "gemm_rope":
        from b200moe.ops import functional as Fn
        x, w = rnd(T, D), rnd(6144, D, scale=0.02)
        cos, sin = Fn.rope_tables(10000.0, 128, 8192, device="cuda")
        return lambda: native.gemm_nt_rope(x, w, cos, sin, 5120, 8192), 2 * T * 6144 * D
    if case == "router":
        x, w = rnd(4 * T, D), rnd(8, D, scale=0.02)

        def route():
            return native.router_top2_fwd(native.gemm_nt(x, w))
        return route, 0
    if case == "embedding":
        ids = torch.randint(0, 32000, (4 * T,), device="cuda")
        table = rnd(32000, D)
        return lambda: native.embedding_fwd(ids, table), 0
    if case == "gemm_nn":
        dy, w = rnd(T, 6144), rnd(6144, D, scale=0.02)
        return lambda: native.gemm_nn(dy, w), 2 * T * 6144 * D
    if case == "gemm_tn":
        dy, x, acc = rnd(T, 6144), rnd(T, D), torch.zeros(6144, D, device="cuda")
        return lambda: native.gemm_tn(dy, x, out=acc, accumulate=True), 2 * T * 6144 * D
    R = 8192
    offs = torch.arange(1, E + 1, device="cuda", dtype=torch.int32) * (R // E)
    tile_expert = torch.arange(R // 128, device="cuda", dtype=torch.int32) // (R // E // 128)
    tiles = torch.tensor([R // 128], device="cuda", dtype=torch.int32)
    if case == "swiglu":
        xp, w1, w3 = rnd(R, D), rnd(E, Fd, D, scale=0.02), rnd(E, Fd, D, scale=0.02)
        return lambda: native.gemm_swiglu(xp, w1, w3, tile_expert, tiles), 2 * R * 2 * Fd * D
    if case == "moe_down":
        h, w2 = rnd(R, Fd, scale=0.1), rnd(E, D, Fd, scale=0.02)
        return (lambda: native.gemm_nt(h, w2, tile_expert=tile_expert, num_m_tiles=tiles, num_experts=E),
                2 * R * D * Fd)
    if case == "wgrad":
        dy, h = rnd(R, D), rnd(R, Fd, scale=0.1)
        acc = torch.zeros(E, D, Fd, device="cuda")
        return (lambda: native.gemm_tn(dy, h, out=acc, accumulate=True, expert_offsets=offs, num_experts=E),
                2 * R * D * Fd)
    if case == "rmsnorm":
        x, w = rnd(T, D), torch.ones(D, device="cuda")
        return lambda: native.rmsnorm_fwd(x, w, 1e-5), 0
    if case == "rmsnorm_bwd":
        x, dy, w = rnd(2 * T, D), rnd(2 * T, D), torch.ones(D, device="cuda")
        _, rstd = native.rmsnorm_fwd(x, w, 1e-5)
        return lambda: native.rmsnorm_bwd(dy, x, w, rstd), 0
    if case == "cross_entropy":
        logits = rnd(4096, 32000)
        targets = torch.randint(0, 32000, (4096,), device="cuda")
        loss = torch.zeros((), device="cuda")
        return lambda: native.cross_entropy_scaled_(logits, targets, loss, 1.0 / 4096, 1.0 / 4096), 0
    if case == "adamw":
        n = 1 << 27
        p_, g_, m_, v_ = (torch.zeros(n, device="cuda", dtype=torch.bfloat16) for _ in range(4))
        return lambda: native.adamw_(p_, g_, m_, v_, 1e-4, 0.9, 0.999, 1e-8, 0.01, 1e-4), 0
    if case == "swiglu_bwd":
        dh, gate, up = rnd(R, Fd, scale=0.1), rnd(R, Fd), rnd(R, Fd)
        return lambda: native.swiglu_bwd(dh, gate, up), 0
    if case in ("fsdp_step", "allreduce"):
        import ctypes
        table = ctypes.c_ulonglong * 8
        pads = [torch.zeros(32 * 8, dtype=torch.int32, device="cuda") for _ in range(2)]
        pads[0].fill_(1 << 20)                      # the emulated peer has "arrived" at every barrier to come
        sig = table(*([s_.data_ptr() for s_ in pads] + [0] * 6))
        counter = torch.zeros(8, dtype=torch.int32, device="cuda")
        status = native.status_word()
        state = {"seq": 0}
        if case == "allreduce":
            n = 1 << 26
            bufs = [torch.randn(n, device="cuda") for _ in range(2)]
            ptrs = table(*([b.data_ptr() for b in bufs] + [0] * 6))

            def launch():
                state["seq"] += 1
                native._call("b2_comm_allreduce", ptrs, sig, ctypes.c_void_p(0), ctypes.c_void_p(0), ctypes.c_int(1),
                             ctypes.c_int(0), ctypes.c_int(2), ctypes.c_int(state["seq"]), ctypes.c_int(12),
                             ctypes.c_longlong(n), ctypes.c_float(0.5), ctypes.c_void_p(counter.data_ptr()),
                             ctypes.c_void_p(status.data_ptr()),
                             ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            return launch, 0
        full = 1 << 27                              # parameters of the emulated stage; this rank owns half
        grads = [torch.randn(full, device="cuda") for _ in range(2)]
        weights = [torch.zeros(full, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
        master, m_, v_, sg = (torch.zeros(full // 2, device="cuda") for _ in range(4))
        entries = torch.tensor([[0, 0, full // 2, 0]], dtype=torch.int64, device="cuda")
        gp = table(*([g_.data_ptr() for g_ in grads] + [0] * 6))
        wp = table(*([w_.data_ptr() for w_ in weights] + [0] * 6))

        def launch():
            state["seq"] += 1
            c = ctypes
            native._call("b2_fsdp_step", gp, wp, sig, c.c_void_p(entries.data_ptr()), c.c_int(1), c.c_int(0),
                         c.c_int(2), c.c_int(state["seq"]), c.c_int(8), c.c_void_p(master.data_ptr()),
                         c.c_void_p(m_.data_ptr()), c.c_void_p(v_.data_ptr()), c.c_void_p(sg.data_ptr()),
                         c.c_float(1e-4), c.c_float(0.9), c.c_float(0.999), c.c_float(1e-8), c.c_float(0.01),
                         c.c_float(1e-4), c.c_int(1), c.c_int(0), c.c_void_p(counter.data_ptr()),
                         c.c_void_p(status.data_ptr()), c.c_void_p(torch.cuda.current_stream().cuda_stream))
        return launch, 0
    if case in ("ep_gateup", "ep_down", "ep_dh", "ep_swiglu_bwd"):
        from b200moe import ops
        from b200moe.comm import ep as EP
        tokens, experts = 4096, 2
        epc = EP.EPPull(None, native.status_word(), torch.device("cuda", torch.cuda.current_device()), tokens, D, Fd,
                        experts)
        x = rnd(tokens, D)
        w1, w3, w2 = rnd(experts, Fd, D, scale=0.02), rnd(experts, Fd, D, scale=0.02), rnd(experts, D, Fd, scale=0.02)
        weights, idx = ops.router_top2(torch.randn(tokens, experts, device="cuda"))
        weights = weights.float().contiguous()
        slot = epc.acquire()
        epc.slot_tensor(slot).copy_(x)
        i32 = dict(dtype=torch.int32, device="cuda")
        row_src, row_tag = torch.empty(epc.cap, **i32), torch.empty(epc.cap, **i32)
        row_w = torch.empty(epc.cap, dtype=torch.float32, device="cuda")
        x_ws, h = epc.ws("x", D), epc.ws("h", Fd)
        state = {}

        def gateup():
            offs, seg_end, tile_expert, meta, seq = epc.plan(idx, weights, "profile")
            state.update(tile_expert=tile_expert, meta=meta, seg_end=seg_end)
            epc.gather_gemm(0, x_ws, w1, w3, 2 * Fd, D, tile_expert, meta, seg_end, 0, epc.pool[slot].table(), 1,
                            epc.land_src.tensor, epc.land_tag.tensor, epc.land_w.tensor, (row_src, row_tag, row_w),
                            EP.SIG_META, seq, 1, h, None, None, None, None, 0)
        if case == "ep_gateup":
            return gateup, 2 * 2 * tokens * 2 * Fd * D
        gateup()
        if case == "ep_dh":
            epc.dout.tensor.view(tokens, D).copy_(rnd(tokens, D))
            dy_ws = epc.ws("dy", D)

            def dh():
                seq = epc.g.next_seq(EP.SIG_BDATA)
                epc.gather_gemm(1, dy_ws, w2, None, Fd, D, state["tile_expert"], state["meta"], state["seg_end"], 0,
                                epc.dout.table(), 1, row_src, row_tag, None, None, EP.SIG_BDATA, seq, 2, h, None,
                                None, None, None, 0)
            return dh, 2 * 2 * tokens * D * Fd
        if case == "ep_swiglu_bwd":
            gate, up, dgu = rnd(epc.cap, Fd), rnd(epc.cap, Fd), epc.ws("dgu", 2 * Fd)
            return (lambda: native.ep_swiglu_bwd(h, gate, up, None, None, epc.cap, dgu, state["meta"], row_tag,
                                                 row_src, row_w, epc.dw_ret.table(), 1)), 0

        def down():
            seq = epc.g.next_seq(EP.SIG_RET_F)
            native.gemm_nt_push(h, w2, state["tile_expert"], state["meta"][0:1], experts, epc.ret_f.table(), row_tag,
                                row_src, row_w, epc.g.sig.table(), EP.SIG_RET_F, seq, 0, 1, epc.tickets[4:])
        return down, 2 * 2 * tokens * D * Fd
    B, S, Hq, Hkv, hd = 2, 8192, 32, 8, 128
    q, k, v = rnd(B, S, Hq, hd), rnd(B, S, Hkv, hd), rnd(B, S, Hkv, hd)
    flops = 4 * B * Hq * S * S * hd // 2
    if case == "sdpa":
        import torch.nn.functional as F
        qh, kh, vh = (t.transpose(1, 2) for t in (q, k, v))
        return lambda: F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, enable_gqa=True), flops
    if case == "sdpa_bwd":
        import torch.nn.functional as F
        qh, kh, vh = (t.transpose(1, 2).detach().requires_grad_(True) for t in (q, k, v))
        out = F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, enable_gqa=True)
        g = torch.randn_like(out)
        return lambda: torch.autograd.grad(out, (qh, kh, vh), g, retain_graph=True), int(flops * 2.5)
    if case == "attention_fwd":
        return lambda: native.attention_fwd(q, k, v, None, None), flops
    if case == "attention_bwd":
        out, lse, qr, kr = native.attention_fwd(q, k, v, None, None)
        g = rnd(B, S, Hq, hd)
        return lambda: native.attention_bwd(g, qr, kr, v, out, lse, None, None), int(flops * 2.5)
    raise SystemExit(f"unknown case {case}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True)
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    native.require()
    fn, flops = build(args.case)
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(args.iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    ms = begin.elapsed_time(end) / args.iters
    print(f"{args.case}: {ms:.4f} ms" + (f", {flops / ms / 1e9:.1f} TFLOP/s" if flops else ""))


if __name__ == "__main__":
    main()
