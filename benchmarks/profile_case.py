"""Launch one kernel a few times on a small case, for profiler captures.

``python benchmarks/profile_case.py --case gemm_nt`` allocates only what that
case needs (operands larger than L2, well under a few GB), runs two warm-up
launches and three measured ones and prints the CUDA-event time.  Cases:
gemm_nt, gemm_nn, gemm_tn, gemm_pair (gemm_nt on CTA pairs), ag_gemm (the all-gather + GEMM kernel as rank 0 of
two emulated ranks: the "peer" is a second buffer on this GPU and its ready signal is written by the host, so no
launch waits for another), swiglu, moe_down, wgrad, rmsnorm, attention_fwd, attention_bwd, sdpa.
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
