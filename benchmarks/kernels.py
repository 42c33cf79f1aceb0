"""Kernel microbenchmarks on the shapes of the headline configuration.

``python benchmarks/kernels.py [--filter gemm] [--iters 10]`` times each kernel
with CUDA events after warm-up, rotating among input copies larger than L2 so
operands come from HBM, and prints achieved TFLOP/s or GB/s next to the
measured peaks in ``MEASURED_PEAKS.json`` when that file exists.
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OUT_DIR = os.environ.get("B200MOE_BENCH_OUT", os.getcwd())
sys.path.insert(0, ROOT)

from b200moe.ops import native  # noqa: E402


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p["bf16_tflops"], p["hbm_gbs"], "of measured"
    return 1590.0, 6650.0, "of fallback"


def timeit(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / iters


def rnd(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--filter", default="")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--compare", action="store_true", help="also time the PyTorch library op")
    ap.add_argument("--experts", type=int, default=8, help="local experts of the grouped cases")
    ap.add_argument("--ab-tiles", action="store_true",
                    help="time every GEMM case with 128x256, single-CTA 256x256 and CTA-pair tiles, back to back")
    ap.add_argument("--tile-mode", type=int, default=0, help="GEMM CTA tile: 0 auto (single-CTA kinds), 1 128x256, 2 256x256 on one CTA, 3 CTA pairs, 4 auto with pairs")
    args = ap.parse_args()
    native.require()
    native.set_gemm_tile_mode(args.tile_mode)
    tf_peak, bw_peak, tag = peaks()
    T, D, Fd, E = args.tokens, 4096, 14336, args.experts
    rows = []

    def gemm_case(name, flops, fn, ref=None):
        if args.filter and args.filter not in name:
            return
        ms = timeit(fn, args.iters)
        line = {"kernel": name, "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1),
                "frac": round(flops / ms / 1e9 / tf_peak, 3), "of": tag}
        if args.ab_tiles:
            # the clocks drift with the power cap over a long run, so the three tile kinds are timed right after
            # one another (twice, interleaved) and only their ratios are meaningful
            for label, mode in (("tflops_128x256", 1), ("tflops_256x256_one_cta", 2), ("tflops_cta_pair", 3)) * 2:
                native.set_gemm_tile_mode(mode)
                t = timeit(fn, args.iters)
                line[label] = max(line.get(label, 0.0), round(flops / t / 1e9, 1))
            native.set_gemm_tile_mode(args.tile_mode)
        if ref is not None and args.compare:
            rms = timeit(ref, args.iters)
            line["library_ms"] = round(rms, 4)
        rows.append(line)
        print(json.dumps(line), flush=True)

    x = rnd(T, D)
    wqkv, wo = rnd(6144, D, scale=0.02), rnd(D, D, scale=0.02)
    gemm_case("gemm_nt qkv 16384x6144x4096", 2 * T * 6144 * D, lambda: native.gemm_nt(x, wqkv), lambda: x @ wqkv.t())
    from b200moe.ops import functional as Fn
    cos, sin = Fn.rope_tables(10000.0, 128, 8192, device="cuda")
    gemm_case("gemm_nt qkv + RoPE in the epilogue 16384x6144x4096", 2 * T * 6144 * D,
              lambda: native.gemm_nt_rope(x, wqkv, cos, sin, 5120, 8192))
    gemm_case("gemm_nt out 16384x4096x4096", 2 * T * D * D, lambda: native.gemm_nt(x, wo), lambda: x @ wo.t())
    hk, wk = rnd(T, Fd, scale=0.1), rnd(D, Fd, scale=0.02)
    gemm_case("gemm_nt K=14336 16384x4096x14336", 2 * T * D * Fd, lambda: native.gemm_nt(hk, wk))
    del hk, wk
    dy = rnd(T, 6144)
    gemm_case("gemm_nn dx 16384x4096x6144", 2 * T * 6144 * D, lambda: native.gemm_nn(dy, wqkv), lambda: dy @ wqkv)
    acc = torch.zeros(6144, D, device="cuda")
    gemm_case("gemm_tn dw 6144x4096x16384 (+= fp32)", 2 * T * 6144 * D,
              lambda: native.gemm_tn(dy, x, out=acc, accumulate=True), lambda: acc.addmm_(dy.t().float(), x.float()))
    # grouped expert GEMMs: 2T rows spread evenly over E experts
    R = 2 * T
    per = R // E
    offs = torch.arange(1, E + 1, device="cuda", dtype=torch.int32) * per
    tile_expert = torch.arange(R // 128, device="cuda", dtype=torch.int32) // (per // 128)
    tiles = torch.tensor([R // 128], device="cuda", dtype=torch.int32)
    xp = rnd(R, D)
    w1, w3, w2 = rnd(E, Fd, D, scale=0.02), rnd(E, Fd, D, scale=0.02), rnd(E, D, Fd, scale=0.02)
    gemm_case("moe gate/up + swiglu 32768x(2x14336)x4096", 2 * R * 2 * Fd * D,
              lambda: native.gemm_swiglu(xp, w1, w3, tile_expert, tiles, save_gate_up=True, align256=True))
    gemm_case("moe gate/up + swiglu (h only)", 2 * R * 2 * Fd * D,
              lambda: native.gemm_swiglu(xp, w1, w3, tile_expert, tiles, save_gate_up=False, align256=True))
    h = rnd(R, Fd, scale=0.1)
    gemm_case("moe down 32768x4096x14336", 2 * R * D * Fd,
              lambda: native.gemm_nt(h, w2, tile_expert=tile_expert, num_m_tiles=tiles, num_experts=E, align256=True))
    dyp = rnd(R, D)
    gemm_case("moe dh = dy W2 32768x14336x4096", 2 * R * D * Fd,
              lambda: native.gemm_nn(dyp, w2, tile_expert=tile_expert, num_m_tiles=tiles, num_experts=E, align256=True))
    dgu = rnd(R, 2 * Fd, scale=0.1)
    gemm_case("moe dx = dg W1 + du W3 32768x4096x28672", 2 * R * D * 2 * Fd,
              lambda: native.gemm_nn(dgu, w1, w2=w3, tile_expert=tile_expert, num_m_tiles=tiles, num_experts=E,
                                     align256=True))
    g32 = torch.zeros(E, D, Fd, device="cuda", dtype=torch.bfloat16)
    gemm_case("moe dW2 += dy^T h (bf16 acc)", 2 * R * D * Fd,
              lambda: native.gemm_tn(dyp, h, out=g32, accumulate=True, expert_offsets=offs, num_experts=E))
    g1 = torch.zeros(E, Fd, D, device="cuda", dtype=torch.bfloat16)
    gemm_case("moe dW1 += dg^T x (bf16 acc)", 2 * R * D * Fd,
              lambda: native.gemm_tn(dgu[:, :Fd], xp, out=g1, accumulate=True, expert_offsets=offs, num_experts=E))
    native.check_status()

    def bw_case(name, nbytes, fn):
        if args.filter and args.filter not in name:
            return
        ms = timeit(fn, args.iters)
        line = {"kernel": name, "ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1),
                "frac": round(nbytes / ms / 1e6 / bw_peak, 3), "of": tag}
        rows.append(line)
        print(json.dumps(line), flush=True)

    wn = torch.ones(D, device="cuda")
    bw_case("rmsnorm_fwd 16384x4096", 2 * T * D * 2, lambda: native.rmsnorm_fwd(x, wn, 1e-5))
    bw_case("add_rmsnorm_fwd 16384x4096", 4 * T * D * 2, lambda: native.add_rmsnorm_fwd(x, x, wn, 1e-5))
    _, rstd = native.rmsnorm_fwd(x, wn, 1e-5)
    bw_case("rmsnorm_bwd 16384x4096", 3 * T * D * 2, lambda: native.rmsnorm_bwd(x, x, wn, rstd))
    gate, up = rnd(R, Fd), rnd(R, Fd)
    bw_case("swiglu_bwd 32768x14336", 6 * R * Fd * 2, lambda: native.swiglu_bwd(h, gate, up))
    logits = rnd(T, 32000)
    tgt = torch.randint(0, 32000, (T,), device="cuda")
    ce_loss = torch.zeros((), device="cuda")
    bw_case("cross_entropy fwd+bwd 16384x32000 (row in registers)", 2 * T * 32000 * 2,
            lambda: native.cross_entropy_scaled_(logits, tgt, ce_loss, 1.0 / T, 1.0 / T))
    n = 1 << 28
    p, g, m, v = (torch.zeros(n, device="cuda", dtype=torch.bfloat16) for _ in range(4))
    bw_case("adamw bf16 x4 256Mi", 7 * n * 2, lambda: native.adamw_(p, g, m, v, 1e-3, 0.9, 0.999, 1e-8, 0.01, 1e-3))
    idx = torch.stack([torch.randperm(E, device="cuda")[:2] for _ in range(1024)]).repeat(T // 1024, 1)
    from b200moe.ops.moe_fused import capacity_rows
    cap = capacity_rows(2 * T, E)
    bw_case("moe_plan 32768 slots", 1, lambda: native.moe_plan(idx, E, cap))
    slot_row, row_slot, offs2, te2, meta, _ = native.moe_plan(idx, E, cap)
    bw_case("moe_gather 32768x4096", 2 * R * D * 2, lambda: native.moe_gather(x, row_slot, meta, cap))
    wts = torch.rand(T, 2, device="cuda")
    bw_case("moe_combine 16384x4096", 3 * T * D * 2, lambda: native.moe_combine(xp, slot_row, wts, T))
    os.makedirs(OUT_DIR, exist_ok=True)
    with open(os.path.join(OUT_DIR, f"kernels_mode{args.tile_mode}.json"), "w") as f:
        json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
