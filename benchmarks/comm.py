"""Multi-GPU microbenchmarks of the peer-memory paths (run under torchrun).

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/comm.py [--skip-nccl]

Times, with CUDA events on each rank and the maximum over ranks:
  * the MoE block of one layer, forward + backward (16384 tokens per rank, d_model 4096, d_ff 14336, 8 experts
    spread over the N ranks, top-2): peer-memory dispatch/return against the NCCL all-to-all path;
  * the row dispatch + return alone, against its NVLink roofline (bytes that must cross ÷ 770 GB/s measured
    peer-copy bandwidth per direction);
  * the replica all-reduce kernels (one-shot, two-shot, NVLS) against ``dist.all_reduce`` at several sizes;
  * the all-gather fused with its consuming GEMM (weight row-sharded over the N ranks) against the same GEMM on
    an already gathered weight and against NCCL ``all_gather_into_tensor`` followed by that GEMM.
Rank 0 prints one JSON line per measurement and writes them to ``$B200MOE_BENCH_OUT/comm_N.json`` (default: the current directory).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OUT_DIR = os.environ.get("B200MOE_BENCH_OUT", os.getcwd())
sys.path.insert(0, ROOT)
NVLINK_GBS = 770.0


def timed(fn, iters=5, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    ms = torch.tensor([begin.elapsed_time(end) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--skip-nccl", action="store_true")
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--only", default="", help="comma-separated subset of: moe, aggemm, allreduce")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    from b200moe import ops
    from b200moe.comm import make_comm
    from b200moe.ops import native
    from b200moe.ops.moe import moe_ffn
    from b200moe.topology import build_groups
    rows = []
    only = set(filter(None, args.only.split(",")))
    want = lambda name: not only or name in only  # noqa: E731

    def emit(**record):
        record["n_gpus"] = world
        rows.append(record)
        if rank == 0:
            print(json.dumps(record), flush=True)

    # ---- expert parallel over all ranks
    mesh = build_groups({"fsdp_parallel_num": world, "data_parallel_num": 1, "pipeline_parallel_stages": 1},
                        rank, world, world)
    comm = make_comm(mesh, device)
    group = mesh.group("fsdp")
    T, D, Fd, E = args.tokens, 4096, 14336, 8
    e_local = E // world
    if want("moe"):
        torch.manual_seed(rank)
        x = torch.randn(T, D, device=device).bfloat16()
        logits = torch.randn(T, E, device=device)
        w1, w3, w2 = ((torch.randn(e_local, Fd, D, device=device) * 0.02).bfloat16().requires_grad_(True),
                      (torch.randn(e_local, Fd, D, device=device) * 0.02).bfloat16().requires_grad_(True),
                      (torch.randn(e_local, D, Fd, device=device) * 0.02).bfloat16().requires_grad_(True))
        for p in (w1, w2, w3):
            p.main_grad = torch.zeros_like(p, dtype=torch.float32)
        dout = torch.randn(T, D, device=device).bfloat16()
        ctx = comm.ep_context(T, D, E)

        def block(fused):
            xs, lg = x.clone().requires_grad_(True), logits.clone().requires_grad_(True)
            weights, idx = ops.router_top2(lg)
            ops.set_native(fused)
            try:
                out = moe_ffn(xs, weights, idx, w1, w2, w3, group=group, ep_ctx=ctx if fused else None)
                out.backward(dout)
            finally:
                ops.set_native(True)

        flops = 3 * 3 * 2 * T * 2 * D * Fd          # fwd + 2x bwd of three GEMMs over 2T rows (per rank, balanced)
        ms = timed(lambda: block(True), iters=3)
        emit(case="moe block fwd+bwd, peer-memory", ms=round(ms, 3), tflops_per_gpu=round(flops / ms / 1e9, 1))
        if not args.skip_nccl:
            ms_nccl = timed(lambda: block(False), iters=2, warmup=1)
            emit(case="moe block fwd+bwd, NCCL all-to-all + library grouped GEMM", ms=round(ms_nccl, 3),
                 tflops_per_gpu=round(flops / ms_nccl / 1e9, 1))
        # dispatch + return alone
        weights, idx = ops.router_top2(logits)

        def round_trip():
            route = ctx.dispatch(x, idx, key="bench")
            ctx.combine(route, route.x_perm, weights, T)

        ms = timed(round_trip)
        crossing = 2 * (2 * T * D * 2) * (world - 1) / world        # there and back, bytes leaving this rank
        emit(case="EP dispatch + return (rows only)", ms=round(ms, 4), nvlink_bytes_per_rank=int(crossing),
             achieved_gbs_per_direction=round(crossing / 2 / ms / 1e6, 1),
             frac_of_nvlink_roofline=round((crossing / 2 / (NVLINK_GBS * 1e9)) * 2 / (ms / 1e3), 3))
    # ---- all-gather fused with the consuming GEMM (weight row-sharded over all ranks)
    if want("aggemm"):
        for name, N, K in (("qkv", 6144, 4096), ("attn out", 4096, 4096)):
            M = args.tokens
            shard = N // world
            w = comm.alloc_flat(N * K, torch.bfloat16).view(N, K)
            torch.manual_seed(7 + rank)
            own = (torch.randn(shard, K, device=device) * 0.02).bfloat16()
            xs = torch.randn(M, K, device=device).bfloat16()
            w[rank * shard:(rank + 1) * shard] = own
            flops = 2 * M * N * K
            ms_fused = timed(lambda: comm.allgather_gemm(xs, w), iters=10)
            ms_plain = timed(lambda: native.gemm_nt(xs, w), iters=10)
            remote = (world - 1) * shard * K * 2
            emit(case=f"all-gather + GEMM in one kernel ({name})", M=M, N=N, K=K, ms=round(ms_fused, 4),
                 tflops=round(flops / ms_fused / 1e9, 1), gemm_alone_ms=round(ms_plain, 4),
                 nvlink_bytes_in=remote, link_time_ms=round(remote / (NVLINK_GBS * 1e6), 4),
                 frac_of_roofline=round(max(ms_plain, remote / (NVLINK_GBS * 1e6)) / ms_fused, 3))
            if not args.skip_nccl:
                def separate():
                    dist.all_gather_into_tensor(w, own, group=group)
                    return native.gemm_nt(xs, w)
                ms_sep = timed(separate, iters=10)
                emit(case=f"NCCL all_gather then GEMM ({name})", M=M, N=N, K=K, ms=round(ms_sep, 4),
                     tflops=round(flops / ms_sep / 1e9, 1))
        native.check_status()
    native.check_status()
    del comm
    if want("allreduce"):
        # ---- replica all-reduce over all ranks
        mesh2 = build_groups({"fsdp_parallel_num": 1, "data_parallel_num": world, "pipeline_parallel_stages": 1},
                             rank, world, world)
        comm2 = make_comm(mesh2, device)
        for n in (1 << 12, 1 << 18, 1 << 22, 1 << 26):
            buf = torch.randn(n, device=device)
            for kind in ("oneshot", "twoshot", "nvls"):
                if kind == "oneshot" and n > (1 << 22):
                    continue
                try:
                    ms = timed(lambda: comm2.allreduce_avg(buf, mesh2.group("ddp"), kind=kind))
                except RuntimeError:
                    continue
                emit(case=f"allreduce {kind}", floats=n, ms=round(ms, 4),
                     busbw_gbs=round(2 * (world - 1) / world * n * 4 / ms / 1e6, 1))
            if not args.skip_nccl:
                ms = timed(lambda: dist.all_reduce(buf, op=dist.ReduceOp.AVG))
                emit(case="allreduce NCCL", floats=n, ms=round(ms, 4), busbw_gbs=round(2 * (world - 1) / world * n * 4 / ms / 1e6, 1))
        native.check_status()
    if rank == 0:
        os.makedirs(OUT_DIR, exist_ok=True)
        with open(os.path.join(OUT_DIR, f"comm_{world}.json"), "w") as f:
            json.dump(rows, f, indent=1)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
