"""Multi-GPU microbenchmarks of the peer-memory paths (run under torchrun).

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/comm.py [--skip-nccl]

Times, with CUDA events on each rank and the maximum over ranks:
  * the MoE block of one layer, forward + backward (16384 tokens per rank, d_model 4096, d_ff 14336, 8 experts
    spread over the N ranks, top-2): the exchange fused with the expert GEMMs against the NCCL all-to-all path;
  * the two fused exchange kernels alone against their rooflines: gather + gate/up GEMM + SwiGLU (dispatch) and
    down-projection GEMM with the weighted return in its epilogue; the roofline of each is the slower of the
    same GEMM on rows that are already in place and the bytes that must cross NVLink ÷ 770 GB/s (measured
    peer-copy bandwidth per direction);
  * the end-of-step kernel of the sharded parameters (gradient reduce-scatter + AdamW + weight all-gather in one
    launch) against the slower of its NVLink bytes ÷ 770 GB/s and its HBM bytes ÷ the measured copy bandwidth;
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


def timed(fn, iters=5, warmup=3):
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
    ap.add_argument("--only", default="", help="comma-separated subset of: moe, fsdp, aggemm, allreduce, pp")
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
    # the NVLS all-reduce needs buffers bound to a multicast address, and the binding is decided at the first rendezvous
    comm = make_comm(mesh, device, wait_seconds=5.0, multicast=want("allreduce"))
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
        from b200moe.comm import ep as EP
        from b200moe.ops.moe_fused import moe_ffn_pull
        epc = comm.ep_context(T, D, E, Fd)

        def block(fused):
            xs, lg = x.clone().requires_grad_(True), logits.clone().requires_grad_(True)
            if fused:
                out, _, _ = moe_ffn_pull(xs, lambda staged: ops.router_top2(lg), w1, w2, w3, epc, key="bench")
            else:
                weights, idx = ops.router_top2(lg)
                ops.set_native(False)
                try:
                    out = moe_ffn(xs, weights, idx, w1, w2, w3, group=group)
                finally:
                    ops.set_native(True)
            out.backward(dout)

        flops = 3 * 3 * 2 * T * 2 * D * Fd          # fwd + 2x bwd of three GEMMs over 2T rows (per rank, balanced)
        ms = timed(lambda: block(True), iters=3)
        emit(case="moe block fwd+bwd, exchange fused with the expert GEMMs", ms=round(ms, 3),
             tflops_per_gpu=round(flops / ms / 1e9, 1), max_rows_over_balanced=round(epc.worst_load(), 3))
        if not args.skip_nccl:
            ms_nccl = timed(lambda: block(False), iters=2, warmup=3)
            emit(case="moe block fwd+bwd, NCCL all-to-all + library grouped GEMM", ms=round(ms_nccl, 3),
                 tflops_per_gpu=round(flops / ms_nccl / 1e9, 1))
        # the two fused kernels alone, on one fixed routing
        weights, idx = ops.router_top2(logits)
        weights = weights.float().contiguous()
        slot = epc.acquire()
        epc.slot_tensor(slot).copy_(x)
        g = epc.g
        i32 = dict(dtype=torch.int32, device=device)
        row_src, row_tag = torch.empty(epc.cap, **i32), torch.empty(epc.cap, **i32)
        row_w = torch.empty(epc.cap, dtype=torch.float32, device=device)
        x_ws, h = epc.ws("x", D), epc.ws("h", Fd)
        state = {}

        def dispatch_gateup():
            offs, seg_end, tile_expert, meta, seq = epc.plan(idx, weights, "bench2")
            state.update(tile_expert=tile_expert, meta=meta)
            epc.gather_gemm(0, x_ws, w1, w3, 2 * Fd, D, tile_expert, meta, seg_end, 0, epc.pool[slot].table(), 1,
                            epc.land_src.tensor, epc.land_tag.tensor, epc.land_w.tensor, (row_src, row_tag, row_w),
                            EP.SIG_META, seq, 1, h, None, None, None, None, 0)

        def down_return():
            seq = g.next_seq(EP.SIG_RET_F)
            native.gemm_nt_push(h, w2, state["tile_expert"], state["meta"][0:1], e_local, epc.ret_f.table(), row_tag,
                                row_src, row_w, g.sig.table(), EP.SIG_RET_F, seq, g.rank, world, epc.tickets[4:])
            epc.combine(epc.ret_f, EP.SIG_RET_F, seq, with_scalars=False)

        ms_dispatch = timed(dispatch_gateup)
        ms_gateup = timed(lambda: native.gemm_swiglu(x_ws, w1, w3, state["tile_expert"], state["meta"][0:1],
                                                     save_gate_up=False, align256=True))
        ms_return = timed(down_return)
        ms_down = timed(lambda: native.gemm_nt(h, w2, tile_expert=state["tile_expert"],
                                               num_m_tiles=state["meta"][0:1], num_experts=e_local, align256=True))
        rows_here = int(state["meta"][1].item())
        crossing = 2 * T * D * 2 * (world - 1) / world                # bytes that enter (or leave) a rank, balanced
        link_ms = crossing / (NVLINK_GBS * 1e6)
        emit(case="gather + gate/up GEMM + SwiGLU in one kernel (plan included)", ms=round(ms_dispatch, 4),
             gemm_alone_ms=round(ms_gateup, 4), nvlink_bytes_in=int(crossing), link_time_ms=round(link_ms, 4),
             rows=rows_here, tflops=round(2 * rows_here * D * 2 * Fd / ms_dispatch / 1e9, 1),
             frac_of_roofline=round(max(ms_gateup, link_ms) / ms_dispatch, 3))
        emit(case="down GEMM with the weighted return in its epilogue + combine", ms=round(ms_return, 4),
             gemm_alone_ms=round(ms_down, 4), nvlink_bytes_out=int(crossing), link_time_ms=round(link_ms, 4),
             tflops=round(2 * rows_here * D * Fd / ms_return / 1e9, 1),
             frac_of_roofline=round(max(ms_down, link_ms) / ms_return, 3))
        epc.release(slot)
        native.check_status()
    if want("pp") and world > 1:
        # ---- pipeline link: every rank stores one microbatch (2 x 8192 tokens, 128 MiB) into the landing ring of its
        # right neighbour and waits for the one from its left neighbour, so every GPU sends and receives at once
        from b200moe.comm.pp import DeviceTransport, PeerLink
        spec = [2, 8192, D]
        slot_bytes = PeerLink.slot_bytes(spec, torch.bfloat16)
        transport = DeviceTransport(group, device, comm.status, slot_bytes, 2, 5.0)
        payload = torch.randn(spec, device=device).bfloat16()
        state = {"n": 0}

        def hop():
            state["n"] += 1
            n = state["n"]
            slot = (n - 1) % 2
            # bandwidth only: nothing reads the slots, so no acknowledgements (need_ack = 0); a neighbour that runs
            # ahead overwrites a slot and raises its message number, which the wait accepts
            transport.send(payload, (rank + 1) % world, slot, slot, 32, n, 0)
            transport.wait(slot, n)
        ms = timed(hop, iters=20)
        nbytes = payload.numel() * 2
        emit(case="pipeline link: 128 MiB to the right neighbour + wait for the left one", ms=round(ms, 4),
             gbs_per_direction=round(nbytes / ms / 1e6, 1), frac_of_nvlink=round(nbytes / ms / 1e6 / NVLINK_GBS, 3))
        if not args.skip_nccl:
            recv = torch.empty_like(payload)

            def nccl_hop():
                ops_ = [dist.P2POp(dist.isend, payload, (rank + 1) % world), dist.P2POp(dist.irecv, recv, (rank - 1) % world)]
                for work in dist.batch_isend_irecv(ops_):
                    work.wait()
            ms_nccl = timed(nccl_hop, iters=20)
            emit(case="NCCL batched isend/irecv, same ring", ms=round(ms_nccl, 4),
                 gbs_per_direction=round(nbytes / ms_nccl / 1e6, 1))
        native.check_status()
    if want("fsdp") and world > 1:
        # ---- end of step: reduce-scatter + AdamW + all-gather of one stage's dense weights in one kernel
        from b200moe.parallel.fsdp import FlatShards
        shapes = []
        for _ in range(8):                                       # eight blocks: q, k, v, output projection, router
            shapes += [(4096, 4096), (1024, 4096), (1024, 4096), (4096, 4096), (8, 4096)]
        entries, shard_off, full_off = [], 0, 0
        for rows_, cols in shapes:
            numel = rows_ * cols
            entries.append({"param": object(), "full_numel": numel, "shard_numel": numel // world,
                            "shard_off": shard_off, "full_off": full_off,
                            "shard_shape": (rows_ // world, cols), "full_shape": (rows_, cols)})
            shard_off += numel // world
            full_off += numel
        flat = FlatShards(entries, world, rank, torch.bfloat16, device, comm.alloc_flat)
        flat.full_g.normal_()
        ms = timed(lambda: comm.fused_update(flat, True, 1e-4, 0.9, 0.999, 1e-8, 0.01, 1e-4), iters=10)
        shard = shard_off
        link_in, link_out = (world - 1) * shard * 4, (world - 1) * shard * 2
        hbm = shard * (4 + 4 * 3 + 4 * 4 + 2)      # own gradient, master/m/v in, master/m/v/shard_grad out, own weights
        hbm_gbs = 6541.8
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                hbm_gbs = float(json.load(f)["hbm_gbs"])
        except (OSError, KeyError, ValueError):
            pass
        bound_ms = max(link_in / (NVLINK_GBS * 1e6), hbm / (hbm_gbs * 1e6))
        emit(case="reduce-scatter + AdamW + all-gather in one kernel", parameters=full_off, ms=round(ms, 4),
             nvlink_bytes_in=link_in, nvlink_bytes_out=link_out, hbm_bytes=hbm,
             achieved_link_in_gbs=round(link_in / ms / 1e6, 1), frac_of_roofline=round(bound_ms / ms, 3))
        if not args.skip_nccl:
            shard_grad = torch.empty(shard, device=device)

            def separate():
                dist.reduce_scatter_tensor(shard_grad, flat.full_g[:shard * world], op=dist.ReduceOp.AVG, group=group)
                native.adamw_(flat.master, shard_grad, flat.m, flat.v, 1e-4, 0.9, 0.999, 1e-8, 0.01, 1e-4)
                dist.all_gather_into_tensor(flat.full_w[:shard * world], flat.master.bfloat16(), group=group)
            ms_sep = timed(separate, iters=10)
            emit(case="NCCL reduce_scatter + AdamW + cast + NCCL all_gather", parameters=full_off, ms=round(ms_sep, 4))
        native.check_status()
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
        comm2 = make_comm(mesh2, device, multicast=True)
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
