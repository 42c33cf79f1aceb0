"""Worker bodies for multi-GPU tests (one process per GPU, NCCL); not collected."""
import os
import sys
import traceback

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _setup(rank, world, port):
    import torch
    import torch.distributed as dist
    os.environ.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    return torch.device("cuda", rank)


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def _guarded(fn, rank, world, port, out_dir, *args):
    import torch.distributed as dist
    try:
        fn(rank, world, port, out_dir, *args)
        with open(os.path.join(out_dir, f"ok_{rank}"), "w") as f:
            f.write("ok")
    except Exception:
        with open(os.path.join(out_dir, f"err_{rank}.txt"), "w") as f:
            f.write(traceback.format_exc())
        raise
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _allreduce(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    from b200moe.comm import make_comm
    from b200moe.ops import native
    from b200moe.topology import build_groups
    device = _setup(rank, world, port)
    mesh = build_groups({"fsdp_parallel_num": 1, "data_parallel_num": world, "pipeline_parallel_stages": 1},
                        rank, world, world)
    # the in-switch reduction needs the staging buffer bound to a multicast address (off by default elsewhere)
    comm = make_comm(mesh, device, multicast=True)
    kinds = ["oneshot", "twoshot"] + (["nvls"] if comm.ddp is not None else [])
    for n in (1000, 262144, 5_000_000):
        for kind in kinds:
            torch.manual_seed(100 + rank)
            x = torch.randn(n, device=device)
            want = x.clone()
            dist.all_reduce(want, op=dist.ReduceOp.AVG)
            got = x.clone()
            try:
                comm.allreduce_avg(got, mesh.group("ddp"), kind=kind)
            except RuntimeError as error:
                if kind == "nvls" and "-11" in str(error):
                    continue          # no multicast address on this system
                raise
            assert _rel(got, want) < 1e-6, (n, kind, _rel(got, want))
    auto = torch.randn(3_000_001, device=device)
    want = auto.clone()
    dist.all_reduce(want, op=dist.ReduceOp.AVG)
    comm.allreduce_avg(auto, mesh.group("ddp"))
    assert _rel(auto, want) < 1e-6
    native.check_status()


def _moe_pull_once(epc, x, logits, params, dout, keep_rows=None, recompute=False):
    """One forward/backward of the pull-based block; returns out and the gradients."""
    import torch
    from b200moe import ops
    from b200moe.ops.moe_fused import moe_ffn_pull
    xs, lg = x.clone().requires_grad_(True), logits.clone().requires_grad_(True)
    ps = [p.clone().requires_grad_(True) for p in params]
    if keep_rows is not None:
        epc.expected_rows = lambda key: keep_rows       # force a partial keep of the gate/up rows
    out, _, _ = moe_ffn_pull(xs, lambda staged: ops.router_top2(lg), *ps, epc, recompute=recompute)
    out.backward(dout)
    torch.cuda.synchronize()
    return [out.detach(), xs.grad, lg.grad] + [p.grad for p in ps]


def _moe_ep(rank, world, port, out_dir):
    """Expert-parallel block against the NCCL all-to-all path, forward and backward: the exchange fused with the
    expert GEMMs with the gate/up rows all kept, partly kept and all rebuilt, under an unbalanced router and under one
    that sends every row of every rank to rank 0."""
    import torch
    from b200moe import ops
    from b200moe.comm import make_comm
    from b200moe.ops import native
    from b200moe.ops.moe import moe_ffn
    from b200moe.topology import build_groups
    device = _setup(rank, world, port)
    mesh = build_groups({"fsdp_parallel_num": world, "data_parallel_num": 1, "pipeline_parallel_stages": 1},
                        rank, world, world)
    comm = make_comm(mesh, device, wait_seconds=3.0)
    group = mesh.group("fsdp")
    T, D, Fd, E_total = 1024, 256, 512, 8
    e_local = E_total // world
    torch.manual_seed(5 + rank)
    x = (torch.randn(T, D, device=device)).bfloat16()
    w1, w3, w2 = ((torch.randn(e_local, Fd, D, device=device) * 0.06).bfloat16(),
                  (torch.randn(e_local, Fd, D, device=device) * 0.06).bfloat16(),
                  (torch.randn(e_local, D, Fd, device=device) * 0.06).bfloat16())
    dout = torch.randn(T, D, device=device).bfloat16()
    epc = comm.ep_context(T, D, E_total, Fd)
    for case in ("unbalanced", "all_to_rank0"):
        logits = torch.randn(T, E_total, device=device)
        if case == "unbalanced":
            if rank == 0:
                logits[:, 0] += 2.0
        else:
            logits[:, :e_local] += 30.0              # every token of every rank picks two experts of rank 0
        xs, lg = x.clone().requires_grad_(True), logits.clone().requires_grad_(True)
        params = [p.clone().requires_grad_(True) for p in (w1, w2, w3)]
        weights, idx = ops.router_top2(lg)
        ops.set_native(False)
        try:
            out = moe_ffn(xs, weights, idx, *params, group=group)          # NCCL all-to-all, PyTorch statements
            out.backward(dout)
        finally:
            ops.set_native(True)
        want = [out.detach(), xs.grad, lg.grad] + [p.grad for p in params]
        for keep_rows, recompute in ((None, False), (256, False), (None, True), (None, False)):
            got = _moe_pull_once(epc, x, logits, (w1, w2, w3), dout, keep_rows, recompute)
            for name, a, b in zip(("out", "dx", "dlogits", "dw1", "dw2", "dw3"), got, want):
                assert _rel(a, b) < 2e-2, (case, keep_rows, recompute, name, _rel(a, b))
            native.check_status()
            epc.__dict__.pop("expected_rows", None)
        assert len(epc.free) == len(epc.pool) >= 1                           # every pool slot came back
        if case == "all_to_rank0" and rank == 0:
            assert epc.worst_load() >= float(world)                          # every slot of every rank landed here


def _train_parity(rank, world, port, out_dir, pp, ddp=1, skew=False):
    """A few training steps: fused peer-memory backend against the NCCL backend.  ``skew``: every token of every
    rank is routed to the two first experts (both on shard rank 0), the worst case for the expert buffers."""
    import warnings

    import torch
    from b200moe.comm import make_comm
    from b200moe.ops import native
    from b200moe.ops.functional import cross_entropy
    from b200moe.parallel import pipelined_train_overlap
    from b200moe.topology import build_groups
    from b200moe.trainer import build_model
    device = _setup(rank, world, port)
    fsdp = world // (pp * ddp)
    if skew:
        from b200moe import ops
        plain_top2 = ops.router_top2

        def biased_top2(logits):
            bias = torch.zeros(logits.shape[-1], device=logits.device, dtype=logits.dtype)
            bias[:2] = 40.0
            return plain_top2(logits + bias)
        ops.router_top2 = biased_top2
    config = {
        "general": {"device": "gpu"}, "data": {"vocab_size": 2048},
        "model": {"num_head": 4, "d_model": 512, "d_ff": 1024, "context_len": 256, "num_layers": 2,
                  "num_expert_per_node": 8 // fsdp},
        "train": {"fsdp_parallel_num": fsdp, "data_parallel_num": ddp, "pipeline_parallel_stages": pp,
                  "learning_rate": 1e-3, "optimizer": {"beta1": 0.9, "beta2": 0.999, "lambda": 0.01}},
    }
    mesh = build_groups(config["train"], rank, world, world)
    comm = make_comm(mesh, device, wait_seconds=5.0)
    losses = {}
    weights = {}
    for variant, backend, gather in (("fused", "fused", "step"), ("first_use", "fused", "first_use"),
                                     ("nccl", "nccl", "step")):
        config["comm"] = {"backend": backend}
        config["train"]["fsdp_gather"] = gather
        torch.manual_seed(77 + mesh.stage)
        model, opt = build_model(config, mesh, device, mesh.group("fsdp"), mesh.group("ddp"), torch.bfloat16,
                                 comm if backend == "fused" else None)
        assert model.fused == (backend == "fused")
        torch.manual_seed(1000 + mesh.dp_idx)
        ids = torch.randint(0, 2048, (4, 257), device=device)
        run = []
        before = native.launch_count()
        for step in range(3):
            x = ids[:, :-1] if mesh.stage == 0 else None
            y = ids[:, 1:] if mesh.stage == pp - 1 else None
            # third step of the fused backend: nothing inside a step may make the host wait for the device
            watch = backend == "fused" and gather == "step" and step == 2
            with warnings.catch_warnings(record=True) as seen:
                warnings.simplefilter("always")
                if watch:
                    torch.cuda.set_sync_debug_mode(1)
                try:
                    loss = pipelined_train_overlap(model, opt, x, y, [4, 256, 512], 2, mesh.stage, cross_entropy,
                                                   dtype=torch.bfloat16, device=device, pp_group=mesh.group("pp"),
                                                   dp_group=mesh.group("data"))
                finally:
                    torch.cuda.set_sync_debug_mode(0)
            syncs = [str(w.message) for w in seen if "synchroniz" in str(w.message).lower()]
            assert not (watch and syncs), syncs
            run.append(float(loss))
        losses[variant] = run
        weights[variant] = model.flat.master.clone()
        if gather == "first_use":
            # steps 2 and 3 gathered q/k/v and the output projection of both blocks inside their first GEMM
            epochs = [state["epoch"] for state in comm._ag_state.values()]
            assert len(epochs) == 4 and all(e == 2 for e in epochs), epochs
            assert all(w.pending_gather is not None for w, _ in model._lazy)
        assert native.launch_count() > before
    if mesh.stage == pp - 1:
        for other in ("first_use", "nccl"):
            for a, b in zip(losses["fused"], losses[other]):
                assert abs(a - b) < 5e-2, losses
    assert _rel(weights["fused"], weights["nccl"]) < 2e-2
    assert _rel(weights["fused"], weights["first_use"]) < 2e-3
    native.check_status()


def _pipeline_link(rank, world, port, out_dir):
    """``world`` pipeline stages, eight microbatches per step: the peer-memory link (landing rings in symmetric
    memory, peer stores, message numbers) against the batched NCCL send/recv.  Same kernels and same data on both
    sides, so losses and weights must agree to rounding of the atomics in the embedding gradient."""
    import torch
    from b200moe.comm import make_comm
    from b200moe.comm.pp import PeerLink
    from b200moe.ops import native
    from b200moe.ops.functional import cross_entropy
    from b200moe.parallel import pipelined_train_overlap
    from b200moe.topology import build_groups
    from b200moe.trainer import build_model
    device = _setup(rank, world, port)
    config = {
        "general": {"device": "gpu"}, "data": {"vocab_size": 2048}, "comm": {"backend": "fused"},
        "model": {"num_head": 4, "d_model": 512, "d_ff": 1024, "context_len": 256, "num_layers": 2 * world,
                  "num_expert_per_node": 4},
        "train": {"fsdp_parallel_num": 1, "data_parallel_num": 1, "pipeline_parallel_stages": world,
                  "learning_rate": 1e-3, "optimizer": {"beta1": 0.9, "beta2": 0.999, "lambda": 0.01}},
    }
    mesh = build_groups(config["train"], rank, world, world)
    stage = mesh.stage
    losses, weights = {}, {}
    for kind in ("nccl", "peer"):
        comm = make_comm(mesh, device, wait_seconds=5.0, pipeline_link=kind, pipeline_wait_seconds=20.0)
        torch.manual_seed(77 + stage)
        model, opt = build_model(config, mesh, device, mesh.group("fsdp"), mesh.group("ddp"), torch.bfloat16, comm)
        torch.manual_seed(1000)
        run = []
        for step in range(3):
            ids = torch.randint(0, 2048, (16, 257), device=device)
            loss = pipelined_train_overlap(model, opt, ids[:, :-1] if stage == 0 else None,
                                           ids[:, 1:] if stage == world - 1 else None, [16, 256, 512], 8, stage,
                                           cross_entropy, dtype=torch.bfloat16, device=device,
                                           pp_group=mesh.group("pp"), dp_group=mesh.group("data"))
            run.append(float(loss))
        torch.cuda.synchronize()
        native.check_status()
        links = [link for link in comm._pp.values() if link is not None]
        if kind == "peer":
            assert len(links) == 1 and isinstance(links[0], PeerLink)
            link = links[0]
            # three steps of eight microbatches: every ring wrapped several times
            assert link.done == 24
            assert link.sent_act == (24 if stage < world - 1 else 0) and link.got_act == (24 if stage > 0 else 0)
            assert link.sent_grad == (24 if stage > 0 else 0) and link.got_grad == (24 if stage < world - 1 else 0)
        else:
            assert not links
        losses[kind] = run
        weights[kind] = torch.cat([p.detach().float().reshape(-1) for p in model.parameters()])
    if stage == world - 1:
        assert all(l > 0 for l in losses["nccl"])
        for a, b in zip(losses["nccl"], losses["peer"]):
            assert abs(a - b) < 2e-3, losses
    assert _rel(weights["peer"], weights["nccl"]) < 1e-3


def _allgather_gemm(rank, world, port, out_dir):
    """All-gather fused with its GEMM against NCCL all_gather + fp32 matmul, over several "steps"."""
    import torch
    import torch.distributed as dist
    from b200moe.comm import make_comm
    from b200moe.ops import native
    from b200moe.topology import build_groups
    device = _setup(rank, world, port)
    mesh = build_groups({"fsdp_parallel_num": world, "data_parallel_num": 1, "pipeline_parallel_stages": 1},
                        rank, world, world)
    comm = make_comm(mesh, device)
    for M, segments, K in ((4096, [6144], 4096), (1000, [1984], 512), (2048, [4096, 1024, 1024], 4096)):
        N = sum(segments)
        owner = torch.cat([torch.arange(rows) // (rows // world) for rows in segments]).to(device)
        mine = owner == rank
        flat = comm.alloc_flat(N * K, torch.bfloat16)
        w = flat.view(N, K)
        for step in range(3):
            torch.manual_seed(1000 * step)
            full = (torch.randn(N, K, device=device) * 0.05).bfloat16()      # same on every rank
            torch.manual_seed(1000 * step + rank)
            x = (torch.randn(M, K, device=device) * 0.5).bfloat16()
            w.fill_(float("nan"))
            w[mine] = full[mine]
            y = comm.allgather_gemm(x, w, segments)
            assert torch.equal(w, full), "gathered weight differs"
            assert _rel(y, x.float() @ full.float().t()) < 1e-2
            # nobody rewrites its rows before every rank has finished reading them
            torch.cuda.synchronize()
            dist.barrier()
    native.check_status()


def run_allreduce(rank, world, port, out_dir):
    _guarded(_allreduce, rank, world, port, out_dir)


def run_moe_ep(rank, world, port, out_dir):
    _guarded(_moe_ep, rank, world, port, out_dir)


def run_train_parity(rank, world, port, out_dir, pp, ddp=1, skew=False):
    _guarded(_train_parity, rank, world, port, out_dir, pp, ddp, skew)


def run_pipeline_link(rank, world, port, out_dir):
    _guarded(_pipeline_link, rank, world, port, out_dir)


def run_allgather_gemm(rank, world, port, out_dir):
    _guarded(_allgather_gemm, rank, world, port, out_dir)
