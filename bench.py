"""Headline benchmark: training throughput of the Mixtral-8x7B-like MoE decoder.

``python bench.py --gpus N --steps K --warmup W`` (under ``torch.distributed.run``
for N > 1) runs full training steps (forward, backward, gradient reduction,
AdamW) on synthetic tokens with random-init weights and prints one JSON line.

Model per GPU count (layer count scaled so per-GPU work is constant; d_model
4096, d_ff 14336, 32/8 heads, 8 experts top-2, vocab 32000, sequence 8192,
32 microbatches of 2 sequences per data rank):

  N=1  8 blocks,  PP1 × FSDP1 × EP1, global batch 64
  N=2  8 blocks,  PP1 × FSDP2 × EP2, global batch 128
  N=4  16 blocks, PP2 × FSDP2 × EP2, global batch 128
  N=8  32 blocks, PP4 × FSDP2 × EP2, global batch 128   (the named configuration)

``value`` is tokens/s normalised to the 32-block model: raw tokens/s times
``flops_per_token(blocks) / flops_per_token(32)``; at N=8 it is the raw number.
``tokens_per_s_raw`` and ``mfu`` (of 2.25 PFLOP/s dense bf16 per GPU) are also
reported.  ``--impl reference`` times the unmodified reference package from
``baseline/_ref`` through its own public API on the same configuration.

Both arms run the loop of the reference's ``train()`` (distributed_parallel_
training_pipelined.py:210-257): every step draws a fresh batch on the host,
copies it from pinned memory to the device, sets the learning rate from the
reference's warm-up/cosine schedule (``configs/run_config.yaml``: 0 at iteration
0, 2e-6 per iteration), runs the pipelined step and reads the loss back.  One
timed pass gives both numbers: ``ms_per_step`` from CUDA events around the K
steps, ``e2e`` from the larger of that and the host clock around the same steps.

``--layout`` selects other named configurations on 8 GPUs: ``ddp2`` (PP1 x FSDP4 x
EP4 x DDP2, 8 blocks, global batch 32, RoPE base 1e6) and ``pp2`` (PP2 x FSDP4 x
EP4, 32 blocks, global batch 64 in 16 microbatches).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
BASELINE_TOKENS_PER_S = 75076.0
MODEL = {"d_model": 4096, "d_ff": 14336, "num_head": 32, "experts": 8, "vocab": 32000, "seq": 8192}
LAYOUT = {1: (1, 1, 8, 64), 2: (1, 2, 8, 128), 4: (2, 2, 8, 128), 8: (4, 2, 8, 128)}  # pp, fsdp, blocks/stage, batch
# other named configurations: pp, fsdp, ddp, blocks/stage, global batch, microbatches, rope base
NAMED = {"ddp2": (1, 4, 2, 8, 32, 4, 1e6), "pp2": (2, 4, 1, 16, 64, 16, 1e4),
         # two stages of the one-GPU workload on two GPUs (16 blocks): isolates what the pipeline itself costs
         "pp2x1": (2, 1, 1, 8, 64, 32, 1e4)}
SCHEDULE = {"a_max": 0.01, "a_min": 0.0001, "t_w": 5000, "t_c": 20000}     # the reference's run_config.yaml


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=2)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="b200moe", choices=["b200moe", "reference"])
    # development overrides (change the workload; the JSON line records them)
    p.add_argument("--layers", type=int, default=None, help="blocks per stage")
    p.add_argument("--microbatches", type=int, default=32)
    p.add_argument("--batch", type=int, default=None, help="global batch in sequences")
    p.add_argument("--seq", type=int, default=MODEL["seq"])
    p.add_argument("--recompute", default=None, choices=["none", "swiglu", "block"])
    p.add_argument("--backend", default=None, choices=["fused", "nccl"])
    p.add_argument("--no-e2e", action="store_true",
                   help="accepted for older command lines: both numbers now come from the one timed pass")
    p.add_argument("--layout", default=None, choices=sorted(NAMED), help="a named configuration (see NAMED)")
    p.add_argument("--pipeline-link", default=None, choices=["peer", "nccl"],
                   help="stage-to-stage transfers: this library's peer-store kernels or batched NCCL send/recv "
                        "(default: the library's default)")
    p.add_argument("--kernel-times", default=None, metavar="FILE",
                   help="after the measurement, run one more step with a CUDA-event pair around every launch of this "
                        "library and write rank 0's per-kernel totals to FILE (JSON)")
    return p.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi every 200 ms."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0):
        self.gpu, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, peak, power, reasons = [], None, [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in self.rows:
            if len(row) < 9:
                continue
            try:
                clocks.append(float(row[1]))
                peak = float(row[2])
                power.append(float(row[3]))
            except ValueError:
                continue
            for name, cell in zip(names, row[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": peak,
                "power_w_max": max(power) if power else None, "samples": len(clocks), "reasons": sorted(reasons)}


def run_config(args):
    if args.layout:
        pp, fsdp, ddp, blocks, batch, microbatches, theta = NAMED[args.layout]
        if args.gpus != pp * fsdp * ddp:
            raise SystemExit(f"--layout {args.layout} needs --gpus {pp * fsdp * ddp}")
    else:
        if args.gpus not in LAYOUT:
            raise SystemExit(f"--gpus must be one of {sorted(LAYOUT)}")
        pp, fsdp, blocks, batch = LAYOUT[args.gpus]
        ddp, microbatches, theta = 1, args.microbatches, 1e4
    blocks = args.layers or blocks
    batch = args.batch or batch
    return {"pp": pp, "fsdp": fsdp, "ddp": ddp, "blocks_per_stage": blocks, "batch": batch,
            "microbatches": microbatches, "seq": args.seq, "experts_per_rank": MODEL["experts"] // fsdp,
            "rope_theta": theta}


def init_dist(args, timeout_s=None):
    import datetime
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"WORLD_SIZE={world} does not match --gpus {args.gpus}")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    extra = {"timeout": datetime.timedelta(seconds=timeout_s)} if timeout_s else {}
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device, **extra)
    return rank, world, local, device


def measure(step, args, device, rank, launches_fn):
    """``warmup`` untimed steps, then ``steps`` timed ones in ONE pass.  ``step(i)`` is a whole iteration of the
    training loop: host batch -> pinned memory -> device, learning rate, pipelined step, loss read back.  Returns
    device ms per step (CUDA events, max over ranks), end-to-end ms per step (the larger of the events and the
    host clock around the same steps, max over ranks), the clock record, launches and the last loss."""
    import torch
    import torch.distributed as dist

    def fence():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    fence()
    sampler = ClockSampler(device.index) if rank == 0 else None
    if sampler:
        sampler.start()
    launches_before = launches_fn()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    begin.record()
    last = None
    for i in range(args.steps):
        last = step(args.warmup + i)
    end.record()
    fence()
    wall = (time.perf_counter() - t0) * 1e3
    launches = launches_fn() - launches_before
    clocks = sampler.stop() if sampler else None
    events = begin.elapsed_time(end)
    ms = torch.tensor([events, max(events, wall)], dtype=torch.float64, device=device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    device_ms, e2e_ms = (float(v) / args.steps for v in ms.tolist())
    return device_ms, e2e_ms, clocks, launches, last


def say_failure(impl, args, error, detail=""):
    """First failing rank of a run: one line that names the exception (stderr for people, a JSON line on stdout
    for the reference arm, whose contract is an ``unavailable`` line), then leave non-zero without waiting in
    collective teardown for peers, so that torchrun ends them at once."""
    rank = int(os.environ.get("RANK", "0"))
    text = str(error).strip().splitlines()
    reason = f"{type(error).__name__}: {text[0][:300] if text else ''}"
    print(f"[bench {impl}, rank {rank}] {reason} {detail}".rstrip(), file=sys.stderr, flush=True)
    marker = os.path.join("/tmp", f"b200moe_bench_failed_{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}")
    try:
        os.close(os.open(marker, os.O_CREAT | os.O_EXCL | os.O_WRONLY))
        first = True
    except OSError:
        first = False          # another rank already reported; its line is the root cause
    if first and impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": f"rank {rank}: {reason}", "n_gpus": args.gpus}),
              flush=True)
    # a lone reference process reports and ends normally; under torchrun a non-zero code ends the peers
    os._exit(0 if impl == "reference" and int(os.environ.get("WORLD_SIZE", "1")) == 1 else 1)


def report(args, cfg, device_ms, e2e_ms, clocks, launches, loss, h2d, d2h, impl, extra=None):
    sys.path.insert(0, ROOT) if ROOT not in sys.path else None
    from b200moe.utils.metrics import PEAK_BF16_DENSE, flops_per_token
    blocks_total = cfg["blocks_per_stage"] * cfg["pp"]
    fpt = flops_per_token(MODEL["d_model"], MODEL["d_ff"], MODEL["num_head"], MODEL["experts"], MODEL["vocab"],
                          blocks_total, cfg["seq"])
    fpt32 = flops_per_token(MODEL["d_model"], MODEL["d_ff"], MODEL["num_head"], MODEL["experts"], MODEL["vocab"],
                            32, cfg["seq"])
    tokens = cfg["batch"] * cfg["seq"]

    def rate(ms):
        raw = tokens / (ms / 1e3)
        return raw, raw * fpt / fpt32
    raw, value = rate(device_ms)
    line = {
        "metric": "total tokens/s (32-block-equivalent), Mixtral-8x7B-like MoE, seq 8192, PP/FSDP/EP training step",
        "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": device_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": value / BASELINE_TOKENS_PER_S, "dtype": "bf16" if impl == "b200moe" else "fp16+bf16 (stock)",
        "data": "synthetic uniform token ids, random-init weights", "impl": impl,
        "tokens_per_s_raw": raw, "mfu": raw * fpt / (args.gpus * PEAK_BF16_DENSE),
        "gflops_per_token": fpt / 1e9, "loss": loss,
        "config": {"model": f"{blocks_total}-block 8x7B-like MoE (d_model 4096, d_ff 14336, 32/8 GQA heads, "
                            f"8 experts top-2, vocab 32000)",
                   "global_batch": cfg["batch"], "seq_len": cfg["seq"], "microbatches": cfg["microbatches"],
                   "parallelism": f"pp{cfg['pp']}·fsdp{cfg['fsdp']}·ep{cfg['fsdp']}·ddp{cfg['ddp']}",
                   "blocks_total": blocks_total, "layout": args.layout or "scaling",
                   "rope_theta": cfg["rope_theta"],
                   "loop": "fresh host batch + H2D from pinned memory, lr from the reference's warm-up schedule, "
                           "pipelined step, loss read back: every step, warm-up included",
                   "l2": "no flush: every step streams >20 GB of weights and activations (inputs larger than L2)"},
        "clocks": clocks, "gpu_launches": launches,
    }
    if e2e_ms is not None:
        line["e2e"] = {"value": rate(e2e_ms)[1], "unit": "tokens/s", "ms_per_step": e2e_ms,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
    if extra:
        line.update(extra)
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------ this framework
def bench_b200moe(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    state = {}
    try:
        rank, world, local, device = init_dist(args)
        from b200moe.ops import native
        from b200moe.ops.functional import cross_entropy
        from b200moe.parallel import pipelined_train_overlap
        from b200moe.topology import build_groups
        from b200moe.trainer import build_model
        from b200moe.utils.data import BatchStager
        from b200moe.utils.schedule import learning_rate_schedule_wrapper
        cfg = run_config(args)
        single = cfg["fsdp"] == 1          # all 8 experts of every block on this GPU
        config = {
            "general": {"device": "gpu", "n_workers": world, "gpu_per_node": world, "info_src": 0},
            "data": {"vocab_size": MODEL["vocab"], "mock_data": True, "seed": 42},
            "model": {"num_head": MODEL["num_head"], "d_model": MODEL["d_model"], "d_ff": MODEL["d_ff"],
                      "context_len": cfg["seq"], "num_layers": cfg["blocks_per_stage"],
                      "num_expert_per_node": cfg["experts_per_rank"], "rope_theta": cfg["rope_theta"]},
            "comm": {"backend": args.backend or "fused"},
            "train": {"fsdp_parallel_num": cfg["fsdp"], "data_parallel_num": cfg["ddp"],
                      "pipeline_parallel_stages": cfg["pp"], "microbatch_num": cfg["microbatches"],
                      "batch_size": cfg["batch"], "learning_rate": 1e-4,
                      "optimizer": {"beta1": 0.9, "beta2": 0.999, "lambda": 0.01},
                      # the trainer decides per MoE call, from the HBM it has left, whether the gate/up
                      # pre-activations are kept or rebuilt in the backward pass
                      "activation_recompute": args.recompute or "auto",
                      # one GPU holds all 8 experts of 8 blocks (11.3 G parameters): moments and gradient
                      # accumulators use the reference's bf16 there; fp32 everywhere else
                      "expert_state_dtype": "bfloat16" if single else "float32",
                      "expert_grad_dtype": "bfloat16" if single else "float32"},
        }
        mesh = build_groups(config["train"], rank, world, world)
        comm = None
        if config["comm"]["backend"] == "fused" and native.has("comm"):
            from b200moe.comm import make_comm
            comm = make_comm(mesh, device, pipeline_link=args.pipeline_link)
        state["comm"] = comm
        torch.manual_seed(1234 + mesh.stage)
        model, optimizer = build_model(config, mesh, device, mesh.group("fsdp"), mesh.group("ddp"), torch.bfloat16,
                                       comm)
        width = cfg["fsdp"] * cfg["ddp"]
        local_batch = cfg["batch"] // width
        stager = BatchStager(local_batch, cfg["seq"], device)
        rng = np.random.default_rng(42 + mesh.dp_idx)
        edge = mesh.stage in (0, mesh.pp - 1)
        spec = [local_batch, cfg["seq"], MODEL["d_model"]]
        lr_at = learning_rate_schedule_wrapper(**SCHEDULE)

        def step(iteration):
            x, y = stager.next(None, rng, MODEL["vocab"], mock_data=True) if edge else (None, None)   # H2D
            for group in optimizer.param_groups:
                group["lr"] = lr_at(iteration)
            loss = pipelined_train_overlap(model, optimizer, x, y, spec, cfg["microbatches"], mesh.stage,
                                           cross_entropy, dtype=torch.bfloat16, device=device,
                                           pp_group=mesh.group("pp"), dp_group=mesh.group("data"))
            return float(loss) if torch.is_tensor(loss) else loss      # device -> host read of the step's loss

        device_ms, e2e_ms, clocks, launches, last = measure(step, args, device, rank, native.launch_count)
        native.check_status()      # a device-side wait that ran out is an error
        if args.kernel_times:
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            native.start_launch_timing()
            begin.record()
            step(args.warmup + args.steps)
            end.record()
            table = native.launch_times()
            if rank == 0:
                step_ms = begin.elapsed_time(end)
                rows = sorted(((ms, label, count) for label, (count, ms) in table.items()), reverse=True)
                with open(args.kernel_times, "w") as handle:
                    json.dump({"step_ms": step_ms, "native_ms": sum(r[0] for r in rows), "n_gpus": args.gpus,
                               "kernels": [{"launch": label, "launches": count, "ms": round(ms, 3),
                                            "share": round(ms / step_ms, 4)} for ms, label, count in rows]},
                              handle, indent=1)
        loss = torch.tensor([float(last) if last is not None else 0.0], device=device)
        dist.all_reduce(loss, op=dist.ReduceOp.MAX)
        # allocator peak, and what the device itself reports as taken (symmetric buffers and library workspaces
        # are outside PyTorch's allocator)
        free, total = torch.cuda.mem_get_info(device)
        peak = torch.tensor([torch.cuda.max_memory_allocated() / 2 ** 30, (total - free) / 2 ** 30], device=device)
        dist.all_reduce(peak, op=dist.ReduceOp.MAX)
        load = torch.tensor([_worst_expert_load(comm)], device=device)
        dist.all_reduce(load, op=dist.ReduceOp.MAX)
        budget = getattr(model, "activation_budget", None)
        kept = torch.tensor(list((budget.granted, budget.refused) if budget else (0, 0)), device=device,
                            dtype=torch.float64)
        dist.all_reduce(kept, op=dist.ReduceOp.SUM)
        if rank == 0:
            report(args, cfg, device_ms, e2e_ms, clocks, launches, float(loss), stager.h2d_bytes if edge else 0, 4,
                   "b200moe", {"peak_mem_gib": float(peak[0]), "device_mem_used_gib": float(peak[1]),
                               "activation_recompute": config["train"]["activation_recompute"],
                               "moe_calls_kept_gate_up": int(kept[0]), "moe_calls_rebuilt_gate_up": int(kept[1]),
                               "ep_max_rows_over_balanced": round(float(load), 3),
                               "comm_backend": "fused" if comm is not None else "nccl",
                               "pipeline_link": ("none" if mesh.pp == 1 else
                                                 "nccl" if comm is None or not any(comm._pp.values()) else "peer"),
                               "native_ops": native.available_ops()})
        dist.destroy_process_group()
    except Exception as error:
        import torch
        detail = ""
        try:
            detail = (f"| peak_mem_gib {torch.cuda.max_memory_allocated() / 2 ** 30:.1f} "
                      f"| ep_max_rows_over_balanced {_worst_expert_load(state.get('comm')):.3f}")
        except Exception:
            pass
        say_failure("b200moe", args, error, detail)


def _worst_expert_load(comm) -> float:
    """Rows the busiest rank of any layer received in its last call, relative to a perfectly balanced split."""
    worst = 0.0
    if comm is not None:
        for ctx in comm._ep.values():
            worst = max(worst, ctx.worst_load())
    return worst


# ------------------------------------------------------------------------------ reference arm
def bench_reference(args):
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "implementation")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed"}))
        return
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != ROOT]
    sys.path.insert(0, ref_root)
    try:
        import numpy as np
        import torch
        import torch.distributed as dist
        rank, world, local, device = init_dist(args, timeout_s=240)   # a rank that dies ends the others quickly
        from implementation.distributed.ddp_modules import FSDPWrapperPipelined
        from implementation.layers import TransformerLMPipelined
        from implementation.nnfunctions import cross_entropy, learning_rate_schedule_wrapper
        from implementation.optimizer import AdamW
        from implementation.startup import parallel_rank_groups
        from implementation.train_utils import compile_model, get_batch
        from pipeline import pipelined_train_overlap
        cfg = run_config(args)
        train = {"fsdp_parallel_num": cfg["fsdp"], "data_parallel_num": cfg["ddp"],
                 "pipeline_parallel_stages": cfg["pp"]}
        groups = {}
        for name, lists in parallel_rank_groups(train, world, world).items():
            for ranks in lists:
                g = dist.new_group(ranks=ranks)
                if rank in ranks:
                    groups[name] = g
        width = cfg["fsdp"] * cfg["ddp"]
        stage, dp_idx = rank // width, rank % width
        torch.backends.cuda.matmul.allow_tf32 = True
        torch.backends.cudnn.allow_tf32 = True
        torch.manual_seed(1234 + stage)
        model = TransformerLMPipelined(MODEL["vocab"], cfg["seq"], MODEL["d_model"], cfg["blocks_per_stage"],
                                       MODEL["num_head"], stage, cfg["pp"],
                                       num_expert_per_node=cfg["experts_per_rank"], d_ff=MODEL["d_ff"],
                                       theta=cfg["rope_theta"], dp_group=groups["fsdp"],
                                       moe_compute_dtype=torch.bfloat16)
        model.to(device)
        model = FSDPWrapperPipelined(model, FSDP_communication_group=groups["fsdp"],
                                     DDP_communication_group=groups["ddp"] if cfg["ddp"] > 1 else None,
                                     compute_dtype=torch.float16, moe_compute_dtype=torch.bfloat16)
        optimizer = AdamW(model.parameters(), lr=1e-4, betas=(0.9, 0.999), weight_decay=0.01)
        model = compile_model(model)
        local_batch = cfg["batch"] // width
        rng = np.random.default_rng(42 + dp_idx)
        edge = stage in (0, cfg["pp"] - 1)
        spec = [local_batch, cfg["seq"], MODEL["d_model"]]
        lr_at = learning_rate_schedule_wrapper(**SCHEDULE)

        def step(iteration):         # the body of the reference's own training loop
            x, y = get_batch(None, local_batch, cfg["seq"], device, rng=rng, vocab_size=MODEL["vocab"],
                             mock_data=True) if edge else (None, None)
            for group in optimizer.param_groups:
                group["lr"] = lr_at(iteration)
            loss = pipelined_train_overlap(model, optimizer, x, y, spec, cfg["microbatches"], stage, cross_entropy,
                                           dtype=torch.float16, device=device, pp_group=groups["pp"],
                                           dp_group=groups["data"])
            return float(loss) if torch.is_tensor(loss) else loss

        device_ms, e2e_ms, clocks, _, last = measure(step, args, device, rank, lambda: 0)
        loss = torch.tensor([float(last) if last is not None else 0.0], device=device)
        dist.all_reduce(loss, op=dist.ReduceOp.MAX)
        peak = torch.tensor([torch.cuda.max_memory_allocated() / 2 ** 30], device=device)
        dist.all_reduce(peak, op=dist.ReduceOp.MAX)
        if rank == 0:
            report(args, cfg, device_ms, e2e_ms, clocks, 0, float(loss), 2 * local_batch * cfg["seq"] * 8 if edge else 0,
                   4, "reference", {"peak_mem_gib": float(peak)})
        dist.destroy_process_group()
    except Exception as error:
        say_failure("reference", args, error)


if __name__ == "__main__":
    arguments = parse_args()
    if arguments.impl == "reference":
        bench_reference(arguments)
    else:
        bench_b200moe(arguments)
