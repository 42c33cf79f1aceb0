"""Worker bodies for multi-process CPU (gloo) tests; not collected by pytest."""
import os
import sys
import traceback

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def tiny_config(world, fsdp, ddp, pp, folder, target=10, save=5, batch=4, micro=2, layers=2, experts=None,
                recompute="none", load=""):
    experts = experts if experts is not None else 4 // fsdp if fsdp <= 4 else 1
    return {
        "general": {"device": "cpu", "n_workers": world, "gpu_per_node": world, "info_src": 0,
                    "checkpoint_folder": str(folder)},
        "recovery": {"collective_timeout_seconds": 60},
        "data": {"vocab_size": 1024, "mock_data": True, "seed": 0, "validate_batches": True},
        "model": {"num_head": 4, "d_model": 128, "d_ff": 256, "context_len": 256, "num_layers": layers,
                  "num_expert_per_node": experts, "rope_theta": 10000},
        "train": {"fsdp_parallel_num": fsdp, "data_parallel_num": ddp, "pipeline_parallel_stages": pp,
                  "microbatch_num": micro, "batch_size": batch, "save_interval": save, "target_iteration": target,
                  "learning_rate": 3e-4, "optimizer": {"beta1": 0.9, "beta2": 0.999, "lambda": 0.01},
                  "learning_rate_scheduler": {"a_max": 3e-4, "a_min": 3e-5, "t_w": 2, "t_c": 100},
                  "print_loss_interval": 1, "load_checkpoint_path": load, "activation_recompute": recompute},
    }


def _env(rank, world, port):
    os.environ.update({"RANK": str(rank), "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world),
                       "LOCAL_WORLD_SIZE": str(world), "GROUP_RANK": "0", "MASTER_ADDR": "127.0.0.1",
                       "MASTER_PORT": str(port)})


def run_train(rank, world, port, config, result_dir, fail_at=None):
    """Run ``b200moe.trainer.train``; optionally raise on one rank at an
    iteration (a host-side failure between steps)."""
    import torch
    import torch.distributed as dist
    _env(rank, world, port)
    torch.manual_seed(1234)
    torch.set_num_threads(2)
    from b200moe import trainer
    if fail_at is not None:
        class Boom(RuntimeError):
            pass
        original = trainer.ckpt.verify_pending_checkpoints
        seen = {"n": 0}

        def counting(pending, iteration, *a, **k):
            if not k.get("drain") and iteration == fail_at[1] and rank == fail_at[0]:
                raise Boom(f"injected host failure at iteration {iteration}")
            return original(pending, iteration, *a, **k)
        trainer.ckpt.verify_pending_checkpoints = counting
    try:
        import io
        import contextlib
        buf = io.StringIO()
        with contextlib.redirect_stdout(buf):
            final = trainer.train(rank, 0, world, config)
        with open(os.path.join(result_dir, f"out_{rank}.txt"), "w") as f:
            f.write(buf.getvalue())
            f.write(f"\nFINAL {final}\n")
    except Exception:
        with open(os.path.join(result_dir, f"err_{rank}.txt"), "w") as f:
            f.write(traceback.format_exc())
        raise
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_grad_equivalence(rank, world, port, result_dir, pp):
    """FSDP×EP (and PP) gradients against a single-process model that owns all
    experts and sees the concatenated batch."""
    import torch
    import torch.distributed as dist
    _env(rank, world, port)
    torch.set_num_threads(2)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from b200moe.models import TransformerLMPipelined
        from b200moe.ops.functional import cross_entropy
        from b200moe.optim import AdamW
        from b200moe.parallel import FSDPWrapperPipelined, pipelined_train_overlap
        from b200moe.topology import build_groups
        fsdp = world // pp
        train = {"fsdp_parallel_num": fsdp, "data_parallel_num": 1, "pipeline_parallel_stages": pp}
        mesh = build_groups(train, rank, world, world)
        solo = [dist.new_group([r]) for r in range(world)]
        V, S, D, L, H, E, FF = 256, 32, 64, 2, 4, 4, 96
        torch.manual_seed(7)
        full = TransformerLMPipelined(V, S, D, L * pp, H, 0, 1, num_expert_per_node=E, d_ff=FF,
                                      moe_compute_dtype=torch.float32)
        full_state = {k: v.clone() for k, v in full.state_dict().items()}
        data = torch.randint(0, V, (fsdp * 4, S + 1))
        stage, shard = mesh.stage, mesh.shard_idx
        e_local = E // fsdp
        part = TransformerLMPipelined(V, S, D, L, H, stage, pp, num_expert_per_node=e_local, d_ff=FF,
                                      dp_group=mesh.group("fsdp"), moe_compute_dtype=torch.float32)
        state = {}
        for key in part.state_dict():
            if key.startswith("layers."):
                idx = int(key.split(".")[1])
                src = full_state[key.replace(f"layers.{idx}.", f"layers.{idx + stage * L}.", 1)]
                if ".experts." in key:
                    src = src[shard * e_local:(shard + 1) * e_local]
                state[key] = src.clone()
            else:
                state[key] = full_state[key].clone()
        part.load_state_dict(state)
        wrapped = FSDPWrapperPipelined(part, mesh.group("fsdp"), None, compute_dtype=torch.float32,
                                       moe_compute_dtype=torch.float32)
        opt = AdamW(wrapped.parameters(), lr=0.0, weight_decay=0.0)
        mine = data[shard * 4:(shard + 1) * 4]
        x = mine[:, :-1] if stage == 0 else None
        y = mine[:, 1:] if stage == pp - 1 else None
        loss = pipelined_train_overlap(wrapped, opt, x, y, [4, S, D], 2, stage, cross_entropy, dtype=torch.float32,
                                       device=torch.device("cpu"), pp_group=mesh.group("pp"),
                                       dp_group=mesh.group("data"))
        grads = {}
        for name, p in wrapped.named_parameters():
            g = p.grad if p.grad is not None else getattr(p, "main_grad", None)
            grads[name] = None if g is None else g.detach().float().clone()
        # single-process oracle on rank 0
        out = {"loss": float(loss), "grads": grads, "stage": stage, "shard": shard}
        if rank == 0:
            full.load_state_dict(full_state)
            ref = FSDPWrapperPipelined(full, solo[0], None, compute_dtype=torch.float32, moe_compute_dtype=torch.float32)
            ropt = AdamW(ref.parameters(), lr=0.0, weight_decay=0.0)
            rloss = pipelined_train_overlap(ref, ropt, data[:, :-1], data[:, 1:], [fsdp * 4, S, D], 1, 0,
                                            cross_entropy, dtype=torch.float32, device=torch.device("cpu"))
            out["ref_loss"] = float(rloss)
            out["ref_grads"] = {n: (p.grad if p.grad is not None else p.main_grad).detach().float().clone()
                                for n, p in ref.named_parameters()}
        torch.save(out, os.path.join(result_dir, f"grads_{rank}.pt"))
    except Exception:
        with open(os.path.join(result_dir, f"err_{rank}.txt"), "w") as f:
            f.write(traceback.format_exc())
        raise
    finally:
        dist.destroy_process_group()


def run_reference_layout(rank, world, port, result_dir, pp, ref_dir):
    """The run of ``_ref_oracle_multi.py`` with this framework: same per-rank initial state, data and steps."""
    import numpy as np
    import torch
    import torch.distributed as dist
    _env(rank, world, port)
    torch.set_num_threads(2)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from b200moe.models import TransformerLMPipelined
        from b200moe.ops.functional import cross_entropy
        from b200moe.optim import AdamW
        from b200moe.parallel import FSDPWrapperPipelined, pipelined_train_overlap
        from b200moe.topology import build_groups
        from b200moe.utils.data import get_batch
        fsdp = world // pp
        mesh = build_groups({"fsdp_parallel_num": fsdp, "data_parallel_num": 1, "pipeline_parallel_stages": pp},
                            rank, world, world)
        stage, shard = mesh.stage, mesh.shard_idx
        ref = torch.load(os.path.join(ref_dir, f"ref_{rank}.pt"))
        assert (ref["stage"], ref["shard"]) == (stage, shard)
        V, S, D, L, H, E, FF, B, STEPS = 512, 64, 64, 2, 4, 4, 128, 4, 4
        model = TransformerLMPipelined(V, S, D, L, H, stage, pp, num_expert_per_node=E // fsdp, d_ff=FF,
                                       dp_group=mesh.group("fsdp"), moe_compute_dtype=torch.bfloat16)
        model.load_state_dict(ref["init"])
        wrapped = FSDPWrapperPipelined(model, mesh.group("fsdp"), None, compute_dtype=torch.float32,
                                       expert_grad_dtype=torch.bfloat16, expert_state_dtype=torch.bfloat16)
        optimizer = AdamW(wrapped.parameters(), lr=1e-3, betas=(0.9, 0.999), weight_decay=0.01)
        rng = np.random.default_rng(shard)
        losses = []
        for _ in range(STEPS):
            x = y = None
            if stage in (0, pp - 1):
                x, y = get_batch(None, B, S, "cpu", rng=rng, vocab_size=V, mock_data=True)
            loss = pipelined_train_overlap(wrapped, optimizer, x if stage == 0 else None,
                                           y if stage == pp - 1 else None, [B, S, D], 2, stage, cross_entropy,
                                           dtype=torch.float32, device=torch.device("cpu"),
                                           pp_group=mesh.group("pp"), dp_group=mesh.group("data"))
            losses.append(float(loss))
        final = {k: v.detach().float().clone() for k, v in wrapped.state_dict().items()}
        torch.save({"losses": losses, "final": final, "ref_losses": ref["losses"], "ref_final": ref["final"],
                    "stage": stage}, os.path.join(result_dir, f"mine_{rank}.pt"))
    except Exception:
        with open(os.path.join(result_dir, f"err_{rank}.txt"), "w") as f:
            f.write(traceback.format_exc())
        raise
    finally:
        dist.destroy_process_group()
