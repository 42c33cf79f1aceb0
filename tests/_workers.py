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


class HostTransport:
    """Stand-in for ``b200moe.comm.pp.DeviceTransport`` on CPU ranks: the landing rings and flag words are files
    mapped by every rank, a send runs at call time (it blocks the rank exactly where the kernel would block the
    stream), and the ring discipline is checked: a slot that its receiver still uses must never be written."""

    def __init__(self, folder, stage, stages, slot_bytes, act_slots, grad_slots, timeout=60.0):
        import torch
        import torch.distributed as dist
        self.stage, self.stages, self.slot_bytes = stage, stages, slot_bytes
        self.act_slots, self.grad_slots = act_slots, grad_slots
        self.timeout = timeout
        slots = act_slots + grad_slots
        for name, size in (("data", slot_bytes * slots), ("flags", 4 * 64), ("busy", 4 * slots)):
            with open(os.path.join(folder, f"{name}_{stage}.bin"), "wb") as f:
                f.write(b"\0" * size)
        dist.barrier()
        self.data = [torch.from_file(os.path.join(folder, f"data_{r}.bin"), shared=True, size=slot_bytes * slots,
                                     dtype=torch.uint8) for r in range(stages)]
        self.flags = [torch.from_file(os.path.join(folder, f"flags_{r}.bin"), shared=True, size=64,
                                      dtype=torch.int32) for r in range(stages)]
        self.busy = [torch.from_file(os.path.join(folder, f"busy_{r}.bin"), shared=True, size=slots,
                                     dtype=torch.int32) for r in range(stages)]
        self.waits_for_room = 0
        dist.barrier()

    def buffers(self):
        return []

    def _spin(self, word, seq, what):
        import time
        deadline = time.monotonic() + self.timeout
        while int(word[0]) < seq:
            if time.monotonic() > deadline:
                raise TimeoutError(f"stage {self.stage}: {what} {seq} never came")
            time.sleep(0.0005)

    def slot(self, index, spec, dtype):
        import math
        begin = index * self.slot_bytes
        return self.data[self.stage][begin:begin + math.prod(spec) * dtype.itemsize].view(dtype).view(spec)

    def send(self, payload, peer, slot, flag, ack_word, seq, need_ack):
        mine = self.flags[self.stage]
        if need_ack > 0 and int(mine[ack_word]) < need_ack:
            self.waits_for_room += 1
            self._spin(mine[ack_word:ack_word + 1], need_ack, "acknowledgement")
        if int(self.busy[peer][slot]) != 0:
            raise AssertionError(f"stage {self.stage} overwrites slot {slot} of stage {peer} while message "
                                 f"{int(self.busy[peer][slot])} is still in use (sending {seq})")
        raw = payload.contiguous().view(-1).view(torch_uint8())
        begin = slot * self.slot_bytes
        self.data[peer][begin:begin + raw.numel()].copy_(raw)
        self.flags[peer][flag] = seq

    def wait(self, flag, seq):
        self._spin(self.flags[self.stage][flag:flag + 1], seq, "message")
        if int(self.flags[self.stage][flag]) != seq:
            raise AssertionError(f"stage {self.stage}: slot of flag {flag} holds message "
                                 f"{int(self.flags[self.stage][flag])}, expected {seq}")
        slot = flag if flag < 16 else self.act_slots + (flag - 16)
        self.busy[self.stage][slot] = seq

    def ack(self, upstream, downstream, value):
        if upstream is not None:
            self.busy[self.stage][(value - 1) % self.act_slots] = 0
            self.flags[upstream][32] = value
        if downstream is not None:
            self.busy[self.stage][self.act_slots + (value - 1) % self.grad_slots] = 0
            self.flags[downstream][33] = value


def torch_uint8():
    import torch
    return torch.uint8


def run_peer_link_schedule(rank, world, port, result_dir, microbatches, steps, act_slots):
    """The 1F1B scheduler over ``world`` stages, once with the NCCL-style link (gloo) and once with the peer link
    over ``HostTransport``: same losses and gradients, no ring overrun, no deadlock."""
    import torch
    import torch.distributed as dist
    _env(rank, world, port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from b200moe.comm.pp import GRAD_SLOTS, PeerLink
        from b200moe.models import TransformerLMPipelined
        from b200moe.ops.functional import cross_entropy
        from b200moe.optim import AdamW
        from b200moe.parallel import FSDPWrapperPipelined, pipelined_train_overlap
        from b200moe.topology import build_groups
        mesh = build_groups({"fsdp_parallel_num": 1, "data_parallel_num": 1, "pipeline_parallel_stages": world},
                            rank, world, world)
        stage = mesh.stage
        V, S, D, H, E, FF, B = 128, 16, 32, 4, 2, 48, 2 * microbatches
        spec = [B // microbatches, S, D]
        results = {}
        for kind in ("nccl", "peer"):
            torch.manual_seed(11 + stage)
            model = TransformerLMPipelined(V, S, D, 1, H, stage, world, num_expert_per_node=E, d_ff=FF,
                                           dp_group=mesh.group("fsdp"), moe_compute_dtype=torch.float32)
            wrapped = FSDPWrapperPipelined(model, mesh.group("fsdp"), None, compute_dtype=torch.float32,
                                           moe_compute_dtype=torch.float32)
            transport = None
            if kind == "peer":
                folder = os.path.join(result_dir, "rings")
                os.makedirs(folder, exist_ok=True)
                transport = HostTransport(folder, stage, world, PeerLink.slot_bytes(spec, torch.float32),
                                          act_slots, GRAD_SLOTS)
                link = PeerLink(stage, world, spec, torch.float32, transport, act_slots=act_slots)

                class _Offer:
                    def pp_link(self, group, stage_, spec_, dtype_):
                        assert (stage_, list(spec_), dtype_) == (stage, spec, torch.float32)
                        return link
                wrapped.comm = _Offer()
            opt = AdamW(wrapped.parameters(), lr=1e-3, weight_decay=0.0)
            gen = torch.Generator().manual_seed(5)
            losses = []
            for _ in range(steps):
                data = torch.randint(0, V, (B, S + 1), generator=gen)
                loss = pipelined_train_overlap(wrapped, opt, data[:, :-1] if stage == 0 else None,
                                               data[:, 1:] if stage == world - 1 else None, [B, S, D], microbatches,
                                               stage, cross_entropy, dtype=torch.float32, device=torch.device("cpu"),
                                               pp_group=mesh.group("pp"), dp_group=mesh.group("data"))
                losses.append(float(loss))
            results[kind] = {"losses": losses,
                             "weights": {k: v.detach().clone() for k, v in wrapped.state_dict().items()},
                             "waits_for_room": 0 if transport is None else transport.waits_for_room}
            dist.barrier()
        torch.save({"stage": stage, **results}, os.path.join(result_dir, f"link_{rank}.pt"))
    except Exception:
        with open(os.path.join(result_dir, f"err_{rank}.txt"), "w") as f:
            f.write(traceback.format_exc())
        raise
    finally:
        dist.destroy_process_group()


def run_weight_hooks(rank, world, port, result_dir):
    """Two row-sharded linear modules in sequence with the gather / prefetch / free hooks of
    ``b200moe.parallel.hooks`` against the same modules holding full weights."""
    import collections
    import torch
    import torch.distributed as dist
    _env(rank, world, port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from implementation.distributed import ddp_modules as H
        torch.manual_seed(3)
        full = [torch.nn.Linear(8, 12, bias=False), torch.nn.Linear(12, 6, bias=False)]
        x = torch.randn(5, 8)
        want = full[1](full[0](x))
        want.sum().backward()
        sharded = [torch.nn.Linear(8, 12, bias=False), torch.nn.Linear(12, 6, bias=False)]
        for whole, part in zip(full, sharded):
            rows = whole.weight.shape[0] // world
            part.weight.data = whole.weight.data[rank * rows:(rank + 1) * rows].clone()
        first, second = sharded
        works, works_back = collections.deque(), collections.deque()
        # forward: the first module gathers itself and prefetches the second, which only waits for its prefetch
        first.register_forward_pre_hook(H.sync_weight_wrapper(torch.float32, None))
        first.register_forward_pre_hook(H.async_weight_wrapper_next(second, works, torch.float32, None))
        second.register_forward_pre_hook(H.wait_prefetched_weight(works))
        # backward: mirrored, the second module gathers itself and prefetches the first
        second.register_full_backward_pre_hook(H.sync_weight_wrapper_backward(torch.float32, None))
        second.register_full_backward_pre_hook(H.async_weight_wrapper_backward_next(first, works_back, torch.float32, None))
        first.register_full_backward_pre_hook(H.wait_prefetched_weight_backward(works_back))
        for module in sharded:
            module.register_forward_hook(H.free_weight)
            module.register_full_backward_hook(H.free_weight_backward)
        xs = x.clone().requires_grad_(True)
        got = second(first(xs))
        assert torch.allclose(got, want, atol=1e-6)
        assert first.weight.shape[0] == 12 // world and second.weight.shape[0] == 6 // world     # shards are back
        got.sum().backward()
        assert not works and not works_back
        assert first.weight.shape[0] == 12 // world and first.weight.data_original is None
        for whole, part in zip(full, sharded):
            assert part.weight.grad.shape == whole.weight.shape
            assert torch.allclose(part.weight.grad, whole.weight.grad, atol=1e-6)
        with open(os.path.join(result_dir, f"hooks_ok_{rank}"), "w") as f:
            f.write("ok")
    except Exception:
        with open(os.path.join(result_dir, f"err_{rank}.txt"), "w") as f:
            f.write(traceback.format_exc())
        raise
    finally:
        dist.destroy_process_group()


def run_moe_two_step(rank, world, port, result_dir):
    """``MoELayerMulti._dispatch_tokens`` → grouped experts → ``_combine_tokens`` over ``world`` gloo ranks against
    the layer's own forward pass, values and gradients."""
    import torch
    import torch.distributed as dist
    _env(rank, world, port)
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from b200moe import ops
        from b200moe.models.layers import MoELayerMulti
        torch.manual_seed(5)
        layer = MoELayerMulti(32, 48, num_expert_per_node=2, dtype=torch.float32, dp_group=dist.group.WORLD)
        torch.manual_seed(100 + rank)
        for p in layer.experts.parameters():
            p.data.normal_(0, 0.2)                        # every rank owns different experts
        x = torch.randn(3, 8, 32)
        x1 = x.clone().requires_grad_(True)
        want, want_aux = layer(x1, return_aux_loss=True)
        (want.sum() + want_aux).backward()
        want_grads = [x1.grad.clone()] + [p.grad.clone() for p in layer.parameters()]
        layer.zero_grad()
        x2 = x.clone().requires_grad_(True)
        flat = x2.reshape(-1, 32)
        logits = layer.router(flat)
        weights, idx = ops.router_top2(logits)
        (expert_input, offsets, expert_splits, recv_splits, order, probs, aux) = layer._dispatch_tokens(
            flat, logits, weights, idx, True)
        assert int(offsets[-1]) == expert_input.shape[0] and len(expert_splits) == 2 * world
        got = layer._combine_tokens(layer.experts(expert_input, offsets), expert_splits, recv_splits, order, probs,
                                    3, 8, x.dtype)
        assert torch.allclose(got, want, atol=1e-5) and torch.allclose(aux, want_aux, atol=1e-6)
        (got.sum() + aux).backward()
        got_grads = [x2.grad] + [p.grad for p in layer.parameters()]
        for a, b in zip(got_grads, want_grads):
            assert torch.allclose(a, b, atol=1e-4), (a - b).abs().max()
        with open(os.path.join(result_dir, f"two_step_ok_{rank}"), "w") as f:
            f.write("ok")
    except Exception:
        with open(os.path.join(result_dir, f"err_{rank}.txt"), "w") as f:
            f.write(traceback.format_exc())
        raise
    finally:
        dist.destroy_process_group()
