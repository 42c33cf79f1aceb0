"""Loss curve, first-step gradients and checkpoint interchange (both directions) against the unmodified
reference package (CPU, tiny configuration, same weights and data).  Skipped when the reference is not installed
under ``baseline/_ref``."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "implementation")), reason="reference not installed")
def test_tiny_model_matches_reference(tmp_path, free_port):
    out = tmp_path / "ref.pt"
    env = {k: v for k, v in os.environ.items() if k != "PYTHONPATH"}
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "_ref_oracle.py"), REF, str(out), str(free_port)],
                          env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    ref = torch.load(out)
    from b200moe.models import TransformerLMPipelined
    from b200moe.ops.functional import cross_entropy
    from b200moe.optim import AdamW
    from b200moe.parallel import FSDPWrapperPipelined, pipelined_train_overlap
    from b200moe.utils.data import get_batch
    model = TransformerLMPipelined(1024, 256, 128, 2, 4, 0, 1, num_expert_per_node=4, d_ff=256,
                                   moe_compute_dtype=torch.bfloat16)
    model.load_state_dict(ref["init"])          # same keys and shapes as the reference's stage model
    wrapped = FSDPWrapperPipelined(model, compute_dtype=torch.float32, expert_grad_dtype=torch.bfloat16,
                                   expert_state_dtype=torch.bfloat16)
    optimizer = AdamW(wrapped.parameters(), lr=3e-4, betas=(0.9, 0.999), weight_decay=0.01)
    rng = np.random.default_rng(0)
    losses, grads = [], None
    for _ in range(6):
        x, y = get_batch(None, 4, 256, "cpu", rng=rng, vocab_size=1024, mock_data=True)
        loss = pipelined_train_overlap(wrapped, optimizer, x, y, [4, 256, 128], 2, 0, cross_entropy,
                                       dtype=torch.float32, device=torch.device("cpu"))
        losses.append(float(loss))
        if grads is None:
            grads = {n: (p.grad if p.grad is not None else p.main_grad).detach().float().clone()
                     for n, p in wrapped.named_parameters()}
    assert losses == pytest.approx(ref["losses"], abs=3e-3)
    checked = 0
    for name, want in ref["grads"].items():
        got = grads[name]
        rel = float((got - want).norm() / (want.norm() + 1e-12))
        assert rel < 0.1, (name, rel)      # both sides run the experts in bf16 with different op order
        checked += 1
    assert checked >= 20
    # ---- checkpoint interchange.  The reference wrote a checkpoint after its sixth step: a fresh model of this
    # framework loads it with its own loader and its seventh step gives the reference's seventh loss.
    from b200moe.utils.checkpoint import load_checkpoint_async_dist, save_checkpoint
    mine7 = float(pipelined_train_overlap(wrapped, optimizer, *get_batch(None, 4, 256, "cpu", rng=rng, vocab_size=1024,
                                                                         mock_data=True),
                                          [4, 256, 128], 2, 0, cross_entropy, dtype=torch.float32,
                                          device=torch.device("cpu")))
    assert mine7 == pytest.approx(ref["loss7"], abs=3e-3)
    torch.manual_seed(123)
    other = TransformerLMPipelined(1024, 256, 128, 2, 4, 0, 1, num_expert_per_node=4, d_ff=256,
                                   moe_compute_dtype=torch.bfloat16)
    resumed = FSDPWrapperPipelined(other, compute_dtype=torch.float32, expert_grad_dtype=torch.bfloat16,
                                   expert_state_dtype=torch.bfloat16)
    resumed_opt = AdamW(resumed.parameters(), lr=3e-4, betas=(0.9, 0.999), weight_decay=0.01)
    assert load_checkpoint_async_dist(str(out) + ".ckpt", resumed, resumed_opt) == 6
    rng2 = np.random.default_rng(0)
    for _ in range(6):
        get_batch(None, 4, 256, "cpu", rng=rng2, vocab_size=1024, mock_data=True)
    x7, y7 = get_batch(None, 4, 256, "cpu", rng=rng2, vocab_size=1024, mock_data=True)
    from_ref = float(pipelined_train_overlap(resumed, resumed_opt, x7, y7, [4, 256, 128], 2, 0, cross_entropy,
                                             dtype=torch.float32, device=torch.device("cpu")))
    assert from_ref == pytest.approx(ref["loss7"], abs=3e-3)
    # ---- and the other way round: a checkpoint of this framework after six steps, loaded by the reference's loader
    torch.manual_seed(0)
    again = TransformerLMPipelined(1024, 256, 128, 2, 4, 0, 1, num_expert_per_node=4, d_ff=256,
                                   moe_compute_dtype=torch.bfloat16)
    again.load_state_dict(ref["init"])
    w2 = FSDPWrapperPipelined(again, compute_dtype=torch.float32, expert_grad_dtype=torch.bfloat16,
                              expert_state_dtype=torch.bfloat16)
    o2 = AdamW(w2.parameters(), lr=3e-4, betas=(0.9, 0.999), weight_decay=0.01)
    rng3 = np.random.default_rng(0)
    for _ in range(6):
        xb, yb = get_batch(None, 4, 256, "cpu", rng=rng3, vocab_size=1024, mock_data=True)
        pipelined_train_overlap(w2, o2, xb, yb, [4, 256, 128], 2, 0, cross_entropy, dtype=torch.float32,
                                device=torch.device("cpu"))
    mine_ckpt = tmp_path / "mine.ckpt"
    save_checkpoint(w2, o2, 6, str(mine_ckpt))
    back = tmp_path / "ref_resume.pt"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "_ref_oracle.py"), REF, str(back),
                           str(free_port), "resume", str(mine_ckpt)], env=env, capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    resumed_by_ref = torch.load(back)
    assert resumed_by_ref["iteration"] == 6
    assert resumed_by_ref["loss7"] == pytest.approx(mine7, abs=3e-3)


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "implementation")), reason="reference not installed")
def test_router_auxiliary_loss_and_metrics_match_reference(tmp_path, free_port):
    """``router_aux_loss_coef`` and ``return_metrics`` of the pipeline step: task, auxiliary and total loss of two
    steps against the reference (the auxiliary term also steers the second step through its gradient)."""
    env = {k: v for k, v in os.environ.items() if k != "PYTHONPATH"}
    base, aux = tmp_path / "base.pt", tmp_path / "aux.pt"
    for out, mode in ((base, "train"), (aux, "aux")):
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "_ref_oracle.py"), REF, str(out),
                               str(free_port), mode], env=env, capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
    init, want = torch.load(base)["init"], torch.load(aux)["metrics"]
    from b200moe.models import TransformerLMPipelined
    from b200moe.ops.functional import cross_entropy
    from b200moe.optim import AdamW
    from b200moe.parallel import FSDPWrapperPipelined, pipelined_train_overlap
    from b200moe.utils.data import get_batch
    model = TransformerLMPipelined(1024, 256, 128, 2, 4, 0, 1, num_expert_per_node=4, d_ff=256,
                                   moe_compute_dtype=torch.bfloat16)
    model.load_state_dict(init)
    wrapped = FSDPWrapperPipelined(model, compute_dtype=torch.float32, expert_grad_dtype=torch.bfloat16,
                                   expert_state_dtype=torch.bfloat16)
    optimizer = AdamW(wrapped.parameters(), lr=3e-4, betas=(0.9, 0.999), weight_decay=0.01)
    rng = np.random.default_rng(0)
    for step in range(2):
        x, y = get_batch(None, 4, 256, "cpu", rng=rng, vocab_size=1024, mock_data=True)
        got = pipelined_train_overlap(wrapped, optimizer, x, y, [4, 256, 128], 2, 0, cross_entropy,
                                      dtype=torch.float32, device=torch.device("cpu"), router_aux_loss_coef=0.05,
                                      return_metrics=True)
        assert set(got) == set(want[step])
        for key, value in want[step].items():
            assert float(got[key]) == pytest.approx(value, abs=3e-3), (step, key)


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "implementation")), reason="reference not installed")
@pytest.mark.parametrize("world,pp", [(2, 1), (4, 2)])
def test_multi_rank_training_matches_reference(tmp_path, free_port, world, pp):
    """FSDP2 x EP2 (and PP2) on gloo: the unmodified reference and this framework start from the same per-rank
    state, see the same batches and must produce the same losses and, after four optimizer steps, the same
    parameter shards (same checkpoint keys) on every rank."""
    import torch.multiprocessing as mp

    import _workers as W
    ref_dir = tmp_path / "ref"
    ref_dir.mkdir()
    env = {k: v for k, v in os.environ.items() if k != "PYTHONPATH"}
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "_ref_oracle_multi.py"), REF, str(ref_dir),
                               str(free_port), str(world), str(pp), str(rank)], env=env, stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True) for rank in range(world)]
    for proc in procs:
        _, err = proc.communicate(timeout=900)
        assert proc.returncode == 0, err[-3000:]
    mine_dir = tmp_path / "mine"
    mine_dir.mkdir()
    mp.spawn(W.run_reference_layout, args=(world, free_port + 1, str(mine_dir), pp, str(ref_dir)), nprocs=world,
             join=True)
    checked = 0
    for rank in range(world):
        out = torch.load(mine_dir / f"mine_{rank}.pt")
        if out["stage"] == pp - 1:
            assert out["losses"] == pytest.approx(out["ref_losses"], abs=5e-3), (rank, out["losses"], out["ref_losses"])
        assert set(out["final"]) == set(out["ref_final"])
        for key, want in out["ref_final"].items():
            got = out["final"][key]
            assert got.shape == want.shape, key
            rel = float((got - want).norm() / (want.norm() + 1e-12))
            assert rel < 2e-2, (rank, key, rel)
            checked += 1
    assert checked >= 20 * world // pp


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "implementation")), reason="reference not installed")
def test_host_side_utilities_match_reference(tmp_path):
    """Data sampling (bit-exact batches and generator state), learning-rate schedule, rank layout, configuration
    validation verdicts, elementwise statements, the AdamW rule and checkpoint discovery: the reference's outputs
    for a fixed set of inputs against this framework's own functions."""
    import copy

    import yaml
    out = tmp_path / "utils.pt"
    env = {k: v for k, v in os.environ.items() if k != "PYTHONPATH"}
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "_ref_oracle_utils.py"), REF, str(out),
                           str(tmp_path)], env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    ref = torch.load(out, weights_only=False)
    from b200moe import config as cfg
    from b200moe.ops.functional import cross_entropy, silu, softmax
    from b200moe.optim import AdamW
    from b200moe.topology import parallel_rank_groups, parallel_sizes
    from b200moe.utils.checkpoint import latest_checkpoint
    from b200moe.utils.data import get_batch
    from b200moe.utils.schedule import learning_rate_schedule_wrapper
    # data
    tokens = (np.arange(5000, dtype=np.int64) * 7) % 1000
    rng = np.random.default_rng(11)
    calls = (dict(mock_data=True, vocab_size=1000), dict(), dict(start_idx=100), dict(serial_sampling=True, start_idx=64),
             dict(serial_sampling=True, start_idx=4900), dict(mock_data=True, vocab_size=17))
    for kwargs, (want_x, want_y) in zip(calls, ref["batches"]):
        x, y = get_batch(None if kwargs.get("mock_data") else tokens, 6, 32, "cpu", rng=rng, **kwargs)
        assert x.dtype == want_x.dtype and torch.equal(x, want_x) and torch.equal(y, want_y), kwargs
    mine_state, ref_state = rng.bit_generator.state, ref["rng_after"]
    assert mine_state["state"] == ref_state["state"]
    # schedule
    sched = learning_rate_schedule_wrapper(0.01, 0.0001, 50, 400)
    assert [sched(t) for t in (0, 1, 25, 49, 50, 51, 200, 399, 400, 401, 10000)] == pytest.approx(ref["lr"], rel=1e-12)
    # rank layout
    for (fsdp, ddp, pp, world, local), want in ref["layouts"].items():
        train = {"fsdp_parallel_num": fsdp, "data_parallel_num": ddp, "pipeline_parallel_stages": pp}
        try:
            got = parallel_rank_groups(train, world, local)
        except ValueError:
            got = "ValueError"
        assert got == want, (fsdp, ddp, pp, world, local)
    assert parallel_sizes({"data_parallel_num": 4}) == tuple(ref["legacy_sizes"])
    # validation verdicts on the same mutations of the same (reference) configuration file
    with open(os.path.join(REF, "configs", "run_config.yaml"), encoding="utf-8") as handle:
        base = yaml.safe_load(handle)
    mutations = {
        "unchanged": lambda c: None,
        "batch_100": lambda c: c["train"].__setitem__("batch_size", 100),
        "info_src_8": lambda c: c["general"].__setitem__("info_src", 8),
        "d_model_4100": lambda c: c["model"].__setitem__("d_model", 4100),
        "ctx_8190": lambda c: c["model"].__setitem__("context_len", 8190),
        "warmup_after_cosine": lambda c: c["train"]["learning_rate_scheduler"].__setitem__("t_w", 30000),
        "two_nodes": lambda c: c["general"].__setitem__("n_workers", 16),
        "vocab_odd": lambda c: c["data"].__setitem__("vocab_size", 32001),
        "layers_0": lambda c: c["model"].__setitem__("num_layers", 0),
        "heads_24": lambda c: c["model"].__setitem__("num_head", 24),
        "one_expert": lambda c: (c["model"].__setitem__("num_expert_per_node", 1),
                                 c["train"].__setitem__("fsdp_parallel_num", 1),
                                 c["train"].__setitem__("pipeline_parallel_stages", 8)),
        "cpu_device": lambda c: c["general"].__setitem__("device", "cpu"),
        "bool_batch": lambda c: c["train"].__setitem__("batch_size", True),
    }
    assert set(mutations) == set(ref["validation"])
    for name, mutate in mutations.items():
        config = copy.deepcopy(base)
        mutate(config)
        try:
            cfg.validate_config(config, allow_cpu=False)      # the reference's GPU-only rule
            verdict = "ok"
        except ValueError:
            verdict = "ValueError"
        assert verdict == ref["validation"][name], name
    # elementwise statements and AdamW
    torch.manual_seed(5)
    logits = torch.randn(7, 13) * 3
    assert torch.allclose(softmax(logits, -1), ref["softmax"], atol=1e-7)
    assert torch.allclose(silu(logits), ref["silu"], atol=1e-7)
    assert torch.allclose(cross_entropy(logits, torch.randint(0, 13, (7,))), ref["cross_entropy"], atol=1e-6)
    adam = ref["adamw"]
    p = torch.nn.Parameter(adam["start"].clone())
    opt = AdamW([p], lr=0.01, betas=(0.9, 0.95), weight_decay=0.1)
    for g in adam["grads"]:
        p.grad = g.clone()
        opt.step()
    assert torch.allclose(p.detach(), adam["end"], atol=1e-6)
    state = opt.state_dict()
    assert sorted(state["state"][0].keys()) == adam["state_keys"]
    assert sorted(k for k in state["param_groups"][0] if k != "params") == adam["group_keys"]
    assert state["param_groups"][0]["t"] == adam["t"]
    # checkpoint discovery on the tree the oracle prepared
    root = tmp_path / "checkpoint"
    found = {"any": latest_checkpoint(root, 2, 2), "first_run": latest_checkpoint(root, 2, 2, run="20240101000000000000"),
             "none": latest_checkpoint(root, 4, 2)}
    got = {k: (None if v is None else os.path.relpath(str(v), root)) for k, v in found.items()}
    assert got == ref["discovery"]
