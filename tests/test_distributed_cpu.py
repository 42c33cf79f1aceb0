"""Multi-process plumbing on CPU (gloo): FSDP × EP × PP gradients against a
single-process oracle, the full worker with checkpoint save/commit/resume, and
recovery from a host-side failure."""
import os
import re

import pytest
import torch
import torch.multiprocessing as mp

import _workers as W


def _spawn(fn, world, args):
    mp.spawn(fn, args=args, nprocs=world, join=True)


@pytest.mark.parametrize("world,pp", [(2, 1), (4, 2)])
def test_gradients_match_single_process(tmp_path, free_port, world, pp):
    _spawn(W.run_grad_equivalence, world, (world, free_port, str(tmp_path), pp))
    outs = [torch.load(tmp_path / f"grads_{r}.pt") for r in range(world)]
    ref_grads, ref_loss = outs[0]["ref_grads"], outs[0]["ref_loss"]
    fsdp, L = world // pp, 2
    last = [o for o in outs if o["stage"] == pp - 1]
    assert abs(sum(o["loss"] for o in last) / len(last) - ref_loss) < 1e-5
    checked = 0
    for o in outs:
        stage, shard = o["stage"], o["shard"]
        for name, g in o["grads"].items():
            key = name
            m = re.match(r"module\.layers\.(\d+)\.(.*)", name)
            if m:
                key = f"module.layers.{int(m.group(1)) + stage * L}.{m.group(2)}"
            want = ref_grads[key]
            if ".experts." in name:
                e = want.shape[0] // fsdp
                want = want[shard * e:(shard + 1) * e] * fsdp     # expert grads are summed over sources
            elif g.shape != want.shape:
                rows = want.shape[0] // fsdp
                want = want[shard * rows:(shard + 1) * rows]
            assert torch.allclose(g, want, atol=2e-5, rtol=1e-4), name
            checked += 1
    assert checked > 20


def _losses(text):
    return [float(v) for v in re.findall(r"Loss from last 1 iterations is (?:tensor\()?([0-9.]+)", text)]


@pytest.mark.parametrize("world,fsdp,ddp,pp", [(2, 2, 1, 1), (4, 2, 1, 2), (4, 2, 2, 1)])
def test_worker_checkpoint_commit_and_resume(tmp_path, free_port, world, fsdp, ddp, pp):
    folder = tmp_path / "run"
    cfg = W.tiny_config(world, fsdp, ddp, pp, folder, target=10, save=5, batch=4 * ddp)
    res = tmp_path / "res1"
    res.mkdir()
    _spawn(W.run_train, world, (world, free_port, cfg, str(res)))
    out0 = (res / "out_0.txt").read_text()
    assert "Checkpoint at iteration 5 committed" in out0 and "Checkpoint at iteration 10 committed" in out0
    runs = list((folder / "checkpoint").iterdir())
    assert len(runs) == 1
    for step in ("5", "10"):
        files = sorted(p.name for p in (runs[0] / step).iterdir())
        want = sorted([f"shaded_dp_{d}_pp_{p}.ckpt" for d in range(fsdp * ddp) for p in range(pp)] + ["COMMITTED"])
        assert files == want
    last_rank = world - 1
    first = _losses((res / f"out_{last_rank}.txt").read_text())
    assert len(first) == 10 and all(6.5 < v < 7.5 for v in first)
    shard = torch.load(runs[0] / "10" / "shaded_dp_0_pp_0.ckpt", weights_only=False)
    assert set(shard) == {"model.state_dict", "optimizer.state_dict", "iteration", "rng"}
    assert shard["iteration"] == 10 and set(shard["rng"]) == {"data", "torch", "cuda", "python"}
    keys = shard["model.state_dict"].keys()
    assert "module.token_embeddings.weight" in keys and "module.layers.0.ffn.experts.w1" in keys
    assert shard["model.state_dict"]["module.layers.0.attn.q_proj.weight"].shape == (128 // fsdp, 128)
    # resume: newest committed step is discovered, run id is reused, training continues to 12
    cfg2 = W.tiny_config(world, fsdp, ddp, pp, folder, target=12, save=50, batch=4 * ddp)
    res2 = tmp_path / "res2"
    res2.mkdir()
    _spawn(W.run_train, world, (world, free_port + 1 if free_port < 65000 else free_port - 1, cfg2, str(res2)))
    text = (res2 / "out_0.txt").read_text()
    assert "loaded checkpoint at 10 iterations" in text and runs[0].name in text
    resumed = _losses((res2 / f"out_{last_rank}.txt").read_text())
    assert len(resumed) == 2


def test_resume_reproduces_uninterrupted_run(tmp_path, free_port):
    """Steps 6-8 after restoring step 5 equal steps 6-8 of a run that never stopped."""
    a, b = tmp_path / "a", tmp_path / "b"
    ra, rb, rc = tmp_path / "ra", tmp_path / "rb", tmp_path / "rc"
    for d in (ra, rb, rc):
        d.mkdir()
    _spawn(W.run_train, 2, (2, free_port, W.tiny_config(2, 2, 1, 1, a, target=8, save=100), str(ra)))
    _spawn(W.run_train, 2, (2, free_port, W.tiny_config(2, 2, 1, 1, b, target=5, save=5), str(rb)))
    _spawn(W.run_train, 2, (2, free_port, W.tiny_config(2, 2, 1, 1, b, target=8, save=100), str(rc)))
    straight = _losses((ra / "out_1.txt").read_text())
    resumed = _losses((rc / "out_1.txt").read_text())
    assert len(straight) == 8 and len(resumed) == 3
    assert resumed == pytest.approx(straight[5:], abs=1e-6)


def test_host_failure_then_restart_resumes_from_last_commit(tmp_path, free_port):
    folder = tmp_path / "run"
    res = tmp_path / "res"
    res.mkdir()
    cfg = W.tiny_config(2, 2, 1, 1, folder, target=12, save=3)
    cfg["recovery"]["collective_timeout_seconds"] = 10
    with pytest.raises(Exception):
        _spawn(W.run_train, 2, (2, free_port, cfg, str(res), (1, 9)))
    assert "injected host failure" in (res / "err_1.txt").read_text()
    runs = list((folder / "checkpoint").iterdir())
    committed = sorted(int(p.parent.name) for p in runs[0].glob("*/COMMITTED"))
    assert committed == [3]                      # step 6 was saved but never committed (commits lag 5 iterations)
    os.environ["TORCHELASTIC_RESTART_COUNT"] = "1"
    try:
        res2 = tmp_path / "res2"
        res2.mkdir()
        _spawn(W.run_train, 2, (2, free_port, cfg, str(res2)))
    finally:
        os.environ.pop("TORCHELASTIC_RESTART_COUNT")
    text = (res2 / "out_0.txt").read_text()
    assert f"loaded checkpoint at {committed[-1]} iterations" in text
    assert "FINAL 12" in text


@pytest.mark.parametrize("world,microbatches,act_slots", [(4, 8, 4), (2, 6, 2), (3, 7, 2)])
def test_peer_link_schedule_matches_nccl_link(tmp_path, free_port, world, microbatches, act_slots):
    """The pipeline's peer-memory link (message numbers, landing rings, acknowledgements) under the real 1F1B
    scheduler, with a host transport in place of the kernels: bit-identical training to the send/recv link, no slot
    written while in use, no deadlock — also with the smallest activation ring the schedule allows (``pp − 1`` slots), where senders wait."""
    _spawn(W.run_peer_link_schedule, world, (world, free_port, str(tmp_path), microbatches, 3, act_slots))
    outs = [torch.load(tmp_path / f"link_{r}.pt") for r in range(world)]
    for o in outs:
        assert o["nccl"]["losses"] == o["peer"]["losses"]
        for key, value in o["nccl"]["weights"].items():
            assert torch.equal(value, o["peer"]["weights"][key]), key
    assert any(o["stage"] == world - 1 and o["peer"]["losses"][0] > 0 for o in outs)
    if act_slots >= world:
        # a ring of ``pp`` activation slots never makes a sender wait for room under 1F1B
        assert all(o["peer"]["waits_for_room"] == 0 or o["stage"] > 0 for o in outs)


def test_gather_and_free_hooks_on_hand_sharded_modules(tmp_path, free_port):
    _spawn(W.run_weight_hooks, 2, (2, free_port, str(tmp_path)))
    assert all((tmp_path / f"hooks_ok_{r}").exists() for r in range(2))


@pytest.mark.parametrize("world", [1, 2])
def test_two_step_dispatch_and_combine_match_the_layer(tmp_path, free_port, world):
    _spawn(W.run_moe_two_step, world, (world, free_port, str(tmp_path)))
    assert all((tmp_path / f"two_step_ok_{r}").exists() for r in range(world))
