"""Host-side safety rules, checked without a GPU: the activation budget, the refusal of self-kill fault injection
while buffers are bound to an NVLink multicast object, the watchdog's release hook, and the commit vote that counts a
device-side failure as "not saved"."""
from concurrent.futures import Future

import pytest
import torch

from b200moe.parallel.memory import ActivationBudget, fixed_bytes_per_block, stage_activation_budget
from b200moe.utils import chaos
from b200moe.utils.checkpoint import verify_pending_checkpoints
from b200moe.utils.watchdog import StatusWatchdog


def test_budget_keeps_optional_tensors_only_while_they_fit_beside_the_calls_to_come():
    budget = ActivationBudget(total_bytes=100, max_live_calls=4, routed_bytes_per_call=10)
    # call 1: 10 routed + 40 optional + reserve for 3 more calls (30) = 80 <= 100 -> kept
    assert budget.enter(10, 40) is True and budget.used == 50
    # call 2: 50 + 10 + 40 + reserve 20 = 120 > 100 -> rebuilt in the backward pass, only the routed part counts
    assert budget.enter(10, 40) is False and budget.used == 60
    # a skewed call (3x the balanced rows) is still accounted for
    assert budget.enter(25, 5) is True and budget.used == 90
    budget.leave(25, 5, True)
    budget.leave(10, 40, False)
    budget.leave(10, 40, True)
    assert budget.used == 0 and budget.live_calls == 0
    assert budget.summary() == {"budget_gib": 0.0, "kept": 2, "recomputed": 1}
    budget.enter(10, 40)
    budget.reset()
    assert budget.used == 0 and budget.live_calls == 0


def test_budget_cross_checks_its_plan_against_what_the_device_really_has_left():
    room = {"bytes": 1000}
    budget = ActivationBudget(total_bytes=10_000, max_live_calls=3, fixed_bytes_per_call=100, floor_bytes=50,
                              probe=lambda: room["bytes"], cold_floor_bytes=400, cold_calls=1)
    # first call (cold): 1000 - 300 optional must cover 2 calls x 100 + floor 50 + cold 400 = 650 -> kept
    assert budget.enter(0, 300) is True
    room["bytes"] = 500
    # second call (warm): 500 - 300 = 200 >= 1 x 100 + 50 -> kept;  with 420 optional it would not be
    assert budget.enter(0, 420) is False
    assert budget.enter(0, 300) is True
    budget = ActivationBudget(total_bytes=10_000, max_live_calls=3, fixed_bytes_per_call=100, floor_bytes=50,
                              probe=lambda: 900, cold_floor_bytes=400, cold_calls=1)
    assert budget.enter(0, 300) is False        # the plan says yes, the cold device says no: 600 < 650


def test_stage_budget_shrinks_with_the_microbatches_a_stage_keeps_alive():
    common = dict(tokens_per_microbatch=16384, d_model=4096, d_ff=14336, num_heads=32, experts_total=8, ep=2,
                  blocks=8, pp=4, microbatches=32, vocab=32000, free_bytes=95 << 30)
    first = stage_activation_budget(stage=0, **common)
    last = stage_activation_budget(stage=3, **common)
    assert first.max_live_calls == 32 and last.max_live_calls == 8
    assert first.total < last.total          # stage 0 keeps four microbatches alive, the last stage one
    per_block = fixed_bytes_per_block(16384, 4096, 32, 8)
    assert 0.9 * 2 ** 30 < per_block < 1.3 * 2 ** 30
    # nothing left: the budget is empty, never negative, and every call rebuilds
    empty = stage_activation_budget(stage=0, **{**common, "free_bytes": 1 << 30})
    assert empty.total == 0 and empty.enter(1, 1) is False


def test_random_kill_is_refused_while_a_buffer_is_bound_to_multicast():
    config = {"random_kill": {"enabled": True, "chance": 0.0}, "random_delay": {"enabled": True, "delay_time": 0,
                                                                                "chance": 0.0}, "wired": True}
    with pytest.raises(ValueError, match="multicast"):
        chaos.ChaosEnginnerTrigger(config, multicast_bound=lambda: True)
    assert len(chaos.ChaosEnginnerTrigger(config, multicast_bound=lambda: False)) == 2
    config["random_kill"]["enabled"] = False
    assert len(chaos.ChaosEnginnerTrigger(config, multicast_bound=lambda: True)) == 1


def test_comm_reports_multicast_and_releases_its_buffers():
    from b200moe.comm import Comm

    class FakeBuffer:
        def __init__(self, mc):
            self.mc_ptr, self.handle, self.tensor = mc, object(), object()

    comm = Comm.__new__(Comm)
    plain, bound = FakeBuffer(0), FakeBuffer(0xdead0000)
    class FakeLink:
        def __init__(self, *buffers):
            self.held = list(buffers)

        def buffers(self):
            return self.held

    ring = FakeBuffer(0)
    comm._symm, comm._ar_stage, comm._ep, comm._pp = {1: plain}, {}, {}, {"link": FakeLink(ring), "none": None}
    comm.fsdp = comm.ddp = None
    comm.device = torch.device("cpu")
    assert comm.any_multicast() is False
    comm._ar_stage["f32"] = bound
    assert comm.any_multicast() is True
    comm.release()
    assert comm.any_multicast() is False and bound.tensor is None and bound.handle is None and not comm._symm
    assert ring.tensor is None and ring.handle is None and not comm._pp


def test_watchdog_runs_the_release_hook_before_it_ends_the_process():
    order = []
    dog = StatusWatchdog(lambda: 105, interval_s=0.01, grace_s=0.05, exit_process=lambda code: order.append(code),
                         log=lambda *a, **k: None, before_exit=lambda: order.append("released"))
    dog.start()
    dog._thread.join(timeout=5)
    assert order == ["released", 75]


def test_a_rank_that_saw_a_device_failure_votes_against_the_commit(tmp_path, capsys):
    done = Future()
    done.set_result(None)
    for healthy, committed in ((lambda: True, True), (lambda: False, False), (None, True)):
        directory = tmp_path / f"step_{committed}_{healthy is None}"
        directory.mkdir()
        pending = [(5, str(directory), done)]
        verify_pending_checkpoints(pending, 10, 0, 0, torch.device("cpu"), healthy=healthy)
        assert not pending and (directory / "COMMITTED").exists() is committed
    assert "votes against" in capsys.readouterr().out
