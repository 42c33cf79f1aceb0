"""Launchers, tools, chaos hooks and the side car, all on CPU with fakes."""
import os
import random

import pytest
import yaml

import modal_wrapper
import run_experiment
from b200moe.utils import chaos
from b200moe.utils.metrics import MetricsSink, flops_per_token, mfu
from rl.worker_node.prompt_loader import DatabasePromptLoader, PromptLoader, read_data_source
from rl.worker_node.start_vllm import build_command, find_vllm_servers, kill_existing_vllm_server, start_server


def test_flops_per_token_matches_published_figure():
    fpt = flops_per_token(4096, 14336, 32, 8, 32000, 32, 8192)
    assert abs(fpt / 1e9 - 84.01) < 0.01
    assert abs(mfu(75076, fpt, 8) - 0.350) < 0.001


def test_metrics_sink(tmp_path):
    sink = MetricsSink(tmp_path / "m.jsonl")
    sink.write(iteration=1, tokens_per_s=10.0)
    assert (tmp_path / "m.jsonl").read_text().count("\n") == 1 and sink.records[0]["iteration"] == 1


def test_torchrun_and_nsys_commands():
    config = {"general": {"n_workers": 8, "gpu_per_node": 8}, "recovery": {"max_restarts": 2},
              "profile": {"enabled": True, "output_dir": "/p", "nsight_trace": "cuda-sw,nvtx"}}
    cmd = modal_wrapper.torchrun_command(config, "c.yaml")
    assert "--nproc-per-node=8" in cmd and "--max-restarts=2" in cmd and "--monitor-interval=1" in cmd
    assert cmd[-4:] == ["--module", "distributed_parallel_training_pipelined", "--config-path", "c.yaml"]
    prefix = modal_wrapper.nsys_prefix(config, "run")
    assert prefix[:2] == ["nsys", "profile"] and "--trace=cuda-sw,nvtx" in prefix
    assert modal_wrapper.nsys_prefix({"profile": {"enabled": False}}, "run") == []
    assert modal_wrapper.nccl_environment()["NCCL_IB_DISABLE"] == "1"


def test_experiment_config_validation(tmp_path):
    good = {"experiment": {"device": "cuda:0", "dtype": "bfloat16", "input_shapes": [[2, 8, 16]], "warmup": 0,
                           "iterations": 1, "mode": "training"}}
    path = tmp_path / "e.yaml"
    path.write_text(yaml.safe_dump(good))
    assert run_experiment.load_experiment_config(path)["experiment"]["mode"] == "training"
    for key, value in [("dtype", "int8"), ("mode", "x"), ("iterations", 0), ("input_shapes", [[0]]), ("warmup", -1)]:
        bad = {"experiment": {**good["experiment"], key: value}}
        path.write_text(yaml.safe_dump(bad))
        with pytest.raises(ValueError):
            run_experiment.load_experiment_config(path)
    with pytest.raises(ValueError, match="CUDA"):
        run_experiment.cuda_device("cpu")


def test_make_module_step_runs_on_cpu():
    import torch
    from b200moe.models import ModuleStack
    from b200moe.utils.profiling import make_module_step
    module = ModuleStack(16, 16, d_ff=32)
    x = torch.randn(2, 3, 16)
    step = make_module_step(module, [x], "training")
    assert step().dim() == 0 and x.grad is None and all(p.grad is None for p in module.parameters())
    assert make_module_step(module, [x], "evaluation")().shape == (2, 3, 16)


def test_chaos_triggers_and_leak_cap(monkeypatch):
    slept = []
    monkeypatch.setattr(chaos.time, "sleep", slept.append)
    trig = chaos.ChaosEnginnerTrigger({"random_delay": {"enabled": True, "delay_time": 3, "chance": 1.0},
                                       "random_kill": {"enabled": False, "chance": 1.0},
                                       "random_gpu_memory_leak": {"enabled": True, "size_mb": 1, "chance": 1.0,
                                                                  "max_total_mb": 2}})
    assert len(trig) == 2
    assert trig.trigger() == 2 and slept == [3]
    trig.trigger()
    assert trig.trigger() == 1          # the leak stopped at its cap
    assert chaos.release_leaks() == 2 and chaos.release_leaks() == 0
    with pytest.raises(ValueError, match="Unknown chaos"):
        chaos.ChaosEnginnerTrigger({"nope": {"enabled": True}})
    random.seed(0)
    assert chaos.random_delay(1, chance=0.0) is False


def test_chaos_kill_sends_sigkill_to_self(monkeypatch):
    sent = []
    monkeypatch.setattr(chaos.os, "kill", lambda pid, sig: sent.append((pid, sig)))
    assert chaos.random_kill(chance=1.0) is True
    assert sent == [(chaos.os.getpid(), chaos.signal.SIGKILL)]


def test_prompt_loader_with_fake_connection(tmp_path):
    class Cursor:
        def __init__(self, rows):
            self.rows, self.seen = rows, []

        def __enter__(self):
            return self

        def __exit__(self, *exc):
            return False

        def execute(self, query):
            self.seen.append(query)

        def fetchone(self):
            return self.rows.pop(0) if self.rows else None

    class Conn:
        def __init__(self, conninfo):
            self.conninfo, self.closed = conninfo, False
            self.cur = Cursor([{"id": 7, "prompt_text": "hello", "priority": 2}])

        def cursor(self):
            return self.cur

        def close(self):
            self.closed = True

    good = {"database": {"host": "h", "port": 1, "dbname": "d", "user": "u", "password": "p", "sslmode": "prefer"},
            "prompt_query": "SELECT id, prompt_text, priority FROM prompts LIMIT 1;"}
    path = tmp_path / "ds.yaml"
    path.write_text(yaml.safe_dump(good, sort_keys=False))
    made = []
    with DatabasePromptLoader(path, connect=lambda info: made.append(Conn(info)) or made[-1]) as loader:
        assert isinstance(loader, PromptLoader) and PromptLoader().samplePrompt() is None
        assert loader.samplePrompt() == {"id": 7, "prompt_text": "hello", "priority": 2}
        assert made[0].conninfo == "host=h port=1 dbname=d user=u password=p sslmode=prefer"
        assert made[0].cur.seen == [good["prompt_query"]]
        assert loader.samplePrompt() is None
        made[0].closed = True                              # the server dropped us: the next call reconnects
        assert loader.samplePrompt() == {"id": 7, "prompt_text": "hello", "priority": 2} and len(made) == 2
    assert made[1].closed
    for broken, error in (({**good, "database": {"host": "h"}}, ValueError), ({**good, "prompt_query": " "}, ValueError),
                          ({"prompt_query": "x"}, TypeError), (["not", "a", "mapping"], TypeError)):
        path.write_text(yaml.safe_dump(broken))
        with pytest.raises(error):
            DatabasePromptLoader(path)
    with pytest.raises(FileNotFoundError):
        DatabasePromptLoader(tmp_path / "absent.yaml")
    # the example file of this repository is a valid data source
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    example = read_data_source(os.path.join(root, "configs", "data_source.example.yaml"))
    assert "prompt_text" in example["prompt_query"]


def test_vllm_launcher_pins_gpu_and_ends_only_the_servers_on_its_port():
    calls = []
    start_server("m", "0.0.0.0", 9000, 3, seed=5, load_format="dummy", logging_level="DEBUG",
                 popen=lambda cmd, env, start_new_session: calls.append((cmd, env, start_new_session)) or "proc")
    cmd, env, own_session = calls[0]
    assert cmd[:3] == ["vllm", "serve", "m"] and own_session is True
    for flag, value in (("--host", "0.0.0.0"), ("--port", "9000"), ("--seed", "5"), ("--load-format", "dummy"),
                        ("--tensor-parallel-size", "1"), ("--gpu-memory-utilization", "0.9"),
                        ("--weight-transfer-config", '{"backend": "nccl"}')):
        assert cmd[cmd.index(flag) + 1] == value
    assert "--enable-prefix-caching" in cmd
    assert (env["CUDA_VISIBLE_DEVICES"], env["VLLM_SERVER_DEV_MODE"], env["VLLM_LOGGING_LEVEL"]) == ("3", "1", "DEBUG")
    assert "--max-model-len" in build_command("m", max_model_len=128)
    table = [(11, ["/usr/bin/python", "/opt/bin/vllm", "serve", "m", "--port", "9000"]),
             (12, ["vllm", "serve", "m", "--port", "9001"]),
             (13, ["vllm", "serve", "m", "--host", "x", "--port=9000"]),
             (14, ["grep", "vllm serve m --port 9000"]),
             (os.getpid(), ["vllm", "serve", "m", "--port", "9000"])]
    assert find_vllm_servers(9000, table) == [11, 13]
    sent, naps = [], []
    assert kill_existing_vllm_server(9000, table, send=lambda pid, sig: sent.append((pid, int(sig))),
                                     sleep=naps.append) == [11, 13]
    assert sent == [(11, 15), (13, 15), (11, 9), (13, 9)] and naps == [2.0]
    assert kill_existing_vllm_server(7, table, send=lambda *a: sent.append(a), sleep=naps.append) == [] and len(sent) == 4


def test_helm_values_hold_a_valid_run_config():
    """The chart's values use the reference chart's keys, its run configuration passes this framework's checks with
    the topology the helper derives, and every ``.Values.*`` path a template reads exists in values.yaml."""
    import re
    from b200moe import config as cfg
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    chart = os.path.join(root, "kubernetes", "chart")
    with open(os.path.join(chart, "values.yaml")) as f:
        values = yaml.safe_load(f)
    for key in ("image", "numNodes", "gpusPerNode", "runtimeRef", "resourcesPerNode", "memlock", "failurePolicy",
                "sharedMemory", "ncclDebug", "runConfig"):
        assert key in values, key
    assert set(values["runtimeRef"]) == {"name", "kind", "apiGroup"} and set(values["memlock"]) == {"enabled", "createRuntime"}
    run = values["runConfig"]
    run["general"]["n_workers"] = values["numNodes"] * values["gpusPerNode"]
    run["general"]["gpu_per_node"] = values["gpusPerNode"]
    cfg.validate_config(run)
    for name in os.listdir(os.path.join(chart, "templates")):
        with open(os.path.join(chart, "templates", name)) as f:
            text = f.read()
        assert text.count("{{") == text.count("}}"), name
        actions = re.findall(r"\{\{-?\s*(.*?)\s*-?\}\}", re.sub(r"\{\{-?\s*/\*.*?\*/\s*-?\}\}", "", text, flags=re.S),
                             flags=re.S)
        opened = sum(1 for a in actions if re.match(r"(if|range|with|define)\b", a))
        assert opened == sum(1 for a in actions if re.match(r"end\b", a)), name
        for path in set(re.findall(r"\.Values\.([A-Za-z_.]+)", text)):
            node = values
            for part in path.rstrip(".").split("."):
                assert isinstance(node, dict) and part in node, f"{name}: .Values.{path}"
                node = node[part]


def test_checked_build_compiles_and_exports_its_readers():
    """``B200MOE_DEBUG=1 python -m b200moe.build`` gives a second library with the debug-record readers."""
    import ctypes
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    subprocess.run([sys.executable, "-m", "b200moe.build"], check=True, cwd=root,
                   env={**os.environ, "B200MOE_DEBUG": "1"})
    path = os.path.join(root, "b200moe", "_C", "debug", "libb200moe_debug.so")
    assert os.path.exists(path)
    try:
        lib = ctypes.CDLL(path)
    except OSError as error:          # no CUDA runtime on this machine: the build itself is what was checked
        pytest.skip(str(error))
    assert hasattr(lib, "b2_moe_debug_read") and hasattr(lib, "b2_comm_debug_read") and hasattr(lib, "b2_gemm_nt")


def test_status_watchdog_reports_to_the_loop_and_exits_when_the_loop_is_stuck():
    import threading
    import time
    from b200moe.utils.watchdog import WATCHDOG_EXIT_CODE, StatusWatchdog
    # healthy: nothing happens
    dog = StatusWatchdog(lambda: 0, interval_s=0.01, grace_s=0.2, exit_process=lambda code: None, log=lambda *a, **k: None).start()
    time.sleep(0.1)
    dog.raise_if_failed()
    dog.stop()
    # a timed-out device wait is picked up by the loop: the process is not killed
    exits, seen = [], []
    code = {"value": 0}
    dog = StatusWatchdog(lambda: code["value"], interval_s=0.01, grace_s=1.0, exit_process=exits.append,
                         on_failure=seen.append, log=lambda *a, **k: None).start()
    code["value"] = 105
    deadline = time.monotonic() + 2.0
    while not dog.code and time.monotonic() < deadline:
        time.sleep(0.01)
    with pytest.raises(RuntimeError, match="105"):
        dog.raise_if_failed()
    time.sleep(0.2)
    dog.stop()
    assert seen == [105] and exits == []
    # the loop never comes back (stuck in a host-side wait): the watchdog ends the process for the launcher
    gone = threading.Event()
    dog = StatusWatchdog(lambda: 301, interval_s=0.01, grace_s=0.1,
                         exit_process=lambda c: (exits.append(c), gone.set()), log=lambda *a, **k: None).start()
    assert gone.wait(3.0)
    dog.stop()
    assert exits == [WATCHDOG_EXIT_CODE]
    # a reader that raises (lost context) counts as a failure too
    def broken():
        raise OSError("context lost")
    dog = StatusWatchdog(broken, interval_s=0.01, grace_s=5.0, exit_process=exits.append, log=lambda *a, **k: None).start()
    deadline = time.monotonic() + 2.0
    while not dog.code and time.monotonic() < deadline:
        time.sleep(0.01)
    with pytest.raises(RuntimeError):
        dog.raise_if_failed()
    dog.stop()


def test_allgather_gemm_schedule_on_the_host():
    """The native host code that orders the column blocks of the all-gather + GEMM kernel: every block exactly once,
    the blocks whose weight rows all belong to this rank first, peers' blocks rotated so that ranks start on
    different peers; row ownership follows the per-segment sharding (a fused q/k/v weight has three segments)."""
    from b200moe.ops import native
    try:
        native.require()
    except RuntimeError as error:
        pytest.skip(str(error))
    cases = [([6144], 2), ([4096, 1024, 1024], 2), ([4096, 1024, 1024], 4), ([1984], 2), ([32000], 8),
             ([1024, 512, 512, 384], 4), ([256], 2), ([512], 1)]
    for segments, world in cases:
        total = sum(segments)
        blocks = (total + 255) // 256
        want_owner = []
        for rows in segments:
            want_owner += [r // (rows // world) for r in range(rows)]
        firsts = []
        for rank in range(world):
            order, n_local, owner = native.ag_gemm_plan(segments, world, rank)
            assert owner == want_owner
            assert sorted(order) == list(range(blocks))
            local = [b for b in range(blocks) if all(o == rank for o in want_owner[b * 256:(b + 1) * 256])]
            assert order[:n_local] == local
            rest = order[n_local:]
            if rest:
                # the peers' blocks keep their cyclic order, starting after this rank's last own block
                base = [b for b in range(blocks) if b not in local]
                shift = base.index(rest[0])
                assert rest == base[shift:] + base[:shift]
                assert not local or rest[0] > local[-1] or all(b < local[-1] for b in base)
                firsts.append(rest[0])
        if world > 1 and blocks >= 2 * world and len(segments) == 1:
            assert len(set(firsts)) == world          # every rank starts copying from a different block
    for bad in (([100], 3), ([0], 2), ([256 * 200], 2)):
        with pytest.raises(ValueError):
            native.ag_gemm_plan(bad[0], bad[1], 0)


def test_modal_launcher_nodes_rendezvous_and_profiler(tmp_path, monkeypatch):
    for name in ("MASTER_ADDR", "MASTER_PORT", "NCCL_HOSTID"):
        monkeypatch.delenv(name, raising=False)
    two_nodes = {"general": {"n_workers": 16, "gpu_per_node": 8}, "recovery": {"max_restarts": 1}}
    # the reference's builder and its checks
    with pytest.raises(ValueError, match="MASTER_ADDR"):
        modal_wrapper._build_torchrun_command("c.json", 1, 16, 8)
    for bad in (dict(cluster_rank=2), dict(world_size=12), dict(max_restarts=-1), dict(max_restarts=True)):
        args = {"config_path": "c.json", "cluster_rank": 0, "world_size": 16, "gpu_per_node": 8, **bad}
        with pytest.raises(ValueError):
            modal_wrapper._build_torchrun_command(**args)
    cmd = modal_wrapper.torchrun_command(two_nodes, "c.yaml", 1, "fd00::7", 29511, "job")
    assert "--nnodes=2" in cmd and "--node-rank=1" in cmd and "--rdzv-endpoint=[fd00::7]:29511" in cmd
    assert "--rdzv-id=job" in cmd and "MASTER_ADDR" not in os.environ
    # one node of two: rendezvous on the first container, one host id per node, IPv6 sockets for an IPv6 cluster
    calls = []

    def runner(command, check, env, cwd):
        with open(command[command.index("--config-path") + 1], encoding="utf-8") as handle:
            seen = yaml.safe_load(handle)
        calls.append((command, env, seen))
    modal_wrapper.run_node(two_nodes, 1, ["fd00::7", "fd00::8"], "cl9", runner=runner)
    command, env, seen = calls[-1]
    assert seen == two_nodes and "--master-addr=fd00::7" in command and "--max-restarts=1" in command
    assert env["NCCL_HOSTID"] == "cl9-node-1" and env["NCCL_SOCKET_FAMILY"] == "AF_INET6" and "--rdzv-id=cl9" in command
    with pytest.raises(ValueError, match="addresses"):
        modal_wrapper.run_node(two_nodes, 0, None, runner=runner)
    # a single node meets itself on loopback whatever the cluster says
    one = {"general": {"n_workers": 8, "gpu_per_node": 8},
           "profile": {"enabled": True, "output_dir": str(tmp_path), "nsight_trace": "cuda-sw,nvtx"}}
    monkeypatch.setattr(modal_wrapper.shutil, "which", lambda name: None)
    with pytest.raises(RuntimeError, match="nsys"):
        modal_wrapper.run_node(one, 0, ["10.0.0.5"], runner=runner)
    monkeypatch.setattr(modal_wrapper.shutil, "which", lambda name: "/opt/nsys")
    with pytest.raises(RuntimeError, match="did not write"):
        modal_wrapper.run_node(one, 0, ["10.0.0.5"], runner=runner)
    committed = []

    def writes_report(command, check, env, cwd):
        output = [c for c in command if c.startswith("--output=")][0].split("=", 1)[1]
        open(output + ".nsys-rep", "w").close()
        calls.append((command, env, None))
    modal_wrapper.run_node(one, 0, ["10.0.0.5"], runner=writes_report, commit_profile=lambda: committed.append(1))
    command, env, _ = calls[-1]
    assert command[:2] == ["/opt/nsys", "profile"] and "--kill=none" in command and "--wait=all" in command
    assert "--master-addr=127.0.0.1" in command and env["MASTER_ADDR"] == "127.0.0.1" and committed == [1]
    assert command[command.index("--module") + 1] == "distributed_parallel_training_pipelined"


def test_packaging_lists_every_importable_top_level_name():
    """``pip install .`` must carry the package, the reference's import names and entry modules, the run
    configuration, the SQL of the side car and the CUDA sources."""
    import tomllib
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, "pyproject.toml"), "rb") as handle:
        meta = tomllib.load(handle)
    tool = meta["tool"]["setuptools"]
    for module in tool["py-modules"]:
        assert os.path.isfile(os.path.join(root, module + ".py")), module
    patterns = tool["packages"]["find"]["include"]
    for package in ("b200moe", "implementation", "pipeline", "configs", "rl"):
        assert os.path.isfile(os.path.join(root, package, "__init__.py")), package
        assert any(p.rstrip("*") == package for p in patterns), package
    assert "csrc/*.cu" in tool["package-data"]["b200moe"] and "*.yaml" in tool["package-data"]["configs"]
    assert meta["project"]["name"] == "b200moe" and any(d.startswith("torch") for d in meta["project"]["dependencies"])
