"""Outputs of the reference's host-side utilities for a fixed set of inputs, saved for comparison with this
framework's own implementations.  Runs with only the reference (``baseline/_ref``) on ``sys.path``.
Arguments: reference root, output file, scratch directory."""
import copy
import os
import sys

ref_root, out_path, scratch = sys.argv[1], sys.argv[2], sys.argv[3]
here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != here]
sys.path.insert(0, ref_root)
os.chdir(ref_root)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import yaml  # noqa: E402

from distributed_parallel_training_pipelined import _latest_checkpoint  # noqa: E402
from implementation.nnfunctions import (cross_entropy, learning_rate_schedule_wrapper, silu,  # noqa: E402
                                        softmax)
from implementation.optimizer import AdamW  # noqa: E402
from implementation.startup import parallel_rank_groups, parallel_sizes, validate_config  # noqa: E402
from implementation.train_utils import get_batch  # noqa: E402

out = {}
# ---- data sampling: mock, random windows, serial windows, with a shared generator
tokens = (np.arange(5000, dtype=np.int64) * 7) % 1000
rng = np.random.default_rng(11)
batches = []
for kwargs in (dict(mock_data=True, vocab_size=1000), dict(), dict(start_idx=100), dict(serial_sampling=True, start_idx=64),
               dict(serial_sampling=True, start_idx=4900), dict(mock_data=True, vocab_size=17)):
    x, y = get_batch(None if kwargs.get("mock_data") else tokens, 6, 32, "cpu", rng=rng, **kwargs)
    batches.append((x.clone(), y.clone()))
out["batches"] = batches
out["rng_after"] = copy.deepcopy(rng.bit_generator.state)
# ---- learning-rate schedule
sched = learning_rate_schedule_wrapper(0.01, 0.0001, 50, 400)
out["lr"] = [sched(t) for t in (0, 1, 25, 49, 50, 51, 200, 399, 400, 401, 10000)]
# ---- rank layout
layouts = {}
for fsdp, ddp, pp, world, local in ((2, 1, 4, 8, 8), (4, 2, 1, 8, 8), (2, 2, 2, 8, 8), (1, 1, 1, 1, 1), (8, 1, 1, 8, 8),
                                    (2, 1, 2, 4, 4), (2, 1, 4, 8, 4), (4, 1, 2, 8, 2), (2, 2, 2, 16, 8)):
    train = {"fsdp_parallel_num": fsdp, "data_parallel_num": ddp, "pipeline_parallel_stages": pp}
    try:
        layouts[(fsdp, ddp, pp, world, local)] = parallel_rank_groups(train, world, local)
    except ValueError:
        layouts[(fsdp, ddp, pp, world, local)] = "ValueError"
out["layouts"] = layouts
out["legacy_sizes"] = parallel_sizes({"data_parallel_num": 4})
# ---- config validation: which mutations of the shipped configuration are rejected
with open(os.path.join(ref_root, "configs", "run_config.yaml"), encoding="utf-8") as handle:
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
    "one_expert": lambda c: (c["model"].__setitem__("num_expert_per_node", 1), c["train"].__setitem__("fsdp_parallel_num", 1),
                             c["train"].__setitem__("pipeline_parallel_stages", 8)),
    "cpu_device": lambda c: c["general"].__setitem__("device", "cpu"),
    "bool_batch": lambda c: c["train"].__setitem__("batch_size", True),
}
verdicts = {}
for name, mutate in mutations.items():
    config = copy.deepcopy(base)
    mutate(config)
    try:
        validate_config(config)
        verdicts[name] = "ok"
    except ValueError:
        verdicts[name] = "ValueError"
out["validation"] = verdicts
# ---- elementwise statements and one AdamW trajectory
torch.manual_seed(5)
logits = torch.randn(7, 13) * 3
out["softmax"] = softmax(logits, -1)
out["silu"] = silu(logits)
out["cross_entropy"] = cross_entropy(logits, torch.randint(0, 13, (7,)))
p = torch.nn.Parameter(torch.randn(5, 3))
start = p.detach().clone()
opt = AdamW([p], lr=0.01, betas=(0.9, 0.95), weight_decay=0.1)
grads = [torch.randn(5, 3) for _ in range(4)]
for g in grads:
    p.grad = g.clone()
    opt.step()
out["adamw"] = {"start": start, "grads": grads, "end": p.detach().clone(),
                "state_keys": sorted(opt.state_dict()["state"][0].keys()),
                "group_keys": sorted(k for k in opt.state_dict()["param_groups"][0] if k != "params"),
                "t": opt.state_dict()["param_groups"][0]["t"]}
# ---- checkpoint discovery on a prepared directory tree
root = os.path.join(scratch, "checkpoint")


def make(run, step, shards, committed=True):
    directory = os.path.join(root, run, str(step))
    os.makedirs(directory, exist_ok=True)
    for dp, pp_ in shards:
        open(os.path.join(directory, f"shaded_dp_{dp}_pp_{pp_}.ckpt"), "w").close()
    if committed:
        open(os.path.join(directory, "COMMITTED"), "w").close()


full = [(d, s) for d in range(2) for s in range(2)]
make("20240101000000000000", 50, full)
make("20240101000000000000", 100, full)
make("20240101000000000000", 150, full, committed=False)          # written but never committed
make("20240101000000000000", 200, full[:3])                       # committed marker but one shard missing
make("20240202000000000000", 50, full)
make("20240202000000000000", "tmp", full)                         # not a step number
found = {
    "any": _latest_checkpoint(root, 2, 2),
    "first_run": _latest_checkpoint(root, 2, 2, run="20240101000000000000"),
    "none": _latest_checkpoint(root, 4, 2),
}
out["discovery"] = {k: (None if v is None else os.path.relpath(str(v), root)) for k, v in found.items()}
torch.save(out, out_path)
