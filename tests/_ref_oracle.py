"""Runs the unmodified reference package (installed under ``baseline/_ref``) on
CPU/gloo for a tiny configuration and saves its initial state, losses and
first-step gradients.  Executed as a separate process with only the reference on
``sys.path`` so its module names do not collide with this repository's."""
import os
import sys

ref_root, out_path = sys.argv[1], sys.argv[2]
sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != os.path.dirname(os.path.dirname(os.path.abspath(__file__)))]
sys.path.insert(0, ref_root)
os.chdir(ref_root)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
os.environ.setdefault("MASTER_PORT", sys.argv[3])
dist.init_process_group("gloo", rank=0, world_size=1)
from implementation.distributed.ddp_modules import FSDPWrapperPipelined  # noqa: E402
from implementation.layers import TransformerLMPipelined  # noqa: E402
from implementation.nnfunctions import cross_entropy  # noqa: E402
from implementation.optimizer import AdamW  # noqa: E402
from implementation.train_utils import get_batch  # noqa: E402
from pipeline import pipelined_train_overlap  # noqa: E402

mode = sys.argv[4] if len(sys.argv) > 4 else "train"
torch.manual_seed(0)
group = dist.new_group([0])
model = TransformerLMPipelined(1024, 256, 128, 2, 4, 0, 1, num_expert_per_node=4, d_ff=256, dp_group=group,
                               moe_compute_dtype=torch.bfloat16)
init = {k: v.clone() for k, v in model.state_dict().items()}
wrapped = FSDPWrapperPipelined(model, FSDP_communication_group=group, compute_dtype=torch.float32,
                               moe_compute_dtype=torch.bfloat16)
optimizer = AdamW(wrapped.parameters(), lr=3e-4, betas=(0.9, 0.999), weight_decay=0.01)
rng = np.random.default_rng(0)


def one_step():
    x, y = get_batch(None, 4, 256, "cpu", rng=rng, vocab_size=1024, mock_data=True)
    return float(pipelined_train_overlap(wrapped, optimizer, x, y, [4, 256, 128], 2, 0, cross_entropy,
                                         dtype=torch.float32, device=torch.device("cpu"), pp_group=group,
                                         dp_group=group))


if mode == "train":
    # six steps, a checkpoint written by the reference's own (synchronous) writer, then a seventh step
    from implementation.train_utils import save_checkpoint  # noqa: E402
    losses, grads = [], None
    for step in range(6):
        losses.append(one_step())
        if grads is None:
            grads = {n: p.grad.detach().float().clone() for n, p in wrapped.named_parameters() if p.grad is not None}
    save_checkpoint(wrapped, optimizer, 6, out_path + ".ckpt")
    torch.save({"init": init, "losses": losses, "grads": grads, "loss7": one_step()}, out_path)
elif mode == "aux":
    # two steps with the router auxiliary loss switched on and the metrics dictionary returned
    rows = []
    for _ in range(2):
        x, y = get_batch(None, 4, 256, "cpu", rng=rng, vocab_size=1024, mock_data=True)
        metrics = pipelined_train_overlap(wrapped, optimizer, x, y, [4, 256, 128], 2, 0, cross_entropy,
                                          dtype=torch.float32, device=torch.device("cpu"), pp_group=group,
                                          dp_group=group, router_aux_loss_coef=0.05, return_metrics=True)
        rows.append({k: float(v) for k, v in metrics.items()})
    torch.save({"metrics": rows}, out_path)
else:
    # resume from a checkpoint written by the other framework with the reference's own loader, run step seven
    from implementation.train_utils import load_checkpoint_async_dist  # noqa: E402
    iteration = load_checkpoint_async_dist(sys.argv[5], wrapped, optimizer)
    for _ in range(6):
        get_batch(None, 4, 256, "cpu", rng=rng, vocab_size=1024, mock_data=True)
    torch.save({"iteration": iteration, "loss7": one_step()}, out_path)
dist.destroy_process_group()
