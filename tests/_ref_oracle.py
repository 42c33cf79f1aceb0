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

torch.manual_seed(0)
group = dist.new_group([0])
model = TransformerLMPipelined(1024, 256, 128, 2, 4, 0, 1, num_expert_per_node=4, d_ff=256, dp_group=group,
                               moe_compute_dtype=torch.bfloat16)
init = {k: v.clone() for k, v in model.state_dict().items()}
wrapped = FSDPWrapperPipelined(model, FSDP_communication_group=group, compute_dtype=torch.float32,
                               moe_compute_dtype=torch.bfloat16)
optimizer = AdamW(wrapped.parameters(), lr=3e-4, betas=(0.9, 0.999), weight_decay=0.01)
rng = np.random.default_rng(0)
losses, grads = [], None
for step in range(6):
    x, y = get_batch(None, 4, 256, "cpu", rng=rng, vocab_size=1024, mock_data=True)
    loss = pipelined_train_overlap(wrapped, optimizer, x, y, [4, 256, 128], 2, 0, cross_entropy, dtype=torch.float32,
                                   device=torch.device("cpu"), pp_group=group, dp_group=group)
    losses.append(float(loss))
    if grads is None:
        grads = {n: p.grad.detach().float().clone() for n, p in wrapped.named_parameters() if p.grad is not None}
torch.save({"init": init, "losses": losses, "grads": grads}, out_path)
dist.destroy_process_group()
