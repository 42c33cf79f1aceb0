"""One rank of the unmodified reference package (``baseline/_ref``) on CPU/gloo, several ranks per run: FSDP x EP
(and PP) training steps on a tiny configuration.  Saves the rank's initial state (before wrapping), its losses and
its parameter shards after the last step.  Started once per rank as a separate process that has only the reference
on ``sys.path``.  Arguments: reference root, output directory, port, world size, pipeline stages, rank."""
import os
import sys

ref_root, out_dir, port, world, pp, rank = sys.argv[1], sys.argv[2], sys.argv[3], int(sys.argv[4]), int(sys.argv[5]), \
    int(sys.argv[6])
here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != here]
sys.path.insert(0, ref_root)
os.chdir(ref_root)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": port})
torch.set_num_threads(2)
dist.init_process_group("gloo", rank=rank, world_size=world)
from implementation.distributed.ddp_modules import FSDPWrapperPipelined  # noqa: E402
from implementation.layers import TransformerLMPipelined  # noqa: E402
from implementation.nnfunctions import cross_entropy  # noqa: E402
from implementation.optimizer import AdamW  # noqa: E402
from implementation.train_utils import get_batch  # noqa: E402
from pipeline import pipelined_train_overlap  # noqa: E402

fsdp = world // pp
stage, shard = rank // fsdp, rank % fsdp
fsdp_groups = [dist.new_group(list(range(s * fsdp, (s + 1) * fsdp))) for s in range(pp)]
pp_groups = [dist.new_group(list(range(o, world, fsdp))) for o in range(fsdp)]
fsdp_group, pp_group = fsdp_groups[stage], pp_groups[shard]
V, S, D, L, H, E, FF, B, STEPS = 512, 64, 64, 2, 4, 4, 128, 4, 4
torch.manual_seed(100 + rank)                 # every rank has its own experts
model = TransformerLMPipelined(V, S, D, L, H, stage, pp, num_expert_per_node=E // fsdp, d_ff=FF, dp_group=fsdp_group,
                               moe_compute_dtype=torch.bfloat16)
init = {k: v.clone() for k, v in model.state_dict().items()}
wrapped = FSDPWrapperPipelined(model, FSDP_communication_group=fsdp_group, compute_dtype=torch.float32,
                               moe_compute_dtype=torch.bfloat16)
optimizer = AdamW(wrapped.parameters(), lr=1e-3, betas=(0.9, 0.999), weight_decay=0.01)
rng = np.random.default_rng(shard)
losses = []
for _ in range(STEPS):
    x = y = None
    if stage in (0, pp - 1):
        x, y = get_batch(None, B, S, "cpu", rng=rng, vocab_size=V, mock_data=True)
    loss = pipelined_train_overlap(wrapped, optimizer, x if stage == 0 else None, y if stage == pp - 1 else None,
                                   [B, S, D], 2, stage, cross_entropy, dtype=torch.float32, device=torch.device("cpu"),
                                   pp_group=pp_group, dp_group=fsdp_group)
    losses.append(float(loss))
final = {k: v.detach().float().clone() for k, v in wrapped.state_dict().items()}
torch.save({"init": init, "losses": losses, "final": final, "stage": stage, "shard": shard},
           os.path.join(out_dir, f"ref_{rank}.pt"))
dist.barrier()
dist.destroy_process_group()
