"""Rank mesh ``[pipeline, replica (ddp), shard (fsdp = ep)]``.

Rank ``r`` sits at stage ``r // (fsdp*ddp)``; inside a stage block the replica
index is the slow axis and the shard index the fast one (reference
implementation/startup.py:26-52).  The expert-parallel group is the FSDP group
(reference distributed_parallel_training_pipelined.py:172).
"""
from __future__ import annotations

from dataclasses import dataclass, field

__all__ = ["parallel_sizes", "parallel_rank_groups", "Mesh", "build_groups"]


def parallel_sizes(train: dict) -> tuple[int, int]:
    """``(fsdp, ddp)``.  A config without ``fsdp_parallel_num`` is the legacy
    FSDP-only form: ``fsdp = data_parallel_num`` and one replica."""
    if "fsdp_parallel_num" in train:
        sizes = (train["fsdp_parallel_num"], train["data_parallel_num"])
    else:
        sizes = (train["data_parallel_num"], 1)
    for size in sizes:
        if type(size) is not int or size < 1:
            raise ValueError("FSDP and DDP sizes must be positive integers")
    return sizes


def parallel_rank_groups(train: dict, world_size: int, local_world_size: int) -> dict[str, list[list[int]]]:
    """Families of rank lists: ``fsdp``, ``ddp``, ``data`` (a whole stage block)
    and ``pp``.  A stage block never straddles a node."""
    fsdp, ddp = parallel_sizes(train)
    pp = train["pipeline_parallel_stages"]
    if type(pp) is not int or pp < 1 or world_size != pp * fsdp * ddp:
        raise ValueError(
            "fsdp_parallel_num * data_parallel_num * pipeline_parallel_stages must equal world size")
    width = fsdp * ddp
    if local_world_size < 1 or world_size % local_world_size or local_world_size % width:
        raise ValueError("FSDP * DDP must divide gpu_per_node to keep each stage block node-local")
    blocks = [list(range(base, base + width)) for base in range(0, world_size, width)]
    families: dict[str, list[list[int]]] = {"fsdp": [], "ddp": [], "data": blocks, "pp": []}
    for block in blocks:
        for replica in range(ddp):
            families["fsdp"].append(block[replica * fsdp:(replica + 1) * fsdp])
        for shard in range(fsdp):
            families["ddp"].append(block[shard::fsdp])
    for offset in range(width):
        families["pp"].append(list(range(offset, world_size, width)))
    return families


@dataclass
class Mesh:
    """Where one rank sits and the process groups it belongs to."""
    rank: int
    world_size: int
    fsdp: int
    ddp: int
    pp: int
    groups: dict = field(default_factory=dict)
    rank_lists: dict = field(default_factory=dict)

    @property
    def width(self) -> int:
        return self.fsdp * self.ddp

    @property
    def stage(self) -> int:
        return self.rank // self.width

    @property
    def dp_idx(self) -> int:
        """Flattened data index inside the stage block; names checkpoint shards
        and seeds the sampler (reference main:147,183)."""
        return self.rank % self.width

    @property
    def shard_idx(self) -> int:
        return self.dp_idx % self.fsdp

    @property
    def replica_idx(self) -> int:
        return self.dp_idx // self.fsdp

    def group(self, family: str):
        return self.groups.get(family)

    def ranks(self, family: str) -> list[int]:
        return self.rank_lists[family]


def build_groups(train: dict, rank: int, world_size: int, local_world_size: int, timeout=None) -> Mesh:
    """Create every group of every family on every rank (``new_group`` is
    collective) and keep the ones this rank belongs to (reference main:148-155)."""
    import torch.distributed as dist
    fsdp, ddp = parallel_sizes(train)
    mesh = Mesh(rank, world_size, fsdp, ddp, train["pipeline_parallel_stages"])
    for family, lists in parallel_rank_groups(train, world_size, local_world_size).items():
        for ranks in lists:
            kwargs = {"timeout": timeout} if timeout is not None else {}
            group = dist.new_group(ranks=ranks, **kwargs)
            if rank in ranks:
                mesh.groups[family] = group
                mesh.rank_lists[family] = ranks
    return mesh
