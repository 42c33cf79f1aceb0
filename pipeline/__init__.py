"""Pipeline training schedules (names of the reference's ``pipeline`` package)."""
from b200moe.parallel.pipeline import pipelined_train, pipelined_train_overlap

__all__ = ["pipelined_train", "pipelined_train_overlap"]
